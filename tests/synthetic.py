"""Seeded synthetic weights and activations for the benchmark configurations.

No dataset or checkpoint is involved: like the reference's own per-layer bench
(neuropress/tools/bench.py:121-128, 291-305) every tensor is random, with the shapes, dtypes
and value distributions the benchmark configurations state.  Each tensor family has its own
``torch.Generator`` so that a tensor does not depend on which other tensors were drawn; all
are generated on the CPU and moved by the caller.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from neuropress_b200.transforms.vq_packing import IndexPacking


def _gen(seed: int, family: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed * 1000003 + family)
    return g


@dataclass
class VQLayerData:
    """One VQ-coded linear layer (CPU tensors)."""

    out_features: int
    in_features: int
    vector_len: int
    bits: int
    centroids: torch.Tensor                       # fp16 [NC, VL] or [n_cb, NC, VL]
    indices: torch.Tensor                         # int64 [N, G]
    packed: torch.Tensor                          # uint8 1-D bit-stream
    cols_per_codebook: int = 0
    residual_centroids: torch.Tensor | None = None
    residual_indices_raw: torch.Tensor | None = None
    residual_indices: torch.Tensor | None = None  # packed uint8
    residual_bits: int = 8
    row_scale: torch.Tensor | None = None         # fp16 [N]
    bias: torch.Tensor | None = None

    def ext(self) -> dict:
        """Keyword arguments for the extended weight forms (empty for the plain form)."""
        d: dict = {}
        if self.residual_indices is not None:
            d.update(residual_indices=self.residual_indices,
                     residual_centroids=self.residual_centroids,
                     residual_bits=self.residual_bits)
        if self.row_scale is not None:
            d["row_scale"] = self.row_scale
        if self.cols_per_codebook:
            d["cols_per_codebook"] = self.cols_per_codebook
        return d

    def to(self, device) -> "VQLayerData":
        kw = {}
        for k, v in self.__dict__.items():
            kw[k] = v.to(device) if isinstance(v, torch.Tensor) else v
        return VQLayerData(**kw)

    def packed_bytes(self) -> int:
        """Algorithmic weight bytes of one forward: index streams + row scale."""
        n = self.packed.numel()
        if self.residual_indices is not None:
            n += self.residual_indices.numel()
        if self.row_scale is not None:
            n += self.row_scale.numel() * 2
        return n


def make_vq_layer(out_features: int, in_features: int, *, num_centroids: int, bits: int | None = None,
                  vector_len: int = 8, centroid_std: float = 0.02, seed: int = 0,
                  residual_centroids: int = 0, residual_std: float = 0.005,
                  row_scale: bool = False, cols_per_codebook: int = 0,
                  bias: bool = False) -> VQLayerData:
    """Random VQ layer: centroids N(0, std) stored fp16, indices uniform over the codebook."""
    if bits is None:
        bits = IndexPacking.bits_for(num_centroids)
    G = in_features // vector_len
    n_cb = (in_features + cols_per_codebook - 1) // cols_per_codebook if cols_per_codebook else 0
    shape = (n_cb, num_centroids, vector_len) if n_cb else (num_centroids, vector_len)
    cent = (torch.randn(shape, generator=_gen(seed, 1)) * centroid_std).to(torch.float16)
    idx = torch.randint(0, num_centroids, (out_features, G), generator=_gen(seed, 2))
    data = VQLayerData(out_features, in_features, vector_len, bits, cent, idx,
                       IndexPacking.pack(idx, bits), cols_per_codebook=cols_per_codebook)
    if residual_centroids:
        data.residual_centroids = (
            torch.randn(residual_centroids, vector_len, generator=_gen(seed, 3)) * residual_std
        ).to(torch.float16)
        data.residual_bits = IndexPacking.bits_for(residual_centroids)
        data.residual_indices_raw = torch.randint(0, residual_centroids, (out_features, G),
                                                  generator=_gen(seed, 4))
        data.residual_indices = IndexPacking.pack(data.residual_indices_raw, data.residual_bits)
    if row_scale:
        data.row_scale = torch.exp(torch.randn(out_features, generator=_gen(seed, 5)) * 0.1).to(torch.float16)
    if bias:
        data.bias = torch.randn(out_features, generator=_gen(seed, 7)) * 0.1
    return data


@dataclass
class QLayerData:
    """One group-affine (Q4_0 / HQQ) linear layer (CPU tensors)."""

    out_features: int
    in_features: int
    nbits: int
    group_size: int
    codes: torch.Tensor                 # uint8 [N, K*nbits/8]
    scale: torch.Tensor                 # fp16 [N*K/g]
    zero_point: torch.Tensor | None     # fp16 [N*K/g] or None (symmetric)
    bias: torch.Tensor | None = None
    extra: dict = field(default_factory=dict)

    def to(self, device) -> "QLayerData":
        kw = {}
        for k, v in self.__dict__.items():
            kw[k] = v.to(device) if isinstance(v, torch.Tensor) else v
        return QLayerData(**kw)

    def packed_bytes(self) -> int:
        n = self.codes.numel() + self.scale.numel() * 2
        if self.zero_point is not None:
            n += self.zero_point.numel() * 2
        return n


def make_q_layer(out_features: int, in_features: int, *, group_size: int, asym: bool,
                 nbits: int = 4, seed: int = 0, bias: bool = False) -> QLayerData:
    """Q4_0 (``asym=False``: symmetric, implicit zero-point 8) or HQQ-style (``asym=True``: fp16
    zero-point uniform in [0, 15]); codes uniform, scale lognormal(-4, 0.3) fp16."""
    vpb = 8 // nbits
    vals = torch.randint(0, 1 << nbits, (out_features, in_features), generator=_gen(seed, 11),
                         dtype=torch.int64)
    g = vals.reshape(out_features, in_features // vpb, vpb)
    codes = torch.zeros(out_features, in_features // vpb, dtype=torch.int64)
    for i in range(vpb):
        codes |= g[:, :, i] << (i * nbits)
    n_groups = out_features * (in_features // group_size)
    scale = torch.exp(torch.randn(n_groups, generator=_gen(seed, 12)) * 0.3 - 4.0).to(torch.float16)
    zp = None
    if asym:
        zp = (torch.rand(n_groups, generator=_gen(seed, 13)) * 15.0).to(torch.float16)
    b = torch.randn(out_features, generator=_gen(seed, 14)) * 0.1 if bias else None
    return QLayerData(out_features, in_features, nbits, group_size, codes.to(torch.uint8), scale, zp, b)


def make_activations(rows: int, in_features: int, dtype: torch.dtype = torch.bfloat16,
                     seed: int = 0) -> torch.Tensor:
    """``[rows, in_features]`` N(0, 1) activations."""
    return torch.randn(rows, in_features, generator=_gen(seed, 6)).to(dtype)


# The large-codebook benchmark layer: in 4096, out 14336, 65536 x 8 fp16 main codebook with
# uint16 indices, 256-entry residual codebook with uint8 indices, fp16 per-row scale.
def make_c2_layer(seed: int = 0, out_features: int = 14336, in_features: int = 4096) -> VQLayerData:
    return make_vq_layer(out_features, in_features, num_centroids=65536, bits=16, seed=seed,
                         residual_centroids=256, row_scale=True)


C2_ROWS = (1, 2, 16, 128, 384, 2048)


# ---- drawn on the device (the full-size layers of the benchmark and of the full-size tests) ----
def device_bytes(n: int, device, seed: int) -> torch.Tensor:
    """``n`` uniform random bytes drawn on the device from a seeded generator."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.randint(0, 256, (n,), dtype=torch.uint8, device=device, generator=g)


def pack_indices_device(idx: torch.Tensor, bits: int) -> torch.Tensor:
    """LSB-first bit-stream of ``idx`` (any shape, flattened) for 16- or 12-bit indices, built on
    the device: 16 bits = little-endian uint16; 12 bits = two indices a, b in three bytes
    ``a & 255, (a >> 8) | ((b & 15) << 4), b >> 4``."""
    v = idx.reshape(-1).to(torch.int32)
    if bits == 16:
        return torch.stack([v & 0xFF, v >> 8], dim=1).to(torch.uint8).reshape(-1)
    if bits == 12 and v.numel() % 2 == 0:
        a, b = v[0::2], v[1::2]
        return torch.stack([a & 0xFF, (a >> 8) | ((b & 0xF) << 4), b >> 4], dim=1).to(torch.uint8).reshape(-1)
    raise ValueError("pack_indices_device: 16-bit, or 12-bit with an even count")


def device_normal(shape, device, seed: int, std: float = 1.0, dtype=torch.bfloat16) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return (torch.randn(shape, device=device, generator=g) * std).to(dtype)
