"""NPVQLinear: ``nn.Linear`` replacement whose weight is packed codebook indices.

    ``W[n, g*VL + v] = centroids[packed_indices[n * n_groups + g], v]``

Same module surface as the reference (neuropress/nn/np_vq_linear.py): :class:`VQProxy`
(:399-455) holds the shared fp16 codebook and is *not* a sub-module of the layers that use it;
:class:`NPVQLinear` (:463-1424) resolves its backend once in the constructor, keeps the buffers
``packed_indices`` / ``bias`` / ``column_perm`` and routes each call by its row count:

    rows <= fused max        -> fused index-decode GEMV           (``_forward_cuda*``)
    rows <= tile-decode max  -> tile-decode tensor-core GEMM      (``_forward_triton``)
    otherwise                -> one-pass decode + dense GEMM      (``_forward_dequant_gemm``)

with the thresholds read from ``NEUROPRESS_VQ_FUSED_MAX_TOKENS``, ``NEUROPRESS_VQ_LUT_MAX_TOKENS``
and ``NEUROPRESS_VQ_TRITON_MAX_TOKENS`` at import time (reference :67-98, dispatch :1029-1037,
edges inclusive, leading dimensions count as rows).  Every band is a CUDA kernel of this
package; there is no Triton, no ``torch.compile`` and no CPU path.

Differences from the reference, all deliberate:
  * ``backend="auto"`` does not fall back to ``compile`` for ``vector_len != 4`` (the reference
    does, :154-157, because its tensor-core / LUT kernels are compiled for 4 only).
  * ``cuda_lut`` layers use the same bands as ``cuda_wmma`` layers: their fused maximum
    defaults to 2 rows instead of 0 and they do not skip the tile-decode band (:75-79, :1035).
  * ``default`` / ``compile`` and the entropy-coded backends (``cuda_tiered``, ``cuda_ntier``,
    ``cuda_zero_escape``) are accepted as names but not implemented: ``forward`` raises.
  * optional extended weight forms: ``residual_proxy`` + ``residual_indices`` (a second
    codebook added in fp16), ``row_scale`` (fp16 per output row, multiplied in fp16) and
    ``cols_per_codebook`` (the proxy holds ``[n_cb, NC, VL]``: one codebook per block of
    input columns).
"""

from __future__ import annotations

import logging
import os

import torch
import torch.nn as nn

from .backends import Backend, VQBackend, is_cuda_jit_available

log = logging.getLogger(__name__)

# Minimum out_features / num_centroids ratio for AUTO to choose CUDA_LUT (reference :67).
_LUT_COV_MIN: float = 4.0

# Row-count bands (reference :73, :79, :87).  The reference's values were measured on a GB10;
# these are the B200 defaults.
_FUSED_MAX_TOKENS: int = int(os.environ.get("NEUROPRESS_VQ_FUSED_MAX_TOKENS", "2"))
_LUT_MAX_TOKENS: int = int(os.environ.get("NEUROPRESS_VQ_LUT_MAX_TOKENS", "2"))
_TRITON_MAX_TOKENS: int = int(os.environ.get("NEUROPRESS_VQ_TRITON_MAX_TOKENS", "384"))

# Not in the reference: between the GEMV band and the tile-decode band, batches up to this many
# rows run the tensor-core small-batch kernel (decode in registers, mma.sync) where the weight
# form allows it (see NPVQLinear._small_batch_ok); 0 switches the band off.
_SMALL_BATCH_MAX_TOKENS: int = int(os.environ.get("NEUROPRESS_B200_VQ_SMALL_BATCH_MAX_TOKENS", "16"))

# cuda_lut layers take the tile-decode band too (the reference skips it for them).
_LUT_SKIPS_TILE_BAND: bool = False

_FUSED_BACKENDS = frozenset({VQBackend.CUDA_WMMA, VQBackend.CUDA_LUT, VQBackend.CUDA})
_ENTROPY_BACKENDS = frozenset({VQBackend.CUDA_TIERED, VQBackend.CUDA_NTIER, VQBackend.CUDA_ZERO_ESCAPE})
_UNIMPLEMENTED = frozenset({VQBackend.DEFAULT, VQBackend.COMPILE})


def _fused_max_tokens(backend: VQBackend) -> int:
    """Largest row count for which *backend*'s fused GEMV is used."""
    return _LUT_MAX_TOKENS if backend == VQBackend.CUDA_LUT else _FUSED_MAX_TOKENS


def _resolve_vq_backend(
    backend: str | VQBackend | Backend | None,
    use_tiered: bool = False,
    use_ntier: bool = False,
    use_zero_escape: bool = False,
    bits: int = 8,
    out_features: int = 0,
    num_centroids: int = 0,
    vector_len: int = 4,
) -> VQBackend:
    """Resolve a backend alias to a concrete :class:`VQBackend`, once, at construction.

    AUTO priority (reference :158-169): zero-escape > n-tier > tiered > ``bits > 12`` -> LUT >
    ``out_features / num_centroids >= 4`` -> LUT > WMMA; ``compile`` when the kernels are not
    available.  ``None`` / ``"torch"`` mean DEFAULT; unknown strings raise ``ValueError``.
    ``vector_len`` is accepted for signature compatibility and does not change the result.
    """
    if backend is None or backend == "torch":
        return VQBackend.DEFAULT
    if isinstance(backend, VQBackend | Backend):
        val = backend.value
    elif isinstance(backend, str):
        val = backend
    else:
        val = str(backend)
    if val != "auto":
        return VQBackend(val)
    if is_cuda_jit_available():
        if use_zero_escape:
            return VQBackend.CUDA_ZERO_ESCAPE
        if use_ntier:
            return VQBackend.CUDA_NTIER
        if use_tiered:
            return VQBackend.CUDA_TIERED
        if bits > 12:
            return VQBackend.CUDA_LUT
        if num_centroids > 0 and out_features / num_centroids >= _LUT_COV_MIN:
            return VQBackend.CUDA_LUT
        return VQBackend.CUDA_WMMA
    return VQBackend.COMPILE


class VQProxy(nn.Module):
    """Shared VQ codebook holder: buffer ``centroids``, always stored fp16 (reference :399-455).

    ``centroids`` is ``[num_centroids, vector_len]``, or ``[n_codebooks, num_centroids,
    vector_len]`` for layers that use one codebook per block of input columns.  One proxy is
    shared by every layer quantized with the same codebook; the model owner registers it on
    the model root so it appears once in ``state_dict``.
    """

    centroids: torch.Tensor

    def __init__(self, centroids: torch.Tensor) -> None:
        super().__init__()
        if centroids.dim() not in (2, 3):
            raise ValueError("centroids must be [NC, VL] or [n_codebooks, NC, VL].")
        self.register_buffer("centroids", centroids.to(torch.float16).contiguous())

    @property
    def num_centroids(self) -> int:
        return self.centroids.shape[-2]

    @property
    def vector_len(self) -> int:
        return self.centroids.shape[-1]

    def extra_repr(self) -> str:
        return f"num_centroids={self.num_centroids}, vector_len={self.vector_len}"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise RuntimeError(
            "VQProxy.forward() should not be called.  Access centroids directly via "
            "self.proxy.centroids."
        )


class NPVQLinear(nn.Module):
    """Linear layer whose weight is packed VQ indices plus a shared :class:`VQProxy`.

    Constructor arguments follow the reference (:493-513).  With ``use_tiered``, ``tier_bits`` or
    ``zero_escape`` the ``packed_indices`` buffer holds an entropy-coded stream
    (``TieredIndexPacking`` / ``NTieredIndexPacking`` / ``ZeroEscapePacking``) and the per-row
    offsets are buffers named as in the reference (``hot_row_offsets``, ``cold_row_offsets``,
    ``ntier_row_off_{k}``, ``zesc_row_off_{k}``; computed here when not passed).  Such a layer
    expands its stream to plain 16-bit indices on the GPU at every forward
    (``npb_vq_entropy_expand``) and then takes the same row-count bands as a plain layer; the
    coded buffer stays whole (the reference splits it into per-stream buffers, :644-801).
    Keyword-only extensions: ``residual_proxy``, ``residual_indices``, ``residual_bits``,
    ``row_scale``, ``cols_per_codebook``.
    """

    def __init__(
        self,
        proxy: VQProxy,
        packed_indices: torch.Tensor,
        bits: int,
        out_features: int,
        in_features: int,
        vector_len: int,
        backend: str | VQBackend | None,
        bias: torch.Tensor | None = None,
        column_perm: torch.Tensor | None = None,
        use_tiered: bool = False,
        cold_bits: int = 8,
        hot_row_offsets: torch.Tensor | None = None,
        cold_row_offsets: torch.Tensor | None = None,
        qtensor_meta: dict[str, str] | None = None,
        tier_bits: list[int] | None = None,
        ntier_row_offsets: list[torch.Tensor] | None = None,
        zero_escape: bool = False,
        zesc_row_offsets: list[torch.Tensor] | None = None,
        *,
        residual_proxy: VQProxy | None = None,
        residual_indices: torch.Tensor | None = None,
        residual_bits: int | None = None,
        row_scale: torch.Tensor | None = None,
        cols_per_codebook: int = 0,
    ) -> None:
        super().__init__()
        if in_features % vector_len:
            raise ValueError("in_features must be a multiple of vector_len.")
        if proxy.vector_len != vector_len:
            raise ValueError("vector_len does not match the proxy's codebook.")
        if (proxy.centroids.dim() == 3) != (cols_per_codebook > 0):
            raise ValueError("a 3-D codebook and cols_per_codebook > 0 go together.")
        if (residual_proxy is None) != (residual_indices is None):
            raise ValueError("residual_proxy and residual_indices must be given together.")
        self._qtensor_meta = qtensor_meta
        self.out_features = out_features
        self.in_features = in_features
        self.vector_len = vector_len
        self.bits = bits
        self.n_vectors = out_features * (in_features // vector_len)
        self.use_tiered = use_tiered
        self.cold_bits = cold_bits
        self.tier_bits: list[int] | None = tier_bits
        self.zero_escape: bool = zero_escape
        self.cols_per_codebook = int(cols_per_codebook)
        self.backend = _resolve_vq_backend(
            backend,
            use_tiered=use_tiered,
            use_ntier=tier_bits is not None,
            use_zero_escape=zero_escape,
            bits=bits,
            out_features=out_features,
            num_centroids=proxy.num_centroids,
            vector_len=vector_len,
        )
        # Plain attributes, not sub-modules: shared codebooks must not be duplicated in
        # state_dict (reference :588-590).
        object.__setattr__(self, "proxy", proxy)
        object.__setattr__(self, "residual_proxy", residual_proxy)

        self.register_buffer("packed_indices", packed_indices.contiguous())
        self.register_buffer("bias", None if bias is None else bias.contiguous())
        self.register_buffer("column_perm",
                             None if column_perm is None else column_perm.to(torch.int64))
        self.register_buffer("residual_indices",
                             None if residual_indices is None else residual_indices.contiguous())
        self.register_buffer("row_scale",
                             None if row_scale is None
                             else row_scale.to(torch.float16).reshape(-1).contiguous())
        if residual_proxy is not None:
            from ..transforms.vq_packing import IndexPacking

            self.residual_bits = (residual_bits if residual_bits is not None
                                  else IndexPacking.bits_for(residual_proxy.num_centroids))
        else:
            self.residual_bits = 8
        if self.row_scale is not None and self.row_scale.numel() != out_features:
            raise ValueError("row_scale must have out_features elements.")
        self._bias_f32: torch.Tensor | None = None
        self._bias_key = None
        self._entropy_scheme: str | None = None
        self._entropy_layout: dict | None = None
        self._decode_ahead = None   # a decode_ahead.DecodeAhead that prefetches this layer's dense weight
        if zero_escape or tier_bits is not None or use_tiered:
            self._init_entropy(hot_row_offsets, cold_row_offsets, ntier_row_offsets, zesc_row_offsets)

    def _init_entropy(self, hot, cold, ntier, zesc) -> None:
        """Row-offset buffers (reference names, :604-625) and the host-side description of where
        the coded buffer's sub-streams sit; offsets that were not passed are computed by the
        packers, as ``from_qtensor_linear`` does in the reference (:878-895)."""
        from ..transforms.entropy_packing import (NTieredIndexPacking, TieredIndexPacking, ZeroEscapePacking,
                                                  describe_entropy_buffer)

        groups = self.in_features // self.vector_len
        if self.zero_escape:
            scheme, names = "zero_escape", [f"zesc_row_off_{i}" for i in range(4)]
            offs = zesc if zesc is not None else ZeroEscapePacking.compute_row_offsets(
                self.packed_indices, self.out_features, groups)
        elif self.tier_bits is not None:
            scheme, names = "ntier", [f"ntier_row_off_{i}" for i in range(len(self.tier_bits))]
            offs = ntier if ntier is not None else NTieredIndexPacking.compute_row_offsets(
                self.packed_indices, self.out_features, groups)
        else:
            scheme, names = "tiered", ["hot_row_offsets", "cold_row_offsets"]
            offs = [hot, cold] if hot is not None and cold is not None else list(
                TieredIndexPacking.compute_row_offsets(self.packed_indices, self.out_features, groups))
        layout = describe_entropy_buffer(self.packed_indices, scheme)
        if len(offs) != len(names) or len(layout["bits"]) != len(names):
            raise ValueError("row offsets do not match the coded buffer's tiers.")
        if layout["n"] != self.n_vectors:
            raise ValueError(f"coded buffer holds {layout['n']} indices, the layer needs {self.n_vectors}.")
        if max(layout["bits"]) > 16 or self.proxy.num_centroids > 65536:
            raise ValueError("entropy-coded layers are expanded to 16-bit indices: tiers wider than 16 bits "
                             "and codebooks beyond 65536 entries are not supported.")
        for name, off in zip(names, offs):
            self.register_buffer(name, off.to(device=self.packed_indices.device, dtype=torch.int32).contiguous())
        self._entropy_scheme, self._entropy_layout, self._entropy_names = scheme, layout, names

    def _stream(self) -> tuple[torch.Tensor, int]:
        """The plain index stream the band kernels read and its width: the ``packed_indices``
        buffer itself, or, for an entropy-coded layer, its expansion to 16-bit indices."""
        if self._entropy_scheme is None:
            return self.packed_indices, self.bits
        from .. import kernels

        plain = kernels.vq_entropy_expand(self.packed_indices, self._entropy_layout,
                                          [getattr(self, n) for n in self._entropy_names], self.out_features,
                                          self.in_features // self.vector_len)
        return plain, 16

    # ------------------------------------------------------------------ factory / serde
    @classmethod
    def from_qtensor_linear(cls, linear: nn.Linear, proxy: VQProxy,
                            backend: str | VQBackend | None = VQBackend.AUTO) -> "NPVQLinear":
        """Build from an ``nn.Linear`` whose ``weight`` is a VQ QTensor (reference :831-921).

        The weight is read by attribute, the way the reference reads it:
        ``weight.qscheme.{centroids, vector_len, is_packed_indices, column_permutation,
        use_tiered, tier_bits, zero_escape}`` and ``weight.u8_blob``.  Any object with those
        attributes is accepted; anything else raises ``TypeError``.
        """
        weight_q = linear.weight
        qscheme = getattr(weight_q, "qscheme", None)
        if qscheme is None or not hasattr(qscheme, "centroids") or not hasattr(weight_q, "u8_blob"):
            raise TypeError(f"Expected a VQ QTensor weight, got {type(weight_q).__name__!r}.")
        bias = linear.bias.detach().clone() if linear.bias is not None else None
        perm = getattr(qscheme, "column_permutation", None)
        meta = weight_q.serde_metadata() if hasattr(weight_q, "serde_metadata") else {}
        return cls(
            proxy=proxy,
            packed_indices=weight_q.u8_blob.detach().clone(),
            bits=qscheme.is_packed_indices,
            out_features=linear.out_features,
            in_features=linear.in_features,
            vector_len=qscheme.vector_len,
            backend=backend,
            bias=bias,
            column_perm=None if perm is None else perm.detach().clone(),
            use_tiered=bool(getattr(qscheme, "use_tiered", False)),
            cold_bits=qscheme.is_packed_indices,
            qtensor_meta=meta,
            tier_bits=getattr(qscheme, "tier_bits", None),
            zero_escape=bool(getattr(qscheme, "zero_escape", False)),
        )

    def to_qtensor(self):
        """Rebuild the VQ QTensor stand-in for saving / unlowering (reference :977-1008).

        Raises ``RuntimeError`` when the module was not built by :meth:`from_qtensor_linear`.
        """
        if self._qtensor_meta is None:
            raise RuntimeError(
                "Cannot reconstruct QTensor: no serde metadata stored. "
                "Build via NPVQLinear.from_qtensor_linear() to enable to_qtensor()."
            )
        from ..qtensor import VQQTensor, VQScheme

        scheme = VQScheme(centroids=self.proxy.centroids, vector_len=self.vector_len,
                          is_packed_indices=self.bits, column_permutation=self.column_perm,
                          use_tiered=self.use_tiered, tier_bits=self.tier_bits, zero_escape=self.zero_escape,
                          original_shape=(self.out_features, self.in_features))
        meta = {k: v for k, v in self._qtensor_meta.items() if k not in ("type", "shape")}
        return VQQTensor(u8_blob=self.packed_indices, qscheme=scheme,
                         shape=(self.out_features, self.in_features), meta=meta)

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, gather=None) -> torch.Tensor:
        """Route by row count exactly as the reference does (:1014-1058).

        ``gather`` (not in the reference) is a ``sharding.PushGather``: this module then holds
        an out-feature shard, and the result is the all-gathered ``[..., N_full]``.  Where the
        band's kernel can store into the peers' buffers itself it does (fused all-gather);
        otherwise the local result is pushed by a separate kernel."""
        if self.column_perm is not None:
            x = x[..., self.column_perm]
        if self.backend in _ENTROPY_BACKENDS and self._entropy_scheme is None:
            raise RuntimeError(f"backend {self.backend.value!r} needs an entropy-coded packed_indices buffer "
                               "(use_tiered / tier_bits / zero_escape).")
        if self.backend in _FUSED_BACKENDS or self.backend in _ENTROPY_BACKENDS:
            m = x.numel() // self.in_features
            if m > _fused_max_tokens(self.backend):
                if m <= _SMALL_BATCH_MAX_TOKENS and self._small_batch_ok(x, m):
                    return self._forward_gemv(x, gather)
                skip_tile = _LUT_SKIPS_TILE_BAND and self.backend == VQBackend.CUDA_LUT
                if not skip_tile and m <= _TRITON_MAX_TOKENS:
                    return self._forward_triton(x, gather)
                return self._forward_dequant_gemm(x, gather)
        if self.backend == VQBackend.CUDA_LUT:
            return self._forward_cuda_lut(x, gather)
        if self.backend == VQBackend.CUDA_WMMA:
            return self._forward_cuda_wmma(x, gather)
        if self.backend == VQBackend.CUDA or self.backend in _ENTROPY_BACKENDS:
            return self._forward_cuda(x, gather)
        raise NotImplementedError(
            f"backend {self.backend.value!r} is not implemented by this package: only the CUDA "
            "backends exist here; there is no eager or compiled path."
        )

    # -- helpers
    def _ext(self) -> dict:
        d: dict = {}
        if self.residual_indices is not None:
            d.update(residual_indices=self.residual_indices,
                     residual_centroids=self.residual_proxy.centroids,
                     residual_bits=self.residual_bits)
        if self.row_scale is not None:
            d["row_scale"] = self.row_scale
        if self.cols_per_codebook:
            d["cols_per_codebook"] = self.cols_per_codebook
        return d

    def _bias32(self) -> torch.Tensor | None:
        """fp32 copy of the bias.  The reference re-casts on every call
        (vq_linear_wmma.cu:512-515); here the copy is kept and remade whenever the ``bias``
        buffer was replaced, moved or written in place (``load_state_dict`` copies in place
        and bumps the tensor's version counter)."""
        if self.bias is None:
            return None
        key = (self.bias.data_ptr(), self.bias._version, self.bias.device)
        if self._bias_f32 is None or self._bias_key != key:
            self._bias_f32 = self.bias.detach().to(torch.float32).contiguous()
            self._bias_key = key
        return self._bias_f32

    def _apply(self, fn, recurse: bool = True):
        self._bias_f32 = None
        return super()._apply(fn, recurse)

    def _flat(self, x: torch.Tensor) -> tuple[torch.Tensor, list[int]]:
        *leading, _ = x.shape
        return x.reshape(-1, self.in_features).contiguous(), leading

    def _small_batch_ok(self, x: torch.Tensor, m: int) -> bool:
        """Whether ``npb_vq_gemv`` takes *m* (3..16) rows of *x* on its tensor-core path: the
        conditions of ``vq_gemv_mma`` (csrc/vq_gemv_mma.cu) plus its shared-memory budget."""
        k = self.in_features
        if x.dtype not in (torch.bfloat16, torch.float16) or self.vector_len != 8:
            return False
        bits = 16 if self._entropy_scheme is not None else self.bits
        if bits not in (8, 12, 16) or k % 1024 or k > (4096 if m > 8 else 8192):
            return False
        if self.cols_per_codebook and self.cols_per_codebook % 256:
            return False
        if self.residual_indices is not None and (self.residual_bits != 8
                                                  or self.residual_proxy.num_centroids > 256):
            return False
        return True

    # -- band (a): fused index-decode GEMV
    def _forward_gemv(self, x: torch.Tensor, gather=None) -> torch.Tensor:
        from .. import kernels

        x2, leading = self._flat(x)
        fused = gather is not None and gather.accepts(x2.shape[0], x2.dtype)
        packed, bits = self._stream()
        y = kernels.vq_gemv(x2, packed, self.proxy.centroids, bits,
                            self.out_features, self._bias32(), gather=gather if fused else None,
                            **self._ext())
        if gather is not None and not fused:
            y = gather(y)
        return y.reshape(*leading, y.shape[-1])

    def _forward_cuda(self, x: torch.Tensor, gather=None) -> torch.Tensor:
        """Fused GEMV, fp16 / bf16 / fp32 activations natively (reference :1173-1187)."""
        return self._forward_gemv(x, gather)

    def _forward_cuda_wmma(self, x: torch.Tensor, gather=None) -> torch.Tensor:
        """Reference :1250-1267.  The reference casts fp32 activations to fp16 first; the GEMV
        here accumulates in fp32 from any activation dtype, so no cast is needed."""
        return self._forward_gemv(x, gather)

    def _forward_cuda_lut(self, x: torch.Tensor, gather=None) -> torch.Tensor:
        """Reference :1189-1248 builds an ``[M, G, NC]`` table in global memory and gathers
        from it, which loses to decoding at every row count (:75-79).  Here ``cuda_lut`` layers
        (large codebooks, large ``N / NC``) run the same fused GEMV, which gathers 16-byte
        centroids through L1 / L2 instead."""
        return self._forward_gemv(x, gather)

    # -- band (b): tile-decode tensor-core GEMM (the reference's Triton band)
    def _forward_triton(self, x: torch.Tensor, gather=None) -> torch.Tensor:
        """Tile-decode GEMM on the tcgen05 tensor cores; the method keeps the reference's
        name (:1097-1125).  Shapes or dtypes the kernel does not take go to decode + GEMM."""
        from .. import kernels

        if (not kernels.VQ_TILE_DECODE_GEMM or x.dtype not in (torch.bfloat16, torch.float16)
                or self.vector_len != 8 or self.in_features % 64
                or (self.cols_per_codebook and self.cols_per_codebook % 64)
                or (self.residual_indices is not None and self.residual_proxy.num_centroids > 256)):
            return self._forward_dequant_gemm(x, gather)
        x2, leading = self._flat(x)
        packed, bits = self._stream()
        y = kernels.vq_gemm_fused(x2, packed, self.proxy.centroids, bits,
                                  self.out_features, self._bias32(), **self._ext())
        if gather is not None:
            y = gather(y)
        return y.reshape(*leading, y.shape[-1])

    # -- band (c): one-pass decode + dense tensor-core GEMM
    def _forward_dequant_gemm(self, x: torch.Tensor, gather=None) -> torch.Tensor:
        """Decode the weight once into a temporary ``[N, K]`` tensor in the activation dtype
        and run the dense GEMM (reference :1127-1148).  fp32 activations are computed in fp16,
        as the reference's tensor-core path does (:1254-1256)."""
        from .. import kernels

        orig = x.dtype
        if orig == torch.float32:
            x = x.to(torch.float16)
        x2, leading = self._flat(x)
        ahead = self._decode_ahead
        w = ahead.weight_for(self, x2.dtype) if ahead is not None else None
        if w is None:
            ahead = None
            w = self._decode_dense(x2.dtype)
        fused = gather is not None and orig == x2.dtype and gather.accepts(x2.shape[0], x2.dtype)
        y = kernels.gemm(x2, w, self._bias32(), gather=gather if fused else None)
        if ahead is not None:
            ahead.release(self)
        y = y.to(orig) if y.dtype != orig else y
        if gather is not None and not fused:
            y = gather(y)
        return y.reshape(*leading, y.shape[-1])

    def _decode_dense(self, dtype: torch.dtype, out: torch.Tensor | None = None) -> torch.Tensor:
        """The whole weight as a dense ``[N, K]`` matrix of ``dtype`` on the current stream (an
        entropy-coded stream is expanded first)."""
        from .. import kernels

        packed, bits = self._stream()
        return kernels.vq_dequant(packed, self.proxy.centroids, bits, self.out_features, self.in_features,
                                  dtype, out=out, **self._ext())

    def extra_repr(self) -> str:
        perm = ", perm=True" if self.column_perm is not None else ""
        ext = ""
        if self.residual_indices is not None:
            ext += f", residual={self.residual_proxy.num_centroids}"
        if self.row_scale is not None:
            ext += ", row_scale=True"
        if self.cols_per_codebook:
            ext += f", cols_per_codebook={self.cols_per_codebook}"
        if self._entropy_scheme is not None:
            ext += f", index_stream={self._entropy_scheme}"
        return (f"in={self.in_features}, out={self.out_features}, vector_len={self.vector_len}, "
                f"num_centroids={self.proxy.num_centroids}, bits={self.bits}, "
                f"backend={self.backend.value}{perm}{ext}")


def _is_vq_weight(w) -> bool:
    q = getattr(w, "qscheme", None)
    return q is not None and hasattr(q, "centroids") and hasattr(w, "u8_blob")


def linearize_vq_weights(model: nn.Module,
                         backend: str | VQBackend | None = VQBackend.AUTO) -> nn.Module:
    """Replace every ``nn.Linear`` whose weight is a VQ QTensor by an :class:`NPVQLinear`
    (reference :1432-1517).  Layers whose ``qscheme.centroids`` is the same tensor object share
    one :class:`VQProxy`; each proxy is registered on the model root as ``_vq_proxy_<i>``.
    Layers that cannot be converted are skipped with a warning.  Returns *model*."""
    proxy_cache: dict[int, VQProxy] = {}
    replacements: list[tuple[str, NPVQLinear]] = []
    for name, module in model.named_modules():
        if not isinstance(module, nn.Linear) or not _is_vq_weight(module._parameters.get("weight")):
            continue
        centroids = module.weight.qscheme.centroids
        proxy = proxy_cache.get(id(centroids))
        created = proxy is None
        if created:
            proxy = VQProxy(centroids)
        try:
            layer = NPVQLinear.from_qtensor_linear(module, proxy, backend)
        except (TypeError, ValueError) as exc:
            log.warning("linearize_vq_weights: skipping %s — %s", name, exc)
            continue
        if created:
            proxy_cache[id(centroids)] = proxy
        replacements.append((name, layer))
    if not replacements:
        log.info("linearize_vq_weights: no VQ-weight linear layers found.")
        return model
    for i, proxy in enumerate(proxy_cache.values()):
        model.add_module(f"_vq_proxy_{i}", proxy)
    for name, layer in replacements:
        parent = model.get_submodule(name.rsplit(".", 1)[0]) if "." in name else model
        setattr(parent, name.rsplit(".", 1)[-1], layer)
    counts: dict[str, int] = {}
    for _, layer in replacements:
        counts[layer.backend.value] = counts.get(layer.backend.value, 0) + 1
    log.info("linearize_vq_weights: replaced %d layer(s) [%s], %d unique proxy/ies",
             len(replacements), ", ".join(f"{v}x{k}" for k, v in sorted(counts.items())),
             len(proxy_cache))
    return model
