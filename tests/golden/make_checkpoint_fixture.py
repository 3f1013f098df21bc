"""Write ``reference_checkpoint.safetensors`` with the reference's own checkpoint code.

    python tests/golden/make_checkpoint_fixture.py /path/to/reference

The reference's ``save_quantized_model`` (neuropress/t2n/model_io.py:214-312) and its serde
handlers (neuropress/t2n/qtensors.py) are run unmodified on a tiny model whose quantized
weights are objects carrying exactly the attributes those handlers read (``u8_blob``,
``qscheme.*``, ``u8_compressors``, ``dequant_to_dtype`` ...), named like the reference's QTensor
classes because the handlers are looked up by class name.  ``torch_to_nnef`` is not installed;
the only thing the reference needs from it on this path is the empty base class
``U8Compressor`` of its ``BitPacking``, which is stubbed.  The file is therefore byte for byte
what the reference writes for this model; the tests load it into this package's modules and
save it back.
"""

from __future__ import annotations

import enum
import importlib
import sys
import types
from pathlib import Path

import torch
from torch import nn

HERE = Path(__file__).resolve().parent


def load_reference_io(root: Path):
    pkg = root / "neuropress"
    for name, sub in (("neuropress", ""), ("neuropress.t2n", "t2n"), ("neuropress.transforms", "transforms"),
                      ("neuropress.nn", "nn")):
        m = types.ModuleType(name)
        m.__path__ = [str(pkg / sub) if sub else str(pkg)]
        sys.modules[name] = m
    for name in ("torch_to_nnef", "torch_to_nnef.tensor", "torch_to_nnef.tensor.quant"):
        sys.modules[name] = types.ModuleType(name)
    base = types.ModuleType("torch_to_nnef.tensor.quant.base")
    base.U8Compressor = type("U8Compressor", (), {})   # abstract base only: no behaviour
    sys.modules["torch_to_nnef.tensor.quant.base"] = base
    return (importlib.import_module("neuropress.t2n.model_io"), importlib.import_module("neuropress.t2n.packing"),
            importlib.import_module("neuropress.transforms.vq_packing"))


def gen(seed: int) -> torch.Generator:
    g = torch.Generator()
    g.manual_seed(seed)
    return g


class _Hashable:
    __hash__ = object.__hash__


def build_model(packing, vq_packing):
    """q_proj / k_proj share one codebook (VQ, 12-bit and 8-bit streams, one with a column
    permutation); o_proj is Q4_0 group 32; up_proj is zero-point group 64; embed_tokens is a Q4_0
    table; norm is a plain parameter; one plain buffer."""
    Selector = enum.StrEnum("ProxySelector", {"L2": "l2"})

    class VQScheme(_Hashable):
        def __init__(self, centroids, bits, original_shape, perm=None):
            self.centroids, self.is_packed_indices, self.original_shape = centroids, bits, original_shape
            self.vector_len = centroids.shape[1]
            self.column_permutation, self.proxy_selector = perm, Selector.L2
            self.use_tiered, self.zero_escape, self.tier_bits = False, False, None

    class QTensorTractVQ(_Hashable):
        def __init__(self, blob, scheme, dtype):
            self.u8_blob, self.qscheme, self.dequant_to_dtype = blob, scheme, dtype
            self.u8_compressors, self.nnef_name = [], None

    class AffineScheme(_Hashable):
        def __init__(self, n_bits, group_size, scale, zero_point=None):
            self.n_bits, self.group_size, self.scale, self.zero_point = n_bits, group_size, scale, zero_point

    class QTensorTractScaleOnly(_Hashable):
        def __init__(self, blob, scheme, shape, dtype):
            self.u8_blob, self.qscheme, self.decompressed_shape, self.dequant_to_dtype = blob, scheme, shape, dtype
            self.u8_compressors, self.nnef_name = [packing.BitPacking(4)], "w_q40"

    class QTensorScaleZp(QTensorTractScaleOnly):
        export_as_float = False

    model = nn.Module()
    model.q_proj = nn.Linear(64, 48, bias=True)
    model.k_proj = nn.Linear(64, 16, bias=False)
    model.o_proj = nn.Linear(64, 32, bias=False)
    model.up_proj = nn.Linear(128, 24, bias=True)
    model.embed_tokens = nn.Embedding(20, 64)
    model.norm = nn.LayerNorm(64)
    model.register_buffer("steps", torch.arange(3))
    with torch.no_grad():
        for i, p in enumerate(pp for pp in model.parameters()):
            p.copy_(torch.randn(p.shape, generator=gen(50 + i)) * 0.1)
    IndexPacking = vq_packing.IndexPacking
    cent = (torch.randn(4096, 8, generator=gen(1)) * 0.02).to(torch.float16)
    iq = torch.randint(0, 4096, (48, 8), generator=gen(2))
    ik = torch.randint(0, 256, (16, 8), generator=gen(3))
    perm = torch.randperm(64, generator=gen(4))
    model.q_proj._parameters["weight"] = QTensorTractVQ(IndexPacking.pack(iq, 12), VQScheme(cent, 12, (48, 64)),
                                                        torch.bfloat16)
    model.k_proj._parameters["weight"] = QTensorTractVQ(IndexPacking.pack(ik, 8), VQScheme(cent, 8, (16, 64), perm),
                                                        torch.float16)

    def affine(n, k, gs, asym, seed):
        vals = torch.randint(0, 16, (n, k), generator=gen(seed)).to(torch.uint8)
        blob = packing.BitPacking(4).compress(vals)
        ng = n * k // gs
        scale = torch.exp(torch.randn(ng, 1, generator=gen(seed + 1)) * 0.3 - 4.0).to(torch.float16)
        if asym:
            zp = (torch.rand(ng, 1, generator=gen(seed + 2)) * 15).to(torch.float16)
            return QTensorScaleZp(blob, AffineScheme(4, gs, scale, zp), torch.Size((n, k)), torch.bfloat16)
        return QTensorTractScaleOnly(blob, AffineScheme(4, gs, scale), torch.Size((n, k)), torch.bfloat16)

    model.o_proj._parameters["weight"] = affine(32, 64, 32, False, 10)
    model.up_proj._parameters["weight"] = affine(24, 128, 64, True, 20)
    model.embed_tokens._parameters["weight"] = affine(20, 64, 32, False, 30)
    return model


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python make_checkpoint_fixture.py <path to a checkout of the reference repository>")
    model_io, packing, vq_packing = load_reference_io(Path(sys.argv[1]))
    model = build_model(packing, vq_packing)
    out = HERE / "reference_checkpoint.safetensors"
    model_io.save_quantized_model(model, out)
    print(f"wrote {out.name}: {out.stat().st_size} bytes")


if __name__ == "__main__":
    main()
