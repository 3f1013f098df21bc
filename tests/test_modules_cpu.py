"""Host-side logic of the drop-in modules: backend resolution, row-count bands, proxy sharing,
lowering configuration.  No GPU needed: the forward methods are replaced by spies, the way the
reference's own band tests do it (tests/nn/test_np_vq_linear.py:422-521 of the reference).
"""

from pathlib import Path

import numpy as np
import pytest
import torch
import torch.nn as nn

import neuropress_b200.nn.np_vq_linear as vqmod
from neuropress_b200 import _cabi
from neuropress_b200.kernel_lowering import (AutoKernelLowering, LoweringConfig, is_lowered,
                                             unlower_model)
from neuropress_b200.nn import (Backend, LinearBackend, NPLinear, NPVQLinear, VQBackend, VQProxy,
                                linearize_qtensor_weights, linearize_vq_weights)
from neuropress_b200.nn.np_linear import _pack_u8, _resolve_backend, _unpack_u8
from neuropress_b200.nn.np_vq_linear import _resolve_vq_backend
from neuropress_b200.qtensor import AffineQTensor, AffineScheme, VQQTensor, VQScheme
from neuropress_b200.transforms.vq_packing import IndexPacking

G = np.load(Path(__file__).parent / "golden" / "reference_vectors.npz")


def _vq_linear(out_features=16, in_features=32, nc=16, vl=4, centroids=None, bias=False):
    if centroids is None:
        centroids = torch.randn(nc, vl)
    idx = torch.randint(0, centroids.shape[0], (out_features * in_features // vl,))
    bits = IndexPacking.bits_for(centroids.shape[0])
    lin = nn.Linear(in_features, out_features, bias=bias)
    lin._parameters["weight"] = VQQTensor(IndexPacking.pack(idx, bits),
                                          VQScheme(centroids, vl, bits), (out_features, in_features))
    return lin


# ------------------------------------------------------------------ backend resolution
def test_explicit_names_resolve_as_in_reference(monkeypatch):
    monkeypatch.setattr(vqmod, "is_cuda_jit_available", lambda: False)
    got = []
    for name in ["auto", "default", "compile", "cuda", "cuda_wmma", "cuda_lut", None, "torch"]:
        r = _resolve_vq_backend(name, bits=16, out_features=14336, num_centroids=65536, vector_len=8)
        got.append(f"{name}->{r.value}")
    assert got == G["resolve_vq_cpu"].tolist()  # the reference's answers without CUDA kernels


def test_auto_resolution_with_kernels(monkeypatch):
    monkeypatch.setattr(vqmod, "is_cuda_jit_available", lambda: True)
    r = lambda **kw: _resolve_vq_backend("auto", **kw)  # noqa: E731
    assert r(bits=16, out_features=14336, num_centroids=65536, vector_len=8) == VQBackend.CUDA_LUT
    assert r(bits=12, out_features=2048, num_centroids=4096, vector_len=8) == VQBackend.CUDA_WMMA
    assert r(bits=12, out_features=16384, num_centroids=4096, vector_len=8) == VQBackend.CUDA_LUT
    assert r(bits=8, out_features=1023, num_centroids=256, vector_len=4) == VQBackend.CUDA_WMMA
    assert r(bits=8, out_features=1024, num_centroids=256, vector_len=4) == VQBackend.CUDA_LUT
    assert r(bits=8, use_tiered=True) == VQBackend.CUDA_TIERED
    assert r(bits=8, use_tiered=True, use_ntier=True) == VQBackend.CUDA_NTIER
    assert r(bits=8, use_ntier=True, use_zero_escape=True) == VQBackend.CUDA_ZERO_ESCAPE
    # vector length 8 is not demoted to "compile" (the reference's kernels are VL=4 only)
    assert r(bits=8, out_features=64, num_centroids=256, vector_len=8) == VQBackend.CUDA_WMMA


def test_enum_and_unknown_names():
    assert _resolve_vq_backend(Backend.CUDA_TIERED) == VQBackend.CUDA_TIERED
    assert _resolve_vq_backend(VQBackend.CUDA_LUT) == VQBackend.CUDA_LUT
    with pytest.raises(ValueError):
        _resolve_vq_backend("tensorrt")
    assert _resolve_backend("auto") == LinearBackend.CUDA
    assert _resolve_backend(None) == LinearBackend.DEFAULT
    assert _resolve_backend(Backend.GEMLITE) == LinearBackend.GEMLITE
    with pytest.raises(ValueError):
        _resolve_backend("cuda_wmma")


def test_band_defaults_and_env_names():
    fused, lut, tile, cov = (int(v) for v in G["band_defaults"])
    assert (vqmod._FUSED_MAX_TOKENS, vqmod._TRITON_MAX_TOKENS, int(vqmod._LUT_COV_MIN)) == (fused, tile, cov)
    assert lut == 0 and vqmod._LUT_MAX_TOKENS == 2  # documented difference for cuda_lut layers
    src = Path(vqmod.__file__).read_text()
    for var in ("NEUROPRESS_VQ_FUSED_MAX_TOKENS", "NEUROPRESS_VQ_LUT_MAX_TOKENS",
                "NEUROPRESS_VQ_TRITON_MAX_TOKENS"):
        assert var in src


# ------------------------------------------------------------------ row-count bands
def _layer_with_spies(monkeypatch, backend, fused_max=16, lut_max=16, tile_max=0):
    monkeypatch.setattr(vqmod, "_FUSED_MAX_TOKENS", fused_max)
    monkeypatch.setattr(vqmod, "_LUT_MAX_TOKENS", lut_max)
    monkeypatch.setattr(vqmod, "_TRITON_MAX_TOKENS", tile_max)
    lin = _vq_linear()
    layer = NPVQLinear.from_qtensor_linear(lin, VQProxy(lin.weight.qscheme.centroids), backend=backend)
    calls = []
    fused = {Backend.CUDA_WMMA: "_forward_cuda_wmma", Backend.CUDA_LUT: "_forward_cuda_lut",
             Backend.CUDA: "_forward_cuda"}[backend]
    monkeypatch.setattr(layer, fused, lambda x, gather=None: calls.append("fused") or x[..., :16])
    monkeypatch.setattr(layer, "_forward_dequant_gemm", lambda x, gather=None: calls.append("dense") or x[..., :16])
    monkeypatch.setattr(layer, "_forward_triton", lambda x, gather=None: calls.append("tile") or x[..., :16])
    return layer, calls


@pytest.mark.parametrize("backend", [Backend.CUDA_WMMA, Backend.CUDA, Backend.CUDA_LUT])
def test_mid_sized_batches_use_tile_decode_band(monkeypatch, backend):
    layer, calls = _layer_with_spies(monkeypatch, backend, tile_max=64)
    layer(torch.randn(16, 32))   # fused, at its threshold
    layer(torch.randn(17, 32))   # tile-decode GEMM
    layer(torch.randn(64, 32))   # tile-decode GEMM, at its threshold
    layer(torch.randn(65, 32))   # decode + GEMM
    assert calls == ["fused", "tile", "tile", "dense"]


def test_lut_layers_can_skip_tile_band_like_the_reference(monkeypatch):
    monkeypatch.setattr(vqmod, "_LUT_SKIPS_TILE_BAND", True)
    layer, calls = _layer_with_spies(monkeypatch, Backend.CUDA_LUT, lut_max=0, tile_max=64)
    layer(torch.randn(8, 32))
    assert calls == ["dense"]


@pytest.mark.parametrize("backend", [Backend.CUDA_WMMA, Backend.CUDA_LUT, Backend.CUDA])
def test_leading_dims_count_as_rows_and_edges_are_inclusive(monkeypatch, backend):
    layer, calls = _layer_with_spies(monkeypatch, backend)
    layer(torch.randn(1, 32))
    layer(torch.randn(2, 8, 32))   # 16 rows, at the threshold
    layer(torch.randn(17, 32))
    layer(torch.randn(2, 9, 32))   # 18 rows
    assert calls == ["fused", "fused", "dense", "dense"]


def test_column_permutation_is_applied_before_dispatch(monkeypatch):
    lin = _vq_linear()
    perm = torch.randperm(32)
    lin.weight.qscheme.column_permutation = perm
    layer = NPVQLinear.from_qtensor_linear(lin, VQProxy(lin.weight.qscheme.centroids), backend="cuda")
    seen = []
    monkeypatch.setattr(layer, "_forward_cuda", lambda x, gather=None: seen.append(x) or x[..., :16])
    x = torch.randn(1, 32)
    layer(x)
    assert torch.equal(seen[0], x[..., perm])
    assert layer.column_perm.dtype == torch.int64


def test_unimplemented_backends_raise_instead_of_falling_back():
    lin = _vq_linear()
    for name in ("default", "compile", None):
        layer = NPVQLinear.from_qtensor_linear(lin, VQProxy(lin.weight.qscheme.centroids), backend=name)
        with pytest.raises(NotImplementedError):
            layer(torch.randn(1, 32))


def test_cuda_backend_refuses_cpu_tensors():
    if not _cabi.library_available():
        pytest.skip("library not built")
    lin = _vq_linear()
    layer = NPVQLinear.from_qtensor_linear(lin, VQProxy(lin.weight.qscheme.centroids), backend="cuda")
    with pytest.raises(RuntimeError, match="CUDA"):
        layer(torch.randn(1, 32))


# ------------------------------------------------------------------ proxies and lowering
class _Tiny(nn.Module):
    def __init__(self):
        super().__init__()
        shared = torch.randn(16, 4)
        self.a = _vq_linear(centroids=shared)
        self.b = _vq_linear(centroids=shared, bias=True)
        self.c = _vq_linear(centroids=torch.randn(16, 4))
        vals = torch.randint(0, 16, (8, 64), dtype=torch.uint8)
        self.q = nn.Linear(64, 8, bias=True)
        scheme = AffineScheme(4, 32, torch.rand(16).half(), torch.rand(16).half() * 15)
        self.q._parameters["weight"] = AffineQTensor(_pack_u8(vals, 4), scheme, (8, 64))
        self.plain = nn.Linear(4, 4)


def test_lowering_shares_proxies_and_round_trips():
    model = _Tiny()
    blob_a = model.a.weight.u8_blob.clone()
    AutoKernelLowering(vq_backend="cuda_wmma", linear_backend="cuda").apply(model)
    assert is_lowered(model)
    assert isinstance(model.a, NPVQLinear) and isinstance(model.q, NPLinear)
    assert isinstance(model.plain, nn.Linear)
    assert model.a.proxy is model.b.proxy and model.a.proxy is not model.c.proxy
    proxies = [n for n, _ in model.named_children() if n.startswith("_vq_proxy_")]
    assert proxies == ["_vq_proxy_0", "_vq_proxy_1"]
    keys = set(model.state_dict().keys())
    assert {"a.packed_indices", "b.bias", "_vq_proxy_0.centroids", "q.u8_blob", "q.scale",
            "q.zero_point", "q.bias"} <= keys
    assert not any(k.startswith("a.proxy") for k in keys)  # the proxy is not a child of the layer
    assert model.a.proxy.centroids.dtype == torch.float16
    assert model.a.backend == VQBackend.CUDA_WMMA and model.q.backend == LinearBackend.CUDA
    assert model.q.qtype == "asym" and model.q.nbits == 4 and model.q.group_size == 32

    unlower_model(model)
    assert not is_lowered(model)
    assert isinstance(model.a, nn.Linear) and torch.equal(model.a.weight.u8_blob, blob_a)
    assert model.b.bias is not None
    assert not [n for n, _ in model.named_children() if n.startswith("_vq_proxy_")]


def test_linearize_functions_skip_foreign_modules():
    model = nn.Sequential(nn.Linear(4, 4), nn.ReLU())
    assert linearize_vq_weights(model) is model and linearize_qtensor_weights(model) is model
    assert not is_lowered(model)


def test_to_qtensor_requires_factory_metadata():
    proxy = VQProxy(torch.randn(16, 4))
    packed = IndexPacking.pack(torch.randint(0, 16, (16 * 8,)), 4)
    layer = NPVQLinear(proxy, packed, 4, 16, 32, 4, backend="cuda")
    with pytest.raises(RuntimeError, match="serde metadata"):
        layer.to_qtensor()
    with pytest.raises(RuntimeError):
        proxy(torch.zeros(1))


def test_lowering_config_surface(tmp_path):
    assert LoweringConfig.load(None) == LoweringConfig()
    cfg = LoweringConfig.load({"vq_backend": "cuda_lut"})
    assert cfg.vq_backend == "cuda_lut" and cfg.linear_backend == "auto"
    with pytest.raises(ValueError, match="Unknown lowering config"):
        LoweringConfig.from_dict({"vq": "cuda"})
    cfg.save(tmp_path / "x" / "cfg.yaml")
    assert LoweringConfig.from_file(tmp_path / "x" / "cfg.yaml") == cfg
    (tmp_path / "bad.yaml").write_text("- 1\n- 2\n")
    with pytest.raises(ValueError, match="mapping"):
        LoweringConfig.from_file(tmp_path / "bad.yaml")
    low = AutoKernelLowering.from_config(cfg)
    assert low.vq_backend == "cuda_lut" and low.norm_backend == "auto"
    presets = Path(_cabi.__file__).parent / "configs" / "lowering"
    assert LoweringConfig.from_file(presets / "cuda_wmma.yaml").vq_backend == "cuda_wmma"


def test_nplinear_constructor_contract():
    vals = torch.randint(0, 16, (8, 64), dtype=torch.uint8)
    blob = _pack_u8(vals, 4)
    assert torch.equal(_unpack_u8(blob, 4), vals)
    layer = NPLinear(blob, torch.rand(8, 2).half(), 8, 64, 32, 4, "sym", "auto")
    assert layer.backend == LinearBackend.CUDA and layer.scale.dim() == 1 and layer.zero_point is None
    with pytest.raises(ValueError):
        NPLinear(blob, torch.rand(16).half(), 8, 64, 32, 4, "asym", "cuda")  # asym needs zero_point
    with pytest.raises(ValueError):
        NPLinear(blob, torch.rand(16).half(), 8, 64, 32, 4, "sym", "default")  # default needs weight_q
    with pytest.raises(NotImplementedError):
        layer.set_backend("compile")(torch.randn(1, 64))


def test_auto_kernel_lowering_config_builds_the_pass():
    """The serialisable configuration of the lowering pass (reference recipe_config.py:252-286)."""
    import pydantic

    from neuropress_b200.kernel_lowering import AutoKernelLowering
    from neuropress_b200.recipe_config import (KERNEL_LOWERING_CONFIG_REGISTRY, AutoKernelLoweringConfig,
                                               resolve_kernel_lowering_config)

    assert KERNEL_LOWERING_CONFIG_REGISTRY["auto"] is AutoKernelLoweringConfig
    cfg = resolve_kernel_lowering_config({"type": "auto", "vq_backend": "cuda_lut", "linear_backend": "cuda"})
    assert cfg.model_dump(mode="json") == {"type": "auto", "linear_backend": "cuda", "vq_backend": "cuda_lut",
                                           "embedding_backend": "auto", "norm_backend": "auto"}
    lowering = cfg.build()
    assert isinstance(lowering, AutoKernelLowering)
    assert lowering.vq_backend == "cuda_lut" and lowering.linear_backend == "cuda"
    with pytest.raises(pydantic.ValidationError):
        AutoKernelLoweringConfig(vq_backend="gemlite")      # not a VQ backend
    with pytest.raises(ValueError):
        resolve_kernel_lowering_config({"type": "manual"})


# ------------------------------------------------------------------------- RMSNorm ---
class _LlamaStyleRMSNorm(torch.nn.Module):
    def __init__(self, h, eps=1e-5):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.rand(h) + 0.5)
        self.eps = eps

    def forward(self, x):
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


class _GemmaStyleRMSNorm(_LlamaStyleRMSNorm):
    def forward(self, x):
        v = x.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        return (v * (1.0 + self.weight.float())).to(x.dtype)


def test_rms_norm_swap_detects_the_plus_one_convention():
    """linearize_rms_norms (reference np_rms_norm.py:106-208): detection, the '+1' weight folded
    in, the source module kept for the way back; the oracle agrees with both source modules."""
    import oracle
    from neuropress_b200.kernel_lowering import unlower_model
    from neuropress_b200.nn.np_rms_norm import NPRMSNorm, linearize_rms_norms

    torch.manual_seed(0)
    model = torch.nn.Sequential()
    model.add_module("a", _LlamaStyleRMSNorm(48))
    model.add_module("b", _GemmaStyleRMSNorm(48))
    model.add_module("c", torch.nn.LayerNorm(48))          # not an RMSNorm: left alone
    wa, wb = model.a.weight.detach().clone(), model.b.weight.detach().clone()
    x = torch.randn(5, 48)
    ya, yb = model.a(x), model.b(x)
    assert linearize_rms_norms(model, require_cuda=False) == 2
    assert isinstance(model.a, NPRMSNorm) and isinstance(model.b, NPRMSNorm)
    assert isinstance(model.c, torch.nn.LayerNorm)
    assert torch.equal(model.a.weight, wa) and torch.equal(model.b.weight, 1.0 + wb)
    assert list(model.state_dict()) == ["a.weight", "b.weight", "c.weight", "c.bias"]
    torch.testing.assert_close(oracle.rms_norm(x, model.a.weight, model.a.eps), ya, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(oracle.rms_norm(x, model.b.weight, model.b.eps), yb, rtol=1e-5, atol=1e-6)
    with pytest.raises(RuntimeError):
        model.a(x)                                           # CUDA only: no CPU path
    unlower_model(model)
    assert isinstance(model.a, _LlamaStyleRMSNorm) and isinstance(model.b, _GemmaStyleRMSNorm)
    assert torch.equal(model.b.weight, wb)


def test_small_batch_band_sits_between_the_gemv_and_the_tile_band(monkeypatch):
    """3..16 rows go to the fused kernel when the weight form fits the tensor-core small-batch
    kernel (vector length 8, 8/12/16-bit indices, K % 1024 == 0, fp16/bf16), else on to the
    tile-decode band as in the reference."""
    from synthetic import make_vq_layer

    d = make_vq_layer(32, 1024, num_centroids=256, bits=8, seed=3)
    layer = NPVQLinear(VQProxy(d.centroids), d.packed, 8, 32, 1024, 8, backend="cuda_wmma")
    calls = []
    monkeypatch.setattr(layer, "_forward_cuda_wmma", lambda x, gather=None: calls.append("gemv") or x[..., :32])
    monkeypatch.setattr(layer, "_forward_gemv", lambda x, gather=None: calls.append("small") or x[..., :32])
    monkeypatch.setattr(layer, "_forward_triton", lambda x, gather=None: calls.append("tile") or x[..., :32])
    monkeypatch.setattr(layer, "_forward_dequant_gemm", lambda x, gather=None: calls.append("dense") or x[..., :32])
    layer(torch.zeros(2, 1024, dtype=torch.bfloat16))      # reference GEMV band
    layer(torch.zeros(3, 1024, dtype=torch.bfloat16))      # small-batch band
    layer(torch.zeros(16, 1024, dtype=torch.bfloat16))     # ... up to 16 rows
    layer(torch.zeros(17, 1024, dtype=torch.bfloat16))     # tile-decode band
    layer(torch.zeros(16, 1024, dtype=torch.float32))      # fp32 activations: not the tensor-core form
    assert calls == ["gemv", "small", "small", "tile", "tile"]
    assert layer._small_batch_ok(torch.zeros(1, 1024, dtype=torch.float16), 9)
    assert not layer._small_batch_ok(torch.zeros(1, 1024, dtype=torch.float32), 9)
    wide = NPVQLinear(VQProxy(d.centroids), d.packed[: 4 * 1024], 8, 4, 8192, 8, backend="cuda_wmma")
    assert wide._small_batch_ok(torch.zeros(1, 8192, dtype=torch.bfloat16), 8)
    assert not wide._small_batch_ok(torch.zeros(1, 8192, dtype=torch.bfloat16), 9)   # two B tiles do not fit
    monkeypatch.setattr(vqmod, "_SMALL_BATCH_MAX_TOKENS", 0)
    layer(torch.zeros(3, 1024, dtype=torch.bfloat16))
    assert calls[-1] == "tile"
