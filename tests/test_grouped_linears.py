"""Linears that share their input run as one launch (``npb_vq_gemv_grouped``), with the RMSNorm
in front folded into the activation staging: the grouping pass on CPU (structure, fallbacks with
spied kernels) and the kernel on a GPU against the ungrouped modules and the oracle."""

import pytest
import torch
from torch import nn

import oracle
from helpers import assert_output_close
from neuropress_b200 import _cabi
from neuropress_b200.nn import (DeferredNorm, GroupedLinear, NPRMSNorm, NPVQLinear, VQProxy,
                                group_shared_input_linears)
from synthetic import make_activations, make_vq_layer


class Attn(nn.Module):
    def __init__(self, mk):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = mk(256, 1024, 1), mk(64, 1024, 2), mk(64, 1024, 3), mk(1024, 256, 4)

    def forward(self, x):
        return self.q_proj(x), self.k_proj(x), self.v_proj(x)


class Mlp(nn.Module):
    def __init__(self, mk):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = mk(512, 1024, 5), mk(512, 1024, 6), mk(1024, 512, 7)

    def forward(self, x):
        return self.gate_proj(x), self.up_proj(x)


class Layer(nn.Module):
    def __init__(self, mk, dev):
        super().__init__()
        g = torch.Generator().manual_seed(9)
        self.input_layernorm = NPRMSNorm((torch.rand(1024, generator=g) + 0.5).to(torch.bfloat16).to(dev), 1e-5)
        self.post_attention_layernorm = NPRMSNorm((torch.rand(1024, generator=g) + 0.5).to(torch.bfloat16).to(dev), 1e-5)
        self.self_attn, self.mlp = Attn(mk), Mlp(mk)

    def forward(self, x):
        return (*self.self_attn(self.input_layernorm(x)), *self.mlp(self.post_attention_layernorm(x)))


def _maker(dev, data):
    def mk(n, k, seed):
        d = make_vq_layer(n, k, num_centroids=4096, bits=16, seed=seed, cols_per_codebook=1024 if k == 1024 else 0,
                          bias=seed % 2 == 1)
        data[seed] = d
        layer = NPVQLinear(VQProxy(d.centroids), d.packed, 16, n, k, 8, backend="cuda",
                           bias=d.bias, cols_per_codebook=d.cols_per_codebook)
        layer.proxy.to(dev)
        return layer.to(dev)
    return mk


def test_grouping_pass_structure_and_fallbacks(monkeypatch):
    from neuropress_b200 import kernels

    data = {}
    layer = Layer(_maker("cpu", data), "cpu")
    model = nn.Module()
    model.layers = nn.ModuleList([layer])
    assert group_shared_input_linears(model) == 2
    assert isinstance(layer.self_attn.q_proj, GroupedLinear) and isinstance(layer.mlp.up_proj, GroupedLinear)
    assert isinstance(layer.self_attn.o_proj, NPVQLinear) and isinstance(layer.mlp.down_proj, NPVQLinear)
    assert isinstance(layer.input_layernorm, DeferredNorm) and isinstance(layer.post_attention_layernorm, DeferredNorm)
    assert group_shared_input_linears(model) == 0          # nothing left to group
    calls = []

    def fake_grouped(x, weights, bits, cpc=0, norm_weight=None, norm_eps=0.0):
        calls.append(("grouped", len(weights), norm_weight is not None))
        return torch.zeros(x.shape[0], sum(w[2] for w in weights), dtype=x.dtype)

    monkeypatch.setattr(kernels, "vq_gemv_grouped", fake_grouped)
    monkeypatch.setattr(NPVQLinear, "_small_batch_ok", lambda self, x, m: True)
    x = torch.zeros(2, 1024, dtype=torch.bfloat16)
    q, k, v, g, u = layer(x)
    assert (q.shape, k.shape, v.shape, g.shape, u.shape) == ((2, 256), (2, 64), (2, 64), (2, 512), (2, 512))
    assert calls == [("grouped", 3, True), ("grouped", 2, True)]   # one launch per group, norm folded in
    # the kernel declines (returns None): norm kernel + the members' own forwards, still one norm call
    seen = []
    monkeypatch.setattr(kernels, "vq_gemv_grouped", lambda *a, **k: None)
    monkeypatch.setattr(kernels, "rms_norm", lambda x, w, eps: seen.append("norm") or x)
    monkeypatch.setattr(kernels, "vq_gemv", lambda x, p, c, b, n, bias, gather=None, **e: seen.append("gemv") or
                        torch.zeros(x.shape[0], n, dtype=x.dtype))
    layer.self_attn(layer.input_layernorm(x))
    assert seen == ["norm", "gemv", "gemv", "gemv"]
    # 17 rows to the end of the tile-decode band: one norm launch, then one grouped GEMM launch
    seen.clear()

    def fake_tile_grouped(x, weights, bits, cpc=0):
        seen.append(("tile", len(weights)))
        return torch.zeros(x.shape[0], sum(w[2] for w in weights), dtype=x.dtype)

    monkeypatch.setattr(kernels, "vq_gemm_fused_grouped", fake_tile_grouped)
    x40 = torch.zeros(40, 1024, dtype=torch.bfloat16)
    q, k, v = layer.self_attn(layer.input_layernorm(x40))
    assert (q.shape, k.shape, v.shape) == ((40, 256), (40, 64), (40, 64))
    assert seen == ["norm", ("tile", 3)]
    # the grouped GEMM declines: the members' own tile-decode GEMMs
    seen.clear()
    monkeypatch.setattr(kernels, "vq_gemm_fused_grouped", lambda *a, **k: None)
    monkeypatch.setattr(kernels, "vq_gemm_fused", lambda x, p, c, b, n, bias, **e: seen.append("fused") or
                        torch.zeros(x.shape[0], n, dtype=x.dtype))
    layer.mlp(layer.post_attention_layernorm(x40))
    assert seen == ["norm", "fused", "fused"]


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 5, 16, 17, 40, 130, 384, 400])
def test_grouped_launch_matches_the_ungrouped_modules(rows):
    dev = torch.device("cuda", 0)
    data = {}
    plain = Layer(_maker(dev, data), dev)
    grouped = Layer(_maker(dev, {}), dev)
    holder = nn.Module()
    holder.layers = nn.ModuleList([grouped])
    assert group_shared_input_linears(holder) == 2
    x = make_activations(rows, 1024, torch.bfloat16, seed=rows).to(dev)
    want = plain(x)
    got = grouped(x)
    xn_a = oracle.rms_norm(x.cpu(), plain.input_layernorm.weight.cpu(), 1e-5)
    xn_m = oracle.rms_norm(x.cpu(), plain.post_attention_layernorm.weight.cpu(), 1e-5)
    for i, (seed, xn) in enumerate([(1, xn_a), (2, xn_a), (3, xn_a), (5, xn_m), (6, xn_m)]):
        d = data[seed]
        ref = oracle.vq_forward_f32(xn, d.packed, d.centroids, 16, d.out_features, 1024, d.bias, **d.ext())
        assert got[i].shape == want[i].shape == (rows, d.out_features)
        assert_output_close(got[i], ref, torch.bfloat16, tol=1.5e-2)   # the norm's own bf16 rounding is in x
        assert_output_close(want[i], ref, torch.bfloat16, tol=1.5e-2)
        # grouped and ungrouped differ at most by the norm's last-bit differences
        assert float((got[i].float() - want[i].float()).abs().max()) <= 0.05 * float(want[i].float().abs().max())


@pytest.mark.gpu
def test_grouped_launch_without_norm_is_bit_identical_to_single_launches():
    from neuropress_b200 import kernels

    dev = torch.device("cuda", 0)
    data = {}
    mk = _maker(dev, data)
    mods = [mk(256, 2048, 1), mk(64, 2048, 2), mk(80, 2048, 3)]
    for rows in (1, 8, 13):
        x = make_activations(rows, 2048, torch.bfloat16, seed=rows).to(dev)
        y = kernels.vq_gemv_grouped(x, [(m.packed_indices, m.proxy.centroids, m.out_features, m._bias32())
                                        for m in mods], 16, 0)
        assert y is not None and y.shape == (rows, 400)
        c = 0
        for m in mods:
            assert torch.equal(y[:, c:c + m.out_features], m(x))
            c += m.out_features


@pytest.mark.gpu
@pytest.mark.parametrize("bits,nc", [(16, 4096), (12, 4096), (8, 256)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_grouped_tile_decode_gemm_is_bit_identical_to_single_launches(bits, nc, dtype):
    """``npb_vq_gemm_fused_grouped``: ragged member widths (tiles padded per member, odd column
    offsets in y), with and without bias, every row band of the kernel."""
    from neuropress_b200 import kernels

    dev = torch.device("cuda", 0)
    mods = []
    for seed, n in enumerate((264, 72, 1000, 3), start=1):
        d = make_vq_layer(n, 2048, num_centroids=nc, bits=bits, seed=seed, bias=seed % 2 == 1)
        layer = NPVQLinear(VQProxy(d.centroids), d.packed, bits, n, 2048, 8, backend="cuda", bias=d.bias)
        layer.proxy.to(dev)
        mods.append(layer.to(dev))
    weights = [(m.packed_indices, m.proxy.centroids, m.out_features, m._bias32()) for m in mods]
    for rows in (17, 64, 129, 300, 384):
        x = make_activations(rows, 2048, dtype, seed=rows).to(dev)
        for n_w in (4, 2, 1):
            y = kernels.vq_gemm_fused_grouped(x, weights[:n_w], bits, 0)
            assert y is not None and y.shape == (rows, sum(m.out_features for m in mods[:n_w]))
            c = 0
            for m in mods[:n_w]:
                single = kernels.vq_gemm_fused(x, m.packed_indices, m.proxy.centroids, bits, m.out_features,
                                               m._bias32())
                assert torch.equal(y[:, c:c + m.out_features], single)
                c += m.out_features
    assert _cabi.gemm_device_status() == 0


@pytest.mark.gpu
def test_grouped_tile_decode_gemm_declines_what_it_does_not_take():
    from neuropress_b200 import kernels

    dev = torch.device("cuda", 0)
    a = make_vq_layer(64, 1024, num_centroids=4096, bits=16, seed=1)
    b = make_vq_layer(64, 1024, num_centroids=1024, bits=16, seed=2)
    x = make_activations(32, 1024, torch.bfloat16, seed=3).to(dev)
    wa = (a.packed.to(dev), a.centroids.to(dev), 64, None)
    wb = (b.packed.to(dev), b.centroids.to(dev), 64, None)
    assert kernels.vq_gemm_fused_grouped(x, [wa, wb], 16, 0) is None          # another codebook size
    assert kernels.vq_gemm_fused_grouped(x, [wa] * 5, 16, 0) is None          # more than four members
    assert kernels.vq_gemm_fused_grouped(x.float(), [wa, wa], 16, 0) is None  # fp32 activations
