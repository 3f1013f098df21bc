"""Parity at the benchmark configurations' full sizes.

The oracle decodes a sample of output columns (whole weight rows) on the CPU and multiplies them
with the full activations in fp64; the module's output on those columns must be within
``1e-2 * RMS + half an ulp`` of it.  Every row-count band of every configuration is covered:
the large-codebook layer (14336 x 4096) at 1/16/128/384 rows, the group-affine layers
(4096 x 4096 and 14336 x 4096, Q4_0 group 32 and zero-point group 64) at 1/8/256/4096 rows, the
70B-shape linear set at 32 and 4096 rows, and the 16-layer 1B-shape decoder stack with a
512-token prefill and a 64-sequence decoding step.  The achieved error of each case is printed
at the end of the run.
"""

import pytest
import torch

import oracle
from helpers import assert_output_close
from neuropress_b200.nn import NPLinear, NPVQLinear, VQProxy
from synthetic import device_bytes, device_normal, make_c2_layer, pack_indices_device

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _sample(n: int, count: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.unique(torch.cat([torch.tensor([0, n - 1]), torch.randint(0, n, (count,), generator=g)]))


# ------------------------------------------------------------------ c2: large codebook ---
@pytest.fixture(scope="module")
def c2():
    d = make_c2_layer(seed=3)
    layer = NPVQLinear(VQProxy(d.centroids).to(DEV), d.packed, 16, d.out_features, d.in_features, 8,
                       backend="auto", residual_proxy=VQProxy(d.residual_centroids).to(DEV),
                       residual_indices=d.residual_indices, row_scale=d.row_scale).to(DEV)
    cols = _sample(d.out_features, 96, 1)
    G = d.in_features // 8
    packed = d.packed.view(d.out_features, G * 2)[cols].reshape(-1)
    res = d.residual_indices.view(d.out_features, G)[cols].reshape(-1)
    w = oracle.vq_decode(packed, d.centroids, 16, cols.numel(), d.in_features, torch.bfloat16,
                         residual_indices=res, residual_centroids=d.residual_centroids,
                         row_scale=d.row_scale[cols])
    return layer, cols, w.double()


@pytest.mark.parametrize("rows", [1, 2, 16, 128, 384, 2048])
def test_c2_full_size_every_band(c2, rows):
    layer, cols, w = c2
    x = device_normal((rows, 4096), DEV, 50 + rows)
    y = layer(x)
    ref = x.cpu().double() @ w.T
    assert_output_close(y[:, cols.to(DEV)], ref, torch.bfloat16, label=f"c2 14336x4096 NC65536+res+scale rows={rows}")


# ------------------------------------------------------------------ c3: group-affine ---
def _q_layer(n_out: int, asym: bool, seed: int):
    k, gs = 4096, 64 if asym else 32
    codes = device_bytes(n_out * k // 2, DEV, seed).view(n_out, k // 2)
    ng = n_out * k // gs
    scale = torch.exp(device_normal((ng,), DEV, seed + 1, std=0.3, dtype=torch.float32) - 4.0).to(torch.float16)
    zp = None
    if asym:
        g = torch.Generator(device=DEV)
        g.manual_seed(seed + 2)
        zp = (torch.rand(ng, device=DEV, generator=g) * 15.0).to(torch.float16)
    layer = NPLinear(codes, scale, n_out, k, gs, 4, "asym" if asym else "sym", "auto", zero_point=zp).to(DEV)
    cols = _sample(n_out, 64, seed)
    w = oracle.q_decode(codes[cols.to(DEV)].cpu(), scale.view(n_out, -1)[cols.to(DEV)].reshape(-1).cpu(),
                        None if zp is None else zp.view(n_out, -1)[cols.to(DEV)].reshape(-1).cpu(), 4, gs,
                        torch.bfloat16)
    return layer, cols, w.double()


@pytest.fixture(scope="module", params=[(4096, False), (4096, True), (14336, False), (14336, True)],
                ids=["q40_4096", "hqq_4096", "q40_14336", "hqq_14336"])
def c3(request):
    n_out, asym = request.param
    return (n_out, asym) + _q_layer(n_out, asym, 11 + n_out % 97 + int(asym))


@pytest.mark.parametrize("rows", [1, 8, 256, 4096])
def test_c3_full_size_every_band(c3, rows):
    n_out, asym, layer, cols, w = c3
    x = device_normal((rows, 4096), DEV, 70 + rows)
    y = layer(x)
    ref = x.cpu().double() @ w.T
    assert_output_close(y[:, cols.to(DEV)], ref, torch.bfloat16,
                        label=f"c3 {'hqq g64' if asym else 'q4_0 g32'} {n_out}x4096 rows={rows}")


# ------------------------------------------------------------------ c5: 70B-shape set ---
C5 = {"q": (8192, 8192), "k": (1024, 8192), "o": (8192, 8192), "gate": (28672, 8192), "down": (8192, 28672)}


@pytest.fixture(scope="module", params=list(C5), ids=list(C5))
def c5(request):
    n, k = C5[request.param]
    proxy = VQProxy(device_normal((65536, 8), DEV, 5, std=0.02, dtype=torch.float16))
    layer = NPVQLinear(proxy, device_bytes(n * (k // 8) * 2, DEV, 9 + n % 13), 16, n, k, 8, backend="auto")
    cols = _sample(n, 48, n + k)
    packed = layer.packed_indices.view(n, (k // 8) * 2)[cols.to(DEV)].reshape(-1).cpu()
    w = oracle.vq_decode(packed, proxy.centroids.cpu(), 16, cols.numel(), k, torch.bfloat16)
    return request.param, layer, cols, w.double()


@pytest.mark.parametrize("rows", [32, 4096])
def test_c5_shapes_prefill_and_decode_batch(c5, rows):
    name, layer, cols, w = c5
    x = device_normal((rows, layer.in_features), DEV, 90 + rows)
    y = layer(x)
    ri = _sample(rows, 12, rows)
    ref = x[ri.to(DEV)].cpu().double() @ w.T
    assert_output_close(y[ri.to(DEV)][:, cols.to(DEV)], ref, torch.bfloat16,
                        label=f"c5 {name} {layer.out_features}x{layer.in_features} NC65536 rows={rows}")


# ------------------------------------------------------------------ c4: 16-layer stack ---
def test_c4_sixteen_layer_stack_prefill512_and_batch64():
    transformers = pytest.importorskip("transformers")
    import copy

    from transformers import LlamaConfig, LlamaModel

    cfg = LlamaConfig(hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=512,
                      max_position_embeddings=1024, attn_implementation="sdpa")
    torch.manual_seed(0)
    dense = LlamaModel(cfg).to(torch.bfloat16).to(DEV).eval()
    vq = copy.deepcopy(dense)
    seed = 0
    from neuropress_b200 import kernels

    for (_, mod_d), (_, mod_q) in zip(list(dense.named_modules()), list(vq.named_modules())):
        for child_name, child in list(mod_d.named_children()):
            if not isinstance(child, torch.nn.Linear):
                continue
            n, k = child.out_features, child.in_features
            seed += 1
            cent = device_normal((k // 2048, 4096, 8), DEV, 100 + seed, std=0.02, dtype=torch.float16)
            g = torch.Generator(device=DEV)
            g.manual_seed(200 + seed)
            idx = torch.randint(0, 4096, (n, k // 8), device=DEV, generator=g)
            packed = pack_indices_device(idx, 16)
            layer = NPVQLinear(VQProxy(cent), packed, 16, n, k, 8, backend="auto", cols_per_codebook=2048)
            # the dense twin holds the decoded weight; the decode kernel is bit-exact against the
            # oracle (tests of the decode), and three linears are re-checked against it here
            w = kernels.vq_dequant(packed, cent, 16, n, k, torch.bfloat16, cols_per_codebook=2048)
            if seed in (1, 5, 112):
                rows = _sample(n, 6, seed)
                want = oracle.vq_decode(packed.view(n, -1)[rows.to(DEV)].reshape(-1).cpu(), cent.cpu(), 16,
                                        rows.numel(), k, torch.bfloat16, cols_per_codebook=2048)
                assert torch.equal(w[rows.to(DEV)].cpu(), want)
            child.weight.data = w
            setattr(mod_q, child_name, layer)
    assert seed == 112

    def rel_rms(a, b):
        a, b = a.double(), b.double()
        return float((a - b).pow(2).mean().sqrt() / b.pow(2).mean().sqrt())

    with torch.no_grad():
        prompt = device_normal((1, 512, 2048), DEV, 1)
        od = dense(inputs_embeds=prompt, use_cache=False).last_hidden_state
        oq = vq(inputs_embeds=prompt, use_cache=False).last_hidden_state
        r = rel_rms(oq, od)
        print(f"[c4] 16 layers, prefill 512: rel RMS difference to the dense-weight stack {r:.4g}")
        assert r < 3e-2
        # decoding step of 64 sequences on a 32-token cache
        ctx = device_normal((64, 32, 2048), DEV, 2)
        tok = device_normal((64, 1, 2048), DEV, 3)
        cd = dense(inputs_embeds=ctx, use_cache=True)
        cq = vq(inputs_embeds=ctx, use_cache=True)
        dd = dense(inputs_embeds=tok, past_key_values=cd.past_key_values, use_cache=True).last_hidden_state
        dq = vq(inputs_embeds=tok, past_key_values=cq.past_key_values, use_cache=True).last_hidden_state
        r = rel_rms(dq, dd)
        print(f"[c4] 16 layers, batch-64 decoding step: rel RMS difference {r:.4g}")
        assert r < 3e-2
        # single sequence (GEMV band) for completeness
        c1d = dense(inputs_embeds=ctx[:1], use_cache=True)
        c1q = vq(inputs_embeds=ctx[:1], use_cache=True)
        d1 = dense(inputs_embeds=tok[:1], past_key_values=c1d.past_key_values, use_cache=True).last_hidden_state
        q1 = vq(inputs_embeds=tok[:1], past_key_values=c1q.past_key_values, use_cache=True).last_hidden_state
        assert rel_rms(q1, d1) < 3e-2
