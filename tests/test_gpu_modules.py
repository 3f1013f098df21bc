"""GPU tests of the drop-in modules: ``NPVQLinear`` / ``NPLinear`` forwards against the golden
outputs produced by the reference itself and against the oracle, one case per row-count band.
"""

from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_output_close
from neuropress_b200.nn import NPLinear, NPVQLinear, VQBackend, VQProxy
from synthetic import make_activations, make_c2_layer, make_q_layer, make_vq_layer
from neuropress_b200.transforms.vq_packing import IndexPacking

pytestmark = pytest.mark.gpu
DEV = "cuda"
G = np.load(Path(__file__).parent / "golden" / "reference_vectors.npz")
DT = {0: torch.float16, 1: torch.bfloat16, 2: torch.float32}


def gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


@pytest.mark.parametrize("tag", ["c1_m1", "c1_m16", "b4", "b10", "b12", "b14", "b16"])
@pytest.mark.parametrize("backend", ["cuda", "cuda_wmma", "cuda_lut"])
def test_vq_module_matches_reference_outputs(tag, backend):
    """Same seeded inputs as the golden generator; output of the reference's default path."""
    N, K, vl, nc, bits, rows, seed, has_bias, dcode = (int(v) for v in G[f"vq_{tag}_meta"])
    std = float(G[f"vq_{tag}_std"][0])
    dtype = DT[dcode]
    cent = torch.randn(nc, vl, generator=gen(seed)) * std
    idx = torch.randint(0, nc, (N, K // vl), generator=gen(seed + 1))
    x = torch.randn(rows, K, generator=gen(seed + 2)).to(dtype)
    b = (torch.randn(N, generator=gen(seed + 3)) * 0.1).to(dtype) if has_bias else None
    layer = NPVQLinear(VQProxy(cent).to(DEV), IndexPacking.pack(idx, bits), bits, N, K, vl,
                       backend=backend, bias=b).to(DEV)
    y = layer(x.to(DEV))
    assert y.dtype == dtype and y.shape == (rows, N)
    y_ref = torch.from_numpy(G[f"vq_{tag}_y"]).double()
    # The golden output is already rounded to the activation dtype; allow the rounding of both.
    assert_output_close(y, y_ref, dtype, tol=1e-2)
    torch.testing.assert_close(y.float().cpu(), y_ref.float(), rtol=2e-2, atol=2e-2 * float(y_ref.abs().max()))


@pytest.mark.parametrize("rows", [1, 2, 3, 16, 130, 400])
def test_vq_module_bands_on_extended_layer(rows):
    """All three bands (GEMV / mid / decode + GEMM) with residual + row scale + bias + perm."""
    d = make_vq_layer(384, 1024, num_centroids=65536, bits=16, seed=9, residual_centroids=256,
                      row_scale=True, bias=True)
    perm = torch.randperm(1024, generator=gen(3))
    layer = NPVQLinear(VQProxy(d.centroids).to(DEV), d.packed, 16, 384, 1024, 8, backend="auto",
                       bias=d.bias, column_perm=perm, residual_proxy=VQProxy(d.residual_centroids).to(DEV),
                       residual_indices=d.residual_indices, row_scale=d.row_scale).to(DEV)
    assert layer.backend == VQBackend.CUDA_LUT
    x = make_activations(rows, 1024, torch.bfloat16, seed=rows)
    y = layer(x.reshape(1, rows, 1024).to(DEV))
    assert y.shape == (1, rows, 384)
    ref = oracle.vq_forward_f32(x[:, perm], d.packed, d.centroids, 16, 384, 1024, d.bias, **d.ext())
    assert_output_close(y.reshape(rows, 384), ref, torch.bfloat16)


def test_vq_module_fp32_activations_large_batch():
    d = make_vq_layer(256, 512, num_centroids=256, bits=8, seed=4)
    layer = NPVQLinear(VQProxy(d.centroids).to(DEV), d.packed, 8, 256, 512, 8, backend="cuda_wmma").to(DEV)
    x = make_activations(600, 512, torch.float32, seed=1)
    y = layer(x.to(DEV))
    assert y.dtype == torch.float32
    ref = oracle.vq_forward_f32(x.to(torch.float16), d.packed, d.centroids, 8, 256, 512)
    assert_output_close(y, ref, torch.float16)  # computed in fp16 like the reference's tensor-core path


@pytest.mark.parametrize("asym,gs", [(False, 32), (True, 64)])
@pytest.mark.parametrize("rows", [1, 8, 9, 256, 385, 700])
def test_q_module_bands(asym, gs, rows):
    q = make_q_layer(512, 1024, group_size=gs, asym=asym, seed=rows, bias=True)
    layer = NPLinear(q.codes, q.scale, 512, 1024, gs, 4, "asym" if asym else "sym", "auto",
                     bias=q.bias, zero_point=q.zero_point).to(DEV)
    x = make_activations(rows, 1024, torch.bfloat16, seed=rows)
    y = layer(x.to(DEV))
    ref = oracle.q_forward_f64(x, q.codes, q.scale, 4, gs, q.zero_point, q.bias)
    assert_output_close(y, ref, torch.bfloat16)


@pytest.mark.parametrize("tag", ["q40_f32", "q40_bf16", "hqq_bf16", "hqq_f16"])
def test_q_module_matches_reference_outputs(tag):
    N, K, gs, asym, rows, dcode = (int(v) for v in G[f"q_{tag}_meta"])
    dtype = DT[dcode]
    blob = torch.from_numpy(G[f"q_{tag}_blob"])
    scale = torch.from_numpy(G[f"q_{tag}_scale"].view(np.float16).copy())
    zp = torch.from_numpy(G[f"q_{tag}_zp"].view(np.float16).copy()) if asym else None
    x = torch.from_numpy(G[f"q_{tag}_x"]).to(dtype)
    b = torch.from_numpy(G[f"q_{tag}_bias"]) if f"q_{tag}_bias" in G else None
    layer = NPLinear(blob, scale, N, K, gs, 4, "asym" if asym else "sym", "cuda", bias=b,
                     zero_point=zp).to(DEV)
    y = layer(x.to(DEV))
    assert_output_close(y, torch.from_numpy(G[f"q_{tag}_y"]).double(), dtype)


def test_full_size_layer_properties():
    """Full benchmark size (14336 x 4096, 65536-entry codebook): size-independent properties.
    Decode is linear in the one-hot sense: the GEMV of a unit vector returns a weight column,
    and the three bands agree with each other on the same input."""
    d = make_c2_layer(seed=0)
    layer = NPVQLinear(VQProxy(d.centroids).to(DEV), d.packed, 16, d.out_features, d.in_features, 8,
                       backend="auto", residual_proxy=VQProxy(d.residual_centroids).to(DEV),
                       residual_indices=d.residual_indices, row_scale=d.row_scale).to(DEV)
    from neuropress_b200 import kernels

    w = kernels.vq_dequant(layer.packed_indices, layer.proxy.centroids, 16, 14336, 4096, torch.bfloat16,
                           **layer._ext())
    # spot rows of the decode against the oracle restricted to those rows
    rows = [0, 1, 777, 14335]
    G_ = 4096 // 8
    for r in rows:
        sl = slice(r * G_ * 2, (r + 1) * G_ * 2)
        ref = oracle.vq_decode(d.packed[sl], d.centroids, 16, 1, 4096, torch.bfloat16,
                               residual_indices=d.residual_indices[r * G_:(r + 1) * G_],
                               residual_centroids=d.residual_centroids, row_scale=d.row_scale[r:r + 1])
        assert torch.equal(w[r].cpu(), ref[0])
    # unit vector -> column of W (exact: one product, zeros elsewhere)
    e = torch.zeros(1, 4096, dtype=torch.bfloat16, device=DEV)
    e[0, 1234] = 1
    assert torch.equal(layer(e)[0], w[:, 1234])
    # bands agree: 2 rows via GEMV == the same 2 rows inside a 2048-row decode + GEMM batch
    x = make_activations(2048, 4096, torch.bfloat16, seed=5).to(DEV)
    y_big = layer(x)
    y_gemv = layer(x[:2].contiguous())
    ref = (x[:2].double() @ w.double().T)
    assert_output_close(y_gemv, ref, torch.bfloat16)
    assert_output_close(y_big[:2], ref, torch.bfloat16)
    from neuropress_b200 import _cabi

    assert _cabi.gemm_device_status() == 0


def test_70b_shaped_layer_properties():
    """Largest layer shape of the 70B-shaped configuration (28672 x 8192, one 65536-entry codebook,
    uint16 indices: 58.7 M indices, 117 MB of index bytes): spot rows of the decode against the
    oracle, unit-vector GEMV = weight column, band agreement, and the eight out-feature shards
    reproducing their rows of the full decode bit for bit."""
    from neuropress_b200 import _cabi, kernels
    from neuropress_b200.sharding import shard_vq_linear

    N, K, G_ = 28672, 8192, 8192 // 8
    d = make_vq_layer(N, K, num_centroids=65536, bits=16, seed=70)
    layer = NPVQLinear(VQProxy(d.centroids), d.packed, 16, N, K, 8, backend="auto")
    w = kernels.vq_dequant(d.packed.to(DEV), d.centroids.to(DEV), 16, N, K, torch.bfloat16)
    for r in (0, 1, 12345, N - 1):
        sl = slice(r * G_ * 2, (r + 1) * G_ * 2)
        ref = oracle.vq_decode(d.packed[sl], d.centroids, 16, 1, K, torch.bfloat16)
        assert torch.equal(w[r].cpu(), ref[0])
    for rank in (0, 3, 7):   # shards of an 8-way split decode to exactly their rows
        shard = shard_vq_linear(layer, 8, rank)
        ws = kernels.vq_dequant(shard.packed_indices.to(DEV), d.centroids.to(DEV), 16, N // 8, K,
                                torch.bfloat16)
        assert torch.equal(ws, w[rank * (N // 8):(rank + 1) * (N // 8)])
    layer.proxy.to(DEV)
    layer = layer.to(DEV)
    e = torch.zeros(1, K, dtype=torch.bfloat16, device=DEV)
    e[0, 4321] = 1
    assert torch.equal(layer(e)[0], w[:, 4321])
    x = make_activations(32, K, torch.bfloat16, seed=9).to(DEV)   # the batch-32 decode of that config
    ref = x.double() @ w.double().T
    assert_output_close(layer(x), ref, torch.bfloat16)
    assert_output_close(layer(x[:2].contiguous()), ref[:2], torch.bfloat16)
    assert _cabi.gemm_device_status() == 0
