"""Pin the CPU oracle (and the package's packers) to vectors produced by the reference itself.

``tests/golden/reference_vectors.npz`` was written by ``tests/golden/make_golden.py`` from the
reference's own functions.  Every oracle function is checked against it here, bit-exactly for
bytes, indices and decoded weights; forward outputs must be equal too, because the oracle
performs the same torch operations in the same order.
"""

from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from neuropress_b200.t2n.packing import BitPacking
from neuropress_b200.transforms.vq_packing import IndexPacking

G = np.load(Path(__file__).parent / "golden" / "reference_vectors.npz")
DT = {0: torch.float16, 1: torch.bfloat16, 2: torch.float32}


def gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


@pytest.mark.parametrize("bits", range(4, 21))
def test_index_stream_matches_reference_bytes(bits):
    idx, ref_bytes = G[f"pack_idx_{bits}"], G[f"pack_bytes_{bits}"]
    n = idx.size
    assert np.array_equal(oracle.pack_indices(idx, bits), ref_bytes)
    assert np.array_equal(oracle.unpack_indices(ref_bytes, bits, n), idx)
    assert np.array_equal(oracle.unpack_indices_bitloop(ref_bytes, bits, n), idx)
    # the package's own packer writes the same wire format
    assert np.array_equal(IndexPacking.pack(torch.from_numpy(idx), bits).numpy(), ref_bytes)
    assert np.array_equal(IndexPacking.unpack(torch.from_numpy(ref_bytes), bits, n).numpy(), idx)


def test_known_answer_byte():
    # the reference's one literal known-answer test: indices [3, 11] at 4 bits -> 3 | 11 << 4
    assert G["pack_kat_4bit_3_11"].tolist() == [3 | (11 << 4)]
    assert oracle.pack_indices(np.array([3, 11]), 4).tolist() == [0xB3]
    assert IndexPacking.pack(torch.tensor([3, 11]), 4).tolist() == [0xB3]


def test_bits_for_table():
    for nc, bits in G["bits_for"]:
        assert IndexPacking.bits_for(int(nc)) == int(bits)


def _vq_inputs(tag):
    N, K, vl, nc, bits, rows, seed, has_bias, dcode = (int(v) for v in G[f"vq_{tag}_meta"])
    std = float(G[f"vq_{tag}_std"][0])
    dtype = DT[dcode]
    cent = (torch.randn(nc, vl, generator=gen(seed)) * std).to(torch.float16)
    idx = torch.randint(0, nc, (N, K // vl), generator=gen(seed + 1))
    x = torch.randn(rows, K, generator=gen(seed + 2)).to(dtype)
    b = (torch.randn(N, generator=gen(seed + 3)) * 0.1).to(dtype) if has_bias else None
    return N, K, bits, dtype, cent, idx, x, b


VQ_TAGS = ["c1_m1", "c1_m16", "b4", "b10", "b12", "b14", "b16"]


@pytest.mark.parametrize("tag", VQ_TAGS)
def test_vq_forward_matches_reference(tag):
    N, K, bits, dtype, cent, idx, x, b = _vq_inputs(tag)
    packed = oracle.pack_indices(idx.numpy(), bits)
    y = oracle.vq_forward(x, packed, cent, bits, N, K, b)
    assert y.dtype == dtype
    assert np.array_equal(y.float().numpy(), G[f"vq_{tag}_y"])
    if f"vq_{tag}_w16" in G:
        w16 = oracle.vq_decode(packed, cent, bits, N, K, torch.float16)
        assert np.array_equal(w16.numpy().view(np.uint16), G[f"vq_{tag}_w16"])
        wx = oracle.vq_decode(packed, cent, bits, N, K, dtype)
        assert np.array_equal(wx.float().numpy(), G[f"vq_{tag}_wx"])


def test_extended_forms_reduce_to_reference_form():
    """Residual of zeros, scale of ones and a single column group leave the decode unchanged."""
    N, K, bits, dtype, cent, idx, x, b = _vq_inputs("b16")
    packed = oracle.pack_indices(idx.numpy(), bits)
    base = oracle.vq_decode(packed, cent, bits, N, K, dtype)
    zeros_cb = torch.zeros(256, 8, dtype=torch.float16)
    ridx = oracle.pack_indices(np.zeros(N * K // 8, dtype=np.int64), 8)
    ext = oracle.vq_decode(packed, cent.unsqueeze(0), bits, N, K, dtype, residual_indices=ridx,
                           residual_centroids=zeros_cb, row_scale=torch.ones(N, dtype=torch.float16),
                           cols_per_codebook=K)
    assert torch.equal(base, ext)


def test_extended_forms_arithmetic():
    """Residual add and row scale are fp16 operations with one rounding each."""
    g = gen(5)
    N, K = 6, 16
    cm = torch.randn(32, 8, generator=g).to(torch.float16)
    cr = (torch.randn(16, 8, generator=g) * 0.1).to(torch.float16)
    im = torch.randint(0, 32, (N, 2), generator=g)
    ir = torch.randint(0, 16, (N, 2), generator=g)
    s = torch.exp(torch.randn(N, generator=g) * 0.1).to(torch.float16)
    w = oracle.vq_decode(oracle.pack_indices(im.numpy(), 5), cm, 5, N, K, torch.bfloat16,
                         residual_indices=oracle.pack_indices(ir.numpy(), 4), residual_centroids=cr,
                         residual_bits=4, row_scale=s)
    for n in range(N):
        for gi in range(2):
            for j in range(8):
                a = (cm[im[n, gi], j].float() + cr[ir[n, gi], j].float()).to(torch.float16)
                v = (a.float() * s[n].float()).to(torch.float16).to(torch.bfloat16)
                assert w[n, gi * 8 + j] == v


Q_TAGS = ["q40_f32", "q40_bf16", "hqq_bf16", "hqq_f16"]


@pytest.mark.parametrize("tag", Q_TAGS)
def test_group_affine_matches_reference(tag):
    N, K, gs, asym, rows, dcode = (int(v) for v in G[f"q_{tag}_meta"])
    dtype = DT[dcode]
    vals, blob = G[f"q_{tag}_vals"], G[f"q_{tag}_blob"]
    assert np.array_equal(oracle.pack_codes(vals, 4), blob)
    assert np.array_equal(oracle.unpack_codes(blob, 4), vals)
    assert np.array_equal(BitPacking(4).compress(torch.from_numpy(vals)).numpy(), blob)
    assert np.array_equal(BitPacking(4).decompress(torch.from_numpy(blob)).numpy(), vals)
    scale = torch.from_numpy(G[f"q_{tag}_scale"].view(np.float16).copy())
    zp = torch.from_numpy(G[f"q_{tag}_zp"].view(np.float16).copy()) if asym else None
    x = torch.from_numpy(G[f"q_{tag}_x"]).to(dtype)
    b = torch.from_numpy(G[f"q_{tag}_bias"]).to(dtype) if f"q_{tag}_bias" in G else None
    w = oracle.q_decode(blob, scale, zp, 4, gs, dtype)
    assert np.array_equal(w.float().numpy(), G[f"q_{tag}_w"])
    y = oracle.q_forward(x, blob, scale, 4, gs, zp, b)
    assert np.array_equal(y.float().numpy(), G[f"q_{tag}_y"])
