"""Embedding lookups: the oracle against the outputs of the reference's own modules
(``tests/golden/reference_embedding_vectors.npz``, written by ``make_golden.py``), the CUDA
kernels against both (bit-exact: the lookup is indexing plus fixed roundings), and the lowering
passes that swap embedding modules."""

from pathlib import Path

import numpy as np
import pytest
import torch
import torch.nn as nn

import oracle
from neuropress_b200.nn import (NPEmbedding, NPVQEmbedding, VQProxy, linearize_qtensor_embeddings,
                                linearize_vq_embeddings)
from neuropress_b200.qtensor import AffineQTensor, AffineScheme, VQQTensor, VQScheme
from neuropress_b200.transforms.vq_packing import IndexPacking

G = np.load(Path(__file__).parent / "golden" / "reference_embedding_vectors.npz")
DT = {-1: None, 0: torch.float16, 1: torch.bfloat16, 2: torch.float32}
VQ_TAGS = ["plain", "big_bf16", "scaled_perm", "scaled_f32"]
Q_TAGS = ["q40", "q40_pad_bf16", "hqq_scaled", "hqq_f32"]


def gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def vq_inputs(tag):
    vocab, dim, vl, nc, perm, dcode, seed = (int(v) for v in G[f"vqe_{tag}_meta"])
    cent = (torch.randn(nc, vl, generator=gen(seed)) * 0.05).to(torch.float16)
    idx = torch.randint(0, nc, (vocab, dim // vl), generator=gen(seed + 1)).to(torch.int16)
    ids = torch.from_numpy(G[f"vqe_{tag}_ids"])
    inv = torch.argsort(torch.randperm(dim, generator=gen(seed + 3))) if perm else None
    return dict(ids=ids, idx=idx, cent=cent, dim=dim, vl=vl, scale=float(G[f"vqe_{tag}_scale"][0]), inv=inv,
                out_dtype=DT[dcode], y=torch.from_numpy(G[f"vqe_{tag}_y"]))


def q_inputs(tag):
    vocab, dim, gs, asym, pad, dcode = (int(v) for v in G[f"qe_{tag}_meta"])
    zp = torch.from_numpy(G[f"qe_{tag}_zp"].view(np.float16).copy()) if asym else None
    return dict(ids=torch.from_numpy(G[f"qe_{tag}_ids"]), blob=torch.from_numpy(G[f"qe_{tag}_blob"]),
                scale=torch.from_numpy(G[f"qe_{tag}_scale"].view(np.float16).copy()), zp=zp, vocab=vocab, dim=dim,
                gs=gs, pad=None if pad < 0 else pad, escale=float(G[f"qe_{tag}_escale"][0]),
                out_dtype=DT[dcode], y=torch.from_numpy(G[f"qe_{tag}_y"]))


@pytest.mark.parametrize("tag", VQ_TAGS)
def test_oracle_vq_embedding_matches_the_reference_module(tag):
    c = vq_inputs(tag)
    y = oracle.vq_embedding(c["ids"], c["idx"], c["cent"], c["dim"], c["scale"], c["inv"], c["out_dtype"])
    assert y.shape == (*c["ids"].shape, c["dim"])
    assert torch.equal(y.float(), c["y"])


@pytest.mark.parametrize("tag", Q_TAGS)
def test_oracle_q_embedding_matches_the_reference_module(tag):
    c = q_inputs(tag)
    y = oracle.q_embedding(c["ids"], c["blob"], c["scale"], 4, c["gs"], c["zp"], c["pad"], c["escale"],
                           c["out_dtype"])
    assert torch.equal(y.float(), c["y"])
    if c["pad"] is not None:
        assert float(y[c["ids"] == c["pad"]].abs().max()) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("tag", VQ_TAGS)
def test_vq_embedding_kernel_bit_exact(tag):
    c = vq_inputs(tag)
    m = NPVQEmbedding(c["idx"], VQProxy(c["cent"]).cuda(), c["dim"], c["vl"], scale=c["scale"], inv_perm=c["inv"],
                      out_dtype=c["out_dtype"]).cuda()
    y = m(c["ids"].cuda())
    assert y.dtype == (c["out_dtype"] or torch.float16) and y.shape == (*c["ids"].shape, c["dim"])
    assert torch.equal(y.float().cpu(), c["y"])
    row = m.weight[int(c["ids"][0, 0])]                   # the lazy weight proxy: one row
    assert torch.equal(row.float().cpu(), c["y"][0, 0])


@pytest.mark.gpu
@pytest.mark.parametrize("tag", Q_TAGS)
def test_q_embedding_kernel_bit_exact(tag):
    c = q_inputs(tag)
    m = NPEmbedding(c["blob"], c["scale"], c["vocab"], c["dim"], c["gs"], 4, "asym" if c["zp"] is not None else "sym",
                    "auto", padding_idx=c["pad"], zero_point=c["zp"], embed_scale=c["escale"],
                    out_dtype=c["out_dtype"]).cuda()
    assert m.backend.value == "cuda"
    y = m(c["ids"].cuda())
    assert torch.equal(y.float().cpu(), c["y"])


@pytest.mark.gpu
def test_embedding_kernels_large_table_and_bad_ids():
    """A 32000 x 2048 table (the size of a real vocabulary): sampled rows against the oracle;
    ids outside the table give zero rows instead of reading out of bounds."""
    vocab, dim, nc = 32000, 2048, 65536
    cent = (torch.randn(nc, 8, generator=gen(1)) * 0.05).to(torch.float16)
    idx = torch.randint(0, nc, (vocab, dim // 8), generator=gen(2))
    m = NPVQEmbedding(idx, VQProxy(cent).cuda(), dim, 8, out_dtype=torch.bfloat16).cuda()
    ids = torch.randint(0, vocab, (4, 300), generator=gen(3))
    y = m(ids.cuda())
    want = oracle.vq_embedding(ids, idx.to(torch.int16), cent, dim, out_dtype=torch.bfloat16)
    assert torch.equal(y.cpu(), want)
    bad = torch.tensor([5, vocab, -1, 7])
    yb = m(bad.cuda()).cpu()
    assert float(yb[1].abs().max()) == 0.0 and float(yb[2].abs().max()) == 0.0
    assert torch.equal(yb[0], oracle.vq_embedding(bad[:1], idx.to(torch.int16), cent, dim, out_dtype=torch.bfloat16)[0])


def test_linearize_vq_embeddings_swaps_modules_and_shares_proxies():
    cent = torch.randn(256, 8, generator=gen(5)) * 0.05
    idx = torch.randint(0, 256, (40, 4), generator=gen(6))
    w = VQQTensor(IndexPacking.pack(idx, 8), VQScheme(cent, 8, 8, original_shape=(40, 32)), (40, 32))

    class Scaled(nn.Embedding):
        embed_scale = 4.0

    model = nn.Module()
    model.embed = Scaled(40, 32)
    model.embed._parameters["weight"] = w
    model.other = nn.Linear(4, 4)
    assert linearize_vq_embeddings(model) == 1
    e = model.embed
    assert isinstance(e, NPVQEmbedding) and e.scale == 4.0 and e.embedding_dim == 32
    assert torch.equal(e.all_indices.long() & 0xFFFF, idx)
    assert isinstance(getattr(model, "_vq_emb_proxy_0"), VQProxy) and e.proxy is model._vq_emb_proxy_0
    assert "proxy" not in dict(e.named_children())          # shared codebook: not a sub-module
    assert e.to_qtensor() is w
    assert e.weight.shape == (40, 32)
    assert linearize_vq_embeddings(model) == 0              # idempotent


def test_linearize_qtensor_embeddings_and_unlower_round_trip():
    from neuropress_b200.kernel_lowering import AutoKernelLowering, is_lowered, unlower_model

    vals = torch.randint(0, 16, (30, 64), generator=gen(7)).to(torch.uint8)
    blob = torch.from_numpy(oracle.pack_codes(vals, 4))
    scale = torch.rand(30 * 2, generator=gen(8)).to(torch.float16)
    w = AffineQTensor(blob, AffineScheme(4, 32, scale), (30, 64), torch.bfloat16)
    model = nn.Module()
    model.embed_tokens = nn.Embedding(30, 64, padding_idx=2)
    model.embed_tokens._parameters["weight"] = w
    assert not is_lowered(model)
    AutoKernelLowering().apply(model)
    e = model.embed_tokens
    assert isinstance(e, NPEmbedding) and e.qtype == "sym" and e.padding_idx == 2 and e.out_dtype == torch.bfloat16
    assert torch.equal(e.u8_blob, blob) and is_lowered(model)
    with pytest.raises(NotImplementedError):
        e.set_backend("compile")(torch.zeros(1, dtype=torch.long))
    e.set_backend("cuda")
    with pytest.raises(RuntimeError):
        e.set_backend("default")
    unlower_model(model)
    back = model.embed_tokens
    assert isinstance(back, nn.Embedding) and back.padding_idx == 2
    q = back._parameters["weight"]
    assert torch.equal(q.u8_blob, blob) and torch.equal(q.qscheme.scale, scale) and q.qscheme.zero_point is None
    assert not is_lowered(model)
    linearize_qtensor_embeddings(model)                     # and lowers again from the restored form
    assert isinstance(model.embed_tokens, NPEmbedding)
