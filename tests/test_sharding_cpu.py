"""Host-side logic of the output-feature sharding, on CPU: shard slicing against the oracle
and the all-gather assembly between two gloo ranks."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from neuropress_b200.nn import NPLinear, NPVQLinear, VQProxy
from neuropress_b200.sharding import (ShardedLinear, gather_outputs, shard_q_linear, shard_rows,
                                      shard_vq_linear)
from synthetic import make_q_layer, make_vq_layer


def test_shard_rows():
    assert shard_rows(14336, 8, 0) == (0, 1792) and shard_rows(14336, 8, 7) == (12544, 14336)
    with pytest.raises(ValueError):
        shard_rows(10, 4, 0)
    with pytest.raises(ValueError):
        shard_rows(8, 4, 4)


@pytest.mark.parametrize("bits,world", [(16, 4), (12, 2), (8, 8)])
def test_vq_shards_decode_to_the_rows_of_the_full_layer(bits, world):
    nc = min(1 << bits, 4096)
    d = make_vq_layer(64, 128, num_centroids=nc, bits=bits, seed=bits, residual_centroids=256,
                      row_scale=True, bias=True)
    full = NPVQLinear(VQProxy(d.centroids), d.packed, bits, 64, 128, 8, backend="cuda", bias=d.bias,
                      residual_proxy=VQProxy(d.residual_centroids), residual_indices=d.residual_indices,
                      row_scale=d.row_scale)
    w_full = oracle.vq_decode(d.packed, d.centroids, bits, 64, 128, torch.bfloat16, **d.ext())
    for r in range(world):
        sh = shard_vq_linear(full, world, r)
        b, e = shard_rows(64, world, r)
        assert sh.out_features == e - b and sh.proxy is full.proxy
        w = oracle.vq_decode(sh.packed_indices, sh.proxy.centroids, bits, e - b, 128, torch.bfloat16,
                             residual_indices=sh.residual_indices,
                             residual_centroids=sh.residual_proxy.centroids, row_scale=sh.row_scale)
        assert torch.equal(w, w_full[b:e])
        assert torch.equal(sh.bias, d.bias[b:e])


def test_vq_shard_boundary_must_fall_on_a_byte():
    d = make_vq_layer(6, 8, num_centroids=4096, bits=12, seed=1)   # one 12-bit index per row
    full = NPVQLinear(VQProxy(d.centroids), d.packed, 12, 6, 8, 8, backend="cuda")
    with pytest.raises(ValueError, match="byte"):
        shard_vq_linear(full, 6, 1)


def test_q_shards_decode_to_the_rows_of_the_full_layer():
    q = make_q_layer(32, 128, group_size=64, asym=True, seed=3, bias=True)
    full = NPLinear(q.codes, q.scale, 32, 128, 64, 4, "asym", "cuda", bias=q.bias, zero_point=q.zero_point)
    w_full = oracle.q_decode(q.codes, q.scale, q.zero_point, 4, 64, torch.bfloat16)
    for r in range(4):
        sh = shard_q_linear(full, 4, r)
        w = oracle.q_decode(sh.u8_blob, sh.scale, sh.zero_point, 4, 64, torch.bfloat16)
        assert torch.equal(w, w_full[r * 8:(r + 1) * 8])


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _FakeLocal(torch.nn.Module):
    """Stands in for a rank's shard: returns that rank's columns of a known full output."""

    def __init__(self, full_w, begin, end):
        super().__init__()
        self.w = full_w[begin:end]
        self.in_features = full_w.shape[1]

    def forward(self, x):
        return x @ self.w.T


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        w = torch.randn(12, 8, generator=g)
        b, e = shard_rows(12, world, rank)
        layer = ShardedLinear(_FakeLocal(w, b, e), 12, rank, world)
        ok = True
        for shape in [(1, 8), (5, 8), (2, 3, 8)]:
            x = torch.randn(*shape, generator=g)
            y = layer(x)
            ok &= y.shape == (*shape[:-1], 12) and torch.allclose(y, x @ w.T, atol=1e-6)
        ok &= gather_outputs(torch.zeros(0, 6)).shape == (0, 12)
        local_only = ShardedLinear(_FakeLocal(w, b, e), 12, rank, world, gather=False)
        ok &= local_only(torch.ones(1, 8)).shape == (1, e - b)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_all_gather_assembly_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, True), (1, True)]


class _FakeGather:
    """Stands in for PushGather on CPU: records how the sharded layer used it."""

    def __init__(self, fused_rows: int, world: int = 2) -> None:
        self.fused_rows, self.world, self.dtype, self.max_rows = fused_rows, world, torch.float32, 1 << 20
        self.calls = []

    def can_push(self, m: int, dtype: torch.dtype) -> bool:
        return dtype == self.dtype and 0 < m <= self.max_rows

    def accepts(self, m: int, dtype: torch.dtype) -> bool:
        return m <= self.fused_rows

    def __call__(self, y: torch.Tensor) -> torch.Tensor:
        self.calls.append(("push", tuple(y.shape)))
        return torch.cat([y] * self.world, dim=-1)


def test_sharded_layer_hands_the_gather_to_the_shard_kernels(monkeypatch):
    """With a push gather enabled the shard's forward receives it (so that its kernels can store
    to the peers themselves); a kernel that cannot fuse gets the stand-alone push instead."""
    from neuropress_b200 import kernels

    d = make_vq_layer(32, 64, num_centroids=16, bits=4, seed=1)
    full = NPVQLinear(VQProxy(d.centroids), d.packed, 4, 32, 64, 8, backend="cuda")
    layer = ShardedLinear.from_layer(full, 0, 2)
    fake = _FakeGather(fused_rows=1)
    layer.push = fake
    seen = []

    def fake_gemv(x, packed, centroids, bits, n, bias, gather=None, **ext):
        seen.append(("gemv", x.shape[0], gather is fake))
        if gather is not None:
            return torch.zeros(x.shape[0], n * 2)       # the kernel filled the full-width buffer
        return torch.zeros(x.shape[0], n)

    monkeypatch.setattr(kernels, "vq_gemv", fake_gemv)
    y = layer(torch.zeros(1, 64))                        # 1 row: fused
    assert y.shape == (1, 32) and seen[-1] == ("gemv", 1, True) and fake.calls == []
    y = layer(torch.zeros(2, 1, 64))                     # 2 rows: kernel cannot fuse -> push after it
    assert y.shape == (2, 1, 32) and seen[-1] == ("gemv", 2, False) and fake.calls == [("push", (2, 16))]


def test_sharded_layer_outside_the_push_envelope_uses_the_collective(monkeypatch):
    """More rows than the peer-store buffers hold, or another dtype: the shard runs locally and
    the outputs go through ``gather_outputs`` (NCCL / gloo), never through the push gather."""
    from neuropress_b200 import kernels, sharding

    d = make_vq_layer(32, 64, num_centroids=16, bits=4, seed=1)
    full = NPVQLinear(VQProxy(d.centroids), d.packed, 4, 32, 64, 8, backend="cuda")
    layer = ShardedLinear.from_layer(full, 0, 2)
    fake = _FakeGather(fused_rows=1)
    fake.max_rows = 1
    layer.push = fake
    seen = []

    def fake_gemv(x, packed, centroids, bits, n, bias, gather=None, **ext):
        seen.append(gather)
        return torch.zeros(x.shape[0], n, dtype=x.dtype)

    monkeypatch.setattr(kernels, "vq_gemv", fake_gemv)
    monkeypatch.setattr(sharding, "gather_outputs", lambda y, group=None: torch.cat([y, y], dim=-1))
    y = layer(torch.zeros(2, 64))                        # 2 rows > max_rows = 1
    assert y.shape == (2, 32) and seen[-1] is None and fake.calls == []
    y = layer(torch.zeros(1, 64, dtype=torch.float16))   # dtype differs from the buffers'
    assert y.shape == (1, 32) and seen[-1] is None and fake.calls == []
    y = layer(torch.zeros(1, 64))                        # inside the envelope: fused as before
    assert seen[-1] is fake
