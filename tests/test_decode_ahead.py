"""DecodeAhead: the next layer's weight decoded on a side stream under the current layer's GEMM.
Results must be the bits of the plain back-to-back path in every calling pattern."""

from __future__ import annotations

import pytest
import torch

from neuropress_b200.nn import DecodeAhead, NPVQLinear, VQProxy
from neuropress_b200.transforms.vq_packing import IndexPacking, TieredIndexPacking

pytestmark = pytest.mark.gpu
DEV = "cuda"
SHAPES = [(512, 1024), (768, 512), (1024, 768), (256, 1024)]     # (N, K) of four independent linears


def _layers(entropy_at: int | None = None):
    g = torch.Generator().manual_seed(0)
    proxy = VQProxy((torch.randn(4096, 8, generator=g) * 0.02).half()).to(DEV)
    out = []
    for i, (n, k) in enumerate(SHAPES):
        idx = torch.randint(0, 4096, (n * (k // 8),), generator=g)
        bias = torch.randn(n, generator=g)
        if i == entropy_at:
            m = NPVQLinear(proxy, TieredIndexPacking.pack(idx, 12, 4), 12, n, k, 8, "cuda_tiered", bias=bias,
                           use_tiered=True, cold_bits=12)
        else:
            m = NPVQLinear(proxy, IndexPacking.pack(idx, 12), 12, n, k, 8, "cuda_wmma", bias=bias)
        out.append(m.to(DEV))
    xs = [torch.randn(500, k, generator=g).to(torch.bfloat16).to(DEV) for _, k in SHAPES]
    return out, xs


def test_chain_matches_back_to_back_path():
    layers, xs = _layers(entropy_at=2)
    want = [m(x) for m, x in zip(layers, xs)]
    ahead = DecodeAhead(layers, torch.bfloat16)
    for _ in range(3):                                     # repeated passes reuse both buffers
        got = [m(x) for m, x in zip(layers, xs)]
        ahead.join()
        for a, b in zip(got, want):
            assert torch.equal(a, b)
    # out of order, a layer twice in a row, another dtype (decodes by itself), fewer rows (another band)
    for i in (2, 0, 0, 3, 1):
        assert torch.equal(layers[i](xs[i]), want[i])
    y16 = layers[1](xs[1].half())
    assert y16.dtype == torch.float16
    layers[1](xs[1][:4])                                   # the GEMV band does not involve the buffers
    ahead.join()
    ahead.enabled = False
    assert torch.equal(layers[1](xs[1]), want[1])
    ahead.close()
    assert all(m._decode_ahead is None for m in layers)
    assert torch.equal(layers[3](xs[3]), want[3])


def test_chain_under_cuda_graph_capture():
    layers, xs = _layers()
    want = [m(x) for m, x in zip(layers, xs)]
    ahead = DecodeAhead(layers, torch.bfloat16)
    for _ in range(2):                                     # warm-up outside the capture
        [m(x) for m, x in zip(layers, xs)]
        ahead.join()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            got = [m(x) for m, x in zip(layers, xs)]
            ahead.join()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        for y in got:
            y.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            assert torch.equal(a, b)
    ahead.close()


def test_rejects_other_modules():
    with pytest.raises(TypeError):
        DecodeAhead([torch.nn.Linear(8, 8)])
    with pytest.raises(ValueError):
        DecodeAhead([])
