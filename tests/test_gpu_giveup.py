"""The bounded waits of the all-gather kernels, made to run out on ONE GPU without a fault.

The kernels wait for a flag that a peer rank writes.  Here the "peer" is a second set of local
buffers that nobody ever signals, and the wait limit is lowered to 20 ms
(``npb_set_wait_limit_ns``): the wait runs out, the kernel records it in the status word of its
flag buffer and returns, and the context stays usable — the next ordinary call works.  Nothing
traps, spins without bound or touches a bad address.
"""

import ctypes

import pytest
import torch

from neuropress_b200 import _cabi

pytestmark = pytest.mark.gpu
DEV = "cuda"
WORLD = 2


@pytest.fixture
def short_wait():
    lib = _cabi.load_library()
    before = lib.npb_get_wait_limit_ns()
    assert lib.npb_set_wait_limit_ns(20_000_000) == 0
    yield lib
    assert lib.npb_set_wait_limit_ns(before) == 0


def _fake_world(rows, n_full, dtype):
    """Two local [rows, n_full] buffers and two local flag buffers posing as ranks 0 and 1."""
    outs = [torch.zeros(rows, n_full, dtype=dtype, device=DEV) for _ in range(WORLD)]
    flags = [torch.zeros(WORLD + 3, dtype=torch.int32, device=DEV) for _ in range(WORLD)]
    out_ptrs = torch.tensor([o.data_ptr() for o in outs], dtype=torch.int64, device=DEV)
    flag_ptrs = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=DEV)
    return outs, flags, out_ptrs, flag_ptrs


def test_wait_limit_setter_validates():
    lib = _cabi.load_library()
    before = lib.npb_get_wait_limit_ns()
    assert before == 2_000_000_000
    assert lib.npb_set_wait_limit_ns(10) == 1            # below 1 us: NPB_ERR_INVALID_ARG
    assert lib.npb_set_wait_limit_ns(10 ** 12) == 1      # above 60 s
    assert lib.npb_get_wait_limit_ns() == before


def test_push_gather_gives_up_when_the_peer_never_signals(short_wait):
    lib = short_wait
    rows, n_local = 4, 64
    outs, flags, out_ptrs, flag_ptrs = _fake_world(rows, n_local * WORLD, torch.bfloat16)
    src = torch.randn(rows, n_local, device=DEV).to(torch.bfloat16)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = lib.npb_allgather_push(src.data_ptr(), rows, n_local, 2, out_ptrs.data_ptr(), flag_ptrs.data_ptr(),
                                0, WORLD, 0, _cabi.stream_ptr())
    t1.record()
    assert rc == 0
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1)
    assert 15.0 < ms < 1500.0, ms                        # gave up after ~20 ms, not after 2 s
    mine = flags[0].cpu()
    assert int(mine[WORLD + 1]) == 1                     # status word: a wait ran out
    assert int(mine[0]) == 1 and int(mine[1]) == 0       # own flag landed, the peer's never did
    assert int(flags[1].cpu()[0]) == 1                   # the peer was signalled
    for o in outs:                                       # the data was pushed all the same
        assert torch.equal(o[:, :n_local], src)
    # the context is intact: an ordinary single-rank call completes and reports success
    outs1, flags1, out_ptrs1, flag_ptrs1 = _fake_world(rows, n_local, torch.bfloat16)
    rc = lib.npb_allgather_push(src.data_ptr(), rows, n_local, 2, out_ptrs1.data_ptr(), flag_ptrs1.data_ptr(),
                                0, 1, 0, _cabi.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert int(flags1[0].cpu()[1 + 1]) == 0 and torch.equal(outs1[0], src)


def test_fused_gemm_gather_gives_up_and_the_next_gemm_works(short_wait):
    lib = short_wait
    m, n_local, k = 70, 256, 512
    outs, flags, out_ptrs, flag_ptrs = _fake_world(m, n_local * WORLD, torch.bfloat16)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n_local, k, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    sink = _cabi.GatherSinkStruct(peer_out=out_ptrs.data_ptr(), peer_flags=flag_ptrs.data_ptr(),
                                  ld=n_local * WORLD, col0=0, rank=0, world=WORLD, epoch=0)
    rc = lib.npb_gemm_allgather(x.data_ptr(), w.data_ptr(), None, m, n_local, k, _cabi.NPB_BF16,
                                ctypes.byref(sink), _cabi.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert int(flags[0].cpu()[WORLD + 1]) == 1           # the handshake gave up ...
    ref = (x.double() @ w.double().T)
    for o in outs:                                       # ... after the tiles had been stored and pushed
        err = (o[:, :n_local].double() - ref).abs().max()
        assert float(err) <= 2e-2 * float(ref.abs().max())
    assert _cabi.gemm_device_status() == 0               # no mbarrier wait of the GEMM itself ran out
    # the next plain GEMM is unaffected
    y = torch.empty(m, n_local, dtype=torch.bfloat16, device=DEV)
    assert lib.npb_gemm(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), m, n_local, k, _cabi.NPB_BF16,
                        _cabi.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert float((y.double() - ref).abs().max()) <= 2e-2 * float(ref.abs().max())
    assert _cabi.gemm_device_status() == 0


def test_gemm_output_at_an_odd_offset_takes_the_elementwise_stores():
    """An output that is a view 2 bytes into a buffer is not 16-byte aligned: the epilogue must
    fall back to element stores instead of issuing misaligned vector stores."""
    lib = _cabi.load_library()
    m, n, k = 33, 96, 128
    g = torch.Generator().manual_seed(1)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    buf = torch.zeros(m * n + 8, dtype=torch.bfloat16, device=DEV)
    y = buf[1:1 + m * n].view(m, n)
    assert y.data_ptr() % 16 == 2
    rc = lib.npb_gemm(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), m, n, k, _cabi.NPB_BF16,
                      _cabi.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    ref = x.double() @ w.double().T
    assert float((y.double() - ref).abs().max()) <= 2e-2 * float(ref.abs().max())
    assert float(buf[0]) == 0.0 and float(buf[1 + m * n:].abs().max()) == 0.0
