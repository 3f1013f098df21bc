"""Entropy-coded index streams (two-tier, N-tier, zero escape): the packers against the bytes the
reference's own packers produced (tests/golden/reference_entropy_vectors.npz), the oracle's
sequential decode against the same bytes, and -- on a GPU -- the expansion kernel against the
oracle, and entropy-coded ``NPVQLinear`` layers against the same layers with plain indices."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_output_close
from neuropress_b200.nn import NPVQLinear, VQProxy
from neuropress_b200.nn.backends import VQBackend
from neuropress_b200.transforms.vq_packing import (IndexPacking, NTieredIndexPacking, TieredIndexPacking,
                                                   ZeroEscapePacking, describe_entropy_buffer)

GOLD = np.load(Path(__file__).parent / "golden" / "reference_entropy_vectors.npz")
CASES = ("a", "b", "c", "d")


def _golden_buffers(tag):
    """(name, scheme, packer call, reference bytes, reference row offsets) for one golden case."""
    rows, groups, nc, _seed, cold = (int(v) for v in GOLD[f"{tag}_meta"])
    out = []
    for name in GOLD.files:
        if not name.startswith(f"{tag}_") or "_off" in name or name.endswith(("_meta", "_indices")):
            continue
        kind = name[len(tag) + 1:]
        offs = [GOLD[f"{name}_off{k}"] for k in range(8) if f"{name}_off{k}" in GOLD.files]
        if kind.startswith("tiered"):
            hot = int(kind[len("tiered"):])
            out.append((name, "tiered", lambda i, c=cold, h=hot: TieredIndexPacking.pack(i, c, h), GOLD[name], offs))
        elif kind.startswith("ntier"):
            tiers = [int(v) for v in kind[len("ntier"):].split("_")]
            out.append((name, "ntier", lambda i, t=tiers: NTieredIndexPacking.pack(i, t), GOLD[name], offs))
        else:
            out.append((name, "zero_escape", lambda i, c=cold: ZeroEscapePacking.pack(i, c), GOLD[name], offs))
    return rows, groups, nc, out


PACKERS = {"tiered": TieredIndexPacking, "ntier": NTieredIndexPacking, "zero_escape": ZeroEscapePacking}


@pytest.mark.parametrize("tag", CASES)
def test_packers_reproduce_the_reference_bytes(tag):
    rows, groups, _nc, bufs = _golden_buffers(tag)
    idx = torch.from_numpy(GOLD[f"{tag}_indices"].astype(np.int64))
    assert len(bufs) >= 5
    for name, scheme, pack, ref_bytes, ref_offs in bufs:
        mine = pack(idx)
        assert mine.dtype == torch.uint8 and np.array_equal(mine.numpy(), ref_bytes), name
        ref_t = torch.from_numpy(ref_bytes)
        assert torch.equal(PACKERS[scheme].unpack(ref_t), idx), name
        offs = PACKERS[scheme].compute_row_offsets(ref_t, rows, groups)
        assert len(offs) == len(ref_offs)
        for a, b in zip(offs, ref_offs):
            assert a.dtype == torch.int32 and np.array_equal(a.numpy(), b), name


@pytest.mark.parametrize("tag", CASES)
def test_oracle_decodes_the_reference_bytes(tag):
    rows, groups, _nc, bufs = _golden_buffers(tag)
    idx = GOLD[f"{tag}_indices"].astype(np.int64)
    for name, scheme, _pack, ref_bytes, ref_offs in bufs:
        assert np.array_equal(oracle.entropy_unpack(ref_bytes, scheme), idx), name
        for a, b in zip(oracle.entropy_row_offsets(ref_bytes, scheme, rows, groups), ref_offs):
            assert np.array_equal(a, b), name


def test_effective_bits_and_format_probes():
    ref = GOLD["effective_bits"]
    assert TieredIndexPacking.effective_bits(10, 100, 16, 4) == ref[0]
    assert NTieredIndexPacking.effective_bits([10, 20, 70], [4, 8, 16]) == ref[1]
    assert ZeroEscapePacking.effective_bits(1, 2, 3, 4, 16) == ref[2]
    assert TieredIndexPacking.effective_bits(0, 0, 12) == 12.0
    nt = torch.from_numpy(GOLD["a_ntier4_12"])
    ze = torch.from_numpy(GOLD["a_zesc"])
    assert NTieredIndexPacking.is_ntier_buffer(nt) and not NTieredIndexPacking.is_ntier_buffer(ze)
    assert ZeroEscapePacking.is_zero_escape_buffer(ze) and not ZeroEscapePacking.is_zero_escape_buffer(nt)
    assert not NTieredIndexPacking.is_ntier_buffer(torch.zeros(2, dtype=torch.uint8))
    assert TieredIndexPacking.hot_threshold(8) == 256
    assert NTieredIndexPacking.tier_thresholds([4, 8, 12]) == [16, 256, 4096]


def test_tiered_legacy_header_reads_as_four_hot_bits():
    idx = torch.tensor([0, 3, 200, 15, 99, 1, 7, 4000], dtype=torch.int64)
    buf = TieredIndexPacking.pack(idx, 12, 4)
    legacy = torch.cat([buf[:12], buf[16:]])          # the header without its fourth field
    # the byte after a legacy header is the prefix stream; make its first word implausible as hot_bits
    assert not 4 <= int(legacy[12:16].view(torch.int32)[0]) <= 16
    assert TieredIndexPacking._parse_header(legacy) == (8, 5, 12, 4, 12)
    assert torch.equal(TieredIndexPacking.unpack(legacy), idx)


def test_packers_reject_bad_arguments():
    idx = torch.arange(16)
    with pytest.raises(ValueError):
        TieredIndexPacking.pack(idx, 3)
    with pytest.raises(ValueError):
        TieredIndexPacking.pack(idx, 12, 3)
    with pytest.raises(ValueError):
        NTieredIndexPacking.pack(idx, [8])
    with pytest.raises(ValueError):
        NTieredIndexPacking.pack(idx, [8, 8])
    with pytest.raises(ValueError):
        ZeroEscapePacking.pack(idx, 21)
    with pytest.raises(ValueError):
        NTieredIndexPacking.unpack(torch.zeros(16, dtype=torch.uint8))
    with pytest.raises(ValueError):
        ZeroEscapePacking.unpack(torch.zeros(24, dtype=torch.uint8))
    with pytest.raises(ValueError):
        TieredIndexPacking.compute_row_offsets(TieredIndexPacking.pack(idx, 8), 3, 5)


def _zipf(n, nc, seed):
    w = 1.0 / torch.arange(1, nc + 1, dtype=torch.float64) ** 1.1
    return torch.multinomial(w / w.sum(), n, replacement=True, generator=torch.Generator().manual_seed(seed))


def _coded_layer(scheme, n, k, nc, seed, tiers=None, backend="auto"):
    """An entropy-coded layer and the same layer with plain indices."""
    g = k // 8
    idx = _zipf(n * g, nc, seed)
    cent = (torch.randn(nc, 8, generator=torch.Generator().manual_seed(seed + 1)) * 0.02).half()
    bits = IndexPacking.bits_for(nc)
    proxy = VQProxy(cent)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(seed + 2))
    plain = NPVQLinear(proxy, IndexPacking.pack(idx, 16), 16, n, k, 8, "cuda_wmma", bias=bias)
    if scheme == "tiered":
        coded = NPVQLinear(proxy, TieredIndexPacking.pack(idx, bits, 4), bits, n, k, 8, backend, bias=bias,
                           use_tiered=True, cold_bits=bits)
    elif scheme == "ntier":
        coded = NPVQLinear(proxy, NTieredIndexPacking.pack(idx, tiers), bits, n, k, 8, backend, bias=bias,
                           tier_bits=tiers)
    else:
        coded = NPVQLinear(proxy, ZeroEscapePacking.pack(idx, bits), bits, n, k, 8, backend, bias=bias,
                           zero_escape=True)
    return coded, plain, idx


def test_entropy_coded_module_on_cpu():
    """Construction computes the row offsets under the reference's buffer names; explicit backend
    names resolve as in the reference; there is no CPU forward."""
    coded, _plain, _idx = _coded_layer("tiered", 16, 64, 300, 1, backend="cuda_tiered")
    assert coded.backend == VQBackend.CUDA_TIERED
    assert set(dict(coded.named_buffers())) >= {"packed_indices", "hot_row_offsets", "cold_row_offsets", "bias"}
    assert coded.hot_row_offsets.dtype == torch.int32 and coded.hot_row_offsets.numel() == 17
    coded, _p, _i = _coded_layer("ntier", 16, 64, 300, 2, tiers=[4, 6, 9], backend="cuda_ntier")
    assert [n for n, _ in coded.named_buffers() if n.startswith("ntier_row_off_")] == [f"ntier_row_off_{i}" for i in range(3)]
    coded, _p, _i = _coded_layer("zero_escape", 16, 64, 300, 3, backend="cuda_zero_escape")
    assert sum(n.startswith("zesc_row_off_") for n, _ in coded.named_buffers()) == 4
    assert "index_stream=zero_escape" in coded.extra_repr()
    with pytest.raises(RuntimeError):
        coded(torch.zeros(1, 64))
    with pytest.raises(ValueError):    # a buffer for another shape
        NPVQLinear(coded.proxy, coded.packed_indices, 9, 8, 64, 8, "cuda_zero_escape", zero_escape=True)
    lay = describe_entropy_buffer(coded.packed_indices, "zero_escape")
    assert lay["kind"] == 2 and lay["bits"][:3] == [0, 4, 8] and lay["n"] == 16 * 8


# ------------------------------------------------------------------------------------------ GPU
gpu = pytest.mark.gpu
DEV = "cuda"


def _expand_gpu(buf: torch.Tensor, scheme: str, rows: int, groups: int) -> np.ndarray:
    from neuropress_b200 import kernels

    lay = describe_entropy_buffer(buf, scheme)
    offs = [o.to(DEV) for o in PACKERS[scheme].compute_row_offsets(buf, rows, groups)]
    out = kernels.vq_entropy_expand(buf.to(DEV), lay, offs, rows, groups)
    assert out.dtype == torch.uint8 and out.numel() == rows * groups * 2
    return out.cpu().numpy().view("<u2").astype(np.int64)


@gpu
@pytest.mark.parametrize("tag", CASES)
def test_expand_kernel_on_the_reference_bytes(tag):
    """Bit-exact: the kernel's table equals the indices the reference packed (ragged group counts
    75 and 1100: a row is not a whole number of prefix words; 1100 needs a second chunk)."""
    rows, groups, _nc, bufs = _golden_buffers(tag)
    idx = GOLD[f"{tag}_indices"].astype(np.int64)
    for name, scheme, _pack, ref_bytes, _offs in bufs:
        got = _expand_gpu(torch.from_numpy(ref_bytes), scheme, rows, groups)
        assert np.array_equal(got, idx), name


@gpu
@pytest.mark.parametrize("shape", [(64, 512, 65536), (5, 3584, 65536), (300, 256, 4096), (1, 8, 17), (33, 33, 300)])
def test_expand_kernel_against_the_oracle(shape):
    rows, groups, nc = shape
    idx = _zipf(rows * groups, nc, rows + groups)
    cold = IndexPacking.bits_for(nc)
    bufs = [("tiered", TieredIndexPacking.pack(idx, cold, 4)), ("tiered", TieredIndexPacking.pack(idx, cold, 8)),
            ("zero_escape", ZeroEscapePacking.pack(idx, cold))]
    for tiers in ([4, cold], [5, 9, cold], [4, 7, 10, cold]):
        if sorted(set(tiers)) == tiers:
            bufs.append(("ntier", NTieredIndexPacking.pack(idx, tiers)))
    for scheme, buf in bufs:
        want = oracle.entropy_unpack(buf.numpy(), scheme)
        assert np.array_equal(want, idx.numpy())
        assert np.array_equal(_expand_gpu(buf, scheme, rows, groups), want), scheme


@gpu
def test_expand_kernel_uniform_and_degenerate_streams():
    """All indices in one tier (empty other streams), and all zero."""
    for idx in (torch.zeros(40 * 16, dtype=torch.int64), torch.full((40 * 16,), 4000),
                torch.randint(0, 16, (40 * 16,), generator=torch.Generator().manual_seed(0))):
        for scheme, buf in (("tiered", TieredIndexPacking.pack(idx, 12)), ("zero_escape", ZeroEscapePacking.pack(idx, 12)),
                            ("ntier", NTieredIndexPacking.pack(idx, [4, 8, 12]))):
            assert np.array_equal(_expand_gpu(buf, scheme, 40, 16), idx.numpy()), scheme


@gpu
@pytest.mark.parametrize("scheme,tiers", [("tiered", None), ("ntier", [4, 8, 12, 16]), ("zero_escape", None)])
@pytest.mark.parametrize("rows", [1, 2, 8, 32, 500])
def test_entropy_coded_layer_equals_plain_layer(scheme, tiers, rows):
    """Every row-count band: the coded layer expands its stream and then runs the plain layer's
    kernel on the same indices, so the outputs are bit-identical; the plain layer is checked
    against the oracle."""
    n, k, nc = 512, 2048, 65536
    coded, plain, idx = _coded_layer(scheme, n, k, nc, 7, tiers)
    assert coded.backend in (VQBackend.CUDA_TIERED, VQBackend.CUDA_NTIER, VQBackend.CUDA_ZERO_ESCAPE)
    x = torch.randn(rows, k, generator=torch.Generator().manual_seed(rows)).to(torch.bfloat16)
    coded.proxy.to(DEV)    # the shared codebook is not a sub-module of the layers (the model root owns it)
    y_coded = coded.to(DEV)(x.to(DEV))
    y_plain = plain.to(DEV)(x.to(DEV))
    assert torch.equal(y_coded, y_plain)
    ref = oracle.vq_forward(x, IndexPacking.pack(idx, 16).numpy(), plain.proxy.centroids.cpu(), 16, n, k,
                            bias=plain.bias.cpu())
    assert_output_close(y_coded, ref.double(), torch.bfloat16, tol=2e-2)   # ref is itself bf16-rounded


@gpu
def test_entropy_coded_qtensor_round_trip():
    from neuropress_b200.qtensor import VQQTensor, VQScheme

    n, k, nc = 64, 256, 4096
    idx = _zipf(n * (k // 8), nc, 11)
    cent = (torch.randn(nc, 8, generator=torch.Generator().manual_seed(12)) * 0.02).half()
    blob = TieredIndexPacking.pack(idx, 12, 4)
    lin = torch.nn.Linear(k, n, bias=False)
    lin._parameters["weight"] = VQQTensor(u8_blob=blob, qscheme=VQScheme(centroids=cent, vector_len=8,
                                                                         is_packed_indices=12, use_tiered=True),
                                          shape=(n, k))
    mod = NPVQLinear.from_qtensor_linear(lin, VQProxy(cent).to(DEV), "auto").to(DEV)
    assert mod.backend == VQBackend.CUDA_TIERED and mod.use_tiered
    back = mod.to_qtensor()
    assert back.qscheme.use_tiered and torch.equal(back.u8_blob.cpu(), blob)
    x = torch.randn(3, k, generator=torch.Generator().manual_seed(1)).half()
    ref = oracle.vq_forward(x, IndexPacking.pack(idx, 12).numpy(), cent, 12, n, k)
    y = mod(x.to(DEV))
    assert_output_close(y, ref.double(), torch.float16, tol=2e-2)
