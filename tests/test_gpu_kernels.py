"""GPU parity tests: every kernel, called through the C ABI, against the CPU oracle.

Decode is checked bit-exactly (rtol = atol = 0), as the reference checks its own decode kernel
(tests/nn/test_np_vq_linear.py:546-562 of the reference).  Forward outputs are checked against
the oracle evaluated in fp64 on the weight decoded for the activation dtype, with the bound
max|err| <= 1e-2 * RMS(y_ref) (+ half an ulp of the output dtype).
"""

import pytest
import torch

import oracle
from helpers import assert_output_close
from neuropress_b200 import kernels
from synthetic import make_activations, make_q_layer, make_vq_layer

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _vq_ext_gpu(layer):
    return {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in layer.ext().items()}


def _decode_gpu(layer, dtype):
    return kernels.vq_dequant(layer.packed.to(DEV), layer.centroids.to(DEV), layer.bits,
                              layer.out_features, layer.in_features, dtype, **_vq_ext_gpu(layer))


def _decode_ref(layer, dtype):
    return oracle.vq_decode(layer.packed, layer.centroids, layer.bits, layer.out_features,
                            layer.in_features, dtype, **layer.ext())


# ---------------------------------------------------------------------------- decode ---
@pytest.mark.parametrize("bits", [4, 5, 8, 10, 12, 14, 15, 16])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("vl", [4, 8])
def test_vq_decode_bit_exact(bits, dtype, vl):
    # N = 37: the last index ends mid-byte for odd widths; no padding on the stream.
    layer = make_vq_layer(37, 64, num_centroids=min(1 << bits, 4096), bits=bits, vector_len=vl,
                          centroid_std=1.0, seed=bits)
    out = _decode_gpu(layer, dtype)
    assert out.dtype == dtype
    torch.testing.assert_close(out.cpu(), _decode_ref(layer, dtype), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_vq_decode_extended_forms_bit_exact(dtype):
    layer = make_vq_layer(96, 256, num_centroids=512, bits=16, seed=3, residual_centroids=256,
                          row_scale=True, cols_per_codebook=128)
    torch.testing.assert_close(_decode_gpu(layer, dtype).cpu(), _decode_ref(layer, dtype),
                               rtol=0, atol=0)


def test_vq_decode_large_codebook_bit_exact():
    layer = make_vq_layer(512, 1024, num_centroids=65536, bits=16, seed=5, residual_centroids=256,
                          row_scale=True)
    torch.testing.assert_close(_decode_gpu(layer, torch.bfloat16).cpu(),
                               _decode_ref(layer, torch.bfloat16), rtol=0, atol=0)


def test_vq_decode_empty_and_errors():
    layer = make_vq_layer(8, 64, num_centroids=16, seed=1)
    out = kernels.vq_dequant(layer.packed.to(DEV)[:0], layer.centroids.to(DEV), 4, 0, 64, torch.float16)
    assert out.shape == (0, 64)
    with pytest.raises(RuntimeError, match="shape"):  # stream too short
        kernels.vq_dequant(layer.packed.to(DEV)[:-1], layer.centroids.to(DEV), 4, 8, 64, torch.float16)
    with pytest.raises(RuntimeError):  # CPU tensors are refused: no fallback
        kernels.vq_dequant(layer.packed, layer.centroids, 4, 8, 64, torch.float16)
    with pytest.raises(RuntimeError, match="unsupported"):
        kernels.vq_dequant(layer.packed.to(DEV), layer.centroids.to(DEV), 3, 8, 64, torch.float16)


@pytest.mark.parametrize("asym,gs", [(False, 32), (True, 64), (True, 128), (False, 8)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_q_decode_bit_exact(asym, gs, dtype):
    layer = make_q_layer(48, 256, group_size=gs, asym=asym, seed=gs)
    out = kernels.q_dequant(layer.codes.to(DEV), layer.scale.to(DEV), 4, gs,
                            None if layer.zero_point is None else layer.zero_point.to(DEV), dtype)
    ref = oracle.q_decode(layer.codes, layer.scale, layer.zero_point, 4, gs, dtype)
    torch.testing.assert_close(out.cpu(), ref, rtol=0, atol=0)


def test_q_decode_8bit_bit_exact():
    layer = make_q_layer(16, 128, group_size=32, asym=True, nbits=8, seed=2)
    out = kernels.q_dequant(layer.codes.to(DEV), layer.scale.to(DEV), 8, 32, layer.zero_point.to(DEV),
                            torch.bfloat16)
    ref = oracle.q_decode(layer.codes, layer.scale, layer.zero_point, 8, 32, torch.bfloat16)
    torch.testing.assert_close(out.cpu(), ref, rtol=0, atol=0)


# ------------------------------------------------------------------------------ GEMV ---
def _vq_forward_ref64(layer, x):
    return oracle.vq_forward_f32(x, layer.packed, layer.centroids, layer.bits, layer.out_features,
                                 layer.in_features, layer.bias, **layer.ext())


GEMV_CASES = [
    # (N, K, NC, bits, VL, residual, scale, cols_per_codebook, bias)
    (2048, 2048, 256, 8, 8, 0, False, 0, False),       # small codebook in smem, byte indices
    (300, 1024, 4096, 12, 8, 0, False, 0, True),       # 12-bit packed stream
    (300, 1024, 4096, 16, 8, 0, False, 512, False),    # per-column-group codebooks, 64 KiB total
    (257, 2048, 65536, 16, 8, 256, True, 0, False),    # large codebook + residual + row scale
    (24, 64, 1024, 10, 4, 0, False, 0, False),         # VL 4, generic width
    (24, 96, 16, 4, 8, 0, False, 0, True),             # K not a multiple of 64 -> generic path
    (64, 8192, 4096, 16, 8, 0, False, 2048, False),    # 4 codebooks = 256 KiB -> gathers from L2
]


@pytest.mark.parametrize("case", GEMV_CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows", [1, 2, 5, 8])
def test_vq_gemv_matches_oracle(case, dtype, rows):
    N, K, NC, bits, vl, res, scale, cpc, bias = case
    layer = make_vq_layer(N, K, num_centroids=NC, bits=bits, vector_len=vl, seed=N + K,
                          residual_centroids=res, row_scale=scale, cols_per_codebook=cpc, bias=bias)
    x = make_activations(rows, K, dtype, seed=rows)
    y = kernels.vq_gemv(x.to(DEV), layer.packed.to(DEV), layer.centroids.to(DEV), bits, N,
                        None if layer.bias is None else layer.bias.to(DEV), **_vq_ext_gpu(layer))
    assert y.shape == (rows, N) and y.dtype == dtype
    assert_output_close(y, _vq_forward_ref64(layer, x), dtype)


SMALL_BATCH_CASES = [
    # (N, K, NC, bits, residual, scale, cols_per_codebook, bias): forms the tensor-core kernel takes
    (2048, 2048, 256, 8, 0, False, 0, False),
    (300, 1024, 4096, 12, 0, False, 0, True),
    (300, 1024, 4096, 16, 0, False, 512, False),
    (257, 2048, 65536, 16, 256, True, 0, True),
    (130, 4096, 4096, 16, 256, True, 2048, False),     # two codebooks of 2048 columns + residual
    (5, 1024, 256, 8, 0, True, 0, True),               # fewer output rows than one 16-row group
]


@pytest.mark.parametrize("case", SMALL_BATCH_CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows", [3, 9, 16])
def test_vq_small_batch_tensor_core_kernel_matches_oracle(case, dtype, rows):
    """3..16 rows through npb_vq_gemv: decode in registers + mma.sync (vq_gemv_mma.cu)."""
    N, K, NC, bits, res, scale, cpc, bias = case
    layer = make_vq_layer(N, K, num_centroids=NC, bits=bits, seed=N + K, residual_centroids=res,
                          row_scale=scale, cols_per_codebook=cpc, bias=bias)
    x = make_activations(rows, K, dtype, seed=rows)
    y = kernels.vq_gemv(x.to(DEV), layer.packed.to(DEV), layer.centroids.to(DEV), bits, N,
                        None if layer.bias is None else layer.bias.to(DEV), **_vq_ext_gpu(layer))
    assert y.shape == (rows, N) and y.dtype == dtype
    assert_output_close(y, _vq_forward_ref64(layer, x), dtype)


def test_vq_gemv_rejects_too_many_rows():
    layer = make_vq_layer(16, 64, num_centroids=16, seed=1)
    x = make_activations(9, 64, torch.float16).to(DEV)
    with pytest.raises(RuntimeError, match="unsupported"):
        kernels.vq_gemv(x, layer.packed.to(DEV), layer.centroids.to(DEV), 4, 16)


@pytest.mark.parametrize("asym,gs", [(False, 32), (True, 64), (True, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("shape", [(320, 1024), (67, 4096), (40, 192), (100, 512), (2500, 2048)])
def test_q_gemv_matches_oracle(asym, gs, dtype, rows, shape):
    N, K = shape
    if K % gs:
        pytest.skip("group does not divide K")
    layer = make_q_layer(N, K, group_size=gs, asym=asym, seed=N, bias=True)
    x = make_activations(rows, K, dtype, seed=rows)
    y = kernels.q_gemv(x.to(DEV), layer.codes.to(DEV), layer.scale.to(DEV), 4, gs,
                       None if layer.zero_point is None else layer.zero_point.to(DEV),
                       layer.bias.to(DEV))
    ref = oracle.q_forward_f64(x, layer.codes, layer.scale, 4, gs, layer.zero_point, layer.bias)
    assert_output_close(y, ref, dtype)


@pytest.mark.parametrize("asym,gs", [(False, 32), (True, 64), (True, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows", [1, 2, 3, 6, 8])
@pytest.mark.parametrize("shape", [(67, 4096), (1192, 4096), (200, 8192), (2411, 4096), (16, 4096), (5000, 4096)])
def test_q_gemv_ring_shapes(asym, gs, dtype, rows, shape):
    """K a multiple of 4096 takes the bulk-copy ring GEMV (1-2 rows; 3-8 rows at K = 4096, sixteen
    weight rows per stage): row counts that are not multiples of 8 / 16 (the last ring stage re-reads
    the last row), a single stage, several stages per CTA, two step pairs per warp (K = 8192; 3-8
    rows then take the register-fed kernel)."""
    N, K = shape
    layer = make_q_layer(N, K, group_size=gs, asym=asym, seed=N + gs, bias=True)
    x = make_activations(rows, K, dtype, seed=rows + N)
    y = kernels.q_gemv(x.to(DEV), layer.codes.to(DEV), layer.scale.to(DEV), 4, gs,
                       None if layer.zero_point is None else layer.zero_point.to(DEV), layer.bias.to(DEV))
    ref = oracle.q_forward_f64(x, layer.codes, layer.scale, 4, gs, layer.zero_point, layer.bias)
    assert_output_close(y, ref, dtype)
    from neuropress_b200 import _cabi
    assert _cabi.gemm_device_status() == 0


@pytest.mark.parametrize("asym", [False, True])
@pytest.mark.parametrize("rows", [1, 2, 3, 8])
def test_q_gemv_group_size_that_is_not_a_power_of_two(asym, rows):
    """Groups of 96 (K = 1536): the ring and full-column kernels decline (they shift by the group
    size), the block-diagonal tensor-core kernel takes every row count."""
    N, K, gs = 200, 1536, 96
    layer = make_q_layer(N, K, group_size=gs, asym=asym, seed=N + gs, bias=True)
    x = make_activations(rows, K, torch.bfloat16, seed=rows)
    y = kernels.q_gemv(x.to(DEV), layer.codes.to(DEV), layer.scale.to(DEV), 4, gs,
                       None if layer.zero_point is None else layer.zero_point.to(DEV), layer.bias.to(DEV))
    ref = oracle.q_forward_f64(x, layer.codes, layer.scale, 4, gs, layer.zero_point, layer.bias)
    assert_output_close(y, ref, torch.bfloat16)


# ------------------------------------------------------------------------- LUT gather ---
@pytest.mark.parametrize("bits,nc", [(4, 16), (8, 256), (10, 1000), (12, 4096), (16, 5000)])
@pytest.mark.parametrize("shape", [(37, 96, 1), (256, 512, 3), (100, 40, 16)])
def test_vq_lut_gather_matches_the_reference_formula(bits, nc, shape):
    """y[m, j] = sum_g lut[m, g, idx[j, g]] with lut = x_groups @ C^T, the reference's cuda_lut
    arithmetic (np_vq_linear.py:1189-1248, vq_linear_lut.cu:121-206); fp32, summation order free."""
    n, k, m = shape
    vl = 4
    g = k // vl
    gen = torch.Generator().manual_seed(bits + n)
    cent = (torch.randn(nc, vl, generator=gen) * 0.05).half()
    idx = torch.randint(0, nc, (n, g), generator=gen)
    x = torch.randn(m, k, generator=gen)
    lut = (x.reshape(m * g, vl) @ cent.float().T).reshape(m, g, nc).contiguous()
    packed = torch.from_numpy(oracle.pack_indices(idx.numpy().reshape(-1), bits))
    y = kernels.vq_lut_gather(lut.to(DEV), packed.to(DEV), bits, n)
    assert y.dtype == torch.float32 and y.shape == (m, n)
    ref = lut.double().gather(2, idx.T.unsqueeze(0).expand(m, g, n)).sum(1)      # [m, n]
    assert_output_close(y, ref, torch.float32, tol=1e-5)
    w = cent.float()[idx].reshape(n, k)                                            # the same product, decoded
    assert_output_close(y, x.double() @ w.double().T, torch.float32, tol=1e-4)


# ------------------------------------------------------------------- dense tcgen05 GEMM ---
@pytest.mark.parametrize("shape", [(128, 256, 64), (128, 256, 512), (256, 512, 1024),
                                   (130, 72, 96), (1, 64, 64), (2048, 1024, 512), (300, 14336, 256)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_dense_gemm_matches_fp32_reference(shape, dtype):
    M, N, K = shape
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(dtype)
    w = (torch.randn(N, K, generator=g) * 0.05).to(dtype)
    b = torch.randn(N, generator=g)
    y = kernels.gemm(x.to(DEV), w.to(DEV), b.to(DEV))
    from neuropress_b200 import _cabi
    assert _cabi.gemm_device_status() == 0
    ref = x.double() @ w.double().T + b.double()
    assert_output_close(y, ref, dtype, tol=2e-3)


PAIR_SHAPES = [(256, 512, 1024), (130, 72, 96), (384, 1000, 192), (640, 4096, 512), (1000, 2056, 320),
               (2048, 1024, 512), (300, 14336, 256), (4096, 4736, 1024), (129, 16, 64)]


@pytest.mark.parametrize("shape", PAIR_SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_dense_gemm_cta_pairs(shape, dtype):
    """The cta_group::2 form of the dense GEMM (two CTAs per 256-row tile), forced on for shapes
    the automatic policy would leave to single CTAs too: row counts that leave the second CTA of
    the last pair without rows (130, 384, 640), N and K tails, many tiles per pair (banded walk).
    Against fp64, and bit-for-bit against the single-CTA form (same products, same K order)."""
    from neuropress_b200 import _cabi
    lib = _cabi.load_library()
    M, N, K = shape
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(dtype).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(dtype).to(DEV)
    b = torch.randn(N, generator=g).to(DEV)
    before = lib.npb_get_gemm_pair_mode()
    try:
        assert lib.npb_set_gemm_pair_mode(2) == 0
        y_pair = kernels.gemm(x, w, b)
        assert _cabi.gemm_device_status() == 0
        assert lib.npb_set_gemm_pair_mode(0) == 0
        y_single = kernels.gemm(x, w, b)
        assert _cabi.gemm_device_status() == 0
    finally:
        lib.npb_set_gemm_pair_mode(before)
    ref = x.double().cpu() @ w.double().cpu().T + b.double().cpu()
    assert_output_close(y_pair, ref, dtype, tol=2e-3)
    assert torch.equal(y_pair, y_single)


def test_gemm_pair_mode_setter_validates():
    from neuropress_b200 import _cabi
    lib = _cabi.load_library()
    before = lib.npb_get_gemm_pair_mode()
    assert lib.npb_set_gemm_pair_mode(3) == 1 and lib.npb_set_gemm_pair_mode(-1) == 1
    assert lib.npb_get_gemm_pair_mode() == before


# ----------------------------------------------------------------- tile-decode GEMMs ---
FUSED_CASES = [
    (256, 512, 4096, 16, 0, False, 0),
    (200, 1024, 4096, 12, 0, False, 0),
    (384, 512, 65536, 16, 256, True, 0),
    (1000, 2048, 4096, 12, 16, False, 0),   # residual only, 12-bit, N tail
    (264, 1024, 4096, 16, 0, True, 512),    # row scale only, one codebook per 512 columns
    (128, 2048, 4096, 16, 0, False, 512),
    (130, 256, 256, 8, 0, False, 0),
    (72, 128, 1024, 10, 0, False, 0),
]


@pytest.mark.parametrize("case", FUSED_CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows", [9, 17, 128, 130, 300, 384])
def test_vq_gemm_fused_matches_oracle(case, dtype, rows):
    N, K, NC, bits, res, scale, cpc = case
    layer = make_vq_layer(N, K, num_centroids=NC, bits=bits, seed=N + K, residual_centroids=res,
                          row_scale=scale, cols_per_codebook=cpc, bias=True)
    x = make_activations(rows, K, dtype, seed=rows)
    y = kernels.vq_gemm_fused(x.to(DEV), layer.packed.to(DEV), layer.centroids.to(DEV), bits, N,
                              layer.bias.to(DEV), **_vq_ext_gpu(layer))
    from neuropress_b200 import _cabi
    assert _cabi.gemm_device_status() == 0
    assert_output_close(y, _vq_forward_ref64(layer, x), dtype, tol=2e-3)


COPY_CASES = [  # N, K, NC, bits, cols_per_codebook: plain weights (the copy form's domain)
    (256, 512, 4096, 16, 0),      # indices above the codebook size are clamped
    (200, 1024, 4096, 12, 0),     # N tail, 12-bit stream
    (1000, 2048, 65536, 16, 0),   # full 16-bit codebook: no clamp
    (128, 2048, 4096, 16, 512),   # one codebook per 512 columns
    (130, 256, 256, 8, 0),
    (4096, 8192, 65536, 16, 0),   # many tiles per CTA: every ring stage wraps
]


@pytest.mark.parametrize("case", COPY_CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows", [17, 32, 130, 300])
def test_vq_gemm_fused_copy_form_equals_converting_form(case, dtype, rows, monkeypatch):
    """Plain weights take the asynchronous-copy form of the tile-decode GEMM (codebook cast once,
    entries copied into the operand tile).  It must give the converting form's bits."""
    from neuropress_b200 import _cabi
    N, K, NC, bits, cpc = case
    layer = make_vq_layer(N, K, num_centroids=NC, bits=bits, seed=N + K + bits, cols_per_codebook=cpc, bias=True)
    x = make_activations(rows, K, dtype, seed=rows).to(DEV)
    args = (x, layer.packed.to(DEV), layer.centroids.to(DEV), bits, N, layer.bias.to(DEV))
    ext = _vq_ext_gpu(layer)
    monkeypatch.setattr(kernels, "VQ_COPY_FORM", True)
    y_copy = kernels.vq_gemm_fused(*args, **ext)
    assert _cabi.gemm_device_status() == 0
    monkeypatch.setattr(kernels, "VQ_COPY_FORM", False)
    y_conv = kernels.vq_gemm_fused(*args, **ext)
    assert _cabi.gemm_device_status() == 0
    assert torch.equal(y_copy, y_conv)
    if N <= 1000:
        assert_output_close(y_copy, _vq_forward_ref64(layer, x.cpu()), dtype, tol=2e-3)


DECODE_COPY_CASES = [  # N, K, NC, bits, cols_per_codebook
    (37, 64, 256, 8, 0),          # one ragged chunk (296 vectors)
    (300, 1024, 4096, 12, 0),     # 12-bit stream, 18.75 chunks
    (2048, 2048, 4096, 16, 512),  # one codebook per 512 columns, indices clamped + offset
    (9000, 4096, 65536, 16, 0),   # 2250 chunks over 148 CTAs: every stage wraps many times
    (1000, 8192, 65536, 16, 0),
]


@pytest.mark.parametrize("case", DECODE_COPY_CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_vq_decode_copy_form_equals_converting_form(case, dtype, monkeypatch):
    """Plain weights decode as a pipelined gather-copy from the codebook in the output type
    (npb_vq_decode_cb); the matrix must be the thread-per-vector decode's, bit for bit."""
    from neuropress_b200 import _cabi
    N, K, NC, bits, cpc = case
    layer = make_vq_layer(N, K, num_centroids=NC, bits=bits, seed=N + bits, cols_per_codebook=cpc)
    args = (layer.packed.to(DEV), layer.centroids.to(DEV), bits, N, K, dtype)
    ext = _vq_ext_gpu(layer)
    seen = []
    monkeypatch.setattr(kernels, "_launch", lambda sym, fn, *a: (seen.append(fn.__name__), fn(*a))[1])
    monkeypatch.setattr(kernels, "VQ_COPY_FORM", True)
    w_copy = kernels.vq_dequant(*args, **ext)
    assert seen[-1] == "npb_vq_decode_cb" and _cabi.gemm_device_status() == 0
    monkeypatch.setattr(kernels, "VQ_COPY_FORM", False)
    w_conv = kernels.vq_dequant(*args, **ext)
    assert seen[-1] == "npb_vq_decode"
    assert torch.equal(w_copy, w_conv)
    if N <= 2048:
        ref = oracle.vq_decode(layer.packed, layer.centroids, bits, N, K, dtype, **layer.ext())
        assert torch.equal(w_copy.cpu(), ref)


def test_vq_codebook_cast_matches_torch():
    c = (torch.randn(4096, 8, generator=torch.Generator().manual_seed(3)) * 0.02).half().to(DEV)
    assert torch.equal(kernels.codebook_in_dtype(c, torch.bfloat16), c.to(torch.bfloat16))
    assert kernels.codebook_in_dtype(c, torch.bfloat16) is kernels.codebook_in_dtype(c, torch.bfloat16)  # cached
    assert kernels.codebook_in_dtype(c, torch.float16) is c
    c.mul_(2)  # an in-place change invalidates the cached table
    assert torch.equal(kernels.codebook_in_dtype(c, torch.bfloat16), c.to(torch.bfloat16))


@pytest.mark.parametrize("asym,gs", [(False, 32), (True, 64), (True, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows", [9, 130, 384])
@pytest.mark.parametrize("shape", [(200, 1024), (256, 512), (72, 128)])
def test_q_gemm_fused_matches_oracle(asym, gs, dtype, rows, shape):
    N, K = shape
    layer = make_q_layer(N, K, group_size=gs, asym=asym, seed=gs, bias=True)
    x = make_activations(rows, K, dtype, seed=rows)
    y = kernels.q_gemm_fused(x.to(DEV), layer.codes.to(DEV), layer.scale.to(DEV), 4, gs,
                             None if layer.zero_point is None else layer.zero_point.to(DEV),
                             layer.bias.to(DEV))
    from neuropress_b200 import _cabi
    assert _cabi.gemm_device_status() == 0
    ref = oracle.q_forward_f64(x, layer.codes, layer.scale, 4, gs, layer.zero_point, layer.bias)
    assert_output_close(y, ref, dtype, tol=2e-3)


@pytest.mark.parametrize("asym,gs,rows", [(True, 64, 130), (False, 32, 384)])
def test_q_gemm_fused_full_size_layer(asym, gs, rows):
    """14336 x 4096: 112 CTAs, 64 K blocks each, so every ring stage wraps many times."""
    N, K = 14336, 4096
    layer = make_q_layer(N, K, group_size=gs, asym=asym, seed=gs)
    x = make_activations(rows, K, torch.bfloat16, seed=rows)
    y = kernels.q_gemm_fused(x.to(DEV), layer.codes.to(DEV), layer.scale.to(DEV), 4, gs,
                             None if layer.zero_point is None else layer.zero_point.to(DEV))
    from neuropress_b200 import _cabi
    assert _cabi.gemm_device_status() == 0
    # same weights as the one-pass decode (bit-exact by construction), so compare with the
    # dense path on the GPU exactly and with the oracle on a slice of the output
    w = kernels.q_dequant(layer.codes.to(DEV), layer.scale.to(DEV), 4, gs,
                          None if layer.zero_point is None else layer.zero_point.to(DEV), torch.bfloat16)
    y_dense = kernels.gemm(x.to(DEV), w)
    assert_output_close(y, y_dense.double().cpu(), torch.bfloat16, tol=2e-3)
    sl = slice(5000, 5256)
    ref = oracle.q_forward_f64(x, layer.codes[sl], layer.scale.view(N, -1)[sl].reshape(-1), 4, gs,
                               None if layer.zero_point is None else layer.zero_point.view(N, -1)[sl].reshape(-1),
                               None)
    assert_output_close(y[:, sl], ref, torch.bfloat16, tol=2e-3)


# ------------------------------------------------------------------------- RMSNorm ---
@pytest.mark.parametrize("shape", [(1, 2048), (5, 8192), (3, 100), (7, 2050), (300, 4096), (2, 16384),
                                   (4, 33000)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_rms_norm_matches_oracle(shape, dtype):
    """Fused RMSNorm against the fp64 restatement: within one rounding of the output type plus
    the fp32 error of the sum of squares (rows of every path: cached in registers, re-read,
    scalar for ragged H)."""
    M, H = shape
    g = torch.Generator().manual_seed(M * 7 + H)
    x = (torch.randn(M, H, generator=g) * 3).to(dtype)
    w = (torch.rand(H, generator=g) + 0.5).to(dtype)
    y = kernels.rms_norm(x.to(DEV), w.to(DEV), 1e-5)
    assert y.dtype == dtype and y.shape == (M, H)
    ref = oracle.rms_norm_f64(x, w, 1e-5)
    ulp = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -23}[dtype]
    err = (y.double().cpu() - ref).abs()
    assert bool((err <= ref.abs() * (ulp * 1.01 + 1e-5) + 1e-7).all())
    # and against the fp32 torch expression the reference documents: one output ulp apart at most
    # (fp32 outputs: a few fp32 ulps, the sums are taken in different orders)
    ref32 = oracle.rms_norm(x, w, 1e-5).double()
    rel = max(ulp * 2.01, 2e-6)
    assert bool(((y.double().cpu() - ref32).abs() <= ref32.abs() * rel + 1e-7).all())
