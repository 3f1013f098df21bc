"""The entry point that allocates nothing (``npb_vq_linear_static_scratch``).

It serves hosts that cannot allocate device memory at call time (fixed-budget C / C++ services,
plugins, loops where cudaMalloc's device-wide synchronisation is unacceptable): the temporary
dense weight lives in a 32 MiB array inside the library.  It runs the same two kernels as the
regular decode + GEMM path, so its output must be bit-identical to that path — on a first call,
and on a second call in a row that reuses the array with a different, smaller layer (stale
contents must not matter).  Collected last on purpose: a run that stops at the first failure
has then already run every other test.
"""

import ctypes

import pytest
import torch

from neuropress_b200 import _cabi, kernels
from neuropress_b200.kernels.static_scratch import MAX_WEIGHT_ELEMENTS, vq_linear_static_scratch
from synthetic import make_activations, make_vq_layer

DEV = "cuda"


def _case(n, k, nc, bits, rows, seed, residual=0, scale=False, bias=False, dtype=torch.bfloat16):
    d = make_vq_layer(n, k, num_centroids=nc, bits=bits, seed=seed, residual_centroids=residual,
                      row_scale=scale, bias=bias)
    x = make_activations(rows, k, dtype, seed=seed).to(DEV)
    ext = {key: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for key, v in d.ext().items()}
    args = (x, d.packed.to(DEV), d.centroids.to(DEV), bits, n, None if d.bias is None else d.bias.to(DEV))
    return args, ext


@pytest.mark.gpu
def test_static_scratch_matches_regular_path_on_two_calls_in_a_row():
    # first call: a large layer (8 MiB of decoded weight), residual + row scale + bias
    args1, ext1 = _case(2048, 2048, 65536, 16, 300, seed=1, residual=256, scale=True, bias=True)
    want1 = kernels.vq_dequant_gemm(*args1, **ext1)
    got1 = vq_linear_static_scratch(*args1, **ext1)
    # second call right after it: a smaller, different layer and dtype reusing the same array
    args2, ext2 = _case(200, 512, 4096, 12, 17, seed=2, dtype=torch.float16)
    want2 = kernels.vq_dequant_gemm(*args2, **ext2)
    got2 = vq_linear_static_scratch(*args2, **ext2)
    # and the first one again, into a caller-provided output buffer
    out = torch.empty_like(want1)
    got3 = vq_linear_static_scratch(*args1, out=out, **ext1)
    torch.cuda.synchronize()
    assert got3.data_ptr() == out.data_ptr()
    assert torch.equal(got1, want1)
    assert torch.equal(got2, want2)
    assert torch.equal(got3, want1)
    assert _cabi.gemm_device_status() == 0


@pytest.mark.gpu
def test_static_scratch_rejects_layers_beyond_its_capacity():
    lib = _cabi.load_library()
    n, k = 4096, 4104                      # 16,809,984 elements > 16,777,216
    assert n * k > MAX_WEIGHT_ELEMENTS
    x = torch.zeros(16, k, dtype=torch.bfloat16, device=DEV)
    y = torch.empty(16, n, dtype=torch.bfloat16, device=DEV)
    packed = torch.zeros(n * (k // 8) * 2, dtype=torch.uint8, device=DEV)
    cent = torch.zeros(16, 8, dtype=torch.float16, device=DEV)
    w = _cabi.vq_struct(packed, cent, 16)
    rc = lib.npb_vq_linear_static_scratch(w, x.data_ptr(), _cabi.NPB_BF16, 16, n, k, None, y.data_ptr(),
                                          _cabi.stream_ptr())
    assert rc == 6                         # NPB_ERR_TOO_LARGE, nothing launched
    assert b"capacity" in lib.npb_status_string(rc)
    with pytest.raises(RuntimeError, match="built-in scratch holds"):
        vq_linear_static_scratch(x, packed, cent, 16, n)
    # exactly at the limit is accepted
    x2 = torch.zeros(9, 4096, dtype=torch.bfloat16, device=DEV)
    packed2 = torch.zeros(4096 * 512 * 2, dtype=torch.uint8, device=DEV)
    assert vq_linear_static_scratch(x2, packed2, cent, 16, 4096).shape == (9, 4096)
    torch.cuda.synchronize()


def test_static_scratch_symbol_is_declared():
    assert "npb_vq_linear_static_scratch" in _cabi.EXPORTED_SYMBOLS
    assert _cabi.STATIC_SCRATCH_BYTES == 32 * 1024 * 1024 == 2 * MAX_WEIGHT_ELEMENTS
    if _cabi.library_available():
        assert hasattr(ctypes.CDLL(str(_cabi.LIB_PATH)), "npb_vq_linear_static_scratch")
