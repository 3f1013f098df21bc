"""Python wrapper of ``npb_vq_linear_static_scratch``: the VQ linear for hosts that cannot
allocate device memory.

Plain C / C++ services, plugins living in another process's memory budget, or loops where a
``cudaMalloc`` (a device-wide synchronisation that can also fail) is not acceptable call the C
entry point directly with their own input and output buffers; the temporary dense weight sits in
a 32 MiB array inside the library, so nothing is allocated by the call.  This wrapper exists
for tests and for Python callers that pre-allocate ``out`` themselves; when ``out`` is omitted
it is taken from torch, which is of course an allocation of the *caller*, not of the library.

All calls share the one array: keep them on a single stream.  The first call on a device
performs a one-time address lookup and should happen outside of stream capture.
"""

from __future__ import annotations

import torch

from .. import _cabi
from . import _bias_f32, _launch, _vq_ext

MAX_WEIGHT_ELEMENTS = _cabi.STATIC_SCRATCH_BYTES // 2


def vq_linear_static_scratch(x: torch.Tensor, packed_indices: torch.Tensor, centroids: torch.Tensor,
                             bits: int, out_features: int, bias: torch.Tensor | None = None, *,
                             out: torch.Tensor | None = None, **ext) -> torch.Tensor:
    """``x[M, K] @ W.T (+ bias)`` via decode + tensor-core GEMM with the library's built-in
    scratch.  ``out_features * K`` must not exceed :data:`MAX_WEIGHT_ELEMENTS` (16,777,216);
    larger layers raise ``RuntimeError`` before anything is launched."""
    ext = _vq_ext(ext)
    if x.dim() != 2:
        raise RuntimeError("vq_linear_static_scratch: x must be 2-D [M, K].")
    _cabi.require_cuda("vq_linear_static_scratch", x, packed_indices, centroids, out,
                       ext.get("residual_indices"), ext.get("residual_centroids"), ext.get("row_scale"))
    m, k = x.shape
    n = int(out_features)
    if n * k > MAX_WEIGHT_ELEMENTS:
        raise RuntimeError(
            f"vq_linear_static_scratch: weight of {n} x {k} = {n * k} elements needs {2 * n * k} bytes, "
            f"the built-in scratch holds {_cabi.STATIC_SCRATCH_BYTES} bytes ({MAX_WEIGHT_ELEMENTS} elements)."
        )
    lib = _cabi.load_library()
    w = _cabi.vq_struct(packed_indices, centroids, bits, **ext)
    b = _bias_f32(bias, n, x.device)
    if out is None:
        out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    elif out.shape != (m, n) or out.dtype != x.dtype:
        raise RuntimeError("vq_linear_static_scratch: `out` has the wrong shape or dtype.")
    with torch.cuda.device(x.device):
        rc = _launch("npb_vq_linear_static_scratch", lib.npb_vq_linear_static_scratch, w, x.data_ptr(),
                     _cabi.dtype_code(x.dtype), m, n, k, None if b is None else b.data_ptr(),
                     out.data_ptr(), _cabi.stream_ptr())
    _cabi.check(rc, "vq_linear_static_scratch")
    return out
