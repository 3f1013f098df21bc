"""ctypes binding of ``libneuropress_b200.so`` (the C ABI declared in ``include/neuropress_b200.h``).

PyTorch is used only as the owner of device memory and of the current CUDA stream: every
call passes raw ``data_ptr()`` values, sizes and ``torch.cuda.current_stream().cuda_stream``.
There is no CPU fallback: if the library is missing or a call returns a non-zero status a
``RuntimeError`` is raised (the reference raises ``RuntimeError`` from ``TORCH_CHECK`` in the
same situations, e.g. neuropress/kernels/vq_dequant.cu:112-127).
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libneuropress_b200.so"

NPB_F16, NPB_BF16, NPB_F32 = 0, 1, 2
GEMV_MAX_ROWS = 8
STATIC_SCRATCH_BYTES = 32 * 1024 * 1024

_DTYPE_CODE = {torch.float16: NPB_F16, torch.bfloat16: NPB_BF16, torch.float32: NPB_F32}

# Every symbol include/neuropress_b200.h declares; the CPU test-suite checks that the built
# library exports all of them.
EXPORTED_SYMBOLS = (
    "npb_status_string",
    "npb_last_cuda_error",
    "npb_version",
    "npb_vq_decode",
    "npb_q_decode",
    "npb_vq_gemv",
    "npb_q_gemv",
    "npb_vq_gemv_grouped",
    "npb_gemm",
    "npb_vq_gemm_fused",
    "npb_vq_gemm_fused_cb",
    "npb_vq_codebook_cast",
    "npb_vq_lut_gather",
    "npb_vq_gemm_fused_grouped",
    "npb_vq_decode_cb",
    "npb_vq_entropy_expand",
    "npb_q_gemm_fused",
    "npb_vq_linear_static_scratch",
    "npb_allgather_push",
    "npb_gemm_allgather",
    "npb_vq_gemv_allgather",
    "npb_rms_norm",
    "npb_vq_embedding",
    "npb_q_embedding",
    "npb_gemm_device_status",
    "npb_set_wait_limit_ns",
    "npb_get_wait_limit_ns",
    "npb_set_gemm_pair_mode",
    "npb_get_gemm_pair_mode",
)


class EntropyStreamStruct(Structure):
    """Mirror of ``npb_vq_entropy_stream``."""

    _fields_ = [
        ("buf", c_void_p), ("buf_bytes", c_int64), ("kind", c_int32), ("n_tiers", c_int32),
        ("prefix_off", c_int64 * 3), ("tier_off", c_int64 * 4), ("tier_bits", c_int32 * 4),
        ("tier_lo", c_int32 * 4), ("row_off", c_void_p * 4),
    ]


class VQWeightStruct(Structure):
    """Mirror of ``npb_vq_weight``."""

    _fields_ = [
        ("packed", c_void_p),
        ("packed_bytes", c_int64),
        ("bits", c_int32),
        ("vector_len", c_int32),
        ("centroids", c_void_p),
        ("num_centroids", c_int32),
        ("cols_per_codebook", c_int32),
        ("res_packed", c_void_p),
        ("res_packed_bytes", c_int64),
        ("res_bits", c_int32),
        ("res_num_centroids", c_int32),
        ("res_centroids", c_void_p),
        ("row_scale", c_void_p),
    ]


class QWeightStruct(Structure):
    """Mirror of ``npb_q_weight``."""

    _fields_ = [
        ("codes", c_void_p),
        ("scale", c_void_p),
        ("zero_point", c_void_p),
        ("nbits", c_int32),
        ("group_size", c_int32),
    ]


class GatherSinkStruct(Structure):
    """Mirror of ``npb_gather_sink``."""

    _fields_ = [
        ("peer_out", c_void_p),
        ("peer_flags", c_void_p),
        ("ld", c_int64),
        ("col0", c_int64),
        ("rank", c_int32),
        ("world", c_int32),
        ("epoch", ctypes.c_uint32),
        ("reserved", ctypes.c_uint32),
    ]


_lib: ctypes.CDLL | None = None


def library_available() -> bool:
    """True when the shared library has been built in-tree."""
    return LIB_PATH.is_file()


def load_library() -> ctypes.CDLL:
    """Load (once) and type the shared library.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.is_file():
        raise RuntimeError(
            f"{LIB_PATH.name} is not built: run `python -m neuropress_b200.build` "
            "(needs nvcc with sm_100a support).  There is no CPU fallback."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.npb_status_string.restype = c_char_p
    lib.npb_status_string.argtypes = [c_int]
    lib.npb_last_cuda_error.restype = c_char_p
    lib.npb_last_cuda_error.argtypes = []
    lib.npb_version.restype = c_int
    lib.npb_version.argtypes = []
    vq_p, q_p = POINTER(VQWeightStruct), POINTER(QWeightStruct)
    lib.npb_vq_decode.argtypes = [vq_p, c_int64, c_int64, c_void_p, c_int, c_void_p]
    lib.npb_q_decode.argtypes = [q_p, c_int64, c_int64, c_void_p, c_int, c_void_p]
    gemv_tail = [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]
    lib.npb_vq_gemv.argtypes = [vq_p, *gemv_tail]
    lib.npb_q_gemv.argtypes = [q_p, *gemv_tail]
    lib.npb_vq_gemv_grouped.argtypes = [vq_p, c_int, POINTER(c_int64), POINTER(c_void_p), c_void_p, c_int, c_int64,
                                        c_int64, c_void_p, ctypes.c_float, c_void_p, c_void_p]
    lib.npb_vq_gemm_fused.argtypes = [vq_p, *gemv_tail]
    lib.npb_vq_gemm_fused_cb.argtypes = [vq_p, c_void_p, *gemv_tail]
    lib.npb_vq_codebook_cast.argtypes = [c_void_p, c_int64, c_void_p, c_int, c_void_p]
    lib.npb_vq_gemm_fused_grouped.argtypes = [vq_p, c_int, POINTER(c_void_p), POINTER(c_int64), POINTER(c_void_p),
                                              c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p]
    lib.npb_vq_lut_gather.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int, c_int64,
                                      c_void_p, c_void_p]
    lib.npb_vq_decode_cb.argtypes = [vq_p, c_void_p, c_int64, c_int64, c_void_p, c_int, c_void_p]
    lib.npb_vq_entropy_expand.argtypes = [POINTER(EntropyStreamStruct), c_int64, c_int64, c_void_p, c_void_p]
    lib.npb_vq_linear_static_scratch.argtypes = [vq_p, *gemv_tail]
    lib.npb_q_gemm_fused.argtypes = [q_p, *gemv_tail]
    lib.npb_gemm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                             c_int, c_void_p]
    lib.npb_allgather_push.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int,
                                       c_int, ctypes.c_uint32, c_void_p]
    sink_p = POINTER(GatherSinkStruct)
    lib.npb_gemm_allgather.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                                       sink_p, c_void_p]
    lib.npb_vq_gemv_allgather.argtypes = [vq_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p,
                                          sink_p, c_void_p]
    lib.npb_rms_norm.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, ctypes.c_float, c_int,
                                 c_void_p]
    lib.npb_vq_embedding.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int32, c_int32,
                                     c_void_p, ctypes.c_float, c_void_p, c_int, c_void_p]
    lib.npb_q_embedding.argtypes = [c_void_p, c_int64, q_p, c_int64, c_int64, c_int64, ctypes.c_float, c_void_p,
                                    c_int, c_void_p]
    lib.npb_gemm_device_status.argtypes = [POINTER(c_int)]
    lib.npb_set_wait_limit_ns.argtypes = [ctypes.c_uint64]
    lib.npb_get_wait_limit_ns.argtypes = []
    lib.npb_set_gemm_pair_mode.argtypes = [c_int]
    lib.npb_get_gemm_pair_mode.argtypes = []
    for name in EXPORTED_SYMBOLS[3:]:
        getattr(lib, name).restype = c_int
    lib.npb_get_wait_limit_ns.restype = ctypes.c_uint64
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    """Raise ``RuntimeError`` for a non-zero ``npb_status``."""
    if status == 0:
        return
    lib = load_library()
    msg = lib.npb_status_string(status).decode()
    detail = lib.npb_last_cuda_error().decode() if status == 5 else ""
    raise RuntimeError(f"{what}: {msg}" + (f" [{detail}]" if detail else ""))


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise RuntimeError(f"dtype must be bfloat16, float16 or float32, got {dtype}") from None


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def require_cuda(name: str, *tensors: torch.Tensor | None) -> None:
    """The reference's ``TORCH_CHECK(t.is_cuda() && t.is_contiguous())`` for every operand."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(f"{name}: all tensors must be CUDA tensors (no CPU fallback).")
        if not t.is_contiguous():
            raise RuntimeError(f"{name}: all tensors must be contiguous.")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"{name}: tensors are on different devices ({dev} vs {t.device}).")


def vq_struct(
    packed: torch.Tensor,
    centroids: torch.Tensor,
    bits: int,
    *,
    residual_indices: torch.Tensor | None = None,
    residual_centroids: torch.Tensor | None = None,
    residual_bits: int = 8,
    row_scale: torch.Tensor | None = None,
    cols_per_codebook: int = 0,
) -> VQWeightStruct:
    """Describe one VQ weight.  ``centroids`` is ``[NC, VL]`` fp16, or ``[n_codebooks, NC, VL]``
    when ``cols_per_codebook`` > 0 (one codebook per block of that many input columns)."""
    if packed.dtype != torch.uint8:
        raise RuntimeError("packed indices must be uint8.")
    if centroids.dtype != torch.float16 or centroids.dim() not in (2, 3):
        raise RuntimeError("centroids must be a [NC, VL] (or [n_cb, NC, VL]) float16 tensor.")
    if (centroids.dim() == 3) != (cols_per_codebook > 0):
        raise RuntimeError("3-D centroids and cols_per_codebook > 0 go together.")
    if (residual_indices is None) != (residual_centroids is None):
        raise RuntimeError("residual_indices and residual_centroids must be given together.")
    if residual_centroids is not None and (
        residual_centroids.dtype != torch.float16 or residual_centroids.shape[-1] != centroids.shape[-1]
    ):
        raise RuntimeError("residual centroids must be float16 with the main vector length.")
    if row_scale is not None and row_scale.dtype != torch.float16:
        raise RuntimeError("row_scale must be float16.")
    s = VQWeightStruct()
    s.packed = packed.data_ptr()
    s.packed_bytes = packed.numel()
    s.bits = int(bits)
    s.vector_len = int(centroids.shape[-1])
    s.centroids = centroids.data_ptr()
    s.cols_per_codebook = int(cols_per_codebook)
    s.num_centroids = int(centroids.shape[-2])
    s.res_packed = _ptr(residual_indices)
    s.res_packed_bytes = 0 if residual_indices is None else residual_indices.numel()
    s.res_bits = int(residual_bits)
    s.res_num_centroids = 0 if residual_centroids is None else int(residual_centroids.shape[0])
    s.res_centroids = _ptr(residual_centroids)
    s.row_scale = _ptr(row_scale)
    return s


def q_struct(codes: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor | None,
             nbits: int, group_size: int) -> QWeightStruct:
    if codes.dtype != torch.uint8:
        raise RuntimeError("codes must be uint8.")
    if scale.dtype != torch.float16 or (zero_point is not None and zero_point.dtype != torch.float16):
        raise RuntimeError("scale / zero_point must be float16.")
    s = QWeightStruct()
    s.codes = codes.data_ptr()
    s.scale = scale.data_ptr()
    s.zero_point = _ptr(zero_point)
    s.nbits = int(nbits)
    s.group_size = int(group_size)
    return s


def gemm_device_status() -> int:
    """Synchronise and return (then clear) the GEMM kernels' give-up record (0 = none)."""
    out = c_int(0)
    rc = load_library().npb_gemm_device_status(ctypes.byref(out))
    if rc not in (0, 7):
        check(rc, "npb_gemm_device_status")
    return out.value
