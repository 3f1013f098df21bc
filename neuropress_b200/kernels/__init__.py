"""Python wrappers over the C ABI, named after the reference's ``neuropress.kernels`` functions.

Reference (neuropress/kernels/__init__.py): ``vq_dequant`` :497-529, ``vq_linear`` (GEMV for
any row count), ``vq_linear_wmma`` :335-352, ``q_linear`` :109-151, ``warn_kernel_fallback``
:436-453; ``vq_gemm_triton`` (neuropress/kernels/vq_triton.py:119-179).  Each wrapper allocates
its output with torch (the C ABI never allocates), validates like the reference's
``TORCH_CHECK``s and raises ``RuntimeError`` on any failure.  Nothing here falls back to
PyTorch math.

The optional keyword arguments ``residual_indices``, ``residual_centroids``, ``residual_bits``,
``row_scale`` and ``cols_per_codebook`` select the extended weight forms (residual codebook,
per-output-row fp16 scale, one codebook per block of input columns); they default to the
reference's plain form.
"""

from __future__ import annotations

import ctypes
import logging
import os

import torch

from .. import _cabi

log = logging.getLogger(__name__)

GEMV_MAX_ROWS = _cabi.GEMV_MAX_ROWS

# Optional observer called as hook(symbol, True) right before and hook(symbol, False) right
# after each C-ABI launch (the benchmark records CUDA events with it).  None = no overhead.
_launch_hook = None


def set_launch_hook(fn) -> None:
    """Install (or with ``None`` remove) the launch observer."""
    global _launch_hook
    _launch_hook = fn


def _launch(symbol: str, fn, *args) -> int:
    hook = _launch_hook
    if hook is None:
        return fn(*args)
    hook(symbol, True)
    rc = fn(*args)
    hook(symbol, False)
    return rc

# ---------------------------------------------------------------------------
# Fallback reporting (kept for build-failure reporting only: there is no fallback path)
# ---------------------------------------------------------------------------

_warned_fallbacks: set[str] = set()


def warn_kernel_fallback(kernel: str, fallback: str, exc: BaseException) -> None:
    """Warn once per *kernel* that it is unavailable (reference: kernels/__init__.py:436-453)."""
    if kernel in _warned_fallbacks:
        return
    _warned_fallbacks.add(kernel)
    log.warning(
        "CUDA kernel %s unavailable (%s); %s. Build the library with "
        "`python -m neuropress_b200.build` (nvcc with sm_100a support).",
        kernel, exc, fallback,
    )


def _bias_f32(bias: torch.Tensor | None, n: int, device: torch.device) -> torch.Tensor | None:
    """The reference re-casts the bias to fp32 on every call (vq_linear_wmma.cu:512-515)."""
    if bias is None:
        return None
    if bias.numel() != n:
        raise RuntimeError(f"bias must have {n} elements, got {bias.numel()}.")
    b = bias.detach()
    if b.dtype != torch.float32 or b.device != device or not b.is_contiguous():
        b = b.to(device=device, dtype=torch.float32).contiguous()
    return b


def _vq_ext(ext: dict) -> dict:
    allowed = {"residual_indices", "residual_centroids", "residual_bits", "row_scale",
               "cols_per_codebook"}
    unknown = set(ext) - allowed
    if unknown:
        raise TypeError(f"unknown keyword argument(s): {sorted(unknown)}")
    return {k: v for k, v in ext.items() if v is not None}


def _infer_n(packed: torch.Tensor, bits: int, k: int, vl: int) -> int:
    """Output rows from the stream length, as vq_linear_wmma.cu:501-506 does."""
    if k % vl:
        raise RuntimeError(f"in_features={k} is not a multiple of vector_len={vl}.")
    g = k // vl
    n = (packed.numel() * 8) // (bits * g)
    if n <= 0:
        raise RuntimeError("packed buffer too short for one output row.")
    return n


# ---------------------------------------------------------------------------
# VQ
# ---------------------------------------------------------------------------


def vq_dequant(packed_indices: torch.Tensor, centroids: torch.Tensor, bits: int,
               out_features: int, in_features: int, dtype: torch.dtype, *,
               out: torch.Tensor | None = None, **ext) -> torch.Tensor:
    """Decode a packed VQ weight to a dense ``[out_features, in_features]`` tensor of *dtype*
    in one kernel pass (reference: kernels/__init__.py:497-529, vq_dequant.cu:105-146)."""
    ext = _vq_ext(ext)
    _cabi.require_cuda("vq_dequant", packed_indices, centroids, ext.get("residual_indices"),
                       ext.get("residual_centroids"), ext.get("row_scale"))
    lib = _cabi.load_library()
    w = _cabi.vq_struct(packed_indices, centroids, bits, **ext)
    if out is None:
        out = torch.empty((out_features, in_features), dtype=dtype, device=packed_indices.device)
    elif out.shape != (out_features, in_features) or out.dtype != dtype or not out.is_contiguous():
        raise RuntimeError("vq_dequant: `out` has the wrong shape, dtype or layout.")
    with torch.cuda.device(packed_indices.device):
        if (VQ_COPY_FORM and dtype in (torch.float16, torch.bfloat16) and bits in (8, 12, 16)
                and centroids.shape[-1] == 8 and in_features % 64 == 0 and "residual_indices" not in ext
                and "row_scale" not in ext and centroids.dtype == torch.float16 and centroids.is_contiguous()):
            # plain weight: gather-copy from the codebook in the output type
            table = codebook_in_dtype(centroids, dtype)
            rc = _launch("npb_vq_decode", lib.npb_vq_decode_cb, w, table.data_ptr(), out_features, in_features,
                         out.data_ptr(), _cabi.dtype_code(dtype), _cabi.stream_ptr())
            if rc == 0:
                return out
            if rc not in (2, 4):   # unsupported size / alignment: the converting decode takes it
                _cabi.check(rc, "vq_dequant")
        rc = _launch("npb_vq_decode", lib.npb_vq_decode, w, out_features, in_features, out.data_ptr(),
                               _cabi.dtype_code(dtype), _cabi.stream_ptr())
    _cabi.check(rc, "vq_dequant")
    return out


def _vq_call(fn_name: str, x: torch.Tensor, packed: torch.Tensor, centroids: torch.Tensor,
             bits: int, out_features: int | None, bias: torch.Tensor | None, ext: dict,
             gather=None) -> torch.Tensor:
    ext = _vq_ext(ext)
    if x.dim() != 2:
        raise RuntimeError(f"{fn_name}: x must be 2-D [M, K].")
    _cabi.require_cuda(fn_name, x, packed, centroids, ext.get("residual_indices"),
                       ext.get("residual_centroids"), ext.get("row_scale"))
    lib = _cabi.load_library()
    m, k = x.shape
    vl = centroids.shape[-1]
    n = out_features if out_features is not None else _infer_n(packed, bits, k, vl)
    w = _cabi.vq_struct(packed, centroids, bits, **ext)
    b = _bias_f32(bias, n, x.device)
    if gather is not None:
        # fused all-gather: the kernel stores into every rank's [M, N_full] buffer
        sink, out = gather.begin(m, n, x.dtype)
        with torch.cuda.device(x.device):
            rc = _launch(fn_name + "_allgather", getattr(lib, fn_name + "_allgather"), w, x.data_ptr(),
                         _cabi.dtype_code(x.dtype), m, n, k, None if b is None else b.data_ptr(),
                         ctypes.byref(sink), _cabi.stream_ptr())
        _cabi.check(rc, fn_name + "_allgather")
        return out
    y = torch.empty((m, n), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _launch(fn_name, getattr(lib, fn_name), w, x.data_ptr(), _cabi.dtype_code(x.dtype), m, n, k,
                                   None if b is None else b.data_ptr(), y.data_ptr(),
                                   _cabi.stream_ptr())
    _cabi.check(rc, fn_name)
    return y


def vq_gemv(x: torch.Tensor, packed_indices: torch.Tensor, centroids: torch.Tensor, bits: int,
            out_features: int | None = None, bias: torch.Tensor | None = None, gather=None,
            **ext) -> torch.Tensor:
    """Fused index-decode GEMV, ``x`` is ``[M, K]`` with ``M <= GEMV_MAX_ROWS``; fp16, bf16 or
    fp32 activations; output in ``x.dtype``.  With ``gather`` (a ``sharding.PushGather``) the
    kernel writes this rank's columns into every rank's buffer and the full ``[M, N]`` comes
    back (``npb_vq_gemv_allgather``)."""
    return _vq_call("npb_vq_gemv", x, packed_indices, centroids, bits, out_features, bias, ext, gather)


def vq_gemv_grouped(x: torch.Tensor, weights: list[tuple], bits: int, cols_per_codebook: int = 0,
                    norm_weight: torch.Tensor | None = None, norm_eps: float = 1e-6) -> torch.Tensor | None:
    """Several VQ weights applied to the same ``x`` ``[M, K]`` (M <= 16) in ONE launch, optionally
    with the RMSNorm of ``x`` fused into its staging.  ``weights`` is a list of ``(packed_indices,
    centroids, out_features, bias_f32_or_None)``; returns ``[M, sum(out_features)]`` with the
    weights' outputs side by side -- or ``None`` when the kernel does not take this combination
    (the caller then runs the norm and the linears one by one)."""
    if x.dim() != 2 or not 1 <= len(weights) <= 4:
        return None
    _cabi.require_cuda("vq_gemv_grouped", x, norm_weight, *[t for w in weights for t in (w[0], w[1], w[3])])
    lib = _cabi.load_library()
    m, k = x.shape
    n_w = len(weights)
    structs = (_cabi.VQWeightStruct * n_w)()
    ns = (ctypes.c_int64 * n_w)()
    biases = (ctypes.c_void_p * n_w)()
    for i, (packed, cent, n, bias) in enumerate(weights):
        structs[i] = _cabi.vq_struct(packed, cent, bits, cols_per_codebook=cols_per_codebook)
        ns[i] = int(n)
        biases[i] = None if bias is None else bias.data_ptr()
    if norm_weight is not None and (norm_weight.dtype != x.dtype or norm_weight.numel() != k):
        raise RuntimeError("vq_gemv_grouped: norm_weight must be [K] in the activation dtype.")
    y = torch.empty((m, sum(int(w[2]) for w in weights)), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _launch("npb_vq_gemv_grouped", lib.npb_vq_gemv_grouped, structs, n_w, ns, biases, x.data_ptr(),
                     _cabi.dtype_code(x.dtype), m, k, None if norm_weight is None else norm_weight.data_ptr(),
                     float(norm_eps), y.data_ptr(), _cabi.stream_ptr())
    if rc == 2:   # NPB_ERR_UNSUPPORTED: not a combination the grouped kernel takes
        return None
    _cabi.check(rc, "vq_gemv_grouped")
    return y


def vq_gemm_fused(x: torch.Tensor, packed_indices: torch.Tensor, centroids: torch.Tensor,
                  bits: int, out_features: int | None = None, bias: torch.Tensor | None = None,
                  **ext) -> torch.Tensor:
    """Tile-decode tensor-core GEMM (tcgen05): same signature as the reference's
    ``vq_gemm_triton`` (vq_triton.py:119-179).  bf16 / fp16 activations, vector length 8,
    ``K % 64 == 0``."""
    ext_n = _vq_ext(ext)
    if (VQ_COPY_FORM and ext_n.get("residual_indices") is None and ext_n.get("row_scale") is None
            and bits in (8, 12, 16) and centroids.shape[-1] == 8 and x.dim() == 2
            and x.dtype in (torch.float16, torch.bfloat16) and packed_indices.data_ptr() % 16 == 0):
        y = _vq_gemm_fused_copy(x, packed_indices, centroids, bits, out_features, bias, ext_n)
        if y is not None:
            return y
    return _vq_call("npb_vq_gemm_fused", x, packed_indices, centroids, bits, out_features, bias, ext)


# Plain weights take the copy form of the tile-decode GEMM (``npb_vq_gemm_fused_cb``): the codebook
# is cast once to the activation type and the kernel copies entries instead of converting them.
VQ_COPY_FORM = os.environ.get("NEUROPRESS_B200_VQ_COPY_FORM", "1") != "0"
_cast_codebooks: dict = {}   # id(centroids) -> (weakref to it, its version, {dtype: cast tensor})


def codebook_in_dtype(centroids: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``centroids`` (fp16 codebook) cast to ``dtype`` by ``npb_vq_codebook_cast``, cached per
    codebook tensor (dropped when the tensor dies or is modified in place).  fp16 returns the
    codebook itself."""
    if dtype == torch.float16:
        return centroids
    import weakref
    key = id(centroids)
    hit = _cast_codebooks.get(key)
    if hit is not None and hit[0]() is centroids and hit[1] == centroids._version and dtype in hit[2]:
        return hit[2][dtype]
    _cabi.require_cuda("vq_codebook_cast", centroids)
    lib = _cabi.load_library()
    out = torch.empty(centroids.shape, dtype=dtype, device=centroids.device)
    with torch.cuda.device(centroids.device):
        rc = _launch("npb_vq_codebook_cast", lib.npb_vq_codebook_cast, centroids.data_ptr(), centroids.numel(),
                     out.data_ptr(), _cabi.dtype_code(dtype), _cabi.stream_ptr())
    _cabi.check(rc, "npb_vq_codebook_cast")
    if hit is None or hit[0]() is not centroids or hit[1] != centroids._version:
        ref = weakref.ref(centroids, lambda _r, k=key: _cast_codebooks.pop(k, None))
        hit = (ref, centroids._version, {})
        _cast_codebooks[key] = hit
    hit[2][dtype] = out
    return out


def _vq_gemm_fused_copy(x, packed, centroids, bits, out_features, bias, ext):
    _cabi.require_cuda("npb_vq_gemm_fused_cb", x, packed, centroids)
    if not centroids.is_contiguous() or centroids.dtype != torch.float16:
        raise RuntimeError("vq_gemm_fused: the codebook must be a contiguous fp16 tensor.")
    lib = _cabi.load_library()
    m, k = x.shape
    n = out_features if out_features is not None else _infer_n(packed, bits, k, 8)
    cbx = codebook_in_dtype(centroids, x.dtype)
    w = _cabi.vq_struct(packed, centroids, bits, **ext)
    b = _bias_f32(bias, n, x.device)
    y = torch.empty((m, n), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _launch("npb_vq_gemm_fused", lib.npb_vq_gemm_fused_cb, w, cbx.data_ptr(), x.data_ptr(),
                     _cabi.dtype_code(x.dtype), m, n, k, None if b is None else b.data_ptr(), y.data_ptr(),
                     _cabi.stream_ptr())
    if rc == 2:   # NPB_ERR_UNSUPPORTED: this weight needs the converting form
        return None
    _cabi.check(rc, "npb_vq_gemm_fused_cb")
    return y


def vq_gemm_fused_grouped(x: torch.Tensor, weights: list[tuple], bits: int,
                          cols_per_codebook: int = 0) -> torch.Tensor | None:
    """Several plain VQ weights applied to the same ``x`` ``[M, K]`` by ONE launch of the copy form
    of the tile-decode GEMM.  ``weights`` as in :func:`vq_gemv_grouped`; returns ``[M,
    sum(out_features)]`` with the weights' outputs side by side, the same bits as one
    :func:`vq_gemm_fused` call per weight -- or ``None`` when the kernel does not take this
    combination."""
    if (x.dim() != 2 or not 1 <= len(weights) <= 4 or bits not in (8, 12, 16)
            or x.dtype not in (torch.float16, torch.bfloat16)):
        return None
    _cabi.require_cuda("vq_gemm_fused_grouped", x, *[t for w in weights for t in (w[0], w[1], w[3])])
    lib = _cabi.load_library()
    m, k = x.shape
    n_w = len(weights)
    structs = (_cabi.VQWeightStruct * n_w)()
    ns = (ctypes.c_int64 * n_w)()
    biases = (ctypes.c_void_p * n_w)()
    cbs = (ctypes.c_void_p * n_w)()
    keep = []
    for i, (packed, cent, n, bias) in enumerate(weights):
        if cent.dtype != torch.float16 or not cent.is_contiguous() or cent.shape[-1] != 8:
            return None
        structs[i] = _cabi.vq_struct(packed, cent, bits, cols_per_codebook=cols_per_codebook)
        ns[i] = int(n)
        biases[i] = None if bias is None else bias.data_ptr()
        cbx = codebook_in_dtype(cent, x.dtype)
        keep.append(cbx)
        cbs[i] = cbx.data_ptr()
    y = torch.empty((m, sum(int(w[2]) for w in weights)), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _launch("npb_vq_gemm_fused", lib.npb_vq_gemm_fused_grouped, structs, n_w, cbs, ns, biases,
                     x.data_ptr(), _cabi.dtype_code(x.dtype), m, k, y.data_ptr(), _cabi.stream_ptr())
    if rc in (2, 4):   # unsupported combination / alignment: the caller runs the members one by one
        return None
    _cabi.check(rc, "npb_vq_gemm_fused_grouped")
    return y


# Whether the mid-sized band runs the tile-decode GEMM (``npb_vq_gemm_fused``); when False it
# runs the one-pass decode followed by the dense tensor-core GEMM.
VQ_TILE_DECODE_GEMM = True
VQ_FUSED_MAX_ROWS = 384   # above this every weight tile would be decoded more than three times


def vq_entropy_expand(packed: torch.Tensor, layout: dict, row_offsets: list[torch.Tensor], n_rows: int,
                      n_groups: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """Expand an entropy-coded index buffer (``TieredIndexPacking`` / ``NTieredIndexPacking`` /
    ``ZeroEscapePacking``) into the plain 16-bit index stream: a 1-D ``uint8`` tensor of
    ``n_rows * n_groups * 2`` bytes, i.e. what ``IndexPacking.pack(indices, 16)`` gives.
    ``layout`` is ``transforms.entropy_packing.describe_entropy_buffer(packed, scheme)``,
    ``row_offsets`` the packer's ``compute_row_offsets`` as int32 tensors on the device of
    ``packed``, one per tier.  Stands in for the index decoding of the reference's
    ``vq_linear_tiered`` / ``vq_linear_ntier`` / ``vq_linear_zero_escape`` kernels."""
    _cabi.require_cuda("vq_entropy_expand", packed, *row_offsets)
    lib = _cabi.load_library()
    n_tiers = len(layout["bits"])
    if len(row_offsets) != n_tiers or layout["n"] != n_rows * n_groups:
        raise RuntimeError("vq_entropy_expand: row offsets / sizes do not match the buffer's header.")
    for off in row_offsets:
        if off.dtype != torch.int32 or off.numel() != n_rows + 1 or not off.is_contiguous():
            raise RuntimeError("vq_entropy_expand: row offsets must be contiguous int32 [n_rows + 1].")
    s = _cabi.EntropyStreamStruct()
    s.buf, s.buf_bytes, s.kind, s.n_tiers = packed.data_ptr(), packed.numel(), layout["kind"], n_tiers
    for k, v in enumerate(layout["prefix_off"]):
        s.prefix_off[k] = v
    for k in range(n_tiers):
        s.tier_off[k], s.tier_bits[k], s.tier_lo[k] = layout["tier_off"][k], layout["bits"][k], layout["lo"][k]
        s.row_off[k] = row_offsets[k].data_ptr()
    if out is None:
        out = torch.empty(n_rows * n_groups * 2, dtype=torch.uint8, device=packed.device)
    elif out.dtype != torch.uint8 or out.numel() != n_rows * n_groups * 2 or not out.is_contiguous():
        raise RuntimeError("vq_entropy_expand: `out` must be a contiguous uint8 tensor of 2 bytes per index.")
    with torch.cuda.device(packed.device):
        rc = _launch("npb_vq_entropy_expand", lib.npb_vq_entropy_expand, ctypes.byref(s), n_rows, n_groups,
                     out.data_ptr(), _cabi.stream_ptr())
    _cabi.check(rc, "vq_entropy_expand")
    return out


def vq_lut_gather(lut: torch.Tensor, packed_indices: torch.Tensor, bits: int, out_features: int) -> torch.Tensor:
    """LUT gather phase ``y[m, j] = sum_g lut[m, g, idx[j, g]]`` (reference: ``vq_lut_gather``,
    kernels/__init__.py:405-426, vq_linear_lut.cu:121-206).  ``lut`` is the caller's fp32
    ``[M, n_groups, NC]`` table ``(x.reshape(M * n_groups, VL) @ centroids.T).reshape(M, n_groups, NC)``;
    returns fp32 ``[M, out_features]``."""
    _cabi.require_cuda("vq_lut_gather", lut, packed_indices)
    if lut.dtype != torch.float32 or lut.dim() != 3:
        raise RuntimeError("vq_lut_gather: lut must be a 3-D float32 tensor [M, n_groups, NC].")
    lib = _cabi.load_library()
    m, g, nc = lut.shape
    out = torch.empty((m, out_features), dtype=torch.float32, device=lut.device)
    with torch.cuda.device(lut.device):
        rc = _launch("npb_vq_lut_gather", lib.npb_vq_lut_gather, lut.data_ptr(), m, g, nc, packed_indices.data_ptr(),
                     packed_indices.numel(), bits, out_features, out.data_ptr(), _cabi.stream_ptr())
    _cabi.check(rc, "vq_lut_gather")
    return out


def vq_dequant_gemm(x: torch.Tensor, packed_indices: torch.Tensor, centroids: torch.Tensor,
                    bits: int, out_features: int | None = None, bias: torch.Tensor | None = None,
                    **ext) -> torch.Tensor:
    """One-pass decode to a temporary ``[N, K]`` weight in ``x.dtype``, then the dense
    tensor-core GEMM (reference: ``_forward_dequant_gemm``, np_vq_linear.py:1127-1148)."""
    k = x.shape[1]
    n = out_features if out_features is not None else _infer_n(packed_indices, bits, k,
                                                                centroids.shape[-1])
    w = vq_dequant(packed_indices, centroids, bits, n, k, x.dtype, **ext)
    return gemm(x, w, bias)


def vq_linear(x: torch.Tensor, packed_indices: torch.Tensor, centroids: torch.Tensor, bits: int,
              vector_len: int, bias: torch.Tensor | None = None, **ext) -> torch.Tensor:
    """Fused VQ linear for any row count (reference: ``vq_linear``, vq_linear.cu:344-424).
    Up to ``GEMV_MAX_ROWS`` rows run the GEMV; more rows run the tile-decode GEMM (or, while
    that is switched off, decode + dense GEMM)."""
    if centroids.shape[-1] != vector_len:
        raise RuntimeError("vector_len does not match the codebook.")
    if x.shape[0] <= GEMV_MAX_ROWS:
        return vq_gemv(x, packed_indices, centroids, bits, None, bias, **ext)
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("vq_linear: more than 8 rows need fp16 or bf16 activations.")
    if VQ_TILE_DECODE_GEMM and vector_len == 8 and x.shape[1] % 64 == 0 and x.shape[0] <= VQ_FUSED_MAX_ROWS:
        return vq_gemm_fused(x, packed_indices, centroids, bits, None, bias, **ext)
    return vq_dequant_gemm(x, packed_indices, centroids, bits, None, bias, **ext)


def vq_linear_wmma(x: torch.Tensor, packed_indices: torch.Tensor, centroids: torch.Tensor,
                   bits: int, vector_len: int = 4, bias: torch.Tensor | None = None,
                   **ext) -> torch.Tensor:
    """Drop-in for the reference's ``vq_linear_wmma`` (kernels/__init__.py:335-352): GEMV up to
    8 rows, tensor-core GEMM above (vq_linear_wmma.cu:47,444).  Unlike the reference the
    vector length is honoured (the reference kernel is compiled for 4 only)."""
    return vq_linear(x, packed_indices, centroids, bits, centroids.shape[-1], bias, **ext)


# ---------------------------------------------------------------------------
# Dense tensor-core GEMM
# ---------------------------------------------------------------------------


def gemm(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, gather=None) -> torch.Tensor:
    """``x[M,K] @ w[N,K].T (+ bias)`` on the tcgen05 tensor cores, bf16 / fp16, fp32
    accumulate.  Stands in for ``F.linear`` after the decode (np_vq_linear.py:1148).  With
    ``gather`` (a ``sharding.PushGather``) the epilogue writes this rank's columns into every
    rank's buffer and the full ``[M, N]`` comes back (``npb_gemm_allgather``)."""
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise RuntimeError("gemm: expected x [M, K] and w [N, K].")
    if x.dtype != w.dtype:
        raise RuntimeError("gemm: x and w must have the same dtype.")
    _cabi.require_cuda("gemm", x, w)
    lib = _cabi.load_library()
    m, k = x.shape
    n = w.shape[0]
    b = _bias_f32(bias, n, x.device)
    if gather is not None:
        sink, out = gather.begin(m, n, x.dtype)
        with torch.cuda.device(x.device):
            rc = _launch("npb_gemm_allgather", lib.npb_gemm_allgather, x.data_ptr(), w.data_ptr(),
                         None if b is None else b.data_ptr(), m, n, k, _cabi.dtype_code(x.dtype),
                         ctypes.byref(sink), _cabi.stream_ptr())
        _cabi.check(rc, "gemm_allgather")
        return out
    y = torch.empty((m, n), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _launch("npb_gemm", lib.npb_gemm, x.data_ptr(), w.data_ptr(), None if b is None else b.data_ptr(),
                          y.data_ptr(), m, n, k, _cabi.dtype_code(x.dtype), _cabi.stream_ptr())
    _cabi.check(rc, "gemm")
    return y


# ---------------------------------------------------------------------------
# Group-affine (Q4_0 / HQQ)
# ---------------------------------------------------------------------------


def _q_prepare(name, w_pack, scale, zero_point, nbits, group_size):
    if w_pack.dim() != 2:
        raise RuntimeError(f"{name}: w_pack must be 2-D [N, K*nbits/8].")
    if nbits not in (4, 8):
        raise RuntimeError(f"{name}: nbits must be 4 or 8, got {nbits}.")
    n = w_pack.shape[0]
    k = w_pack.shape[1] * (8 // nbits)
    if group_size <= 0 or k % group_size:
        raise RuntimeError(f"{name}: group_size must divide K={k}.")
    n_groups = n * (k // group_size)
    if scale.numel() != n_groups or (zero_point is not None and zero_point.numel() != n_groups):
        raise RuntimeError(f"{name}: scale / zero_point must have N*K/group_size = {n_groups} elements.")
    return n, k


def q_dequant(w_pack: torch.Tensor, scale: torch.Tensor, nbits: int, group_size: int,
              zero_point: torch.Tensor | None, dtype: torch.dtype) -> torch.Tensor:
    """Dense ``[N, K]`` weight ``((q - zp) * s).to(dtype)`` (np_linear.py:334-351)."""
    _cabi.require_cuda("q_dequant", w_pack, scale, zero_point)
    n, k = _q_prepare("q_dequant", w_pack, scale, zero_point, nbits, group_size)
    lib = _cabi.load_library()
    w = _cabi.q_struct(w_pack, scale, zero_point, nbits, group_size)
    out = torch.empty((n, k), dtype=dtype, device=w_pack.device)
    with torch.cuda.device(w_pack.device):
        rc = _launch("npb_q_decode", lib.npb_q_decode, w, n, k, out.data_ptr(), _cabi.dtype_code(dtype),
                     _cabi.stream_ptr())
    _cabi.check(rc, "q_dequant")
    return out


def _q_call(fn_name, x, w_pack, scale, nbits, group_size, zero_point, bias):
    _cabi.require_cuda(fn_name, x, w_pack, scale, zero_point)
    n, k = _q_prepare(fn_name, w_pack, scale, zero_point, nbits, group_size)
    if x.shape[-1] != k:
        raise RuntimeError(f"{fn_name}: x has {x.shape[-1]} columns, the weight has K={k}.")
    lib = _cabi.load_library()
    *leading, _ = x.shape
    x2 = x.reshape(-1, k)
    m = x2.shape[0]
    w = _cabi.q_struct(w_pack, scale, zero_point, nbits, group_size)
    b = _bias_f32(bias, n, x.device)
    y = torch.empty((m, n), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _launch(fn_name, getattr(lib, fn_name), w, x2.data_ptr(), _cabi.dtype_code(x.dtype), m, n, k,
                                   None if b is None else b.data_ptr(), y.data_ptr(),
                                   _cabi.stream_ptr())
    _cabi.check(rc, fn_name)
    return y.reshape(*leading, n)


def q_gemv(x, w_pack, scale, nbits, group_size, zero_point=None, bias=None) -> torch.Tensor:
    """Fused unpack + dequant + dot for up to ``GEMV_MAX_ROWS`` rows."""
    return _q_call("npb_q_gemv", x, w_pack, scale, nbits, group_size, zero_point, bias)


def q_gemm_fused(x, w_pack, scale, nbits, group_size, zero_point=None, bias=None) -> torch.Tensor:
    """Tile-dequant tensor-core GEMM for 4-bit codes (bf16 / fp16 activations)."""
    return _q_call("npb_q_gemm_fused", x, w_pack, scale, nbits, group_size, zero_point, bias)


# Whether q_linear's mid band (9..Q_FUSED_MAX_ROWS rows) runs the tile-dequant GEMM
# (``npb_q_gemm_fused``) instead of decoding once and running the dense GEMM.  On: with the raw
# codes / scales staged by TMA (csrc/q_gemm_staged.cu) it is the faster of the two on a B200
# (14336 x 4096, Q4_0: 37 / 38 / 46 / 57 us at 16 / 128 / 256 / 384 rows against 49 / 50 / 56 / 75 us).
# NEUROPRESS_B200_Q_TILE_DEQUANT=0 switches it off.
Q_TILE_DEQUANT_GEMM = os.environ.get("NEUROPRESS_B200_Q_TILE_DEQUANT", "1") != "0"
Q_FUSED_MAX_ROWS = 384
Q_FUSED_MIN_WEIGHTS = 1 << 25   # smaller layers (4096 x 4096: 34 us against 31 us at 256 rows) decode + GEMM


def q_linear(x: torch.Tensor, w_pack: torch.Tensor, scale: torch.Tensor, nbits: int,
             group_size: int, zero_point: torch.Tensor | None = None,
             bias: torch.Tensor | None = None, gather=None) -> torch.Tensor:
    """Drop-in for the reference's ``q_linear`` (kernels/__init__.py:109-151): ``x`` is
    ``[..., K]``, output ``[..., N]`` in ``x.dtype``.  The reference runs one GEMV kernel for
    every row count (q4_linear.cu:137-140); here rows are banded: GEMV up to 8 rows, the
    tile-dequant GEMM up to 384 rows, then decode once + dense GEMM.  ``gather``
    (a ``sharding.PushGather``; not in the reference): the weight is an out-feature shard and the
    all-gathered ``[..., N_full]`` is returned -- by the GEMM's own epilogue where it can."""
    k = w_pack.shape[1] * (8 // nbits)
    m = x.numel() // max(k, 1)
    *leading, _ = x.shape

    def pushed(y: torch.Tensor) -> torch.Tensor:
        if gather is None:
            return y
        return gather(y.reshape(-1, y.shape[-1])).reshape(*leading, -1)

    if m <= GEMV_MAX_ROWS:
        return pushed(q_gemv(x, w_pack, scale, nbits, group_size, zero_point, bias))
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("q_linear: more than 8 rows need fp16 or bf16 activations.")
    if (Q_TILE_DEQUANT_GEMM and m <= Q_FUSED_MAX_ROWS and nbits == 4 and k % 64 == 0
            and group_size % 32 == 0 and w_pack.shape[0] * k >= Q_FUSED_MIN_WEIGHTS):
        return pushed(q_gemm_fused(x, w_pack, scale, nbits, group_size, zero_point, bias))
    w = q_dequant(w_pack, scale, nbits, group_size, zero_point, x.dtype)
    if gather is not None and gather.accepts(m, x.dtype):
        return gemm(x.reshape(-1, k), w, bias, gather=gather).reshape(*leading, -1)
    return pushed(gemm(x.reshape(-1, k), w, bias).reshape(*leading, w.shape[0]))


# ---------------------------------------------------------------------------
# RMSNorm
# ---------------------------------------------------------------------------


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Fused single-pass RMSNorm, drop-in for the reference's ``rms_norm``
    (kernels/__init__.py:1091-1110): ``out[m, i] = x[m, i] * rsqrt(mean(x[m, :]**2) + eps) *
    weight[i]`` computed in fp32.  ``x`` is ``[M, H]``, ``weight`` ``[H]`` of the same dtype
    (fp16, bf16 or fp32)."""
    if x.dim() != 2 or weight.dim() != 1 or weight.shape[0] != x.shape[1]:
        raise RuntimeError("rms_norm: expected x [M, H] and weight [H].")
    if x.dtype != weight.dtype:
        raise RuntimeError("rms_norm: x and weight must share dtype.")
    _cabi.require_cuda("rms_norm", x, weight)
    lib = _cabi.load_library()
    x = x.contiguous()
    weight = weight.contiguous()
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        rc = _launch("npb_rms_norm", lib.npb_rms_norm, x.data_ptr(), weight.data_ptr(), out.data_ptr(),
                     x.shape[0], x.shape[1], float(eps), _cabi.dtype_code(x.dtype), _cabi.stream_ptr())
    _cabi.check(rc, "rms_norm")
    return out


# ---------------------------------------------------------------------------
# Embedding lookups
# ---------------------------------------------------------------------------


def vq_embedding(input_ids: torch.Tensor, all_indices: torch.Tensor, centroids: torch.Tensor,
                 embedding_dim: int, scale: float = 1.0, inv_perm: torch.Tensor | None = None,
                 out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """Rows ``input_ids`` of a VQ-compressed embedding table, ``[..., embedding_dim]``.
    ``all_indices`` is the ``[vocab, n_groups]`` 16-bit index table, ``centroids`` the fp16
    ``[NC, VL]`` codebook; arithmetic as ``NPVQEmbedding.forward`` of the reference
    (np_vq_embedding.py:119-141).  Output dtype ``out_dtype`` (fp16 when ``None``)."""
    _cabi.require_cuda("vq_embedding", input_ids, all_indices, centroids, inv_perm)
    if all_indices.dtype not in (torch.int16, torch.uint16) or all_indices.dim() != 2:
        raise RuntimeError("vq_embedding: all_indices must be a [vocab, n_groups] 16-bit tensor.")
    if centroids.dtype != torch.float16 or centroids.dim() != 2:
        raise RuntimeError("vq_embedding: centroids must be a [NC, VL] float16 tensor.")
    v, g = all_indices.shape
    vl = centroids.shape[1]
    if g * vl != embedding_dim:
        raise RuntimeError("vq_embedding: n_groups * vector_len must equal embedding_dim.")
    if inv_perm is not None and (inv_perm.dtype != torch.int64 or inv_perm.numel() != embedding_dim):
        raise RuntimeError("vq_embedding: inv_perm must be int64 with embedding_dim elements.")
    lib = _cabi.load_library()
    ids = input_ids.reshape(-1).to(torch.int64).contiguous()
    dt = out_dtype if out_dtype is not None else torch.float16
    out = torch.empty((ids.numel(), embedding_dim), dtype=dt, device=ids.device)
    with torch.cuda.device(ids.device):
        rc = _launch("npb_vq_embedding", lib.npb_vq_embedding, ids.data_ptr(), ids.numel(),
                     all_indices.data_ptr(), v, g, centroids.data_ptr(), centroids.shape[0], vl,
                     None if inv_perm is None else inv_perm.data_ptr(), float(scale), out.data_ptr(),
                     _cabi.dtype_code(dt), _cabi.stream_ptr())
    _cabi.check(rc, "vq_embedding")
    return out.reshape(*input_ids.shape, embedding_dim)


def q_embedding(input_ids: torch.Tensor, u8_blob: torch.Tensor, scale: torch.Tensor, nbits: int,
                group_size: int, zero_point: torch.Tensor | None = None, padding_idx: int | None = None,
                embed_scale: float = 1.0, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """Rows ``input_ids`` of a group-affine embedding table, gathered in packed space and
    dequantised: ``_emb_dequant`` + the tail of ``NPEmbedding.forward`` of the reference
    (np_embedding.py:120-183, 449-473).  Output dtype ``out_dtype`` (fp16 when ``None``)."""
    _cabi.require_cuda("q_embedding", input_ids, u8_blob, scale, zero_point)
    v, d = _q_prepare("q_embedding", u8_blob, scale, zero_point, nbits, group_size)
    lib = _cabi.load_library()
    w = _cabi.q_struct(u8_blob, scale, zero_point, nbits, group_size)
    ids = input_ids.reshape(-1).to(torch.int64).contiguous()
    dt = out_dtype if out_dtype is not None else torch.float16
    out = torch.empty((ids.numel(), d), dtype=dt, device=ids.device)
    with torch.cuda.device(ids.device):
        rc = _launch("npb_q_embedding", lib.npb_q_embedding, ids.data_ptr(), ids.numel(), w, v, d,
                     -1 if padding_idx is None else int(padding_idx), float(embed_scale), out.data_ptr(),
                     _cabi.dtype_code(dt), _cabi.stream_ptr())
    _cabi.check(rc, "q_embedding")
    return out.reshape(*input_ids.shape, d)
