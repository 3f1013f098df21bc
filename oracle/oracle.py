"""CPU oracle for the quantized-linear forward path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU with numpy (integer / byte work) and torch CPU tensors
(fp16 / bf16 arithmetic), what the reference computes for the lowered quantized linears.  It
is the checker for the CUDA kernels: only the tests, the smoke check and the CPU-baseline leg
of the benchmark may import it.  The library itself never does — it has no CPU path.

Pinned against the reference: ``tests/golden/make_golden.py`` imports the reference's own
modules and stores their outputs for small seeded cases; ``tests/test_oracle_golden.py`` checks
every function here against those files, and against the one literal known-answer byte of the
reference's tests.  The residual-codebook, row-scale and per-column-group codebook forms do
not exist in the reference: for those the parity is unpinned, and the arithmetic below is
composed of reference primitives only (unpack, ``centroids[indices]``, ``.to(dtype)``,
``F.linear``) with fp16 add / multiply rounding once per operation.

Reference locations restated here (paths inside the reference project):
  * index bit-stream            neuropress/transforms/vq_packing.py:135-295
  * VQ decode + linear          neuropress/nn/np_vq_linear.py:178-211, 1060-1095
                                neuropress/kernels/vq_dequant.cu:27-83
  * nibble unpack               neuropress/nn/np_linear.py:78-96
  * group-affine decode+linear  neuropress/nn/np_linear.py:298-353
                                neuropress/kernels/q4_linear.cu:80-131
  * embedding lookups           neuropress/nn/np_vq_embedding.py:119-141
                                neuropress/nn/np_embedding.py:120-183, 449-503
  * entropy-coded index streams neuropress/transforms/vq_packing.py:298-1384
"""

from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

# --------------------------------------------------------------------------------------
# Index bit-stream
# --------------------------------------------------------------------------------------


def pack_indices(indices: np.ndarray, bits: int) -> np.ndarray:
    """LSB-first bit-stream pack: index i occupies bits [i*bits, (i+1)*bits).

    Follows ``IndexPacking.pack`` / ``_pack_bitstream`` (vq_packing.py:135-252): one pass per
    bit, each bit OR-ed into its byte.
    """
    if not 4 <= bits <= 20:
        raise ValueError(f"bits must be in [4, 20], got {bits}.")
    flat = np.asarray(indices, dtype=np.int64).reshape(-1)
    n = flat.size
    if bits == 4 and n % 2:
        raise ValueError("4-bit packing needs an even index count.")
    n_bytes = (n * bits + 7) // 8
    out = np.zeros(n_bytes, dtype=np.uint8)
    i = np.arange(n, dtype=np.int64)
    for b in range(bits):
        pos = i * bits + b
        bit = ((flat >> b) & 1).astype(np.uint8)
        np.bitwise_or.at(out, pos >> 3, bit << (pos & 7).astype(np.uint8))
    return out


def unpack_indices_bitloop(packed: np.ndarray, bits: int, n_indices: int) -> np.ndarray:
    """Faithful restatement of the reference's CPU unpack (vq_packing.py:178-208, 284-295):
    8-bit is a cast, 4-bit splits nibbles, every other width gathers one bit per pass."""
    if not 4 <= bits <= 20:
        raise ValueError(f"bits must be in [4, 20], got {bits}.")
    p = np.asarray(packed, dtype=np.uint8).reshape(-1)
    if bits == 8:
        return p[:n_indices].astype(np.int64)
    if bits == 4:
        lo = (p & 0xF).astype(np.int64)
        hi = (p >> 4).astype(np.int64)
        return np.stack([lo, hi], axis=1).reshape(-1)[:n_indices]
    p64 = p.astype(np.int64)
    i = np.arange(n_indices, dtype=np.int64)
    out = np.zeros(n_indices, dtype=np.int64)
    for b in range(bits):
        pos = i * bits + b
        out |= ((p64[pos >> 3] >> (pos & 7)) & 1) << b
    return out


def unpack_indices(packed: np.ndarray, bits: int, n_indices: int) -> np.ndarray:
    """Same result as :func:`unpack_indices_bitloop`, one pass: read the (at most three)
    bytes that hold an index, shift, mask — the window read of vq_dequant.cu:27-36."""
    if not 4 <= bits <= 20:
        raise ValueError(f"bits must be in [4, 20], got {bits}.")
    p = np.asarray(packed, dtype=np.uint8).reshape(-1)
    if bits == 8:
        return p[:n_indices].astype(np.int64)
    if bits == 16 and p.size >= 2 * n_indices:
        return p[: 2 * n_indices].view("<u2").astype(np.int64)
    p64 = np.concatenate([p.astype(np.int64), np.zeros(4, dtype=np.int64)])
    pos = np.arange(n_indices, dtype=np.int64) * bits
    b0 = pos >> 3
    win = p64[b0] | (p64[b0 + 1] << 8) | (p64[b0 + 2] << 16) | (p64[b0 + 3] << 24)
    return (win >> (pos & 7)) & ((1 << bits) - 1)


# --------------------------------------------------------------------------------------
# VQ decode and forward
# --------------------------------------------------------------------------------------


# --------------------------------------------------------------------------------------
# Entropy-coded index streams (two-tier, N-tier, zero escape)
# --------------------------------------------------------------------------------------


def _stream_bits(buf: np.ndarray) -> np.ndarray:
    return np.unpackbits(np.ascontiguousarray(buf, dtype=np.uint8), bitorder="little")


def _payloads(bits: np.ndarray, first_bit: int, width: int, count: int) -> np.ndarray:
    """``count`` consecutive ``width``-bit values (LSB first) starting at stream bit ``first_bit``."""
    if count == 0 or width == 0:
        return np.zeros(count, dtype=np.int64)
    chunk = bits[first_bit:first_bit + count * width].reshape(count, width).astype(np.int64)
    return (chunk << np.arange(width, dtype=np.int64)).sum(axis=1)


def _u32(buf: np.ndarray, word: int) -> int:
    return int(np.frombuffer(np.ascontiguousarray(buf[4 * word:4 * word + 4]).tobytes(), dtype="<u4")[0])


def entropy_unpack(packed, scheme: str) -> np.ndarray:
    """Indices of an entropy-coded buffer, decoded sequentially the way the formats are defined:
    the prefix stream gives every index its tier, and tier t's payloads are consumed in index
    order from tier t's stream.  ``scheme``: ``"tiered"`` (reference :298-520: header n, n_hot,
    cold_bits[, hot_bits]; prefix bit 0 = hot), ``"ntier"`` (:612-908: magic 0x4E565154, cascaded
    prefixes, tier k stores index - 2**bits[k-1]) or ``"zero_escape"`` (:1037-1276: magic
    0x5A455343, two-bit prefix, payload widths 0/4/8/cold_bits, offsets 0/1/17/257).
    Four-bit streams are padded to whole bytes (an even count), every stream starts on a byte."""
    buf = _as_np_u8(packed)
    bits = _stream_bits(buf)

    def nbytes(count: int, width: int) -> int:
        return (count * width + 7) // 8

    if scheme == "tiered":
        n, n_hot, cold_bits = _u32(buf, 0), _u32(buf, 1), _u32(buf, 2)
        hot_bits, off = 4, 12
        if buf.size >= 16 and 4 <= _u32(buf, 3) <= 16:
            hot_bits, off = _u32(buf, 3), 16
        tier = bits[8 * off:8 * off + n].astype(np.int64)
        off += nbytes(n, 1)
        widths, lows, counts = [hot_bits, cold_bits], [0, 0], [n_hot, n - n_hot]
    elif scheme == "ntier":
        assert _u32(buf, 0) == 0x4E565154, "not an n-tier buffer"
        n, d = _u32(buf, 1), _u32(buf, 2)
        counts = [_u32(buf, 3 + 2 * k) for k in range(d)]
        widths = [_u32(buf, 4 + 2 * k) for k in range(d)]
        lows = [0] + [1 << w for w in widths[:-1]]
        off = 12 + 8 * d
        tier = np.full(n, d - 1, dtype=np.int64)
        alive = np.arange(n)
        for k in range(d - 1):
            later = bits[8 * off:8 * off + alive.size].astype(bool)
            tier[alive[~later]] = k
            off += nbytes(alive.size, 1)
            alive = alive[later]
    elif scheme == "zero_escape":
        assert _u32(buf, 0) == 0x5A455343, "not a zero-escape buffer"
        n, cold_bits = _u32(buf, 1), _u32(buf, 2)
        counts = [_u32(buf, 3), _u32(buf, 4), _u32(buf, 5)]
        counts.append(n - sum(counts))
        widths, lows = [0, 4, 8, cold_bits], [0, 1, 17, 257]
        off = 24
        pre = bits[8 * off:8 * off + 2 * n].reshape(n, 2).astype(np.int64)
        tier = pre[:, 0] + 2 * pre[:, 1]
        off += nbytes(n, 2)
    else:
        raise ValueError(scheme)
    out = np.zeros(n, dtype=np.int64)
    for k, (width, low, count) in enumerate(zip(widths, lows, counts)):
        where = np.flatnonzero(tier == k)
        assert where.size == count, "tier counts in the header do not match the prefix stream"
        out[where] = _payloads(bits, 8 * off, width, count) + low
        off += nbytes(count, width)
    return out


def entropy_row_offsets(packed, scheme: str, n_rows: int, n_groups: int) -> list[np.ndarray]:
    """Per tier, the number of its indices in the rows before row i (int32 ``[n_rows + 1]``): the
    ``compute_row_offsets`` of the three packers (:522-572, :910-973, :1278-1326), restated from
    the decoded indices."""
    idx = entropy_unpack(packed, scheme).reshape(n_rows, n_groups)
    buf = _as_np_u8(packed)
    if scheme == "tiered":
        hot_bits = _u32(buf, 3) if buf.size >= 16 and 4 <= _u32(buf, 3) <= 16 else 4
        bounds = [1 << hot_bits]
    elif scheme == "ntier":
        d = _u32(buf, 2)
        bounds = [1 << _u32(buf, 4 + 2 * k) for k in range(d - 1)]
    else:
        bounds = [1, 17, 257]
    tier = np.searchsorted(np.asarray(bounds), idx, side="right")
    out = []
    for k in range(len(bounds) + 1):
        off = np.zeros(n_rows + 1, dtype=np.int64)
        off[1:] = np.cumsum((tier == k).sum(axis=1))
        out.append(off.astype(np.int32))
    return out


def _as_np_u8(t) -> np.ndarray:
    if isinstance(t, torch.Tensor):
        return t.detach().cpu().contiguous().numpy()
    return np.asarray(t, dtype=np.uint8)


def vq_decode(
    packed,
    centroids: torch.Tensor,
    bits: int,
    out_features: int,
    in_features: int,
    dtype: torch.dtype,
    *,
    residual_indices=None,
    residual_centroids: torch.Tensor | None = None,
    residual_bits: int = 8,
    row_scale: torch.Tensor | None = None,
    cols_per_codebook: int = 0,
    unpack=unpack_indices,
) -> torch.Tensor:
    """Dense weight ``[out_features, in_features]`` in *dtype*.

    Base form (np_vq_linear.py:1091-1095, vq_dequant.cu:50-83):
        ``W = centroids[unpack(packed)].reshape(N, K).to(dtype)``  with fp16 centroids.
    Extensions (not in the reference): per-column-group codebooks
    (``centroids`` is ``[n_cb, NC, VL]``, group ``g`` uses codebook ``g*VL // cols_per_codebook``),
    a residual codebook added in fp16, a per-output-row fp16 scale multiplied in fp16.
    """
    c = centroids.detach().cpu().to(torch.float16)
    vl = c.shape[-1]
    N, K = out_features, in_features
    if K % vl:
        raise ValueError("in_features must be a multiple of the vector length.")
    G = K // vl
    idx = torch.from_numpy(unpack(_as_np_u8(packed), bits, N * G)).reshape(N, G)
    if cols_per_codebook:
        if c.dim() != 3:
            raise ValueError("column-group codebooks need [n_cb, NC, VL] centroids.")
        cb = (torch.arange(G) * vl) // cols_per_codebook
        w16 = c[cb.unsqueeze(0).expand(N, G), idx]
    else:
        w16 = c[idx]
    if residual_indices is not None:
        r = residual_centroids.detach().cpu().to(torch.float16)
        ridx = torch.from_numpy(unpack(_as_np_u8(residual_indices), residual_bits, N * G)).reshape(N, G)
        w16 = w16 + r[ridx]  # fp16 add, one rounding
    w16 = w16.reshape(N, K)
    if row_scale is not None:
        w16 = w16 * row_scale.detach().cpu().to(torch.float16).reshape(N, 1)  # fp16 multiply
    return w16.to(dtype)


def vq_forward(x: torch.Tensor, packed, centroids, bits, out_features, in_features,
               bias: torch.Tensor | None = None, **ext) -> torch.Tensor:
    """``F.linear(x, decode(...).to(x.dtype), bias)`` — the reference's default / dense path
    (np_vq_linear.py:1091-1095, 1127-1148)."""
    x = x.detach().cpu()
    w = vq_decode(packed, centroids, bits, out_features, in_features, x.dtype, **ext)
    b = None if bias is None else bias.detach().cpu().to(x.dtype)
    return F.linear(x, w, b)


def vq_forward_f32(x: torch.Tensor, packed, centroids, bits, out_features, in_features,
                   bias: torch.Tensor | None = None, **ext) -> torch.Tensor:
    """High-precision yardstick: the weight exactly as decoded for ``x.dtype``, product and
    accumulation in fp64.  Used to measure how far a low-precision result is from the truth
    when checking the ``max|err| <= 1e-2 * RMS`` bound."""
    x = x.detach().cpu()
    w = vq_decode(packed, centroids, bits, out_features, in_features, x.dtype, **ext)
    y = x.double() @ w.double().T
    if bias is not None:
        y = y + bias.detach().cpu().double()
    return y


# --------------------------------------------------------------------------------------
# Group-affine (Q4_0 / HQQ) decode and forward
# --------------------------------------------------------------------------------------


def unpack_codes(codes, nbits: int) -> np.ndarray:
    """``[N, K*nbits/8]`` uint8 -> ``[N, K]`` uint8; value j of a byte sits at bits
    [j*nbits, (j+1)*nbits) (np_linear.py:78-96)."""
    c = _as_np_u8(codes)
    vpb = 8 // nbits
    shifts = (np.arange(vpb) * nbits).astype(np.uint8)
    vals = (c[:, :, None] >> shifts[None, None, :]) & ((1 << nbits) - 1)
    return vals.reshape(c.shape[0], c.shape[1] * vpb).astype(np.uint8)


def pack_codes(values, nbits: int) -> np.ndarray:
    """Inverse of :func:`unpack_codes` (np_linear.py:99-117)."""
    v = _as_np_u8(values)
    vpb = 8 // nbits
    g = v.reshape(v.shape[0], v.shape[1] // vpb, vpb).astype(np.uint8)
    out = np.zeros(g.shape[:2], dtype=np.uint8)
    for i in range(vpb):
        out |= g[:, :, i] << np.uint8(i * nbits)
    return out


def q_decode(codes, scale: torch.Tensor, zero_point: torch.Tensor | None, nbits: int,
             group_size: int, dtype: torch.dtype) -> torch.Tensor:
    """``W = ((q.f32 - zp.f32) * s.f32).to(dtype)``; symmetric zero-point ``2**(nbits-1)``
    (np_linear.py:334-351)."""
    vals = torch.from_numpy(unpack_codes(codes, nbits).astype(np.float32))
    N, K = vals.shape
    ng = K // group_size
    v = vals.reshape(N, ng, group_size)
    s = scale.detach().cpu().to(torch.float32).reshape(N, ng, 1)
    if zero_point is not None:
        z = zero_point.detach().cpu().to(torch.float32).reshape(N, ng, 1)
        w = (v - z) * s
    else:
        w = (v - float(1 << (nbits - 1))) * s
    return w.reshape(N, K).to(dtype)


def q_forward(x: torch.Tensor, codes, scale, nbits, group_size, zero_point=None,
              bias=None) -> torch.Tensor:
    """``F.linear(x, q_decode(...), bias)`` (np_linear.py:353)."""
    x = x.detach().cpu()
    w = q_decode(codes, scale, zero_point, nbits, group_size, x.dtype)
    b = None if bias is None else bias.detach().cpu().to(x.dtype)
    return F.linear(x, w, b)


def q_forward_f64(x: torch.Tensor, codes, scale, nbits, group_size, zero_point=None,
                  bias=None) -> torch.Tensor:
    x = x.detach().cpu()
    w = q_decode(codes, scale, zero_point, nbits, group_size, x.dtype)
    y = x.double() @ w.double().T
    if bias is not None:
        y = y + bias.detach().cpu().double()
    return y


# --------------------------------------------------------------------------------------
# Shared error metric
# --------------------------------------------------------------------------------------


def rel_max_err(y: torch.Tensor, y_ref: torch.Tensor) -> float:
    """``max|y - y_ref| / RMS(y_ref)``: the quantity the output tolerance (1e-2 for bf16) is
    stated on."""
    y = y.detach().cpu().double()
    r = y_ref.detach().cpu().double()
    rms = float(torch.sqrt(torch.mean(r * r)))
    return float((y - r).abs().max()) / max(rms, 1e-30)


# ---------------------------------------------------------------------------
# Embedding lookups
# ---------------------------------------------------------------------------


def vq_embedding(input_ids: torch.Tensor, all_indices: torch.Tensor, centroids: torch.Tensor,
                 embedding_dim: int, scale: float = 1.0, inv_perm: torch.Tensor | None = None,
                 out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``NPVQEmbedding.forward`` (neuropress/nn/np_vq_embedding.py:119-141): gather the 16-bit
    index rows, gather fp16 centroids, reshape, optional column permutation, optional multiply by
    a python scalar (fp16 result), optional cast."""
    flat = input_ids.detach().cpu().flatten()
    idx = all_indices.detach().cpu().to(torch.int16)[flat].long()
    out = centroids.detach().cpu().to(torch.float16)[idx].reshape(flat.shape[0], embedding_dim)
    if inv_perm is not None:
        out = out[:, inv_perm.detach().cpu()]
    if scale != 1.0:
        out = out * scale
    if out_dtype is not None:
        out = out.to(out_dtype)
    return out.reshape(*input_ids.shape, embedding_dim)


def q_embedding(input_ids: torch.Tensor, u8_blob, scale: torch.Tensor, nbits: int, group_size: int,
                zero_point: torch.Tensor | None = None, padding_idx: int | None = None,
                embed_scale: float = 1.0, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``_emb_dequant`` followed by the tail of ``NPEmbedding.forward``
    (neuropress/nn/np_embedding.py:120-183, 449-473, 497-503): gather packed rows, unpack,
    ``((q - zp) * s)`` in fp32, cast to the fp16 scale dtype, zero the padding rows, cast to
    ``out_dtype``, multiply by ``embed_scale``."""
    blob = torch.from_numpy(_as_np_u8(u8_blob))
    ids = input_ids.detach().cpu()
    flat = ids.reshape(-1)
    n_emb = blob.shape[0]
    dim = blob.shape[1] * (8 // nbits)
    ng = dim // group_size
    vals = torch.from_numpy(unpack_codes(blob[flat].numpy(), nbits).astype(np.float32)).reshape(-1, ng, group_size)
    sc16 = scale.detach().cpu().to(torch.float16)
    sc = sc16.reshape(n_emb, ng)[flat].to(torch.float32).unsqueeze(-1)
    if zero_point is not None:
        zp = zero_point.detach().cpu().reshape(n_emb, ng)[flat].to(torch.float32).unsqueeze(-1)
        out = (vals - zp) * sc
    else:
        out = (vals - float(1 << (nbits - 1))) * sc
    out = out.reshape(-1, dim).to(sc16.dtype).reshape(*ids.shape, dim)
    if padding_idx is not None:
        out = out.clone()
        out[ids == padding_idx] = 0.0
    if out_dtype is not None:
        out = out.to(out_dtype)
    if embed_scale != 1.0:
        out = out * embed_scale
    return out


# ---------------------------------------------------------------------------
# RMSNorm (the step on the input side of the lowered linears)
# ---------------------------------------------------------------------------


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(mean(x**2, -1) + eps) * weight`` with fp32 arithmetic and one rounding to the
    input dtype, as the reference kernel defines it (neuropress/kernels/rms_norm.cu:40-76:
    fp32 sum of squares, ``rsqrtf(ss / H + eps)``, ``(float)x * scale * (float)weight``) and as
    its module documents it (neuropress/nn/np_rms_norm.py:45-47).  The reference has no CPU
    implementation of this kernel; the torch expression of its docstring is the yardstick."""
    xf = x.to(torch.float32)
    scale = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * scale * weight.to(torch.float32)).to(x.dtype)


def rms_norm_f64(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """The same in float64, unrounded (tolerance checks)."""
    xd = x.to(torch.float64)
    scale = torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + eps)
    return xd * scale * weight.to(torch.float64)
