// One-pass decode of a vector-quantized weight: packed indices -> dense [N, K].
//
//   W16[n, VL*g + j] = hmul(hadd(C[cb(g)][idx[n,g]][j], R[ridx[n,g]][j]), s[n])   (fp16, RN)
//   W = convert(W16)                      (fp16 -> fp32 -> T, one rounding)
//
// Without residual and row scale this is the arithmetic of the reference decode
// (neuropress/kernels/vq_dequant.cu:50-83): pure indexing plus one conversion, so the
// result is bit-exact.  One thread decodes one vector per step; lanes take consecutive
// vectors so that index loads (2 B/lane) and stores (VL*sizeof(T) per lane) are contiguous
// across the warp.  HBM traffic = packed bytes + N*K*sizeof(T).  With a codebook that stays in
// L1 the kernel is write-bound; with a 1 MiB codebook every gather misses L1 and pulls a
// 32-byte sector from L2, and the sum of gather sectors, index reads and output writes runs
// at the L2's throughput (measured: ~8 TB/s), which then bounds it.
#include "common.cuh"

namespace npb {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

struct VqDev {
  const uint8_t* packed;
  int64_t packed_bytes;
  const __half* centroids;
  const uint8_t* res_packed;
  int64_t res_bytes;
  const __half* res_centroids;
  const __half* row_scale;
  int bits, res_bits, num_centroids, groups_per_codebook;  // groups_per_codebook 0: single
  // Whether the optional parts exist.  Their pointers are never null (an absent part aliases
  // the main stream / codebook), so a load hoisted above the test still reads mapped memory.
  int has_res, has_scale;
};

template <int VL>
struct HVec;
template <>
struct HVec<8> { using type = Half8; };
template <>
struct HVec<4> { using type = Half4; };

template <typename T, int VL>
__device__ __forceinline__ void store_vec(T* dst, const __half2 (&h)[VL / 2]) {
  if constexpr (sizeof(T) == 2) {
    struct alignas(VL * 2) Out { T v[VL]; } o;
#pragma unroll
    for (int i = 0; i < VL / 2; ++i) {
      o.v[2 * i] = from_half<T>(__low2half(h[i]));
      o.v[2 * i + 1] = from_half<T>(__high2half(h[i]));
    }
    *reinterpret_cast<Out*>(dst) = o;
  } else {
#pragma unroll
    for (int i = 0; i < VL / 4; ++i) {
      float4 o;
      o.x = __low2float(h[2 * i]);
      o.y = __high2float(h[2 * i]);
      o.z = __low2float(h[2 * i + 1]);
      o.w = __high2float(h[2 * i + 1]);
      reinterpret_cast<float4*>(dst)[i] = o;
    }
  }
}

template <typename T, int VL, int BITS, int RBITS>
__global__ void __launch_bounds__(kThreads)
vq_decode_kernel(VqDev a, T* __restrict__ out, uint32_t n_vectors, uint32_t G) {
  using HV = typename HVec<VL>::type;
  const uint32_t base = blockIdx.x * (kThreads * kUnroll) + threadIdx.x;
  uint32_t idx[kUnroll], ridx[kUnroll];
  const bool has_res = a.has_res != 0;
  const bool has_scale = a.has_scale != 0;
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const uint32_t v = base + u * kThreads;
    idx[u] = 0; ridx[u] = 0;
    if (v < n_vectors) {
      idx[u] = read_index<BITS>(a.packed, a.packed_bytes, v, a.bits);
      if (has_res) ridx[u] = read_index<RBITS>(a.res_packed, a.res_bytes, v, a.res_bits);
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const uint32_t v = base + u * kThreads;
    if (v >= n_vectors) continue;
    uint32_t row_off = idx[u];
    uint32_t n = 0;
    if (a.groups_per_codebook > 0 || has_scale) {
      n = v / G;
      const uint32_t g = v - n * G;
      if (a.groups_per_codebook > 0)
        row_off += (g / (uint32_t)a.groups_per_codebook) * (uint32_t)a.num_centroids;
    }
    HV c = ldg_vec(reinterpret_cast<const HV*>(a.centroids) + row_off);
    __half2 h[VL / 2];
#pragma unroll
    for (int i = 0; i < VL / 2; ++i) h[i] = c.h[i];
    if (has_res) {
      const HV r = ldg_vec(reinterpret_cast<const HV*>(a.res_centroids) + ridx[u]);
#pragma unroll
      for (int i = 0; i < VL / 2; ++i) h[i] = __hadd2_rn(h[i], r.h[i]);
    }
    if (has_scale) {
      const __half2 s = __half2half2(__ldg(a.row_scale + (has_scale ? n : 0u)));
#pragma unroll
      for (int i = 0; i < VL / 2; ++i) h[i] = __hmul2_rn(h[i], s);
    }
    store_vec<T, VL>(out + (size_t)v * VL, h);
  }
}

template <typename T, int VL>
int launch_decode(const VqDev& a, T* out, uint32_t n_vectors, uint32_t G, cudaStream_t st) {
  const uint32_t per_block = kThreads * kUnroll;
  const uint32_t blocks = (n_vectors + per_block - 1) / per_block;
  const bool a16 = a.bits == 16 && aligned_to(a.packed, 2);
  const bool a8 = a.bits == 8;
  const bool r8 = !a.has_res || a.res_bits == 8;
  if (a16 && r8)
    vq_decode_kernel<T, VL, 16, 8><<<blocks, kThreads, 0, st>>>(a, out, n_vectors, G);
  else if (a8 && r8)
    vq_decode_kernel<T, VL, 8, 8><<<blocks, kThreads, 0, st>>>(a, out, n_vectors, G);
  else
    vq_decode_kernel<T, VL, 0, 0><<<blocks, kThreads, 0, st>>>(a, out, n_vectors, G);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

template <typename T>
int dispatch_vl(const VqDev& a, int vl, T* out, uint32_t n_vectors, uint32_t G, cudaStream_t st) {
  if (vl == 8) return launch_decode<T, 8>(a, out, n_vectors, G, st);
  if (vl == 4) return launch_decode<T, 4>(a, out, n_vectors, G, st);
  return NPB_ERR_UNSUPPORTED;
}

}  // namespace

int vq_decode(const npb_vq_weight* w, int64_t N, int64_t K, void* out, int out_dtype,
              cudaStream_t st) {
  if (int rc = validate_vq(w, N, K)) return rc;
  if (out == nullptr && N * K > 0) return NPB_ERR_INVALID_ARG;
  if (N * K == 0) return NPB_OK;
  if (!aligned_to(out, 16)) return NPB_ERR_ALIGNMENT;
  const int64_t G = K / w->vector_len;
  const int64_t n_vectors = N * G;
  if (n_vectors >= (int64_t)1 << 31) return NPB_ERR_UNSUPPORTED;
  VqDev a;
  a.packed = w->packed;
  a.packed_bytes = w->packed_bytes;
  a.centroids = static_cast<const __half*>(w->centroids);
  a.has_res = w->res_packed != nullptr;
  a.has_scale = w->row_scale != nullptr;
  a.res_packed = a.has_res ? w->res_packed : w->packed;
  a.res_bytes = a.has_res ? w->res_packed_bytes : 0;
  a.res_centroids = a.has_res ? static_cast<const __half*>(w->res_centroids) : a.centroids;
  a.row_scale = a.has_scale ? static_cast<const __half*>(w->row_scale) : a.centroids;
  a.bits = w->bits;
  a.res_bits = a.has_res ? w->res_bits : 0;
  a.num_centroids = w->num_centroids;
  a.groups_per_codebook = w->cols_per_codebook > 0 ? w->cols_per_codebook / w->vector_len : 0;
  switch (out_dtype) {
    case NPB_BF16:
      return dispatch_vl<__nv_bfloat16>(a, w->vector_len, static_cast<__nv_bfloat16*>(out),
                                        (uint32_t)n_vectors, (uint32_t)G, st);
    case NPB_F16:
      return dispatch_vl<__half>(a, w->vector_len, static_cast<__half*>(out),
                                 (uint32_t)n_vectors, (uint32_t)G, st);
    case NPB_F32:
      return dispatch_vl<float>(a, w->vector_len, static_cast<float*>(out), (uint32_t)n_vectors,
                                (uint32_t)G, st);
    default:
      return NPB_ERR_UNSUPPORTED;
  }
}

}  // namespace npb
