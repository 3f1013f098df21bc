// Fused RMSNorm over the last dimension:  out[m, i] = T( x[m, i] * rsqrt(mean_i(x[m, :]^2) + eps) * w[i] )
// with all arithmetic in fp32 (the definition of the reference kernel,
// neuropress/kernels/rms_norm.cu:27-76).  The step on the input side of every q/k/v and
// gate/up linear of a lowered decoder layer.
//
// One CTA per row, 128-bit loads.  A row of up to kThreads * kCache * (16 / sizeof(T)) elements
// (8192 for 16-bit types) is read from HBM once and kept in registers between the
// sum-of-squares pass and the scaling pass; longer rows are re-read (from L2).  HBM bytes:
// 2 * M * H * sizeof(T) + H * sizeof(T); the kernel is bandwidth-bound for large M and
// latency-bound for a handful of rows.
#include "common.cuh"

namespace npb {
namespace {

constexpr int kThreads = 256;
constexpr int kCache = 4;  // 16-byte pieces of the row a thread keeps in registers

template <typename T>
__global__ void __launch_bounds__(kThreads)
rms_norm_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out, int H, float eps,
                bool vec) {
  constexpr int EPV = 16 / (int)sizeof(T);  // elements per 16-byte piece
  const T* xm = x + (size_t)blockIdx.x * H;
  T* om = out + (size_t)blockIdx.x * H;
  const int tid = threadIdx.x;
  struct alignas(16) Piece { T v[EPV]; };
  Piece cache[kCache];
  float ss = 0.f;
  const int n_pieces = vec ? H / EPV : 0;  // vec: H % EPV == 0 and 16-byte aligned rows
#pragma unroll
  for (int c = 0; c < kCache; ++c) {
    const int p = tid + c * kThreads;
    if (p < n_pieces) {
      cache[c] = *reinterpret_cast<const Piece*>(xm + (size_t)p * EPV);
#pragma unroll
      for (int e = 0; e < EPV; ++e) { const float f = to_f32(cache[c].v[e]); ss = fmaf(f, f, ss); }
    }
  }
  for (int p = tid + kCache * kThreads; p < n_pieces; p += kThreads) {
    const Piece q = *reinterpret_cast<const Piece*>(xm + (size_t)p * EPV);
#pragma unroll
    for (int e = 0; e < EPV; ++e) { const float f = to_f32(q.v[e]); ss = fmaf(f, f, ss); }
  }
  for (int i = n_pieces * EPV + tid; i < H; i += kThreads) {  // scalar path / ragged tail
    const float f = to_f32(xm[i]);
    ss = fmaf(f, f, ss);
  }
  __shared__ float warp_ss[kThreads / 32];
  __shared__ float scale_sh;
  ss = warp_sum(ss);
  if ((tid & 31) == 0) warp_ss[tid >> 5] = ss;
  __syncthreads();
  if (tid < 32) {
    float t = tid < kThreads / 32 ? warp_ss[tid] : 0.f;
    t = warp_sum(t);
    if (tid == 0) scale_sh = rsqrtf(t / (float)H + eps);
  }
  __syncthreads();
  const float scale = scale_sh;
#pragma unroll
  for (int c = 0; c < kCache; ++c) {
    const int p = tid + c * kThreads;
    if (p < n_pieces) {
      const Piece wv = *reinterpret_cast<const Piece*>(w + (size_t)p * EPV);
      Piece o;
#pragma unroll
      for (int e = 0; e < EPV; ++e)
        o.v[e] = from_f32<T>(__fmul_rn(__fmul_rn(to_f32(cache[c].v[e]), scale), to_f32(wv.v[e])));
      *reinterpret_cast<Piece*>(om + (size_t)p * EPV) = o;
    }
  }
  for (int p = tid + kCache * kThreads; p < n_pieces; p += kThreads) {
    const Piece q = *reinterpret_cast<const Piece*>(xm + (size_t)p * EPV);
    const Piece wv = *reinterpret_cast<const Piece*>(w + (size_t)p * EPV);
    Piece o;
#pragma unroll
    for (int e = 0; e < EPV; ++e)
      o.v[e] = from_f32<T>(__fmul_rn(__fmul_rn(to_f32(q.v[e]), scale), to_f32(wv.v[e])));
    *reinterpret_cast<Piece*>(om + (size_t)p * EPV) = o;
  }
  for (int i = n_pieces * EPV + tid; i < H; i += kThreads)
    om[i] = from_f32<T>(__fmul_rn(__fmul_rn(to_f32(xm[i]), scale), to_f32(w[i])));
}

template <typename T>
int launch(const void* x, const void* w, void* out, int64_t M, int64_t H, float eps, cudaStream_t st) {
  const bool vec = (H % (16 / (int)sizeof(T)) == 0) && aligned_to(x, 16) && aligned_to(w, 16) &&
                   aligned_to(out, 16);
  rms_norm_kernel<T><<<(unsigned)M, kThreads, 0, st>>>(static_cast<const T*>(x), static_cast<const T*>(w),
                                                        static_cast<T*>(out), (int)H, eps, vec);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

}  // namespace

int rms_norm(const void* x, const void* weight, void* out, int64_t M, int64_t H, float eps, int dtype,
             cudaStream_t st) {
  if (M < 0 || H <= 0 || M >= (int64_t)1 << 31 || H >= (int64_t)1 << 31) return NPB_ERR_INVALID_ARG;
  if (M == 0) return NPB_OK;
  if (x == nullptr || weight == nullptr || out == nullptr) return NPB_ERR_INVALID_ARG;
  switch (dtype) {
    case NPB_BF16: return launch<__nv_bfloat16>(x, weight, out, M, H, eps, st);
    case NPB_F16: return launch<__half>(x, weight, out, M, H, eps, st);
    case NPB_F32: return launch<float>(x, weight, out, M, H, eps, st);
    default: return NPB_ERR_UNSUPPORTED;
  }
}

}  // namespace npb
