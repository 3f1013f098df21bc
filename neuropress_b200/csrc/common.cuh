// Shared device/host helpers for the sm_100a quantized-linear kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "neuropress_b200.h"

namespace npb {

// ---- host-side status plumbing ------------------------------------------------------
void set_last_cuda_error(cudaError_t e, const char* where);

#define NPB_CUDA_TRY(expr)                                  \
  do {                                                      \
    cudaError_t _e = (expr);                                \
    if (_e != cudaSuccess) {                                \
      ::npb::set_last_cuda_error(_e, #expr);                \
      return NPB_ERR_CUDA;                                  \
    }                                                       \
  } while (0)

#define NPB_LAUNCH_CHECK()                                  \
  do {                                                      \
    cudaError_t _e = cudaGetLastError();                    \
    if (_e != cudaSuccess) {                                \
      ::npb::set_last_cuda_error(_e, "kernel launch");      \
      return NPB_ERR_CUDA;                                  \
    }                                                       \
  } while (0)

inline bool aligned_to(const void* p, size_t a) {
  return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

// Limit, in nanoseconds, of every bounded in-kernel wait (mbarriers of the GEMMs, peer flags of
// the all-gather): 2 s unless npb_set_wait_limit_ns changed it.  Read at launch time.
uint64_t wait_limit_ns();
// Tile shape policy of the dense GEMM (npb_set_gemm_pair_mode): 0 single CTAs, 1 automatic, 2 pairs.
int gemm_pair_mode();

// Number of SMs of the current device (cached per device id).
int sm_count();
// Opt a kernel into a large dynamic shared-memory size; cached by the caller.
int max_dynamic_smem();

// Resident blocks per SM of `kernel` at (threads, dynamic smem); opts the kernel into the
// shared-memory size on first use.  Cached per (device, kernel, smem): no runtime queries on
// the launch path after the first call.
int blocks_per_sm(const void* kernel, int threads, size_t smem, int* per_sm);

// Host-side validation shared by decode / GEMV / fused GEMM.  Mirrors the checks of
// vq_dequant.cu:112-127 and vq_linear_wmma.cu:475-506 of the reference.
int validate_vq(const npb_vq_weight* w, int64_t N, int64_t K);
int validate_q(const npb_q_weight* w, int64_t N, int64_t K);

// ---- device: dtype conversion ---------------------------------------------------------
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

// fp16 -> T exactly as the reference decode does it (vq_dequant.cu:38-47): bf16 goes
// through fp32 with one round-to-nearest-even.
template <typename T>
__device__ __forceinline__ T from_half(__half h) { return from_f32<T>(__half2float(h)); }
template <>
__device__ __forceinline__ __half from_half<__half>(__half h) { return h; }

// ---- device: LSB-first bit-stream index read -----------------------------------------
// Index v occupies bits [v*bits, (v+1)*bits) of the stream.  bits in [4, 16]; a 3-byte
// window always covers one index.  No padding is assumed: loads are bounds-checked.
__device__ __forceinline__ uint32_t read_index_generic(const uint8_t* __restrict__ p,
                                                       int64_t n_bytes, int64_t v, int bits) {
  const int64_t bit0 = v * (int64_t)bits;
  const int64_t b0 = bit0 >> 3;
  const int sh = (int)(bit0 & 7);
  uint32_t win = __ldg(p + b0);
  if (b0 + 1 < n_bytes) win |= (uint32_t)__ldg(p + b0 + 1) << 8;
  if (b0 + 2 < n_bytes) win |= (uint32_t)__ldg(p + b0 + 2) << 16;
  return (win >> sh) & ((1u << bits) - 1u);
}

// BITS is a compile-time hint: 16 and 8 use aligned scalar loads (the stream base must be
// 2-byte aligned for 16), 0 means "use the runtime width".
template <int BITS>
__device__ __forceinline__ uint32_t read_index(const uint8_t* __restrict__ p, int64_t n_bytes,
                                               int64_t v, int bits) {
  if constexpr (BITS == 16) {
    return __ldg(reinterpret_cast<const uint16_t*>(p) + v);
  } else if constexpr (BITS == 8) {
    return __ldg(p + v);
  } else {
    return read_index_generic(p, n_bytes, v, bits);
  }
}

// Eight consecutive indices starting at a multiple of 8: they occupy exactly `BITS` bytes
// starting at byte (v0/8)*BITS.  Wide loads where the alignment allows it.
template <int BITS>
__device__ __forceinline__ void read_index8(const uint8_t* __restrict__ p, int64_t chunk,
                                            uint32_t (&idx)[8]) {
  const uint8_t* q = p + chunk * BITS;
  if constexpr (BITS == 16) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(q));
    idx[0] = r.x & 0xffffu; idx[1] = r.x >> 16;
    idx[2] = r.y & 0xffffu; idx[3] = r.y >> 16;
    idx[4] = r.z & 0xffffu; idx[5] = r.z >> 16;
    idx[6] = r.w & 0xffffu; idx[7] = r.w >> 16;
  } else if constexpr (BITS == 8) {
    const uint2 r = __ldg(reinterpret_cast<const uint2*>(q));
    idx[0] = r.x & 0xffu; idx[1] = (r.x >> 8) & 0xffu; idx[2] = (r.x >> 16) & 0xffu; idx[3] = r.x >> 24;
    idx[4] = r.y & 0xffu; idx[5] = (r.y >> 8) & 0xffu; idx[6] = (r.y >> 16) & 0xffu; idx[7] = r.y >> 24;
  } else if constexpr (BITS == 4) {
    const uint32_t r = __ldg(reinterpret_cast<const uint32_t*>(q));
#pragma unroll
    for (int i = 0; i < 8; ++i) idx[i] = (r >> (4 * i)) & 0xfu;
  } else if constexpr (BITS % 4 == 0) {  // 12: three aligned 32-bit words
    constexpr int W = BITS / 4;
    uint32_t w[W + 1];
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = __ldg(reinterpret_cast<const uint32_t*>(q) + i);
    w[W] = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int bit = i * BITS;
      const uint64_t two = ((uint64_t)w[bit / 32 + 1] << 32) | w[bit / 32];
      idx[i] = (uint32_t)(two >> (bit % 32)) & ((1u << BITS) - 1u);
    }
  } else if constexpr (BITS % 2 == 0) {  // 6, 10, 14: aligned 16-bit loads
    constexpr int H = BITS / 2;
    uint32_t w[(H + 1) / 2 + 1] = {};
#pragma unroll
    for (int i = 0; i < H; ++i)
      w[i / 2] |= (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(q) + i) << (16 * (i % 2));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int bit = i * BITS;
      const uint64_t two = ((uint64_t)w[bit / 32 + 1] << 32) | w[bit / 32];
      idx[i] = (uint32_t)(two >> (bit % 32)) & ((1u << BITS) - 1u);
    }
  } else {  // odd widths: byte loads
    uint32_t w[BITS / 4 + 2] = {};
#pragma unroll
    for (int i = 0; i < BITS; ++i) w[i / 4] |= (uint32_t)__ldg(q + i) << (8 * (i % 4));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int bit = i * BITS;
      const uint64_t two = ((uint64_t)w[bit / 32 + 1] << 32) | w[bit / 32];
      idx[i] = (uint32_t)(two >> (bit % 32)) & ((1u << BITS) - 1u);
    }
  }
}

// Alignment (bytes) the stream base needs for read_index8<BITS>.
constexpr int index8_alignment(int bits) {
  return bits == 16 ? 16 : bits == 8 ? 8 : (bits % 4 == 0) ? 4 : (bits % 2 == 0) ? 2 : 1;
}

// 16-byte read-only load of eight fp16 values.
struct alignas(16) Half8 { __half2 h[4]; };
struct alignas(8) Half4 { __half2 h[2]; };

__device__ __forceinline__ Half8 ldg_vec(const Half8* p) {
  const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
  return *reinterpret_cast<const Half8*>(&r);
}
__device__ __forceinline__ Half4 ldg_vec(const Half4* p) {
  const uint2 r = __ldg(reinterpret_cast<const uint2*>(p));
  return *reinterpret_cast<const Half4*>(&r);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace npb
