// Shared arithmetic of the 4-bit group-affine decoders: eight nibbles of one 32-bit code word
// -> eight weights ((q - z) * s in fp32, one rounding per operation, then one rounding to the
// output type), two elements per instruction on the packed-fp32 pipe of sm_100.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace npb {

// Packed fp32 (two lanes per instruction), round-to-nearest, one rounding each.
__device__ __forceinline__ float2 fsub2(const float2 a, const float2 b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(reinterpret_cast<const uint64_t&>(a)), "l"(reinterpret_cast<const uint64_t&>(b)));
  return reinterpret_cast<const float2&>(d);
}
__device__ __forceinline__ float2 fmul2(const float2 a, const float2 b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(reinterpret_cast<const uint64_t&>(a)), "l"(reinterpret_cast<const uint64_t&>(b)));
  return reinterpret_cast<const float2&>(d);
}

__device__ __forceinline__ uint32_t pack2(float a, float b, __nv_bfloat16) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, __half) {
  const __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// One code word (nibble e = element e) -> four fp32 pairs (elements 2e, 2e+1).
// 0x4B000000 | q is the float 2^23 + q, so subtracting 2^23 yields q without an int-to-float
// conversion; for a symmetric weight (z = 8) both subtractions fold into one exact one.
template <bool ASYM>
__device__ __forceinline__ void q4_word_f32(uint32_t word, float s, float z, float2 (&out)[4]) {
  const uint32_t lo = word & 0x0f0f0f0fu;         // elements 0, 2, 4, 6 (one per byte)
  const uint32_t hi = (word >> 4) & 0x0f0f0f0fu;  // elements 1, 3, 5, 7
  const float2 s2 = make_float2(s, s);
  const float2 m2 = ASYM ? make_float2(8388608.f, 8388608.f) : make_float2(8388616.f, 8388616.f);
  const float2 z2 = make_float2(z, z);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float2 q = make_float2(__uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7650 + e)),
                           __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7650 + e)));
    q = fsub2(q, m2);
    if (ASYM) q = fsub2(q, z2);
    out[e] = fmul2(q, s2);
  }
}

// Same, rounded to eight 16-bit outputs (one 16-byte chunk).
template <typename T, bool ASYM>
__device__ __forceinline__ uint4 q4_word_to_chunk(uint32_t word, float s, float z) {
  float2 f[4];
  q4_word_f32<ASYM>(word, s, z, f);
  return make_uint4(pack2(f[0].x, f[0].y, T()), pack2(f[1].x, f[1].y, T()),
                    pack2(f[2].x, f[2].y, T()), pack2(f[3].x, f[3].y, T()));
}

}  // namespace npb
