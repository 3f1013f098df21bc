// Group-affine (Q4_0 / HQQ style) weights: one-pass decode and fused GEMV.
//
//   W[n, k] = convert_T( (float(q[n,k]) - zp[n, k/g]) * float(s[n, k/g]) )
//
// q is nbits wide, packed LSB-first inside each byte of codes[N, K*nbits/8]; zp is the fp16
// zero-point or the constant 2^(nbits-1).  The arithmetic (fp32 subtract, fp32 multiply, one
// rounding to T) is that of _q_dequant_linear (neuropress/nn/np_linear.py:334-351) and of the
// reference kernel (neuropress/kernels/q4_linear.cu:101-123); __fmul_rn / __fsub_rn keep the
// compiler from contracting them, so the decode is bit-exact.
//
// GEMV: a warp owns one output row; each lane loads 16 bytes of codes (32 nibbles) per step,
// so a warp reads 512 contiguous bytes.  Per lane and step the dot product uses
//   sum_k x_k (q_k - zp) s  =  s * (sum_k x_k q_k  -  zp * sum_k x_k)
// with sum_k x_k over each 8-element chunk precomputed once per CTA.  fp32 accumulation.
// HBM bytes per call: N*K*nbits/8 + 2*(1 or 2)*N*K/g + activations — pure streaming.
#include <type_traits>

#include "common.cuh"
#include "q4_math.cuh"

namespace npb {

int q4_gemv_ring(const npb_q_weight*, const void*, int, int64_t, int64_t, int64_t, const float*, void*,
                 cudaStream_t);
int q4_gemv_mma(const npb_q_weight*, const void*, int, int64_t, int64_t, int64_t, const float*,
                void*, cudaStream_t);

namespace {

// ------------------------------------------------------------------ decode ------------
constexpr int kDecThreads = 256;

template <typename T, int NBITS>
__global__ void __launch_bounds__(kDecThreads)
q_decode_kernel(const uint8_t* __restrict__ codes, const __half* __restrict__ scale,
                const __half* __restrict__ zp, T* __restrict__ out, int64_t n_chunks,
                int group_size) {
  // One thread decodes 8 consecutive values (one 8-element chunk never straddles a group:
  // group_size % 8 == 0).
  constexpr int BYTES = NBITS;  // 8 values * NBITS / 8
  const int64_t c = (int64_t)blockIdx.x * kDecThreads + threadIdx.x;
  if (c >= n_chunks) return;
  const int64_t e0 = c * 8;
  const int64_t gi = e0 / group_size;
  const float s = __half2float(__ldg(scale + gi));
  const float z = zp ? __half2float(__ldg(zp + gi)) : (float)(1 << (NBITS - 1));
  uint32_t q[8];
  if constexpr (NBITS == 4) {
    const uint32_t r = __ldg(reinterpret_cast<const uint32_t*>(codes + c * BYTES));
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = (r >> (4 * i)) & 0xfu;
  } else {
    const uint2 r = __ldg(reinterpret_cast<const uint2*>(codes + c * BYTES));
#pragma unroll
    for (int i = 0; i < 4; ++i) { q[i] = (r.x >> (8 * i)) & 0xffu; q[4 + i] = (r.y >> (8 * i)) & 0xffu; }
  }
  float w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = __fmul_rn(__fsub_rn((float)q[i], z), s);
  if constexpr (sizeof(T) == 2) {
    struct alignas(16) Out { T v[8]; } o;
#pragma unroll
    for (int i = 0; i < 8; ++i) o.v[i] = from_f32<T>(w[i]);
    *reinterpret_cast<Out*>(out + e0) = o;
  } else {
    reinterpret_cast<float4*>(out + e0)[0] = make_float4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<float4*>(out + e0)[1] = make_float4(w[4], w[5], w[6], w[7]);
  }
}

// 4-bit decode to a 16-bit type, the large-batch path: a thread converts four 8-value chunks
// that lie 256 chunks apart, so every warp-wide code load (4 bytes per lane) and store (16
// bytes per lane) is contiguous; nibble -> fp32 by byte-permute, (q - z) * s in packed fp32
// (q4_math.cuh), 32-bit index arithmetic, group index by shift when the group is a power of
// two.  HBM bytes: codes + scales (+ zero points) in, N*K*2 out; the kernel is write-bound.
constexpr int kDec4Unroll = 4;

template <typename T, bool ASYM>
__global__ void __launch_bounds__(kDecThreads)
q4_decode16_kernel(const uint32_t* __restrict__ codes, const __half* __restrict__ scale,
                   const __half* __restrict__ zp, uint4* __restrict__ out, uint32_t n_chunks,
                   uint32_t chunks_per_group, int cpg_shift) {
  const uint32_t base = blockIdx.x * (kDecThreads * kDec4Unroll) + threadIdx.x;
  uint32_t word[kDec4Unroll];
  __half s[kDec4Unroll], z[kDec4Unroll];
#pragma unroll
  for (int u = 0; u < kDec4Unroll; ++u) {
    const uint32_t c = base + u * kDecThreads;
    // chunks past the end read chunk 0 (always mapped) and are not stored
    const uint32_t cc = c < n_chunks ? c : 0u;
    const uint32_t g = cpg_shift >= 0 ? cc >> cpg_shift : cc / chunks_per_group;
    word[u] = __ldg(codes + cc);
    s[u] = __ldg(scale + g);
    z[u] = __ldg(zp + g);  // symmetric weights pass the scale pointer here: a mapped address
  }
#pragma unroll
  for (int u = 0; u < kDec4Unroll; ++u) {
    const uint32_t c = base + u * kDecThreads;
    if (c < n_chunks)
      out[c] = q4_word_to_chunk<T, ASYM>(word[u], __half2float(s[u]), __half2float(z[u]));
  }
}

template <typename T>
int launch_decode(const npb_q_weight* w, int64_t N, int64_t K, T* out, cudaStream_t st) {
  const int64_t n_chunks = N * K / 8;
  if constexpr (sizeof(T) == 2) {
    if (w->nbits == 4 && n_chunks < ((int64_t)1 << 31) && aligned_to(w->codes, 4) && aligned_to(out, 16)) {
      const uint32_t cpg = (uint32_t)(w->group_size / 8);
      const int shift = (cpg & (cpg - 1)) == 0 ? __builtin_ctz(cpg) : -1;
      const uint32_t per_block = kDecThreads * kDec4Unroll;
      const uint32_t blocks = (uint32_t)((n_chunks + per_block - 1) / per_block);
      const uint32_t* c32 = reinterpret_cast<const uint32_t*>(w->codes);
      const __half* sc = static_cast<const __half*>(w->scale);
      uint4* o = reinterpret_cast<uint4*>(out);
      if (w->zero_point)
        q4_decode16_kernel<T, true><<<blocks, kDecThreads, 0, st>>>(
            c32, sc, static_cast<const __half*>(w->zero_point), o, (uint32_t)n_chunks, cpg, shift);
      else
        q4_decode16_kernel<T, false><<<blocks, kDecThreads, 0, st>>>(c32, sc, sc, o, (uint32_t)n_chunks,
                                                                      cpg, shift);
      NPB_LAUNCH_CHECK();
      return NPB_OK;
    }
  }
  const int64_t blocks = (n_chunks + kDecThreads - 1) / kDecThreads;
  if (blocks >= (int64_t)1 << 31) return NPB_ERR_UNSUPPORTED;
  const __half* s = static_cast<const __half*>(w->scale);
  const __half* z = static_cast<const __half*>(w->zero_point);
  if (w->nbits == 4)
    q_decode_kernel<T, 4><<<(unsigned)blocks, kDecThreads, 0, st>>>(w->codes, s, z, out, n_chunks, w->group_size);
  else
    q_decode_kernel<T, 8><<<(unsigned)blocks, kDecThreads, 0, st>>>(w->codes, s, z, out, n_chunks, w->group_size);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

// ------------------------------------------------------------------ GEMV --------------
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

struct QGemvArgs {
  const uint8_t* codes;
  const __half* scale;
  const __half* zp;
  const float* bias;
  const void* x;
  void* y;
  int M, N, K, group_size;
};

// Shared memory: x as fp32?  No: x stays in T, [MT][K] with the same XOR swizzle on 8-element
// chunks as the VQ GEMV (a lane's 32 values are 4 consecutive chunks), plus fp32 chunk sums
// xsum[MT][K/8].
__device__ __forceinline__ int swz8(int j) { return (j ^ ((j >> 3) & 7)) * 8; }

template <typename T>
__device__ __forceinline__ void load8f(const T* p, float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&r);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = to_f32(e[i]);
  } else {
    const float4 a = reinterpret_cast<const float4*>(p)[0];
    const float4 b = reinterpret_cast<const float4*>(p)[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
}

// Two fp32 FMAs in one instruction (sm_100 packed-fp32 pipe): d += a * b, component-wise.
__device__ __forceinline__ void ffma2(float2& d, const float2 a, const float2 b) {
  uint64_t dd = reinterpret_cast<const uint64_t&>(d);
  asm("fma.rn.f32x2 %0, %1, %2, %0;"
      : "+l"(dd)
      : "l"(reinterpret_cast<const uint64_t&>(a)), "l"(reinterpret_cast<const uint64_t&>(b)));
  d = reinterpret_cast<const float2&>(dd);
}

// Eight activations (one swizzled chunk) as four fp32 pairs (x0,x1) (x2,x3) (x4,x5) (x6,x7).
template <typename T>
__device__ __forceinline__ void load_x_pairs(const T* p, float2 (&xp)[4]) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)  // bf16 -> fp32 is a 16-bit shift
      xp[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
  } else if constexpr (std::is_same<T, __half>::value) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) xp[i] = __half22float2(h[i]);
  } else {
    const float4 a = reinterpret_cast<const float4*>(p)[0];
    const float4 b = reinterpret_cast<const float4*>(p)[1];
    xp[0] = make_float2(a.x, a.y); xp[1] = make_float2(a.z, a.w);
    xp[2] = make_float2(b.x, b.y); xp[3] = make_float2(b.z, b.w);
  }
}

// A warp owns ROWS output rows at a time; a lane takes 32 consecutive k (16 bytes of codes,
// exactly one scale group when group_size % 32 == 0) per step, 1024 k per warp step.
// Nibble q becomes the fp32 value 128 + q with one byte-permute (byte 0x0q dropped into the
// top mantissa byte of 128.0f), products run on the packed-fp32 pipe (two FMAs per
// instruction), and the zero-point / scale are applied once per lane step:
//   acc += s * (sum_k (128 + q_k) x_k  -  (128 + zp) * sum_k x_k).
template <typename T, int MT, int ROWS>
__global__ void __launch_bounds__(kThreads) q4_gemv_kernel(QGemvArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int K = a.K;
  T* xs = reinterpret_cast<T*>(smem);                                         // [MT][K]
  float* xsum = reinterpret_cast<float*>(smem + (size_t)MT * K * sizeof(T));  // [MT][K/32]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gs = a.group_size;
  const int groups = K / gs;
  const int row_bytes = K / 2;
  const int ksteps = K / 1024;
  const int stride = gridDim.x * kWarps * ROWS;

  // One lane step of ROWS rows: 16 bytes of codes, scale and zero-point per row.
  struct Step { uint4 code[ROWS]; __half s[ROWS]; __half z[ROWS]; };
  auto load_step = [&](Step& st, int n0, int ks) {
    const int k0 = ks * 1024 + lane * 32;
    const int g = k0 / gs;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int n = n0 + r < a.N ? n0 + r : a.N - 1;
      st.code[r] = __ldg(reinterpret_cast<const uint4*>(a.codes + (size_t)n * row_bytes + k0 / 2));
      st.s[r] = __ldg(a.scale + (size_t)n * groups + g);
      st.z[r] = a.zp ? __ldg(a.zp + (size_t)n * groups + g) : __float2half_rn(8.f);
    }
  };

  // The first weight loads are issued before the activations are staged, so their HBM
  // latency overlaps the staging; after that the loop always has the next step in flight.
  int n0 = (blockIdx.x * kWarps + warp) * ROWS, ks = 0;
  bool have = n0 < a.N;
  Step cur;
  if (have) load_step(cur, n0, 0);
  {
    const T* x = static_cast<const T*>(a.x);
    for (int t = tid; t < MT * (K / 32); t += kThreads) {
      const int m = t / (K / 32), j4 = t - m * (K / 32);
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int j = j4 * 4 + c;
        struct alignas(16) V8 { T v[8]; } v;
        if (m < a.M) {
          v = *reinterpret_cast<const V8*>(x + (size_t)m * K + j * 8);  // K % 1024 == 0, x 16 B aligned
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) v.v[e] = from_f32<T>(0.f);
        }
        *reinterpret_cast<V8*>(xs + (size_t)m * K + swz8(j)) = v;
#pragma unroll
        for (int e = 0; e < 8; ++e) s += to_f32(v.v[e]);
      }
      xsum[t] = s;
    }
  }
  __syncthreads();

  float acc[ROWS][MT];
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;

  while (have) {
    int nn0 = n0, nks = ks + 1;
    if (nks == ksteps) { nks = 0; nn0 = n0 + stride; }
    const bool have_next = nn0 < a.N;
    Step nxt;
    if (have_next) load_step(nxt, nn0, nks);

    const int k0 = ks * 1024 + lane * 32;
    float2 d[ROWS][MT];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m) d[r][m] = make_float2(0.f, 0.f);
    const int j0 = k0 / 8;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      float2 xp[MT][4];
#pragma unroll
      for (int m = 0; m < MT; ++m) load_x_pairs<T>(xs + (size_t)m * K + swz8(j0 + ch), xp[m]);
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const uint32_t word = ch == 0 ? cur.code[r].x : ch == 1 ? cur.code[r].y
                            : ch == 2 ? cur.code[r].z : cur.code[r].w;
        const uint32_t lo = word & 0x0f0f0f0fu;          // nibbles 0, 2, 4, 6 (one per byte)
        const uint32_t hi = (word >> 4) & 0x0f0f0f0fu;   // nibbles 1, 3, 5, 7
        float2 q[4];
        q[0] = make_float2(__uint_as_float(__byte_perm(lo, 0x43000000u, 0x7044)),
                           __uint_as_float(__byte_perm(hi, 0x43000000u, 0x7044)));
        q[1] = make_float2(__uint_as_float(__byte_perm(lo, 0x43000000u, 0x7144)),
                           __uint_as_float(__byte_perm(hi, 0x43000000u, 0x7144)));
        q[2] = make_float2(__uint_as_float(__byte_perm(lo, 0x43000000u, 0x7244)),
                           __uint_as_float(__byte_perm(hi, 0x43000000u, 0x7244)));
        q[3] = make_float2(__uint_as_float(__byte_perm(lo, 0x43000000u, 0x7344)),
                           __uint_as_float(__byte_perm(hi, 0x43000000u, 0x7344)));
#pragma unroll
        for (int m = 0; m < MT; ++m) {
#pragma unroll
          for (int i = 0; i < 4; ++i) ffma2(d[r][m], q[i], xp[m][i]);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const float xs32 = xsum[m * (K / 32) + k0 / 32];
#pragma unroll
      for (int r = 0; r < ROWS; ++r)
        acc[r][m] = fmaf(__half2float(cur.s[r]),
                         (d[r][m].x + d[r][m].y) - (128.f + __half2float(cur.z[r])) * xs32, acc[r][m]);
    }

    if (ks == ksteps - 1) {  // row group finished: reduce over the warp and write
#pragma unroll
      for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = warp_sum(acc[r][m]);
      if (lane == 0) {
        T* y = static_cast<T*>(a.y);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          const int n = n0 + r;
          if (n >= a.N) continue;
          const float b = a.bias ? __ldg(a.bias + n) : 0.f;
#pragma unroll
          for (int m = 0; m < MT; ++m)
            if (m < a.M) y[(size_t)m * a.N + n] = from_f32<T>(acc[r][m] + b);
        }
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;
    }
    cur = nxt;
    n0 = nn0;
    ks = nks;
    have = have_next;
  }
}

// Fallback for shapes the streaming kernel does not take (K % 32 != 0, 8-bit codes):
// a warp per row, one 8-value chunk per lane and step.
template <typename T, int NBITS>
__global__ void __launch_bounds__(kThreads) q_gemv_generic_kernel(QGemvArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int K = a.K, gs = a.group_size, groups = K / gs;
  const int row_bytes = K * NBITS / 8;
  const T* x = static_cast<const T*>(a.x);
  T* y = static_cast<T*>(a.y);
  for (int n = blockIdx.x * kWarps + warp; n < a.N; n += gridDim.x * kWarps) {
    for (int m = 0; m < a.M; ++m) {
      float acc = 0.f;
      for (int j = lane; j < K / 8; j += 32) {
        const int g = (j * 8) / gs;
        const float s = __half2float(__ldg(a.scale + (size_t)n * groups + g));
        const float z = a.zp ? __half2float(__ldg(a.zp + (size_t)n * groups + g))
                             : (float)(1 << (NBITS - 1));
        const uint8_t* cp = a.codes + (size_t)n * row_bytes + (size_t)j * NBITS;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          uint32_t q;
          if constexpr (NBITS == 4) q = (__ldg(cp + e / 2) >> (4 * (e & 1))) & 0xfu;
          else q = __ldg(cp + e);
          acc = fmaf(((float)q - z) * s, to_f32(x[(size_t)m * K + j * 8 + e]), acc);
        }
      }
      acc = warp_sum(acc);
      if (lane == 0) y[(size_t)m * a.N + n] = from_f32<T>(acc + (a.bias ? a.bias[n] : 0.f));
    }
  }
}

template <typename KernT>
int launch_persistent(KernT kern, const QGemvArgs& a, size_t smem, int rows_per_warp,
                      cudaStream_t st) {
  int per_sm = 0;
  if (int rc = blocks_per_sm(reinterpret_cast<const void*>(kern), kThreads, smem, &per_sm)) return rc;
  if (per_sm < 1) return NPB_ERR_UNSUPPORTED;
  const int rows_per_block = kWarps * rows_per_warp;
  const int want = (a.N + rows_per_block - 1) / rows_per_block;
  const int cap = sm_count() * per_sm;
  kern<<<want < cap ? want : cap, kThreads, smem, st>>>(a);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

template <typename T>
int run_gemv(const npb_q_weight* w, QGemvArgs a, cudaStream_t st) {
  const bool fast = w->nbits == 4 && a.K % 1024 == 0 && w->group_size % 32 == 0 &&
                    aligned_to(a.codes, 16) && aligned_to(a.x, 16);
  if (!fast) {
    if (w->nbits == 4) return launch_persistent(q_gemv_generic_kernel<T, 4>, a, 0, 1, st);
    return launch_persistent(q_gemv_generic_kernel<T, 8>, a, 0, 1, st);
  }
  const int M = a.M;
  int batch = 8;
  auto need = [&](int mt) { return (size_t)mt * a.K * sizeof(T) + (size_t)mt * (a.K / 32) * 4; };
  while (batch > 1 && need(batch) > (size_t)max_dynamic_smem() / 2) batch >>= 1;
  if (need(batch) > (size_t)max_dynamic_smem()) return NPB_ERR_TOO_LARGE;
  for (int m0 = 0; m0 < M; m0 += batch) {
    QGemvArgs b = a;
    b.M = (M - m0) < batch ? (M - m0) : batch;
    b.x = static_cast<const T*>(a.x) + (size_t)m0 * a.K;
    b.y = static_cast<T*>(a.y) + (size_t)m0 * a.N;
    const int mt = b.M <= 1 ? 1 : b.M <= 2 ? 2 : b.M <= 4 ? 4 : 8;
    int rc;
    switch (mt) {
      case 1: rc = launch_persistent(q4_gemv_kernel<T, 1, 4>, b, need(1), 4, st); break;
      case 2: rc = launch_persistent(q4_gemv_kernel<T, 2, 2>, b, need(2), 2, st); break;
      case 4: rc = launch_persistent(q4_gemv_kernel<T, 4, 1>, b, need(4), 1, st); break;
      default: rc = launch_persistent(q4_gemv_kernel<T, 8, 1>, b, need(8), 1, st); break;
    }
    if (rc) return rc;
  }
  return NPB_OK;
}

}  // namespace

int q_decode(const npb_q_weight* w, int64_t N, int64_t K, void* out, int out_dtype,
             cudaStream_t st) {
  if (int rc = validate_q(w, N, K)) return rc;
  if (N * K == 0) return NPB_OK;
  if (out == nullptr) return NPB_ERR_INVALID_ARG;
  if (!aligned_to(out, 16) || !aligned_to(w->codes, w->nbits == 4 ? 4 : 8)) return NPB_ERR_ALIGNMENT;
  switch (out_dtype) {
    case NPB_BF16: return launch_decode<__nv_bfloat16>(w, N, K, static_cast<__nv_bfloat16*>(out), st);
    case NPB_F16: return launch_decode<__half>(w, N, K, static_cast<__half*>(out), st);
    case NPB_F32: return launch_decode<float>(w, N, K, static_cast<float*>(out), st);
    default: return NPB_ERR_UNSUPPORTED;
  }
}

int q_gemv(const npb_q_weight* w, const void* x, int x_dtype, int64_t M, int64_t N, int64_t K,
           const float* bias, void* y, cudaStream_t st) {
  if (int rc = validate_q(w, N, K)) return rc;
  if (M < 0 || M > NPB_GEMV_MAX_ROWS) return NPB_ERR_UNSUPPORTED;
  if (M == 0 || N == 0) return NPB_OK;
  if (x == nullptr || y == nullptr) return NPB_ERR_INVALID_ARG;
  if (N >= (int64_t)1 << 31 || K >= (int64_t)1 << 24) return NPB_ERR_UNSUPPORTED;
  QGemvArgs a{};
  a.codes = w->codes;
  a.scale = static_cast<const __half*>(w->scale);
  a.zp = static_cast<const __half*>(w->zero_point);
  a.bias = bias;
  a.x = x;
  a.y = y;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.group_size = w->group_size;
  {
    // the weight streamed through a shared-memory ring by bulk async copies (it declines what it does not take)
    const int rc = q4_gemv_ring(w, x, x_dtype, M, N, K, bias, y, st);
    if (rc != NPB_ERR_UNSUPPORTED) return rc;
  }
  {
    // Tensor-core GEMV first (bf16 / fp16, K % 512 == 0); it declines other shapes.
    const int rc = q4_gemv_mma(w, x, x_dtype, M, N, K, bias, y, st);
    if (rc != NPB_ERR_UNSUPPORTED) return rc;
  }
  switch (x_dtype) {
    case NPB_BF16: return run_gemv<__nv_bfloat16>(w, a, st);
    case NPB_F16: return run_gemv<__half>(w, a, st);
    case NPB_F32: return run_gemv<float>(w, a, st);
    default: return NPB_ERR_UNSUPPORTED;
  }
}

}  // namespace npb
