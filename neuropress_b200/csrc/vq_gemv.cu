// Fused index-decode GEMV for 1..8 activation rows (the decode band).
//
//   y[m, n] = s[n] * sum_g  x[m, VL*g : VL*g+VL] . (C[cb(g)][idx[n,g]] + R[ridx[n,g]])  + bias[n]
//
// One warp owns one output row at a time (rows are strided over all warps of a persistent
// grid).  Lanes stream the row's packed indices with 128-bit loads (eight 16-bit indices,
// or the 12 / 8 bytes holding eight 12- / 8-bit ones), gather 16-byte centroids from shared
// memory (codebooks up to 64 KiB) or through L1/L2 (large codebooks), multiply with the
// activation chunk held in shared memory (XOR-swizzled so that the 128-byte lane stride of
// the 8-index chunks is conflict-free) and reduce with warp shuffles.  fp32 accumulation.
//
// Algorithmic HBM bytes per call: packed indices (+ residual indices, + 2N scale)
// + M*K + M*N activations; the codebook is read once per CTA and stays in L2.
//
// Replaces _vq_linear / _vq_linear_h2 (neuropress/kernels/vq_linear.cu:139-224), _vq_gemv
// (vq_linear_wmma.cu:187-240) and the LUT gather (vq_linear_lut.cu:121-142).
#include <type_traits>

#include "common.cuh"
#include "gather_sink.cuh"

namespace npb {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kSmemCodebookMax = 64 * 1024;

struct GemvArgs {
  const uint8_t* packed;
  int64_t packed_bytes;
  const __half* centroids;
  const uint8_t* res_packed;
  int64_t res_bytes;
  const __half* res_centroids;
  const __half* row_scale;
  const float* bias;
  const void* x;
  void* y;
  int bits, res_bits, num_centroids, res_num_centroids, groups_per_codebook, n_codebooks;
  int M, N, K, Kp, G;
  int res_rep;  // copies of the residual table in shared memory (1 or 8, see the kernel)
  GatherSink sink;  // peer_out != null: y goes to every rank's buffer, then the handshake
};

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
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

// The weight values of one vector exactly as the one-pass decode produces them for
// activation dtype T: fp16 add of the residual, fp16 multiply by the row scale, one rounding
// to T (bf16 through fp32); returned as fp32 for the accumulation.
template <typename T, int NH>
__device__ __forceinline__ void weight_f32(const __half2 (&c)[NH], bool has_res,
                                           const __half2 (&r)[NH], bool has_scale, __half2 s2,
                                           float (&w)[2 * NH]) {
#pragma unroll
  for (int i = 0; i < NH; ++i) {
    __half2 h = c[i];
    if (has_res) h = __hadd2_rn(h, r[i]);
    if (has_scale) h = __hmul2_rn(h, s2);
    float2 f = __half22float2(h);
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
      f = __bfloat1622float2(b);
    }
    w[2 * i] = f.x;
    w[2 * i + 1] = f.y;
  }
}

// Position (in elements) of 8-element chunk j inside a swizzled activation row.
__device__ __forceinline__ int swz(int j) { return (j ^ ((j >> 3) & 7)) * 8; }

template <typename T, int VL, int BITS, int MT, bool CB_SMEM>
__global__ void __launch_bounds__(kThreads) vq_gemv_kernel(GemvArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  T* xs = reinterpret_cast<T*>(smem);
  __half* rcs = reinterpret_cast<__half*>(smem + (size_t)MT * a.Kp * sizeof(T));
  __half* cbs = rcs + (a.res_packed ? a.res_num_centroids * VL * a.res_rep : 0);
  // With res_rep == 8 entry e is stored eight times, at 16-byte slots 8 e .. 8 e + 7, and a lane
  // reads slot 8 e + (lane & 7): the eight lanes that share a pass of a 128-bit shared-memory
  // load then always hit eight different bank groups, so the random gather is conflict-free.
  const int rep_shift = a.res_rep == 8 ? 3 : 0;
  const int rep_lane = (threadIdx.x & 7) & (a.res_rep - 1);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool has_res = a.res_packed != nullptr;

  // ---- stage activations (zero rows beyond M), residual codebook, main codebook --------
  {
    const T* x = static_cast<const T*>(a.x);
    const int chunks = a.Kp / 8;
    for (int t = tid; t < MT * chunks; t += kThreads) {
      const int m = t / chunks, j = t - m * chunks;
      T* dst = xs + (size_t)m * a.Kp + swz(j);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int k = j * 8 + e;
        dst[e] = (m < a.M && k < a.K) ? x[(size_t)m * a.K + k] : from_f32<T>(0.f);
      }
    }
    if (has_res) {
      if (a.res_rep == 8) {  // VL == 8 here: one entry is one 16-byte word
        const int nw = a.res_num_centroids * 8;
        for (int t = tid; t < nw; t += kThreads)
          reinterpret_cast<uint4*>(rcs)[t] = __ldg(reinterpret_cast<const uint4*>(a.res_centroids) + (t >> 3));
      } else {
        const int nw = a.res_num_centroids * VL / 2;
        for (int t = tid; t < nw; t += kThreads)
          reinterpret_cast<uint32_t*>(rcs)[t] =
              __ldg(reinterpret_cast<const uint32_t*>(a.res_centroids) + t);
      }
    }
    if constexpr (CB_SMEM) {
      const int nw = a.n_codebooks * a.num_centroids * VL / 8;  // 16-byte words
      for (int t = tid; t < nw; t += kThreads)
        reinterpret_cast<uint4*>(cbs)[t] = __ldg(reinterpret_cast<const uint4*>(a.centroids) + t);
    }
  }
  __syncthreads();

  const int G = a.G;
  const int gpc = a.groups_per_codebook;
  const int warps_total = gridDim.x * kWarps;
  for (int n = blockIdx.x * kWarps + warp; n < a.N; n += warps_total) {
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    const bool has_scale = a.row_scale != nullptr;
    const __half2 s2 = has_scale ? __half2half2(__ldg(a.row_scale + n)) : __float2half2_rn(1.f);

    if constexpr (BITS != 0) {
      static_assert(VL == 8, "vector index path is VL=8 only");
      const int chunks = G >> 3;
      const int64_t chunk0 = (int64_t)n * chunks;
      for (int c = lane; c < chunks; c += 32) {
        uint32_t idx[8], ridx[8];
        read_index8<BITS>(a.packed, chunk0 + c, idx);
        if (has_res) read_index8<8>(a.res_packed, chunk0 + c, ridx);
        if (gpc > 0) {
          const uint32_t off = (uint32_t)((c * 8) / gpc) * (uint32_t)a.num_centroids;
#pragma unroll
          for (int i = 0; i < 8; ++i) idx[i] += off;  // gpc is a multiple of 8 on this path
        }
        Half8 cv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if constexpr (CB_SMEM)
            cv[i] = reinterpret_cast<const Half8*>(cbs)[idx[i]];
          else
            cv[i] = ldg_vec(reinterpret_cast<const Half8*>(a.centroids) + idx[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float w[8];
          Half8 rv = cv[i];
          if (has_res) rv = reinterpret_cast<const Half8*>(rcs)[(ridx[i] << rep_shift) + rep_lane];
          weight_f32<T, 4>(cv[i].h, has_res, rv.h, has_scale, s2, w);
          const int pos = swz(c * 8 + i);
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            float xv[8];
            load8<T>(xs + (size_t)m * a.Kp + pos, xv);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[m] = fmaf(xv[e], w[e], acc[m]);
          }
        }
      }
    } else {
      // Generic widths / VL=4 / rows whose group count is not a multiple of 8.
      const int64_t v0 = (int64_t)n * G;
      for (int g = lane; g < G; g += 32) {
        uint32_t idx = read_index_generic(a.packed, a.packed_bytes, v0 + g, a.bits);
        if (gpc > 0) idx += (uint32_t)(g / gpc) * (uint32_t)a.num_centroids;
        float w[VL];
        const __half2* cp =
            reinterpret_cast<const __half2*>((CB_SMEM ? cbs : a.centroids) + (size_t)idx * VL);
        __half2 ch[VL / 2], rh[VL / 2];
#pragma unroll
        for (int e = 0; e < VL / 2; ++e) { ch[e] = cp[e]; rh[e] = cp[e]; }
        if (has_res) {
          const uint32_t ri = read_index_generic(a.res_packed, a.res_bytes, v0 + g, a.res_bits);
          const __half2* rp = reinterpret_cast<const __half2*>(rcs + (size_t)ri * VL);
#pragma unroll
          for (int e = 0; e < VL / 2; ++e) rh[e] = rp[e];
        }
        weight_f32<T, VL / 2>(ch, has_res, rh, has_scale, s2, w);
        const int k = g * VL;
        const int pos = swz(k >> 3) + (k & 7);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const T* xp = xs + (size_t)m * a.Kp + pos;
#pragma unroll
          for (int e = 0; e < VL; ++e) acc[m] = fmaf(to_f32(xp[e]), w[e], acc[m]);
        }
      }
    }

#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = warp_sum(acc[m]);
    if (lane == 0) {
      const float b = a.bias ? __ldg(a.bias + n) : 0.f;
      if (a.sink.peer_out == nullptr) {
        T* y = static_cast<T*>(a.y);
#pragma unroll
        for (int m = 0; m < MT; ++m)
          if (m < a.M) y[(size_t)m * a.N + n] = from_f32<T>(acc[m] + b);
      } else {
        // fused all-gather: into this rank's own [M, ld] buffer first
        T* y = static_cast<T*>(a.sink.peer_out[a.sink.rank]);
#pragma unroll
        for (int m = 0; m < MT; ++m)
          if (m < a.M) y[(size_t)m * a.sink.ld + a.sink.col0 + n] = from_f32<T>(acc[m] + b);
      }
    }
  }
  if (a.sink.peer_out != nullptr) gather_tail_small<T>(a.sink, a.M, a.N);
}

template <typename T, int VL, int BITS, int MT, bool CB_SMEM>
int launch(const GemvArgs& a, size_t smem, cudaStream_t st) {
  auto kern = vq_gemv_kernel<T, VL, BITS, MT, CB_SMEM>;
  int per_sm = 0;
  if (int rc = blocks_per_sm(reinterpret_cast<const void*>(kern), kThreads, smem, &per_sm)) return rc;
  if (per_sm < 1) return NPB_ERR_UNSUPPORTED;
  const int want = (a.N + kWarps - 1) / kWarps;
  const int grid = want < sm_count() * per_sm ? want : sm_count() * per_sm;
  kern<<<grid, kThreads, smem, st>>>(a);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

template <typename T, int VL, int BITS, int MT>
int launch_cb(const GemvArgs& a, bool cb_smem, size_t smem, cudaStream_t st) {
  return cb_smem ? launch<T, VL, BITS, MT, true>(a, smem, st)
                 : launch<T, VL, BITS, MT, false>(a, smem, st);
}

template <typename T, int VL, int BITS>
int launch_mt(const GemvArgs& a, int mt, bool cb_smem, size_t smem, cudaStream_t st) {
  switch (mt) {
    case 1: return launch_cb<T, VL, BITS, 1>(a, cb_smem, smem, st);
    case 2: return launch_cb<T, VL, BITS, 2>(a, cb_smem, smem, st);
    case 4: return launch_cb<T, VL, BITS, 4>(a, cb_smem, smem, st);
    default: return launch_cb<T, VL, BITS, 8>(a, cb_smem, smem, st);
  }
}

template <typename T>
int run_rows(const npb_vq_weight* w, GemvArgs a, cudaStream_t st) {
  const int VL = w->vector_len;
  a.Kp = (a.K + 63) / 64 * 64;
  const int mt = a.M <= 1 ? 1 : a.M <= 2 ? 2 : a.M <= 4 ? 4 : 8;
  const size_t x_bytes = (size_t)mt * a.Kp * sizeof(T);
  size_t res_bytes = a.res_packed ? (size_t)a.res_num_centroids * VL * 2 : 0;
  const size_t cb_bytes = (size_t)a.n_codebooks * a.num_centroids * VL * 2;
  const size_t cap = (size_t)max_dynamic_smem();

  // Vector index path: VL 8, whole 8-index chunks per row, aligned streams, 8-bit residual.
  int vbits = 0;
  if (VL == 8 && a.G % 8 == 0 && (a.bits == 16 || a.bits == 12 || a.bits == 8) &&
      aligned_to(a.packed, index8_alignment(a.bits)) && aligned_to(a.centroids, 16) &&
      (a.groups_per_codebook % 8 == 0) &&
      (!a.res_packed || (a.res_bits == 8 && aligned_to(a.res_packed, 8) &&
                         aligned_to(a.res_centroids, 16))))
    vbits = a.bits;
  // Replicate a small residual table eight-fold (conflict-free gathers); vector path only.
  a.res_rep = 1;
  if (vbits != 0 && a.res_packed && res_bytes * 8 <= 32 * 1024 && x_bytes + res_bytes * 8 <= cap) {
    a.res_rep = 8;
    res_bytes *= 8;
  }
  if (x_bytes + res_bytes > cap) return NPB_ERR_TOO_LARGE;
  const bool cb_smem = cb_bytes <= (size_t)kSmemCodebookMax && x_bytes + res_bytes + cb_bytes <= cap &&
                       aligned_to(a.centroids, 16) && (res_bytes % 16 == 0);
  const size_t smem = x_bytes + res_bytes + (cb_smem ? cb_bytes : 0);
  if (VL == 8) {
    switch (vbits) {
      case 16: return launch_mt<T, 8, 16>(a, mt, cb_smem, smem, st);
      case 12: return launch_mt<T, 8, 12>(a, mt, cb_smem, smem, st);
      case 8: return launch_mt<T, 8, 8>(a, mt, cb_smem, smem, st);
      default: return launch_mt<T, 8, 0>(a, mt, cb_smem, smem, st);
    }
  }
  if (VL == 4) return launch_mt<T, 4, 0>(a, mt, cb_smem, smem, st);
  return NPB_ERR_UNSUPPORTED;
}

template <typename T>
int run(const npb_vq_weight* w, GemvArgs a, cudaStream_t st) {
  // Rows that do not fit in shared memory together are processed in smaller batches.
  const int M = a.M;
  const int Kp = (a.K + 63) / 64 * 64;
  const size_t res_bytes = a.res_packed ? (size_t)a.res_num_centroids * w->vector_len * 2 : 0;
  int batch = 8;
  while (batch > 1 && (size_t)batch * Kp * sizeof(T) + res_bytes > (size_t)max_dynamic_smem() / 2)
    batch >>= 1;
  if (a.sink.peer_out != nullptr && batch < M) return NPB_ERR_TOO_LARGE;  // one handshake per call
  for (int m0 = 0; m0 < M; m0 += batch) {
    GemvArgs b = a;
    b.M = (M - m0) < batch ? (M - m0) : batch;
    b.x = static_cast<const T*>(a.x) + (size_t)m0 * a.K;
    b.y = static_cast<T*>(a.y) + (size_t)m0 * a.N;
    if (int rc = run_rows<T>(w, b, st)) return rc;
  }
  return NPB_OK;
}

}  // namespace

int vq_gemv_mma(const npb_vq_weight*, const void*, int, int64_t, int64_t, int64_t, const float*, void*,
                const GatherSink*, cudaStream_t);
namespace {
int vq_gemv_impl(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M, int64_t N, int64_t K,
                 const float* bias, void* y, const GatherSink* sink, cudaStream_t st);
}

int vq_gemv(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M, int64_t N, int64_t K,
            const float* bias, void* y, cudaStream_t st) {
  return vq_gemv_impl(w, x, x_dtype, M, N, K, bias, y, nullptr, st);
}

// GEMV whose result goes into columns [col0, col0 + N) of every rank's [M, ld] buffer, closed
// by the all-gather handshake (gather_sink.cuh).  One launch, so M <= 8 rows must fit shared
// memory together (NPB_ERR_TOO_LARGE otherwise).
int vq_gemv_gather(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M, int64_t N, int64_t K,
                   const float* bias, const GatherSink& sink, cudaStream_t st) {
  if (sink.peer_out == nullptr || sink.peer_flags == nullptr || sink.world < 1 ||
      sink.world > kMaxGatherWorld || sink.rank < 0 || sink.rank >= sink.world || sink.ld < N ||
      sink.col0 < 0 || sink.col0 + N > sink.ld)
    return NPB_ERR_INVALID_ARG;
  if (M <= 0 || N <= 0) return NPB_ERR_INVALID_ARG;  // every rank must run the handshake
  const int64_t epc = x_dtype == NPB_F32 ? 4 : 8;    // elements per 16-byte piece of a row
  if (N % epc != 0 || sink.ld % epc != 0 || sink.col0 % epc != 0) return NPB_ERR_ALIGNMENT;
  if (M <= NPB_VQ_SMALL_BATCH_MAX_ROWS) {  // tensor-core kernel where the weight form allows it
    const int rc = vq_gemv_mma(w, x, x_dtype, M, N, K, bias, nullptr, &sink, st);
    if (rc != NPB_ERR_UNSUPPORTED) return rc;
  }
  return vq_gemv_impl(w, x, x_dtype, M, N, K, bias, nullptr, &sink, st);
}

namespace {
int vq_gemv_impl(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M, int64_t N, int64_t K,
                 const float* bias, void* y, const GatherSink* sink, cudaStream_t st) {
  if (int rc = validate_vq(w, N, K)) return rc;
  if (M < 0 || M > NPB_GEMV_MAX_ROWS) return NPB_ERR_UNSUPPORTED;
  if (M == 0 || N == 0) return NPB_OK;
  if (x == nullptr || (y == nullptr && sink == nullptr)) return NPB_ERR_INVALID_ARG;
  if (N >= (int64_t)1 << 31 || K >= (int64_t)1 << 24) return NPB_ERR_UNSUPPORTED;
  GemvArgs a{};
  a.packed = w->packed;
  a.packed_bytes = w->packed_bytes;
  a.centroids = static_cast<const __half*>(w->centroids);
  a.res_packed = w->res_packed;
  a.res_bytes = w->res_packed_bytes;
  a.res_centroids = static_cast<const __half*>(w->res_centroids);
  a.row_scale = static_cast<const __half*>(w->row_scale);
  a.bias = bias;
  a.x = x;
  a.y = y;
  a.bits = w->bits;
  a.res_bits = w->res_bits;
  a.num_centroids = w->num_centroids;
  a.res_num_centroids = w->res_num_centroids;
  a.groups_per_codebook = w->cols_per_codebook > 0 ? w->cols_per_codebook / w->vector_len : 0;
  a.n_codebooks = w->cols_per_codebook > 0
                      ? (int)((K + w->cols_per_codebook - 1) / w->cols_per_codebook) : 1;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.G = (int)(K / w->vector_len);
  if (sink) a.sink = *sink;
  switch (x_dtype) {
    case NPB_BF16: return run<__nv_bfloat16>(w, a, st);
    case NPB_F16: return run<__half>(w, a, st);
    case NPB_F32: return run<float>(w, a, st);
    default: return NPB_ERR_UNSUPPORTED;
  }
}
}  // namespace

}  // namespace npb
