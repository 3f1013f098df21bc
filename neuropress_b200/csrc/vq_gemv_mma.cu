// Fused index-decode linear for 1..16 activation rows on the tensor cores (mma.sync):
//
//   y[m, n] = sum_k x[m, k] * W[n, k] + bias[n],   W decoded on the fly exactly as the one-pass
//   decode produces it (fp16 add of the residual, fp16 multiply by the row scale, one rounding
//   to the activation type), never written to memory.
//
// The weight is the A operand of mma.m16n8k16 (16 output rows x 16 k), the activations the B
// operand (16 k x 8 activation rows; two B tiles for 9..16 rows), so one decoded 16-row slab is
// used by every activation row.  Because a sum over k does not care about the order of its
// terms, the k slots of an mma need not be consecutive k: lane (g, t) of a warp (g = lane / 4,
// t = lane % 4) owns whole centroid vectors -- for its rows g and g + 8, vectors 8 t + s of the
// warp's 32-vector K slice, s = 0..7 -- and feeds elements 0..3 of a vector to one mma and 4..7
// to the next, while the B operand supplies the activations of exactly those k (one 16-byte
// shared-memory load per lane, XOR-swizzled so that it is conflict-free).  So every gather is a
// full 16-byte centroid, every index load a 16-byte (8 x 16-bit) run, as in the GEMV.
//
// CTA = W warps, warp w owns K slice(s) w (256 k each); a CTA walks 16-row groups of W (strided
// by the grid); per group the warps' partial 16 x 16 tiles are summed through shared memory
// (double-buffered, one __syncthreads per group).  Bound by the same centroid-gather rate as
// the GEMV, but independent of the row count up to 16.
//
// Stands in for the GEMM branch of vq_linear_wmma at small batches
// (neuropress/kernels/vq_linear_wmma.cu:261-394) and for _vq_gemv above 2 rows (:187-240).
#include <type_traits>

#include "common.cuh"
#include "mma_sync.cuh"
#include "gather_sink.cuh"

namespace npb {
namespace {

// One weight of a grouped launch: several weights that share the activations (q / k / v, or
// gate / up) are walked by one kernel as if their rows were stacked.
struct MmaSeg {
  const uint8_t* packed;
  const __half* centroids;
  const float* bias;
  int N;        // rows of this weight
  int group0;   // first 16-row group of this weight in the stacked order
  int col0;     // first output column
};
constexpr int kMaxSegs = 4;

struct MmaVqArgs {
  const uint8_t* packed;
  const __half* centroids;
  const uint8_t* res_packed;   // never null: aliases `packed` when there is no residual
  const __half* res_centroids; // never null: aliases `centroids`
  const __half* row_scale;     // never null: aliases `centroids`
  const float* bias;
  const void* x;
  void* y;
  int has_res, has_scale;
  int num_centroids, res_num_centroids, groups_per_codebook;
  int M, N, K, G;
  int slices_per_warp;
  GatherSink sink;  // peer_out != null: y goes to this rank's own [M, ld] buffer, then the tail
  // grouped launch (n_segs > 1): the per-weight fields above are unused; no residual / row scale
  int n_segs, ld_y, total_groups;
  int cb_entries;  // codebook entries over all column blocks (shared-memory staging)
  MmaSeg seg[kMaxSegs];
  // fused RMSNorm of the activations while they are staged (norm_w == null: none):
  // x' = T(x * rsqrt(mean(x^2) + eps) * norm_w), fp32 arithmetic, rounded once like the norm kernel
  const void* norm_w;
  float norm_eps;
};

// fp16 pair -> the activation type, one rounding (bf16 through fp32, as from_half<bf16>).
template <typename T>
__device__ __forceinline__ uint32_t to_operand(__half2 h) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    const float2 f = __half22float2(h);
    const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
    return *reinterpret_cast<const uint32_t*>(&b);
  } else {
    return *reinterpret_cast<const uint32_t*>(&h);
  }
}

// Eight consecutive indices of BITS bits as raw words (loaded one step ahead of their use) ...
template <int BITS>
struct RawIdx { uint32_t w[BITS / 4]; };

template <int BITS>
__device__ __forceinline__ RawIdx<BITS> load_raw(const uint8_t* __restrict__ p, int64_t chunk) {
  RawIdx<BITS> r;
  const uint8_t* q = p + chunk * BITS;
  if constexpr (BITS == 16) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(q));
    r.w[0] = v.x; r.w[1] = v.y; r.w[2] = v.z; r.w[3] = v.w;
  } else if constexpr (BITS == 8) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(q));
    r.w[0] = v.x; r.w[1] = v.y;
  } else {
#pragma unroll
    for (int i = 0; i < BITS / 4; ++i) r.w[i] = __ldg(reinterpret_cast<const uint32_t*>(q) + i);
  }
  return r;
}

// ... and their expansion (LSB-first bit-stream, as read_index8).
template <int BITS>
__device__ __forceinline__ void expand(const RawIdx<BITS>& r, uint32_t (&idx)[8]) {
  if constexpr (BITS == 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { idx[2 * i] = r.w[i] & 0xffffu; idx[2 * i + 1] = r.w[i] >> 16; }
  } else if constexpr (BITS == 8) {
#pragma unroll
    for (int i = 0; i < 8; ++i) idx[i] = (r.w[i >> 2] >> (8 * (i & 3))) & 0xffu;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int bit = i * BITS;
      const uint32_t lo = r.w[bit / 32];
      const uint32_t hi = (bit / 32 + 1 < BITS / 4) ? r.w[bit / 32 + 1] : 0u;
      const uint64_t two = ((uint64_t)hi << 32) | lo;
      idx[i] = (uint32_t)(two >> (bit % 32)) & ((1u << BITS) - 1u);
    }
  }
}

// Physical 16-byte chunk of logical chunk c (= vector index inside the K slice) in a row of
// the activation tile: lanes t = 0..3 of a quad read chunks 8 t + s, which this spreads over
// four different bank groups.
__device__ __forceinline__ int xchunk(int c) { return c ^ ((c >> 3) & 3); }

template <typename T, int BITS, int MT, int WARPS, bool CBS>
__global__ void __launch_bounds__(WARPS * 32, 1) vq_gemv_mma_kernel(MmaVqArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.K;
  // x tile: [MT * 8 rows][K] of T, row stride K * 2 + 64 bytes (rows g and g + 1 of a quarter-warp
  // pass then fall into different halves of the banks); chunks swizzled per 32-vector slice.
  const int xstride = K * (int)sizeof(T) + 64;
  uint8_t* xs = smem;
  float* part = reinterpret_cast<float*>(smem + (size_t)MT * 8 * xstride);  // [2][WARPS][MT][32][4]
  uint4* rtab = reinterpret_cast<uint4*>(part + 2 * WARPS * MT * 128);      // residual table x 8
  // CBS: the whole codebook (all column blocks) staged in shared memory -- a gather from there
  // costs a bank-conflicted LDS instead of one L1 tag lookup per lane (1 per clock per SM)
  const uint4* cbs = rtab + (a.has_res ? a.res_num_centroids * 8 : 0);

  const int n_groups = a.n_segs > 1 ? a.total_groups : (a.N + 15) / 16;
  const int chunks_per_row = a.G >> 3;  // 8-index chunks per W row
  // Weight that owns row group rg: its index stream, codebook, row count and first group.
  struct SegView { const uint8_t* packed; const __half* centroids; const float* bias; int N, group0, col0; };
  auto seg_of = [&](int rg_) -> SegView {
    if (a.n_segs <= 1) return SegView{a.packed, a.centroids, a.bias, a.N, 0, 0};
    int s_ = 0;
#pragma unroll
    for (int i = 1; i < kMaxSegs; ++i)
      if (i < a.n_segs && rg_ >= a.seg[i].group0) s_ = i;
    return SegView{a.seg[s_].packed, a.seg[s_].centroids, a.seg[s_].bias, a.seg[s_].N, a.seg[s_].group0,
                   a.seg[s_].col0};
  };
  const bool has_res = a.has_res != 0, has_scale = a.has_scale != 0;
  // Index words of one (row group, slice) item for this lane's two rows; the next item's are
  // requested before the current item's gathers, so their latency is off the critical path.
  // The row scales of a row group travel with its first slice, unconverted: converting them where
  // they are loaded would make the warp wait for the load at the start of every row group.
  struct Item { RawIdx<BITS> lo, hi; RawIdx<8> rlo, rhi; unsigned short s_lo, s_hi; };
  auto fetch = [&](Item& it, int rg_, int sl_) {
    const SegView sv = seg_of(rg_);
    const int nl = (rg_ - sv.group0) * 16 + g, nh = nl + 8;
    const int rl = nl < sv.N ? nl : sv.N - 1, rh = nh < sv.N ? nh : sv.N - 1;  // rows past N: row N-1
    const int c0 = (warp * a.slices_per_warp + sl_) * 4 + t;               // chunk of 8 indices in the row
    it.lo = load_raw<BITS>(sv.packed, (int64_t)rl * chunks_per_row + c0);
    it.hi = load_raw<BITS>(sv.packed, (int64_t)rh * chunks_per_row + c0);
    if (has_res) {
      it.rlo = load_raw<8>(a.res_packed, (int64_t)rl * chunks_per_row + c0);
      it.rhi = load_raw<8>(a.res_packed, (int64_t)rh * chunks_per_row + c0);
    } else {
      it.rlo.w[0] = it.rlo.w[1] = it.rhi.w[0] = it.rhi.w[1] = 0u;
    }
    if (has_scale && sl_ == 0) {
      const unsigned short* rs = reinterpret_cast<const unsigned short*>(a.row_scale);
      it.s_lo = __ldg(rs + rl);
      it.s_hi = __ldg(rs + rh);
    }
  };
  // The first item's index words are requested before the activations are staged: their latency
  // runs under the staging instead of after it.
  Item nxt;
  if ((int)blockIdx.x < n_groups) fetch(nxt, blockIdx.x, 0);

  // ---- stage activations (zero rows past M) and the replicated residual table ----
  {
    const T* x = static_cast<const T*>(a.x);
    const int chunks = K / 8;
    float* inv_rms = part;  // [MT * 8], reused as the partial-sum area after the barrier below
    if (a.norm_w != nullptr) {
      for (int m = warp; m < a.M; m += WARPS) {  // one warp per activation row
        float ss = 0.f;
        for (int c = lane; c < chunks; c += 32) {
          const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)m * K + c * 8);
          const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
          for (int j = 0; j < 8; ++j) { const float f = to_f32(e[j]); ss = fmaf(f, f, ss); }
        }
        ss = warp_sum(ss);
        if (lane == 0) inv_rms[m] = rsqrtf(ss / (float)K + a.norm_eps);
      }
      __syncthreads();
    }
    for (int i = tid; i < MT * 8 * chunks; i += WARPS * 32) {
      const int m = i / chunks, c = i - m * chunks;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < a.M) {
        v = *reinterpret_cast<const uint4*>(x + (size_t)m * K + c * 8);
        if (a.norm_w != nullptr) {
          const uint4 wv = *reinterpret_cast<const uint4*>(static_cast<const T*>(a.norm_w) + c * 8);
          const T* e = reinterpret_cast<const T*>(&v);
          const T* we = reinterpret_cast<const T*>(&wv);
          struct alignas(16) Out { T o[8]; } r;
          const float inv = inv_rms[m];
#pragma unroll
          for (int j = 0; j < 8; ++j) r.o[j] = from_f32<T>(to_f32(e[j]) * inv * to_f32(we[j]));
          v = *reinterpret_cast<const uint4*>(&r);
        }
      }
      const int phys = (c & ~31) | xchunk(c & 31);
      *reinterpret_cast<uint4*>(xs + (size_t)m * xstride + phys * 16) = v;
    }
    if (a.has_res) {
      // entry e at slots 8 e .. 8 e + 7; a lane reads slot 8 e + (lane & 7): conflict-free
      for (int i = tid; i < a.res_num_centroids * 8; i += WARPS * 32)
        rtab[i] = __ldg(reinterpret_cast<const uint4*>(a.res_centroids) + (i >> 3));
    }
    if constexpr (CBS) {
      uint4* dst = const_cast<uint4*>(cbs);
      for (int i = tid; i < a.cb_entries; i += WARPS * 32)
        dst[i] = __ldg(reinterpret_cast<const uint4*>(a.centroids) + i);
    }
  }
  __syncthreads();

  int buf = 0;
  for (int rg = blockIdx.x; rg < n_groups; rg += gridDim.x, buf ^= 1) {
    const SegView sv = seg_of(rg);
    __half2 s_lo = __float2half2_rn(1.f), s_hi = s_lo;
    if (has_scale) {   // loaded with the first slice's index words (nxt holds slice 0 of this row group here)
      s_lo = __half2half2(__ushort_as_half(nxt.s_lo));
      s_hi = __half2half2(__ushort_as_half(nxt.s_hi));
    }
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;

    for (int sl = 0; sl < a.slices_per_warp; ++sl) {
      const int slice = warp * a.slices_per_warp + sl;  // 32 vectors = 256 k
      const Item cur = nxt;
      if (sl + 1 < a.slices_per_warp) fetch(nxt, rg, sl + 1);
      else if (rg + (int)gridDim.x < n_groups) fetch(nxt, rg + gridDim.x, 0);
      uint32_t idx_lo[8], idx_hi[8], rdx_lo[8], rdx_hi[8];
      expand<BITS>(cur.lo, idx_lo);
      expand<BITS>(cur.hi, idx_hi);
      expand<8>(cur.rlo, rdx_lo);
      expand<8>(cur.rhi, rdx_hi);
      if (a.groups_per_codebook > 0) {  // a multiple of 32 vectors: constant over the slice
        const uint32_t off = (uint32_t)((slice * 32) / a.groups_per_codebook) * (uint32_t)a.num_centroids;
#pragma unroll
        for (int s = 0; s < 8; ++s) { idx_lo[s] += off; idx_hi[s] += off; }
      }
      const uint8_t* xrow = xs + (size_t)g * xstride + (size_t)slice * 512;
#pragma unroll
      for (int h = 0; h < 2; ++h) {  // two batches of four vectors per row: 8 gathers in flight
        Half8 c_lo[4], c_hi[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if constexpr (CBS) {
            c_lo[j] = *reinterpret_cast<const Half8*>(cbs + idx_lo[4 * h + j]);
            c_hi[j] = *reinterpret_cast<const Half8*>(cbs + idx_hi[4 * h + j]);
          } else {
            c_lo[j] = ldg_vec(reinterpret_cast<const Half8*>(sv.centroids) + idx_lo[4 * h + j]);
            c_hi[j] = ldg_vec(reinterpret_cast<const Half8*>(sv.centroids) + idx_hi[4 * h + j]);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int s = 4 * h + j;
          __half2 w_lo[4], w_hi[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) { w_lo[i] = c_lo[j].h[i]; w_hi[i] = c_hi[j].h[i]; }
          if (has_res) {
            const Half8 q_lo = *reinterpret_cast<const Half8*>(&rtab[(rdx_lo[s] << 3) + (lane & 7)]);
            const Half8 q_hi = *reinterpret_cast<const Half8*>(&rtab[(rdx_hi[s] << 3) + (lane & 7)]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              w_lo[i] = __hadd2_rn(w_lo[i], q_lo.h[i]);
              w_hi[i] = __hadd2_rn(w_hi[i], q_hi.h[i]);
            }
          }
          if (has_scale) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              w_lo[i] = __hmul2_rn(w_lo[i], s_lo);
              w_hi[i] = __hmul2_rn(w_hi[i], s_hi);
            }
          }
          // elements 0..3 of the two vectors -> first mma, 4..7 -> second
          const uint32_t a0[4] = {to_operand<T>(w_lo[0]), to_operand<T>(w_hi[0]), to_operand<T>(w_lo[1]),
                                  to_operand<T>(w_hi[1])};
          const uint32_t a1[4] = {to_operand<T>(w_lo[2]), to_operand<T>(w_hi[2]), to_operand<T>(w_lo[3]),
                                  to_operand<T>(w_hi[3])};
          const int phys = xchunk(8 * t + s);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xrow + (size_t)mt * 8 * xstride + phys * 16);
            mma16816<T>(acc[mt], a0, xv.x, xv.y);
            mma16816<T>(acc[mt], a1, xv.z, xv.w);
          }
        }
      }
    }

    // ---- sum the warps' partial tiles and store ----
    float* mine = part + ((size_t)buf * WARPS + warp) * MT * 128;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
      *reinterpret_cast<float4*>(mine + mt * 128 + lane * 4) =
          make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
    __syncthreads();
    for (int i = tid; i < MT * 128; i += WARPS * 32) {  // a 4-warp CTA has fewer threads than outputs
      float sum = 0.f;
      const float* p = part + (size_t)buf * WARPS * MT * 128 + i;
#pragma unroll 4
      for (int w = 0; w < WARPS; ++w) sum += p[(size_t)w * MT * 128];
      const int mt = i >> 7, ln = (i >> 2) & 31, c = i & 3;
      const int n = (rg - sv.group0) * 16 + (ln >> 2) + 8 * (c >> 1);
      const int m = mt * 8 + 2 * (ln & 3) + (c & 1);
      if (n < sv.N && m < a.M) {
        if (sv.bias) sum += __ldg(sv.bias + n);
        if (a.sink.peer_out == nullptr)
          static_cast<T*>(a.y)[(size_t)m * a.ld_y + sv.col0 + n] = from_f32<T>(sum);
        else
          static_cast<T*>(a.sink.peer_out[a.sink.rank])[(size_t)m * a.sink.ld + a.sink.col0 + n] =
              from_f32<T>(sum);
      }
    }
    // No second barrier: the next group writes the other half of `part`, and the barrier of
    // that group orders this group's reads before the writes of the group after it.
  }
  if (a.sink.peer_out != nullptr) gather_tail_small<T>(a.sink, a.M, a.N);
}

template <typename T, int BITS, int MT, int WARPS, bool CBS>
int launch_cb(const MmaVqArgs& a, size_t smem, cudaStream_t st) {
  auto kern = vq_gemv_mma_kernel<T, BITS, MT, WARPS, CBS>;
  int per_sm = 0;
  if (int rc = blocks_per_sm(reinterpret_cast<const void*>(kern), WARPS * 32, smem, &per_sm)) return rc;
  if (per_sm < 1) return NPB_ERR_UNSUPPORTED;
  const int n_groups = a.n_segs > 1 ? a.total_groups : (a.N + 15) / 16;
  const int cap = sm_count() * per_sm;
  kern<<<n_groups < cap ? n_groups : cap, WARPS * 32, smem, st>>>(a);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

template <typename T, int BITS, int MT, int WARPS>
int launch(const MmaVqArgs& a, cudaStream_t st) {
  const size_t xbytes = (size_t)MT * 8 * ((size_t)a.K * sizeof(T) + 64);
  const size_t smem = xbytes + (size_t)2 * WARPS * MT * 128 * 4 + (a.has_res ? 256 * 8 * 16 : 0);
  const size_t cap = (size_t)max_dynamic_smem();
  if (smem > cap) return NPB_ERR_UNSUPPORTED;
  // Codebook in shared memory when it fits beside the activations and every CTA gathers several
  // times more vectors than the staging copies (one weight only: each has its own codebook).
  const size_t cb_bytes = (size_t)a.cb_entries * 16;
  const int n_groups = (a.N + 15) / 16;
  const int64_t ctas = n_groups < sm_count() ? n_groups : sm_count();
  const int64_t gathers_per_cta = (int64_t)(n_groups + ctas - 1) / ctas * 16 * a.G;
  if (a.n_segs <= 1 && a.cb_entries > 0 && smem + cb_bytes <= cap && gathers_per_cta >= 3 * (int64_t)a.cb_entries)
    return launch_cb<T, BITS, MT, WARPS, true>(a, smem + cb_bytes, st);
  return launch_cb<T, BITS, MT, WARPS, false>(a, smem, st);
}

template <typename T, int BITS, int MT>
int launch_warps(MmaVqArgs a, cudaStream_t st) {
  const int slices = a.K / 256;
  if (slices % 16 == 0) { a.slices_per_warp = slices / 16; return launch<T, BITS, MT, 16>(a, st); }
  if (slices % 8 == 0) { a.slices_per_warp = slices / 8; return launch<T, BITS, MT, 8>(a, st); }
  if (slices % 4 == 0) { a.slices_per_warp = slices / 4; return launch<T, BITS, MT, 4>(a, st); }
  return NPB_ERR_UNSUPPORTED;
}

template <typename T, int BITS>
int launch_mt(const MmaVqArgs& a, cudaStream_t st) {
  return a.M <= 8 ? launch_warps<T, BITS, 1>(a, st) : launch_warps<T, BITS, 2>(a, st);
}

template <typename T>
int launch_bits(const MmaVqArgs& a, int bits, cudaStream_t st) {
  switch (bits) {
    case 16: return launch_mt<T, 16>(a, st);
    case 12: return launch_mt<T, 12>(a, st);
    case 8: return launch_mt<T, 8>(a, st);
    default: return NPB_ERR_UNSUPPORTED;
  }
}

}  // namespace

// Returns NPB_ERR_UNSUPPORTED when the weight form / shape is not one this kernel takes; the
// caller then uses the CUDA-core GEMV (up to 8 rows) or decode + dense GEMM.
int vq_gemv_mma(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M, int64_t N, int64_t K,
                const float* bias, void* y, const GatherSink* sink, cudaStream_t st) {
  if (int rc = validate_vq(w, N, K)) return rc;
  if (x_dtype != NPB_BF16 && x_dtype != NPB_F16) return NPB_ERR_UNSUPPORTED;
  if (M < 1 || M > 16 || N < 1 || N >= (int64_t)1 << 31 || K % 1024 != 0 || K > 16384) return NPB_ERR_UNSUPPORTED;
  if (x == nullptr || (y == nullptr && sink == nullptr)) return NPB_ERR_INVALID_ARG;
  if (w->vector_len != 8 || (w->bits != 16 && w->bits != 12 && w->bits != 8)) return NPB_ERR_UNSUPPORTED;
  if (!aligned_to(w->packed, index8_alignment(w->bits)) || !aligned_to(w->centroids, 16) || !aligned_to(x, 16))
    return NPB_ERR_UNSUPPORTED;
  if (w->res_packed && (w->res_bits != 8 || w->res_num_centroids > 256 || !aligned_to(w->res_packed, 8) ||
                        !aligned_to(w->res_centroids, 16)))
    return NPB_ERR_UNSUPPORTED;
  const int gpc = w->cols_per_codebook > 0 ? w->cols_per_codebook / 8 : 0;
  if (gpc % 32 != 0) return NPB_ERR_UNSUPPORTED;
  MmaVqArgs a{};
  a.packed = w->packed;
  a.centroids = static_cast<const __half*>(w->centroids);
  a.has_res = w->res_packed != nullptr;
  a.has_scale = w->row_scale != nullptr;
  a.res_packed = a.has_res ? w->res_packed : w->packed;
  a.res_centroids = a.has_res ? static_cast<const __half*>(w->res_centroids) : a.centroids;
  a.row_scale = a.has_scale ? static_cast<const __half*>(w->row_scale) : a.centroids;
  a.bias = bias;
  a.x = x;
  a.y = y;
  a.num_centroids = w->num_centroids;
  a.res_num_centroids = a.has_res ? w->res_num_centroids : 0;
  a.groups_per_codebook = gpc;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.G = (int)(K / 8);
  a.n_segs = 1;
  a.ld_y = (int)N;
  a.cb_entries = w->num_centroids * (w->cols_per_codebook > 0
                                         ? (int)((K + w->cols_per_codebook - 1) / w->cols_per_codebook) : 1);
  if (sink) a.sink = *sink;
  return x_dtype == NPB_BF16 ? launch_bits<__nv_bfloat16>(a, w->bits, st)
                             : launch_bits<__half>(a, w->bits, st);
}

// Grouped launch: n_w weights of the same K / index width / codebook layout applied to the same
// activations in ONE kernel; y is [M, sum of N_i] with weight i at columns [sum_{j<i} N_j, +N_i).
// Optionally the activations are RMS-normalised while they are staged (norm_w != null).  Plain
// weights only (no residual codebook, no row scale); NPB_ERR_UNSUPPORTED for anything the
// tensor-core small-batch kernel does not take.
int vq_gemv_grouped(const npb_vq_weight* ws, int n_w, const int64_t* Ns, const float* const* biases,
                    const void* x, int x_dtype, int64_t M, int64_t K, const void* norm_w, float norm_eps,
                    void* y, cudaStream_t st) {
  if (ws == nullptr || Ns == nullptr || n_w < 1 || n_w > kMaxSegs) return NPB_ERR_INVALID_ARG;
  if (x_dtype != NPB_BF16 && x_dtype != NPB_F16) return NPB_ERR_UNSUPPORTED;
  if (M < 1 || M > 16 || K % 1024 != 0 || K > 16384) return NPB_ERR_UNSUPPORTED;
  if (x == nullptr || y == nullptr) return NPB_ERR_INVALID_ARG;
  if (!aligned_to(x, 16) || (norm_w && !aligned_to(norm_w, 16))) return NPB_ERR_UNSUPPORTED;
  MmaVqArgs a{};
  int64_t total_n = 0, groups = 0;
  for (int i = 0; i < n_w; ++i) {
    const npb_vq_weight* w = ws + i;
    if (int rc = validate_vq(w, Ns[i], K)) return rc;
    if (Ns[i] < 1) return NPB_ERR_INVALID_ARG;
    if (w->vector_len != 8 || w->bits != ws[0].bits || (w->bits != 16 && w->bits != 12 && w->bits != 8))
      return NPB_ERR_UNSUPPORTED;
    if (w->res_packed != nullptr || w->row_scale != nullptr) return NPB_ERR_UNSUPPORTED;
    if (w->cols_per_codebook != ws[0].cols_per_codebook || w->num_centroids != ws[0].num_centroids)
      return NPB_ERR_UNSUPPORTED;
    if (!aligned_to(w->packed, index8_alignment(w->bits)) || !aligned_to(w->centroids, 16)) return NPB_ERR_UNSUPPORTED;
    a.seg[i].packed = w->packed;
    a.seg[i].centroids = static_cast<const __half*>(w->centroids);
    a.seg[i].bias = biases ? biases[i] : nullptr;
    a.seg[i].N = (int)Ns[i];
    a.seg[i].group0 = (int)groups;
    a.seg[i].col0 = (int)total_n;
    groups += (Ns[i] + 15) / 16;
    total_n += Ns[i];
  }
  if (total_n >= (int64_t)1 << 31) return NPB_ERR_UNSUPPORTED;
  const int gpc = ws[0].cols_per_codebook > 0 ? ws[0].cols_per_codebook / 8 : 0;
  if (gpc % 32 != 0) return NPB_ERR_UNSUPPORTED;
  // single-weight fields: alias the first weight so that every pointer the kernel can form is mapped
  a.packed = ws[0].packed;
  a.centroids = a.seg[0].centroids;
  a.res_packed = a.packed;
  a.res_centroids = a.centroids;
  a.row_scale = a.centroids;
  a.bias = nullptr;
  a.x = x;
  a.y = y;
  a.num_centroids = ws[0].num_centroids;
  a.groups_per_codebook = gpc;
  a.M = (int)M; a.N = (int)Ns[0]; a.K = (int)K; a.G = (int)(K / 8);
  a.n_segs = n_w == 1 ? 1 : n_w;
  if (n_w == 1) { a.bias = a.seg[0].bias; }
  a.ld_y = (int)total_n;
  a.total_groups = (int)groups;
  a.norm_w = norm_w;
  a.norm_eps = norm_eps;
  return x_dtype == NPB_BF16 ? launch_bits<__nv_bfloat16>(a, ws[0].bits, st)
                             : launch_bits<__half>(a, ws[0].bits, st);
}

}  // namespace npb
