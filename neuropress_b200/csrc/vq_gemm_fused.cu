// Tile-decode tensor-core GEMM for vector-quantized weights (the mid-batch band, 17..384 rows):
//
//   y[M, N] = x[M, K] . W[N, K]^T (+ bias),  W decoded on the fly from the packed index stream
//   and the codebook(s) straight into the 128B-swizzled shared-memory operand of tcgen05.mma;
//   the dense weight never exists in HBM.
//
// With at most 384 rows every weight tile is used by one CTA only, so the kernel is bound by the
// decode: one random 16-byte codebook gather per index (an L2 sector each for a 1 MiB codebook)
// plus the index stream from HBM.  The design therefore maximises gathers in flight:
//
//   * CTA tile 128*MT rows x BN columns x 64 k.  BN is a run-time multiple of 16 chosen so that
//     the tiles fill one wave of SMs as evenly as possible (e.g. 112 for N = 14336: 128 CTAs).
//   * warp 0: TMA producer of the x tiles (cp.async.bulk.tensor.2d, no multicast); warp 1: TMEM
//     owner and single-thread tcgen05.mma issuer; warps 2-5: epilogue (tcgen05.ld -> bias -> T
//     -> global); warps 6..: decode warps in GROUPS of four.  Group g serves ring stage g only,
//     i.e. the CTA's (tile, k block) items g, g + GROUPS, ... -- consecutive phases of that
//     stage's barriers -- and its four warps split the BN rows of the W tile between them.
//     All stages are therefore decoded concurrently, and every lane keeps eight gathers in
//     flight while the index words of its NEXT item are already on their way.
//   * One 16-byte centroid (vector length 8) is exactly one swizzle chunk: a decoded vector is a
//     single st.shared.v4 at chunk (c ^ (row & 7)) of its 128-byte row.
//   * Residual codebook (<= 256 entries) staged in shared memory; row scale in a register.
//
// Copy form (plain weights: no residual, no row scale).  A decoded vector of such a weight is the
// codebook entry itself, cast to the activation type -- a pure function of the entry.  Given the
// codebook already in the activation type (npb_vq_codebook_cast; the fp16 codebook itself for
// fp16 activations), decoding a vector is a 16-byte copy from the table to its swizzle chunk,
// and the decode warps issue it as cp.async (global -> shared, no register destination) with
// cp.async.mbarrier.arrive on the stage's full barrier: nothing in the decode warps ever waits
// for a gather, and the number of gathers in flight is bounded by the ring (stages x BN x 8),
// not by registers.
//
// Weights are rounded exactly as the one-pass decode rounds them (fp16 add / multiply, one
// rounding to the activation type), so this band and decode + dense GEMM differ only in the
// order of the fp32 accumulation.  Every mbarrier wait is bounded (see tcgen05.cuh).
//
// Replaces the Triton tile-decode GEMM (neuropress/kernels/vq_triton.py:37-116, called from
// neuropress/nn/np_vq_linear.py:1097-1125) and the wmma GEMM branch of vq_linear_wmma
// (neuropress/kernels/vq_linear_wmma.cu:261-394).
#include <type_traits>

#include "common.cuh"
#include "tcgen05.cuh"

namespace npb {

__device__ int g_vq_fused_status = 0;  // 0 ok; 1..4: the role whose bounded wait gave up

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kAStageBytes = BM * BK * 2;
constexpr int kDecodeWarps = 16;
constexpr int kMaxGroups = kDecodeWarps;            // decode groups = ring stages (1, 2 or 4 warps each)
constexpr int kThreads = 192 + 32 * kDecodeWarps + 32;   // 736: the last warp is the second mma issuer
constexpr int kBarrierBytes = 1024;
constexpr int kResTableBytes = 256 * 16;

// Grouped launch: up to four plain weights that share the activations (q / k / v, gate / up) are the
// row segments of one tall W; a tile never straddles two segments.
constexpr int kMaxSegs = 4;
struct Seg {
  const uint8_t* packed;   // the segment's index stream
  const void* cb_x;        // its codebook in the activation type (copy form), else null
  const __half* centroids; // its fp16 codebook
  const float* bias;       // or null
  int N;                   // its output features
  int tile0;               // first N-tile of the segment
  int col0;                // its first output column
};

struct FusedParams {
  const uint8_t* packed;
  int64_t packed_bytes;
  const __half* centroids;
  const void* cb_x;              // copy form: the codebook in the activation type, else null
  const uint8_t* res_packed;     // never null: aliases `packed` when there is no residual
  int64_t res_bytes;
  const __half* res_centroids;   // never null: aliases `centroids`
  const __half* row_scale;       // never null: aliases `centroids`
  const float* bias;
  void* y;
  uint64_t wait_ns;
  int bits, res_bits, num_centroids, groups_per_codebook, cb_rows, res_rows;
  int has_res, has_scale;
  int clamp;                     // copy form: indices can exceed the codebook (NC < 2^bits) or take an offset
  int M, N, K, BN, tiles_m, tiles_n, groups, warps_per_group;
  int dual;                      // two mma-issuing threads, one accumulator each (narrow tiles)
  int n_segs, ld_y;              // segments of a grouped launch (1: the plain call) and the row pitch of y
  Seg seg[kMaxSegs];
};

__device__ __forceinline__ const Seg& seg_of(const FusedParams& p, int tn) {
  int s = 0;
#pragma unroll
  for (int i = 1; i < kMaxSegs; ++i)
    if (i < p.n_segs && tn >= p.seg[i].tile0) s = i;
  return p.seg[s];
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// fp16 x 8 -> eight values of T, same rounding as from_half<T>
template <typename T>
__device__ __forceinline__ uint4 pack_half8(const __half2 (&h)[4]) {
  uint4 o;
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    __nv_bfloat162 b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      b[i] = __floats2bfloat162_rn(f.x, f.y);
    }
    o.x = *reinterpret_cast<const uint32_t*>(&b[0]);
    o.y = *reinterpret_cast<const uint32_t*>(&b[1]);
    o.z = *reinterpret_cast<const uint32_t*>(&b[2]);
    o.w = *reinterpret_cast<const uint32_t*>(&b[3]);
  } else {
    o.x = *reinterpret_cast<const uint32_t*>(&h[0]);
    o.y = *reinterpret_cast<const uint32_t*>(&h[1]);
    o.z = *reinterpret_cast<const uint32_t*>(&h[2]);
    o.w = *reinterpret_cast<const uint32_t*>(&h[3]);
  }
  return o;
}

// Raw words of the eight indices of one (row, k block): fetched one item ahead of their use.
template <int BITS>
struct RawRow {
  uint32_t w[BITS == 0 ? 1 : BITS / 4];
  uint2 r;  // eight 8-bit residual indices
};

template <int BITS>
__device__ __forceinline__ void fetch_row(RawRow<BITS>& it, const FusedParams& p, const uint8_t* packed, int n,
                                          int kb) {
  if constexpr (BITS != 0) {
    const int64_t chunk = (int64_t)n * (p.K >> 6) + kb;  // 8-index chunks per row = K / 64
    const uint8_t* q = packed + chunk * BITS;
    if constexpr (BITS == 16) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(q));
      it.w[0] = v.x; it.w[1] = v.y; it.w[2] = v.z; it.w[3] = v.w;
    } else if constexpr (BITS == 8) {
      const uint2 v = __ldg(reinterpret_cast<const uint2*>(q));
      it.w[0] = v.x; it.w[1] = v.y;
    } else {
#pragma unroll
      for (int i = 0; i < BITS / 4; ++i) it.w[i] = __ldg(reinterpret_cast<const uint32_t*>(q) + i);
    }
    it.r = p.has_res ? __ldg(reinterpret_cast<const uint2*>(p.res_packed + chunk * 8)) : make_uint2(0u, 0u);
  }
}

template <int BITS>
__device__ __forceinline__ void expand_row(const RawRow<BITS>& it, uint32_t (&idx)[8]) {
  if constexpr (BITS == 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { idx[2 * i] = it.w[i] & 0xffffu; idx[2 * i + 1] = it.w[i] >> 16; }
  } else if constexpr (BITS == 8) {
#pragma unroll
    for (int i = 0; i < 8; ++i) idx[i] = (it.w[i >> 2] >> (8 * (i & 3))) & 0xffu;
  } else if constexpr (BITS != 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int bit = i * BITS;
      const uint32_t lo = it.w[bit / 32];
      const uint32_t hi = (bit / 32 + 1 < BITS / 4) ? it.w[bit / 32 + 1] : 0u;
      idx[i] = (uint32_t)((((uint64_t)hi << 32) | lo) >> (bit % 32)) & ((1u << BITS) - 1u);
    }
  }
}

// Decode the 64-wide k block `kb` of W row n into tile row `row` of the stage at `b_stage`.
template <typename T, int BITS>
__device__ __forceinline__ void emit_row(const RawRow<BITS>& it, const FusedParams& p, int n, int kb,
                                         uint32_t b_stage, int row, const uint4* res_tab) {
  const uint32_t row_addr = b_stage + row * 128;
  const int sw = row & 7;
  if (n >= p.N) {  // rows past N: zeros (their columns are never stored)
    const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int c = 0; c < 8; ++c) st_shared_v4(row_addr + ((c ^ sw) << 4), z);
    return;
  }
  uint32_t idx[8], ridx[8];
  if constexpr (BITS != 0) {
    expand_row<BITS>(it, idx);
#pragma unroll
    for (int i = 0; i < 8; ++i) ridx[i] = ((i < 4 ? it.r.x : it.r.y) >> (8 * (i & 3))) & 0xffu;
  } else {
    const int64_t v0 = (int64_t)n * (p.K >> 3) + kb * 8;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      idx[c] = read_index_generic(p.packed, p.packed_bytes, v0 + c, p.bits);
      ridx[c] = p.has_res ? read_index_generic(p.res_packed, p.res_bytes, v0 + c, p.res_bits) : 0u;
    }
  }
  const uint32_t off = p.groups_per_codebook > 0
                           ? (uint32_t)((kb * 8) / p.groups_per_codebook) * (uint32_t)p.num_centroids : 0u;
  const uint32_t last = (uint32_t)p.cb_rows - 1u;
  Half8 cv[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t e = min(idx[c] + off, last);  // an index past the codebook reads its last entry
    cv[c] = ldg_vec(reinterpret_cast<const Half8*>(p.centroids) + e);
  }
  __half2 s2 = __float2half2_rn(1.f);
  if (p.has_scale) s2 = __half2half2(__ldg(p.row_scale + n));
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    __half2 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = cv[c].h[i];
    if (p.has_res) {
      const uint4 rv = res_tab[min(ridx[c], (uint32_t)p.res_rows - 1u)];
      const __half2* r = reinterpret_cast<const __half2*>(&rv);
#pragma unroll
      for (int i = 0; i < 4; ++i) h[i] = __hadd2_rn(h[i], r[i]);
    }
    if (p.has_scale) {
#pragma unroll
      for (int i = 0; i < 4; ++i) h[i] = __hmul2_rn(h[i], s2);
    }
    st_shared_v4(row_addr + ((c ^ sw) << 4), pack_half8<T>(h));
  }
}

// 16-byte asynchronous copy global -> shared through L2 only; src_bytes = 0 writes zeros.
__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(src), "r"(src_bytes) : "memory");
}
// The barrier gets one arrival from this thread once all its cp.async issued so far have landed
// (counted in the barrier's expected arrivals: .noinc).
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Copy form of emit_row: the eight vectors of (row n, k block kb) go from the activation-type
// codebook to their swizzle chunks as asynchronous copies.
template <int BITS>
__device__ __forceinline__ void emit_row_copy(const RawRow<BITS>& it, const FusedParams& p, const void* cb_x,
                                              bool valid, int kb, uint32_t b_stage, int row) {
  // chunk c of tile row `row` lives at (row * 128) + ((c ^ (row & 7)) << 4) = base ^ (c << 4)
  const uint32_t base = b_stage + row * 128 + ((row & 7) << 4);
  uint32_t idx[8];
  expand_row<BITS>(it, idx);
  if (p.clamp) {
    const uint32_t off = p.groups_per_codebook > 0
                             ? (uint32_t)((kb * 8) / p.groups_per_codebook) * (uint32_t)p.num_centroids : 0u;
    const uint32_t last = (uint32_t)p.cb_rows - 1u;
#pragma unroll
    for (int c = 0; c < 8; ++c) idx[c] = min(idx[c] + off, last);
  }
  const char* cb = static_cast<const char*>(cb_x);
  const uint32_t nbytes = valid ? 16u : 0u;  // rows past N: zeros (their columns are never stored)
#pragma unroll
  for (int c = 0; c < 8; ++c) cp_async_16(base ^ (uint32_t)(c << 4), cb + ((size_t)idx[c] << 4), nbytes);
}

template <typename T, int MT, int BITS, bool COPY>
__global__ void __launch_bounds__(kThreads, 1)
vq_gemm_fused_kernel(const __grid_constant__ CUtensorMap tmap_a, const FusedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);   // [groups]
  uint64_t* empty_bar = full_bar + kMaxGroups;              // [groups]
  uint64_t* tmem_full = empty_bar + kMaxGroups;             // [2]
  uint64_t* tmem_empty = tmem_full + 2;                     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint4* res_tab = reinterpret_cast<uint4*>(smem + kBarrierBytes);
  uint8_t* stage_base = smem + kBarrierBytes + kResTableBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BN = p.BN;
  const int stage_bytes = MT * kAStageBytes + BN * 128;
  const int G = p.groups;                 // ring stages = decode groups
  const int num_kb = p.K / BK;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int acc_cols = MT * BN;
  // Narrow tiles are bound by the rate at which ONE thread issues tcgen05.mma (four K = 16 instructions
  // and a commit per k block, ~70 cycles each).  In the dual form two threads of different warps issue
  // the even and the odd k blocks into accumulators of their own, which the epilogue adds; the stage
  // count is even, so a stage always belongs to the same issuer and each of its barriers sees one
  // waiter on consecutive phases.
  const int nacc = p.dual ? 2 : 1;
  const int nbuf = (2 * nacc * acc_cols <= 512) ? 2 : 1;
  int tmem_cols = 32;
  while (tmem_cols < nbuf * nacc * acc_cols) tmem_cols <<= 1;
  const uint32_t idesc = umma_idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, BM, BN);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < G; ++s) {
      // TMA producer's expect_tx arrive + one per decode warp (copy form: one per decode lane)
      mbar_init(&full_bar[s], 1 + (COPY ? 32 : 1) * p.warps_per_group);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], nacc);
      mbar_init(&tmem_empty[b], 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
  }
  if (p.has_res)
    for (int i = threadIdx.x; i < p.res_rows; i += kThreads)
      res_tab[i] = __ldg(reinterpret_cast<const uint4*>(p.res_centroids) + i);
  if (warp == 1) {
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ================= TMA producer (x tiles) =================
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int tm = t % p.tiles_m;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag, p.wait_ns, 64u)) {
            atomicExch(&g_vq_fused_status, 1);
            ok = false;
            break;
          }
          uint8_t* st = stage_base + (size_t)s * stage_bytes;
          mbar_arrive_expect_tx(&full_bar[s], MT * kAStageBytes);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            tma_load_2d(st + mt * kAStageBytes, &tmap_a, &full_bar[s], kb * BK, (tm * MT + mt) * BM);
          if (++s == G) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1 || (warp == kThreads / 32 - 1 && p.dual)) {
    // ================= MMA issuer(s): issuer j takes the k blocks j, j + nacc, ... of every tile =================
    if (lane == 0) {
      const int j0 = warp == 1 ? 0 : 1;
      // This issuer's items are j0, j0 + nacc, ... of the CTA's item list (in the dual form K / 64 is
      // even, so the list of every tile continues the stride): stage and phase advance without a division.
      int s = j0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int buf = (nbuf == 2) ? (it & 1) : 0;
        const uint32_t buf_ph = (nbuf == 2) ? ((it >> 1) & 1) : (it & 1);
        if (!mbar_wait_bounded(&tmem_empty[buf], buf_ph ^ 1, abort_flag, p.wait_ns)) {
          atomicExch(&g_vq_fused_status, 2);
          break;
        }
        tc_fence_after();
        const uint32_t acc = tmem_base + (buf * nacc + j0) * acc_cols;
        for (int kb = j0; kb < num_kb; kb += nacc) {
          if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag, p.wait_ns)) {
            atomicExch(&g_vq_fused_status, 2);
            ok = false;
            break;
          }
          tc_fence_after();
          if (COPY) fence_proxy_async_smem();  // the W tile was written by cp.async (generic proxy)
          const uint32_t st = smem_u32(stage_base + (size_t)s * stage_bytes);
          const uint64_t bdesc = umma_desc_sw128(st + MT * kAStageBytes);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint64_t adesc = umma_desc_sw128(st + mt * kAStageBytes);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_f16(acc + mt * BN, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > j0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
          s += nacc;
          if (s >= G) { s -= G; ph ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[buf]);
      }
    }
  } else if (warp < 6) {
    // ================= epilogue: TMEM -> registers -> global =================
    const int quad = warp & 3;
    T* y = static_cast<T*>(p.y);
    int it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
      const int tm = t % p.tiles_m, tn = t / p.tiles_m;
      const Seg& sg = seg_of(p, tn);            // the weight this tile belongs to
      const int seg_n0 = (tn - sg.tile0) * BN;  // the tile's first output feature inside it
      const int buf = (nbuf == 2) ? (it & 1) : 0;
      const uint32_t buf_ph = (nbuf == 2) ? ((it >> 1) & 1) : (it & 1);
      const bool got = mbar_wait_bounded(&tmem_full[buf], buf_ph, abort_flag, p.wait_ns, 256u);
      if (!__all_sync(0xffffffffu, got)) {
        atomicExch(&g_vq_fused_status, 3);
        break;
      }
      tc_fence_after();
      const uint32_t acc = tmem_base + buf * nacc * acc_cols + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        if ((tm * MT + mt) * BM >= p.M) break;  // whole sub-tile past M: skipped by all lanes together
        const int m = (tm * MT + mt) * BM + quad * 32 + lane;
#pragma unroll 1
        for (int c = 0; c < BN / 16; ++c) {
          uint32_t v[16];
          tmem_ld_32x32_x16(acc + mt * BN + c * 16, v);
          tmem_ld_wait();
          if (p.dual) {   // the odd k blocks' accumulator
            uint32_t w[16];
            tmem_ld_32x32_x16(acc + acc_cols + mt * BN + c * 16, w);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) + __uint_as_float(w[e]));
          }
          const int n0 = seg_n0 + c * 16;
          if (m < p.M && n0 < sg.N) {
            T* dst = y + (int64_t)m * p.ld_y + sg.col0 + n0;
            if (n0 + 16 <= sg.N && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
              struct alignas(16) Out { T e[8]; } o[2];
#pragma unroll
              for (int q = 0; q < 2; ++q)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  float f = __uint_as_float(v[q * 8 + e]);
                  if (sg.bias) f += __ldg(sg.bias + n0 + q * 8 + e);
                  o[q].e[e] = from_f32<T>(f);
                }
              reinterpret_cast<Out*>(dst)[0] = o[0];
              reinterpret_cast<Out*>(dst)[1] = o[1];
            } else {
#pragma unroll
              for (int e = 0; e < 16; ++e)
                if (n0 + e < sg.N) {
                  float f = __uint_as_float(v[e]);
                  if (sg.bias) f += __ldg(sg.bias + n0 + e);
                  dst[e] = from_f32<T>(f);
                }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
  } else {
    // ================= decode warps =================
    const int dw = warp - 6;
    const int wpg = p.warps_per_group;        // 1, 2 or 4 warps share a stage's BN rows
    const int grp = dw / wpg, part = dw - grp * wpg;
    if (dw < kDecodeWarps && grp < G) {
      const int rows_per_warp = BN / wpg;
      const int row0 = part * rows_per_warp;
      const int my_tiles = (int)blockIdx.x < num_tiles ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
      const int total = my_tiles * num_kb;    // the CTA's (tile, k block) items in ring order
      const uint32_t b_stage = smem_u32(stage_base + (size_t)grp * stage_bytes + MT * kAStageBytes);
      auto tile_tn = [&](int i) { return (int)((blockIdx.x + (i / num_kb) * gridDim.x) / p.tiles_m); };
      constexpr int RPL = 2;                  // rows per lane (second one only when BN > 128)
      const bool two = rows_per_warp > 32;
      RawRow<BITS> cur[RPL], nxt[RPL];
      auto fetch = [&](RawRow<BITS> (&dst)[RPL], int i) {
        const int tn = tile_tn(i), kb = i % num_kb;
        const Seg& sg = seg_of(p, tn);
        const int n0 = (tn - sg.tile0) * BN + row0;     // row inside the segment's weight
#pragma unroll
        for (int r = 0; r < RPL; ++r) {
          const int rr = lane + 32 * r;
          if (r == 0 ? rr < rows_per_warp : (two && rr < rows_per_warp)) {
            const int n = n0 + rr;
            fetch_row<BITS>(dst[r], p, sg.packed, n < sg.N ? n : sg.N - 1, kb);
          }
        }
      };
      if (grp < total) fetch(cur, grp);
      for (int i = grp; i < total; i += G) {
        if (i + G < total) fetch(nxt, i + G);
        const uint32_t ph = (uint32_t)(i / G) & 1u;
        const bool got = mbar_wait_bounded(&empty_bar[grp], ph ^ 1, abort_flag, p.wait_ns, 64u);
        if (!__all_sync(0xffffffffu, got)) {
          atomicExch(&g_vq_fused_status, 4);
          break;
        }
        const int tn = tile_tn(i), kb = i % num_kb;
        const Seg& sg = seg_of(p, tn);
        const int n0 = (tn - sg.tile0) * BN + row0;
        if constexpr (COPY && BITS != 0) {
#pragma unroll
          for (int r = 0; r < RPL; ++r) {
            const int rr = lane + 32 * r;
            if (r == 0 ? rr < rows_per_warp : (two && rr < rows_per_warp))
              emit_row_copy<BITS>(cur[r], p, sg.cb_x, n0 + rr < sg.N, kb, b_stage, row0 + rr);
          }
          cp_async_arrive(&full_bar[grp]);  // every lane, also one without rows
        } else {
#pragma unroll
          for (int r = 0; r < RPL; ++r) {
            const int rr = lane + 32 * r;
            if (r == 0 ? rr < rows_per_warp : (two && rr < rows_per_warp))
              emit_row<T, BITS>(cur[r], p, n0 + rr, kb, b_stage, row0 + rr, res_tab);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_bar[grp]);
        }
#pragma unroll
        for (int r = 0; r < RPL; ++r) cur[r] = nxt[r];
      }
    }
  }

  // ---- teardown: everyone meets here, also after an abort ----
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);  // let issued TMA copies land
  }
  if (COPY) asm volatile("cp.async.wait_all;" ::: "memory");  // none of this thread's copies outlives the CTA
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// out[i] = T(in[i]): the cast the decode applies to a plain weight's codebook entries.
template <typename T>
__global__ void codebook_cast_kernel(const __half* __restrict__ in, T* __restrict__ out, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_half<T>(in[i]);
}

// BN: a multiple of 16 in [16, 256] such that (waves of tiles) x BN -- the decode work of the
// busiest SM -- is smallest; ties go to the wider tile (fewer x-tile re-reads).
int pick_bn(const FusedParams& p, int tiles_m, int mt, int sms) {
  int best_bn = 128;
  double best = 1e30;
  for (int bn = 256; bn >= 16; bn -= 16) {
    if (mt * bn > 512) continue;  // one accumulator buffer must fit TMEM
    int64_t tiles_n = 0;
    for (int i = 0; i < p.n_segs; ++i) tiles_n += (p.seg[i].N + bn - 1) / bn;   // a tile stays inside a segment
    const int64_t tiles = (int64_t)tiles_m * tiles_n;
    const int64_t waves = (tiles + sms - 1) / sms;
    const double cost = (double)waves * bn;
    if (cost < best - 1e-9) { best = cost; best_bn = bn; }
  }
  return best_bn;
}

int make_tmap_x(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, bool bf16) {
  using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  if (fn == nullptr) {
    set_last_cuda_error(cudaErrorSymbolNotFound, "cuTensorMapEncodeTiled lookup");
    return NPB_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)BM};
  const cuuint32_t estr[2] = {1, 1};
  if (fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return NPB_ERR_CUDA;
  }
  return NPB_OK;
}

template <typename T, int MT, int BITS, bool COPY>
int launch(const void* x, FusedParams p, cudaStream_t st) {
  auto kern = vq_gemm_fused_kernel<T, MT, BITS, COPY>;
  const int sms = sm_count();
  p.tiles_m = (p.M + BM * MT - 1) / (BM * MT);
  p.BN = pick_bn(p, p.tiles_m, MT, sms);
  p.tiles_n = 0;
  for (int i = 0, col = 0; i < p.n_segs; ++i) {
    p.seg[i].tile0 = p.tiles_n;
    p.seg[i].col0 = col;
    p.tiles_n += (p.seg[i].N + p.BN - 1) / p.BN;
    col += p.seg[i].N;
  }
  const int stage_bytes = MT * kAStageBytes + p.BN * 128;
  const int cap = max_dynamic_smem();
  // Narrow tiles have few gathers per stage and are bound by the latency of one decode; they get
  // more, smaller groups (more stages decoded concurrently): a warp covers up to 64 rows.
  int wpg = 4;
  if (p.BN <= 32) wpg = 1;
  else if (p.BN <= 64) wpg = 2;
  if (p.BN % wpg != 0) wpg = 4;
  p.warps_per_group = wpg;
  int groups = (cap - kBarrierBytes - kResTableBytes - 1024) / stage_bytes;
  if (groups > kDecodeWarps / wpg) groups = kDecodeWarps / wpg;
  if (groups < 2) return NPB_ERR_UNSUPPORTED;
  // Dual issue for tiles of up to 32 columns with one row tile: from 64 columns on a k block's gathers
  // take as long as its mmas take to issue, and a second issuer only adds contention (8192 x 8192 at
  // 32 rows: 56 -> 63 us; 1024 x 8192: 45 -> 33 us).
  p.dual = (MT == 1 && p.BN <= 32 && (p.K / BK) % 2 == 0 && groups >= 4) ? 1 : 0;
  if (p.dual) groups &= ~1;
  p.groups = groups;
  const int smem = kBarrierBytes + kResTableBytes + 1024 + groups * stage_bytes;
  static int configured[64] = {0};
  int dev = 0;
  NPB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && configured[dev] < smem) {  // per instantiation and device, once
    NPB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cap));
    configured[dev] = cap;
  }
  CUtensorMap ta;
  if (int rc = make_tmap_x(&ta, x, p.M, p.K, std::is_same<T, __nv_bfloat16>::value)) return rc;
  p.wait_ns = wait_limit_ns();
  const int tiles = p.tiles_m * p.tiles_n;
  kern<<<tiles < sms ? tiles : sms, kThreads, smem, st>>>(ta, p);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

template <typename T, int BITS>
int launch_mt(const void* x, const FusedParams& p, cudaStream_t st) {
  if constexpr (BITS != 0) {
    if (p.cb_x != nullptr) {
      if (p.M <= 128) return launch<T, 1, BITS, true>(x, p, st);
      if (p.M <= 256) return launch<T, 2, BITS, true>(x, p, st);
      return launch<T, 3, BITS, true>(x, p, st);
    }
  }
  if (p.M <= 128) return launch<T, 1, BITS, false>(x, p, st);
  if (p.M <= 256) return launch<T, 2, BITS, false>(x, p, st);
  return launch<T, 3, BITS, false>(x, p, st);
}

template <typename T>
int launch_bits(const void* x, const FusedParams& p, int vbits, cudaStream_t st) {
  switch (vbits) {
    case 16: return launch_mt<T, 16>(x, p, st);
    case 12: return launch_mt<T, 12>(x, p, st);
    case 8: return launch_mt<T, 8>(x, p, st);
    default: return launch_mt<T, 0>(x, p, st);
  }
}

}  // namespace

// Reads and clears this kernel's give-up record (synchronises); merged into
// npb_gemm_device_status by gemm_tcgen05.cu.
int vq_gemm_fused_device_status(int* host_out) {
  int v = 0;
  NPB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_vq_fused_status, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    NPB_CUDA_TRY(cudaMemcpyToSymbol(g_vq_fused_status, &zero, sizeof(int)));
  }
  if (host_out) *host_out = v;
  return NPB_OK;
}

int vq_codebook_cast(const void* centroids, int64_t n_values, void* out, int out_dtype, cudaStream_t st) {
  if (n_values < 0) return NPB_ERR_INVALID_ARG;
  if (out_dtype != NPB_BF16 && out_dtype != NPB_F16) return NPB_ERR_UNSUPPORTED;
  if (n_values == 0) return NPB_OK;
  if (centroids == nullptr || out == nullptr) return NPB_ERR_INVALID_ARG;
  const unsigned blocks = (unsigned)((n_values + 255) / 256);
  const __half* in = static_cast<const __half*>(centroids);
  if (out_dtype == NPB_BF16)
    codebook_cast_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(in, static_cast<__nv_bfloat16*>(out), n_values);
  else
    codebook_cast_kernel<__half><<<blocks, 256, 0, st>>>(in, static_cast<__half*>(out), n_values);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

// codebook_x: null, or the codebook in the activation type (vq_codebook_cast) for the copy form.
int vq_gemm_fused(const npb_vq_weight* w, const void* codebook_x, const void* x, int x_dtype, int64_t M, int64_t N,
                  int64_t K, const float* bias, void* y, cudaStream_t st) {
  if (int rc = validate_vq(w, N, K)) return rc;
  if (M < 0) return NPB_ERR_INVALID_ARG;
  if (x_dtype != NPB_BF16 && x_dtype != NPB_F16) return NPB_ERR_UNSUPPORTED;
  if (M == 0 || N == 0) return NPB_OK;
  if (x == nullptr || y == nullptr) return NPB_ERR_INVALID_ARG;
  if (K == 0 || K % 8 != 0) return NPB_ERR_SHAPE;
  if (w->vector_len != 8 || K % 64 != 0) return NPB_ERR_UNSUPPORTED;
  if (M >= (int64_t)1 << 31 || N >= (int64_t)1 << 31 || K >= (int64_t)1 << 31) return NPB_ERR_UNSUPPORTED;
  if (!aligned_to(x, 16)) return NPB_ERR_ALIGNMENT;
  if (!aligned_to(w->centroids, 16) || (w->res_centroids && !aligned_to(w->res_centroids, 16)))
    return NPB_ERR_ALIGNMENT;
  if (w->res_packed && w->res_num_centroids > 256) return NPB_ERR_UNSUPPORTED;  // shared-memory table
  FusedParams p{};
  p.packed = w->packed;
  p.packed_bytes = w->packed_bytes;
  p.centroids = static_cast<const __half*>(w->centroids);
  p.has_res = w->res_packed != nullptr;
  p.has_scale = w->row_scale != nullptr;
  p.res_packed = p.has_res ? w->res_packed : w->packed;
  p.res_bytes = p.has_res ? w->res_packed_bytes : 0;
  p.res_centroids = p.has_res ? static_cast<const __half*>(w->res_centroids) : p.centroids;
  p.row_scale = p.has_scale ? static_cast<const __half*>(w->row_scale) : p.centroids;
  p.bias = bias;
  p.y = y;
  p.bits = w->bits;
  p.res_bits = p.has_res ? w->res_bits : 0;
  p.num_centroids = w->num_centroids;
  p.groups_per_codebook = w->cols_per_codebook > 0 ? w->cols_per_codebook / 8 : 0;
  p.cb_rows = w->num_centroids *
              (w->cols_per_codebook > 0 ? (int)((K + w->cols_per_codebook - 1) / w->cols_per_codebook) : 1);
  p.res_rows = p.has_res ? w->res_num_centroids : 1;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  // Wide index reads need whole 8-index chunks per k block of a row (K % 64 == 0 gives that),
  // an aligned stream, byte-wide residual indices and codebook groups of whole k blocks.
  int vbits = 0;
  if ((w->bits == 16 || w->bits == 12 || w->bits == 8) && aligned_to(w->packed, index8_alignment(w->bits)) &&
      (p.groups_per_codebook % 8 == 0) && (!p.has_res || (w->res_bits == 8 && aligned_to(w->res_packed, 8))))
    vbits = w->bits;
  if (vbits == 0 && p.groups_per_codebook % 8 != 0) return NPB_ERR_UNSUPPORTED;
  if (codebook_x != nullptr) {
    // the copy form covers plain weights with wide index reads; anything else is the caller's mistake
    if (p.has_res || p.has_scale || vbits == 0) return NPB_ERR_UNSUPPORTED;
    if (!aligned_to(codebook_x, 16)) return NPB_ERR_ALIGNMENT;
    p.cb_x = codebook_x;
    p.clamp = (w->num_centroids != (1 << w->bits)) || p.groups_per_codebook > 0;
  }
  p.n_segs = 1;
  p.ld_y = (int)N;
  p.seg[0] = Seg{p.packed, p.cb_x, p.centroids, bias, (int)N, 0, 0};
  return x_dtype == NPB_BF16 ? launch_bits<__nv_bfloat16>(x, p, vbits, st) : launch_bits<__half>(x, p, vbits, st);
}

// Several plain weights applied to the same x in one launch (copy form only): y is [M, sum of Ns], weight i's
// outputs in columns [sum of the Ns before it, + Ns[i]).  The weights must agree in index width, codebook size
// and codebook layout; each brings its own codebook in the activation type.
int vq_gemm_fused_grouped(const npb_vq_weight* ws, int n_weights, const void* const* codebooks_x, const int64_t* Ns,
                          const float* const* biases, const void* x, int x_dtype, int64_t M, int64_t K, void* y,
                          cudaStream_t st) {
  if (ws == nullptr || codebooks_x == nullptr || Ns == nullptr || n_weights < 1 || n_weights > kMaxSegs)
    return NPB_ERR_INVALID_ARG;
  if (M < 0) return NPB_ERR_INVALID_ARG;
  if (x_dtype != NPB_BF16 && x_dtype != NPB_F16) return NPB_ERR_UNSUPPORTED;
  if (K == 0 || K % 64 != 0 || K >= (int64_t)1 << 31 || M >= (int64_t)1 << 31) return NPB_ERR_UNSUPPORTED;
  const npb_vq_weight& w0 = ws[0];
  int64_t total_n = 0;
  for (int i = 0; i < n_weights; ++i) {
    const npb_vq_weight& w = ws[i];
    if (int rc = validate_vq(&w, Ns[i], K)) return rc;
    if (Ns[i] <= 0 || codebooks_x[i] == nullptr) return NPB_ERR_INVALID_ARG;
    if (w.vector_len != 8 || w.res_packed != nullptr || w.row_scale != nullptr) return NPB_ERR_UNSUPPORTED;
    if (w.bits != w0.bits || w.num_centroids != w0.num_centroids || w.cols_per_codebook != w0.cols_per_codebook)
      return NPB_ERR_UNSUPPORTED;
    if (w.bits != 16 && w.bits != 12 && w.bits != 8) return NPB_ERR_UNSUPPORTED;
    if (!aligned_to(w.packed, index8_alignment(w.bits)) || !aligned_to(codebooks_x[i], 16) ||
        !aligned_to(w.centroids, 16))
      return NPB_ERR_ALIGNMENT;
    total_n += Ns[i];
  }
  if (total_n >= (int64_t)1 << 31) return NPB_ERR_UNSUPPORTED;
  if (M == 0) return NPB_OK;
  if (x == nullptr || y == nullptr) return NPB_ERR_INVALID_ARG;
  if (!aligned_to(x, 16)) return NPB_ERR_ALIGNMENT;
  FusedParams p{};
  p.packed = w0.packed;
  p.packed_bytes = w0.packed_bytes;
  p.centroids = static_cast<const __half*>(w0.centroids);
  p.res_packed = w0.packed;
  p.res_centroids = p.centroids;
  p.row_scale = p.centroids;
  p.bias = biases ? biases[0] : nullptr;
  p.y = y;
  p.bits = w0.bits;
  p.num_centroids = w0.num_centroids;
  p.groups_per_codebook = w0.cols_per_codebook > 0 ? w0.cols_per_codebook / 8 : 0;
  if (p.groups_per_codebook % 8 != 0) return NPB_ERR_UNSUPPORTED;
  p.cb_rows = w0.num_centroids *
              (w0.cols_per_codebook > 0 ? (int)((K + w0.cols_per_codebook - 1) / w0.cols_per_codebook) : 1);
  p.res_rows = 1;
  p.M = (int)M; p.N = (int)total_n; p.K = (int)K;
  p.cb_x = codebooks_x[0];
  p.clamp = (w0.num_centroids != (1 << w0.bits)) || p.groups_per_codebook > 0;
  p.n_segs = n_weights;
  p.ld_y = (int)total_n;
  for (int i = 0; i < n_weights; ++i)
    p.seg[i] = Seg{ws[i].packed, codebooks_x[i], static_cast<const __half*>(ws[i].centroids),
                   biases ? biases[i] : nullptr, (int)Ns[i], 0, 0};
  return x_dtype == NPB_BF16 ? launch_bits<__nv_bfloat16>(x, p, w0.bits, st) : launch_bits<__half>(x, p, w0.bits, st);
}

}  // namespace npb
