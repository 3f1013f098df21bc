// Persistent warp-specialised tcgen05 GEMM  y[M,N] = x[M,K] . W[N,K]^T (+ bias)  for sm_100a,
// in two flavours selected at compile time by where the W tile comes from:
//
//   B_TMA : W is a dense [N,K] matrix in HBM (the large-batch band after the one-pass decode);
//           W tiles arrive by TMA like the x tiles.
//   B_Q4  : W tiles are dequantised from 4-bit group-affine codes by decode warps straight into
//           the 128B-swizzled shared-memory stage (the dense weight never exists in HBM).
//
// (The tile-decode GEMM for vector-quantized weights is a kernel of its own: vq_gemm_fused.cu.)
//
// CTA = 128 x (MT*128 rows) x BN tile, K step 64.  Warp roles: warp 0 TMA producer, warp 1
// TMEM owner + single-thread tcgen05.mma issuer, warps 2-5 epilogue (tcgen05.ld -> bias ->
// T -> global), warps 6.. (fused mode) B decoders.  smem ring of STAGES stages guarded by
// full/empty mbarriers; accumulators live in TMEM (MT*BN fp32 columns per buffer, two buffers
// when they fit so the epilogue of tile i overlaps the MMAs of tile i+1).  Every mbarrier wait
// is bounded: on give-up the CTA raises an abort flag, records it in g_gemm_status, lets the
// outstanding copies land, frees its TMEM and returns.
//
// Bounds: fp32 accumulate of bf16/fp16 products; tensor-pipe bound for M >= ~1024, decode bound
// in the fused mode.  FLOPs = 2*M*N*K; HBM bytes = operands once (x tiles are re-read from L2).
//
// Stands in for: cuBLAS via F.linear (neuropress/nn/np_vq_linear.py:1148) and, for group-affine
// weights, the per-row GEMV the reference runs at every batch size
// (neuropress/kernels/q4_linear.cu:80-131).
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "gather_sink.cuh"
#include "q4_math.cuh"
#include "tcgen05.cuh"

namespace npb {

__device__ int g_gemm_status = 0;  // 0 ok; 1..4: the role whose wait gave up; >= 10: a
                                   // decoder refused an out-of-range access (see below)

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;            // 64 x 16-bit = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kAStageBytes = BM * BK * 2;                 // 16 KiB per 128-row A sub-tile
constexpr int kSmemCapAssumed = 232448;                   // opt-in dynamic shared memory per CTA on sm_100

enum BMode { B_TMA = 0, B_Q4 = 2 };

struct FusedQ4 {
  const uint8_t* codes;
  const __half* scale;
  const __half* zp;   // never null: aliases `scale` when the weight is symmetric (has_zp == 0)
  int group_size;     // a multiple of 32 on the fused path
  int has_zp;
};

struct GemmParams {
  const float* bias;
  void* y;
  int M, N, K;
  int tiles_m, tiles_n;
  int group_m;  // tiles are walked in bands of group_m tile rows (see tile_coords)
  FusedQ4 q4;
  GatherSink sink;  // peer_out != null: y goes to every rank's buffer, then the handshake
  uint64_t wait_ns;  // limit of every mbarrier wait (npb_set_wait_limit_ns; 2 s by default)
};

template <int BN, int MT>
struct SmemLayout {
  static constexpr int kStageBytes = MT * kAStageBytes + BN * BK * 2;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int stages(int smem_cap) {
    int s = (smem_cap - kBarrierBytes - 1024 /*alignment slack*/) / kStageBytes;
    return s > 8 ? 8 : s;
  }
};

// Ring depth and decode warps of the 4-bit fused mode: at most six stages so that four warps
// per stage (24 decode warps + 6 role warps = 960 threads) fit one CTA.
constexpr int kQ4DecodeWarps = 24;
template <int BN, int MT>
constexpr int q4_stages() {
  return SmemLayout<BN, MT>::stages(kSmemCapAssumed) > 6 ? 6 : SmemLayout<BN, MT>::stages(kSmemCapAssumed);
}

// Tile order.  Tiles are walked in bands of group_m tile rows: inside a band the tile row runs
// fastest, then the tile column, so a wave of CTAs works on (a few tile columns) x (group_m tile
// rows) and the band's activation rows stay L2-resident while all of W streams past them once.
// group_m == tiles_m is the plain column-by-column walk.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int t, int& tm, int& tn) {
  const int per_band = p.group_m * p.tiles_n;
  const int band = t / per_band, r = t - band * per_band;
  const int m0 = band * p.group_m;
  const int gm = min(p.group_m, p.tiles_m - m0);
  tn = r / gm;
  tm = m0 + (r - tn * gm);
}

// ---- B tile decoders (fused modes) ---------------------------------------------------------
// One decode thread owns one W row of the tile (BN == 128 == decode threads) and writes its
// eight 16-byte chunks of the current 64-wide K block.
__device__ __forceinline__ void st_shared_v4(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// 4-bit group-affine decoder.  Every ring stage has its own decode warp(s): with S stages and
// R warps per stage, warp w serves stage w % S only, i.e. the CTA's (tile, K block) items
// w % S, w % S + S, ... -- consecutive phases of that stage's barriers, which is what makes a
// one-bit parity wait unambiguous -- and decodes rows [128/R * (w / S), +128/R) of the tile.
// The per-stage handshake (empty wait, proxy fence, arrive) is thus paid once per 8192 / R
// elements per warp, and all S stages are decoded concurrently.  A lane owns rows lane + 32 r:
// 32 code bytes per row and K block (one fully used 32-byte sector).  The raw bytes of a
// warp's next item are fetched (q4_fetch) before the current one is converted (q4_emit),
// which keeps the global-load latency off the critical path.
template <int RPL>  // rows per lane
struct Q4Item {
  uint4 c[RPL][2];     // [row][half of the K block]
  __half s[RPL][2], z[RPL][2];  // raw: converting here would wait for the loads at fetch time
};

// n0: first W row of this warp's share of the tile; the lane's rows are n0 + lane + 32 r.
template <int RPL>
__device__ __forceinline__ void q4_fetch(Q4Item<RPL>& it, const FusedQ4& p, int n0, int N, int K, int kb,
                                         int lane) {
  const int groups = K / p.group_size;
  const int g0 = (kb * 64) / p.group_size, g1 = (kb * 64 + 32) / p.group_size;
#pragma unroll
  for (int r = 0; r < RPL; ++r) {
    // Rows past N read row N-1 (always mapped); q4_emit gives them scale 0 and their columns
    // are never stored.
    const int n = n0 + lane + 32 * r;
    const int nn = n < N ? n : N - 1;
    const uint4* cp = reinterpret_cast<const uint4*>(p.codes + (size_t)nn * (K / 2) + kb * 32);
    it.c[r][0] = __ldg(cp);
    it.c[r][1] = __ldg(cp + 1);
    const size_t gb = (size_t)nn * groups;
    it.s[r][0] = __ldg(p.scale + gb + g0);
    it.s[r][1] = __ldg(p.scale + gb + g1);
    it.z[r][0] = __ldg(p.zp + gb + g0);
    it.z[r][1] = __ldg(p.zp + gb + g1);
  }
}

// (q - z) * s in fp32 with one rounding per operation, exactly as the one-pass decode does,
// two elements per instruction (packed fp32).  0x4B000000 | q is the float 2^23 + q, so
// subtracting 2^23 yields q without an int-to-float conversion; for a symmetric weight
// (z = 8) both subtractions fold into one exact one.
template <typename T, bool ASYM>
__device__ __forceinline__ void q4_emit_half(const uint4& codes, __half sh, __half zh, bool valid,
                                             uint32_t row_addr, int sw, int half) {
  const float s = valid ? __half2float(sh) : 0.f;
  const float z = __half2float(zh);
  const uint32_t words[4] = {codes.x, codes.y, codes.z, codes.w};
#pragma unroll
  for (int j = 0; j < 4; ++j)
    st_shared_v4(row_addr + (((half * 4 + j) ^ sw) << 4), q4_word_to_chunk<T, ASYM>(words[j], s, z));
}

// row0: tile row of the warp's first row (n0 = tile's first W row + row0).
template <typename T, bool ASYM, int RPL>
__device__ __forceinline__ void q4_emit(const Q4Item<RPL>& it, int n0, int N, uint32_t b_stage, int row0,
                                        int lane) {
#pragma unroll
  for (int r = 0; r < RPL; ++r) {
    const int row = row0 + lane + 32 * r;
    const bool valid = n0 + lane + 32 * r < N;
#pragma unroll
    for (int h = 0; h < 2; ++h)
      q4_emit_half<T, ASYM>(it.c[r][h], it.s[r][h], it.z[r][h], valid, b_stage + row * 128, row & 7, h);
  }
}

// ---- the kernel ------------------------------------------------------------------------------
// GATHER: the epilogue carries the fused all-gather (dense mode only); a separate instantiation
// so that the plain kernels do not pay for its registers.
// CG = 2 (dense mode, MT = 1): two CTAs of a cluster share one 256 x BN tile -- each loads its own
// 128 rows of x and its own BN/2 rows of W, the even CTA issues tcgen05.mma.cta_group::2 for both,
// each CTA's TMEM gets the accumulator rows of its own x rows.  Half the W bytes per stage and CTA
// means a deeper ring (7 stages instead of 4 at BN = 256) for the same shared memory.
template <typename T, int BN, int MT, int BMODE, int BITS, bool GATHER, int CG = 1>
__global__ void __launch_bounds__(BMODE == B_TMA ? 192 : 192 + 32 * kQ4DecodeWarps, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const GemmParams p, const int stages) {
  constexpr int ACC_COLS = MT * BN;                       // fp32 columns per accumulator buffer
  constexpr int NBUF = (2 * ACC_COLS <= 512) ? 2 : 1;
  constexpr int TMEM_COLS = (NBUF * ACC_COLS <= 32) ? 32 : (NBUF * ACC_COLS <= 64) ? 64
                          : (NBUF * ACC_COLS <= 128) ? 128 : (NBUF * ACC_COLS <= 256) ? 256 : 512;
  constexpr int BUF_STRIDE = (NBUF == 2) ? TMEM_COLS / 2 : 0;
  constexpr int kStageBytes = SmemLayout<BN / CG, MT>::kStageBytes;
  // Q4: S stages x R warps per stage (see the decoder notes); VQ: four warps share every stage.
  constexpr int kQ4Stages = q4_stages<BN, MT>();
  constexpr int kQ4WarpsPerStage = 4;
  constexpr int kNumDecodeWarps = (BMODE == B_TMA) ? 0 : kQ4Stages * kQ4WarpsPerStage;
  constexpr int kFullArrivals = (BMODE == B_TMA) ? 0 : kQ4WarpsPerStage;
  static_assert(BMODE != B_Q4 || kNumDecodeWarps <= kQ4DecodeWarps, "decode warps of the Q4 launch");
  constexpr uint32_t kIdesc = umma_idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, BM * CG, BN);
  static_assert(CG == 1 || (CG == 2 && BMODE == B_TMA && MT == 1 && BN % 32 == 0), "CTA pairs: dense mode only");
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "BN");
  static_assert(BMODE == B_TMA || BN == 128, "fused decode maps one decode thread to one W row");

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: swizzle atoms of TMA and UMMA are anchored at multiples of 1024.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);          // [stages]
  uint64_t* empty_bar = full_bar + 8;                              // [stages]
  uint64_t* tmem_full = empty_bar + 8;                             // [2]
  uint64_t* tmem_empty = tmem_full + 2;                            // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_got = abort_flag + 1;  // [2][4]: outcome of each epilogue warp's wait, per tile parity
  uint8_t* stage_base = smem + SmemLayout<BN / CG, MT>::kBarrierBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK - 1) / BK;
  const int num_tiles = p.tiles_m * p.tiles_n;
  // Tile walk of this CTA (pair): tiles first_tile, first_tile + tile_stride, ...
  const int cta_rank = CG == 2 ? (int)cluster_ctarank() : 0;
  const int first_tile = blockIdx.x / CG, tile_stride = gridDim.x / CG;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1 + kFullArrivals);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4 * CG);  // one arrive per epilogue warp (of both CTAs of a pair)
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    if (BMODE == B_TMA) tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    if (CG == 2) {
      tmem_alloc_pair(tmem_slot, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if (CG == 2) {
    __syncwarp();
    cluster_sync_all();  // the peer's barriers are initialised before anything is sent to them
  } else {
    __syncthreads();
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      // pair mode: all bytes of a stage, both CTAs', are credited to the leader's full barrier
      const uint32_t full0 = CG == 2 ? map_to_cta(smem_u32(&full_bar[0]), 0) : 0u;
      for (int t = first_tile; t < num_tiles && ok; t += tile_stride) {
        int tm, tn;
        tile_coords(p, t, tm, tn);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag, p.wait_ns,
                                 BMODE == B_TMA ? 0u : 128u)) {
            atomicExch(&g_gemm_status, 1);
            ok = false;
            break;
          }
          uint8_t* st = stage_base + (size_t)s * kStageBytes;
          constexpr uint32_t tx = MT * kAStageBytes + (BMODE == B_TMA ? BN * BK * 2 : 0);
          if (CG == 2) {
            if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[s], tx + kAStageBytes);  // 2 A tiles + all of B
            const uint32_t bar = full0 + (uint32_t)s * 8u;
            tma_load_2d_pair(st, &tmap_a, bar, kb * BK, (tm * 2 + cta_rank) * BM);
            tma_load_2d_pair(st + kAStageBytes, &tmap_b, bar, kb * BK, tn * BN + cta_rank * (BN / 2));
          } else {
            mbar_arrive_expect_tx(&full_bar[s], tx);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
              tma_load_2d(st + mt * kAStageBytes, &tmap_a, &full_bar[s], kb * BK,
                          (tm * MT + mt) * BM);
            if (BMODE == B_TMA)
              tma_load_2d(st + MT * kAStageBytes, &tmap_b, &full_bar[s], kb * BK, tn * BN);
          }
          if (++s == stages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0 && cta_rank == 0) {
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = first_tile; t < num_tiles && ok; t += tile_stride, ++it) {
        const int buf = (NBUF == 2) ? (it & 1) : 0;
        const uint32_t buf_ph = (NBUF == 2) ? ((it >> 1) & 1) : (it & 1);
        if (!mbar_wait_bounded(&tmem_empty[buf], buf_ph ^ 1, abort_flag, p.wait_ns)) {
          atomicExch(&g_gemm_status, 2);
          break;
        }
        tc_fence_after();
        const uint32_t acc = tmem_base + buf * BUF_STRIDE;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag, p.wait_ns)) {
            atomicExch(&g_gemm_status, 2);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t st = smem_u32(stage_base + (size_t)s * kStageBytes);
          const uint64_t bdesc = umma_desc_sw128(st + MT * kAStageBytes);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint64_t adesc = umma_desc_sw128(st + mt * kAStageBytes);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // +32 bytes per K step inside the 128-byte swizzle row: +2 in the >>4 field
              if (CG == 2)
                umma_f16_pair(acc, adesc + 2 * k, bdesc + 2 * k, kIdesc, (kb > 0 || k > 0) ? 1u : 0u);
              else
                umma_f16(acc + mt * BN, adesc + 2 * k, bdesc + 2 * k, kIdesc,
                         (kb > 0 || k > 0) ? 1u : 0u);
            }
          }
          // frees the stage (in both CTAs of a pair) once these MMAs have read it
          if (CG == 2) umma_commit_pair(&empty_bar[s]);
          else umma_commit(&empty_bar[s]);
          if (++s == stages) { s = 0; ph ^= 1; }
        }
        if (ok) {
          if (CG == 2) umma_commit_pair(&tmem_full[buf]);
          else umma_commit(&tmem_full[buf]);
        }
      }
    }
  } else if (warp < 6) {
    // ================= epilogue: TMEM -> registers -> global =================
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) are this warp's
    T* y = static_cast<T*>(p.y);
    // Fused all-gather: the tile goes to this rank's own [M, ld] buffer first (below, one
    // output row per lane); once the four epilogue warps have stored it they re-read it
    // row-wise and copy it to every peer with row-contiguous 16-byte stores -- NVLink carries
    // those far better than the epilogue's own 16-bytes-per-row pattern.  The TMEM buffer is
    // released before the copy, so the next tile's MMAs run under it.
    const bool gathered = GATHER && p.sink.peer_out != nullptr;
    const int64_t ld = gathered ? p.sink.ld : p.N;
    const int64_t col0 = gathered ? p.sink.col0 : 0;
    if (gathered) y = static_cast<T*>(p.sink.peer_out[p.sink.rank]);
    int it = 0;
    bool ok = true;
    const uint32_t empty0 = CG == 2 ? map_to_cta(smem_u32(&tmem_empty[0]), 0) : 0u;  // the leader's
    for (int t = first_tile; t < num_tiles && ok; t += tile_stride, ++it) {
      int tm, tn;
      tile_coords(p, t, tm, tn);
      if (CG == 2) tm = tm * 2 + cta_rank;  // this CTA's 128 rows of the pair's 256
      const int buf = (NBUF == 2) ? (it & 1) : 0;
      const uint32_t buf_ph = (NBUF == 2) ? ((it >> 1) & 1) : (it & 1);
      // All lanes wait (each needs the acquire), then agree on the outcome so that the
      // warp-collective tcgen05.ld below is never reached by part of a warp.
      const bool got = mbar_wait_bounded(&tmem_full[buf], buf_ph, abort_flag, p.wait_ns,
                                         BMODE == B_TMA ? 0u : 512u);
      if (gathered) {
        // The four warps meet at a named barrier further down, so they must leave together.
        // The decision rests on words that only the epilogue warps write and that cannot change
        // between the barrier and the reads: each warp publishes the outcome of its own wait
        // (for this tile) before the barrier, all four read all four after it.  The CTA-wide
        // abort flag is not used here: another role may raise it at any moment.
        const bool warp_got = __all_sync(0xffffffffu, got);
        volatile int* slot = epi_got + (it & 1) * 4;  // two sets: a fast warp may already write
        if (lane == 0) slot[quad] = warp_got ? 1 : 0;  // the next tile's word while a slow one reads
        __syncwarp();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool all_got = slot[0] && slot[1] && slot[2] && slot[3];
        if (!all_got) {
          atomicExch(&g_gemm_status, 3);
          break;
        }
      } else if (!__all_sync(0xffffffffu, got)) {
        atomicExch(&g_gemm_status, 3);
        break;
      }
      tc_fence_after();
      const uint32_t acc = tmem_base + buf * BUF_STRIDE + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        const int m = (tm * MT + mt) * BM + quad * 32 + lane;
        // Rows past M hold zeros (TMA zero fill); whole sub-tiles past M are skipped by all
        // lanes together so the tcgen05.ld stays warp-uniform.
        if ((tm * MT + mt) * BM >= p.M) break;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(acc + mt * BN + c * 32, v);
          tmem_ld_wait();
          const int n0 = tn * BN + c * 32;
          if (m < p.M && n0 < p.N) {
            const int64_t off = (int64_t)m * ld + col0 + n0;
            // 16-byte stores only where the destination address itself is 16-byte aligned (an
            // output that is a view at an odd offset takes the element-wise path)
            const bool full = (n0 + 32 <= p.N) && ((reinterpret_cast<uintptr_t>(y + off) & 15u) == 0);
            if (full) {
              struct alignas(16) Out { T e[8]; } o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  float f = __uint_as_float(v[q * 8 + e]);
                  if (p.bias) f += __ldg(p.bias + n0 + q * 8 + e);
                  o[q].e[e] = from_f32<T>(f);
                }
              }
              Out* dst = reinterpret_cast<Out*>(y + off);
#pragma unroll
              for (int q = 0; q < 4; ++q) dst[q] = o[q];
            } else {
              T* dst = y + off;
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                if (n0 + e < p.N) {
                  float f = __uint_as_float(v[e]);
                  if (p.bias) f += __ldg(p.bias + n0 + e);
                  dst[e] = from_f32<T>(f);
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CG == 2) mbar_arrive_remote(empty0 + (uint32_t)buf * 8u);
        else mbar_arrive(&tmem_empty[buf]);
      }
      if (gathered && p.sink.world > 1) {
        // copy the finished tile to the peers (N, ld and col0 are multiples of 8 elements)
        asm volatile("bar.sync 1, 128;" ::: "memory");  // all four warps' rows are stored
        const int rows = min(MT * BM, p.M - tm * MT * BM);
        const int cols = min(BN, p.N - tn * BN);
        const int cpr = cols / 8;  // 16-byte chunks per row
        const int64_t tile_off = (int64_t)(tm * MT * BM) * ld + col0 + (int64_t)tn * BN;
        const int et = threadIdx.x - 64;  // 0..127 over the epilogue warps
        constexpr int U = 16;  // 16-byte pieces in flight per thread (32 KiB per CTA)
        auto piece_off = [&](int i) -> int64_t {
          const int r = i / cpr, c = i - r * cpr;
          return tile_off + (int64_t)r * ld + c * 8;
        };
        for (int i0 = et; i0 < rows * cpr; i0 += 128 * U) {
          uint4 vv[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int i = i0 + u * 128;
            if (i < rows * cpr) vv[u] = __ldcg(reinterpret_cast<const uint4*>(y + piece_off(i)));
          }
          for (int d = 1; d < p.sink.world; ++d) {
            T* peer = static_cast<T*>(p.sink.peer_out[(p.sink.rank + d) % p.sink.world]);
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int i = i0 + u * 128;
              if (i < rows * cpr) *reinterpret_cast<uint4*>(peer + piece_off(i)) = vv[u];
            }
          }
        }
      }
    }
    if (gathered) {
      // Fused all-gather: fence this CTA's peer stores, count the CTA in, and let the last
      // CTA of the grid publish the flags and wait for the peers' slices.
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
      if (warp == 2) {
        int last = 0;
        if (lane == 0) last = gather_cta_arrive(p.sink, gridDim.x) ? 1 : 0;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) gather_signal_and_wait(p.sink, lane);
      }
    }
  } else {
    // ================= B decoders (fused modes only) =================
    if constexpr (BMODE == B_Q4) {
      constexpr int S = kQ4Stages, R = kQ4WarpsPerStage, RPL = 4 / R;
      const int dw = warp - 6;  // warps past S * R have no stage
      if (dw < S * R) {
        const int slot = dw % S, row0 = (dw / S) * (128 / R);
        const int my_tiles = blockIdx.x < num_tiles ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        const int total = my_tiles * num_kb;  // (tile, K block) items of this CTA, in ring order
        const bool asym = p.q4.has_zp != 0;
        const uint32_t b_stage = smem_u32(stage_base + (size_t)slot * kStageBytes + MT * kAStageBytes);
        auto warp_n0 = [&](int i) {
          int tm, tn;
          tile_coords(p, blockIdx.x + (i / num_kb) * gridDim.x, tm, tn);
          return tn * BN + row0;
        };
        // Decode item i from `cur` while this warp's next item, i + S, is fetched into `nxt`.
        auto step = [&](Q4Item<RPL>& cur, Q4Item<RPL>& nxt, int i) -> bool {
          if (i + S < total) q4_fetch<RPL>(nxt, p.q4, warp_n0(i + S), p.N, p.K, (i + S) % num_kb, lane);
          const uint32_t ph = (uint32_t)(i / S) & 1u;
          const bool got = mbar_wait_bounded(&empty_bar[slot], ph ^ 1, abort_flag, p.wait_ns, 128u);
          if (!__all_sync(0xffffffffu, got)) {
            atomicExch(&g_gemm_status, 4);
            return false;
          }
          if (asym) q4_emit<T, true, RPL>(cur, warp_n0(i), p.N, b_stage, row0, lane);
          else q4_emit<T, false, RPL>(cur, warp_n0(i), p.N, b_stage, row0, lane);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_bar[slot]);
          return true;
        };
        Q4Item<RPL> a, b;
        if (slot < total) q4_fetch<RPL>(a, p.q4, warp_n0(slot), p.N, p.K, slot % num_kb, lane);
        for (int i = slot; i < total; i += 2 * S) {
          if (!step(a, b, i)) break;
          if (i + S < total && !step(b, a, i + S)) break;
        }
      }
    }
  }

  // ---- teardown: everyone meets here, also after an abort ----
  if (*abort_flag) {
    // Let TMA copies that were already issued land before the shared memory is released.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  if (CG == 2) {
    // Nothing of the peer may be touched after it left: its TMEM by the leader's MMAs, the
    // leader's barriers by the peer's copies and arrives.
    __syncwarp();
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    if (CG == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side -------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Row-major [rows, cols] matrix of 16-bit elements, box = [box_rows, 64 cols], 128B swizzle.
int make_tmap(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int box_rows,
              bool bf16) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) {
    set_last_cuda_error(cudaErrorSymbolNotFound, "cuTensorMapEncodeTiled lookup");
    return NPB_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return NPB_ERR_CUDA;
  }
  return NPB_OK;
}

// Band height of the tile walk, from a traffic estimate: a band whose activation rows fit the L2
// share that survives next to the streaming W and y traffic is read from HBM once, a larger one
// once per wave of CTAs; W is read once per band.
int pick_group_m(int tiles_m, int tiles_n, int tile_rows, int bn, int K, int ctas) {
  const double kResident = 40e6;
  const double x_tile = (double)tile_rows * K * 2, w_all = (double)tiles_n * bn * K * 2;
  double best = 1e300;
  int best_g = tiles_m;
  for (int g = tiles_m; g >= 1; g = g > 1 ? (g + 1) / 2 : 0) {
    const int bands = (tiles_m + g - 1) / g;
    const double waves = (double)g * tiles_n / ctas;
    const double x_reads = g * x_tile <= kResident ? 1.0 : (waves > 1.0 ? waves : 1.0);
    const double traffic = x_reads * g * x_tile * bands + w_all * bands;
    if (traffic < best * 0.98) { best = traffic; best_g = g; }
  }
  return best_g;
}

template <typename T, int BN, int MT, int BMODE, int BITS, bool GATHER = false, int CG = 1>
int launch_gemm(const void* x, const void* w_dense, GemmParams p, cudaStream_t st) {
  constexpr bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  auto kern = gemm_kernel<T, BN, MT, BMODE, BITS, GATHER, CG>;
  using Layout = SmemLayout<BN / CG, MT>;  // a CTA of a pair holds half of the W tile
  const int cap = max_dynamic_smem();
  int stages = Layout::stages(cap);
  if (stages < 2) return NPB_ERR_UNSUPPORTED;
  // The 4-bit decoder binds its warps to ring stages at compile time.
  if (BMODE == B_Q4) {
    if (stages < q4_stages<BN, MT>()) return NPB_ERR_UNSUPPORTED;
    stages = q4_stages<BN, MT>();
  }
  const int smem = Layout::kBarrierBytes + 1024 + stages * Layout::kStageBytes;
  static int configured[64] = {0};
  int dev = 0;
  NPB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && configured[dev] < smem) {
    NPB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev] = smem;
  }
  CUtensorMap ta, tb;
  if (int rc = make_tmap(&ta, x, p.M, p.K, BM, bf16)) return rc;
  if (BMODE == B_TMA) {
    if (int rc = make_tmap(&tb, w_dense, p.N, p.K, BN / CG, bf16)) return rc;
  } else {
    tb = ta;
  }
  p.wait_ns = wait_limit_ns();
  p.tiles_m = (p.M + BM * MT * CG - 1) / (BM * MT * CG);
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n;
  constexpr int threads = BMODE == B_TMA ? 192 : 192 + 32 * kQ4DecodeWarps;
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr{};
  int slots = sm_count() / CG;  // CTAs, or CTA pairs, that run at once
  if (CG == 2) {
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = CG;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    // pairs that can be resident together (both CTAs of a pair sit in one GPC)
    static int resident_pairs[64] = {0};
    if (dev >= 0 && dev < 64) {
      if (resident_pairs[dev] == 0) {
        cfg.gridDim = dim3(slots * CG);
        int n = 0;
        NPB_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
        resident_pairs[dev] = n > 0 ? n : 1;
      }
      if (resident_pairs[dev] < slots) slots = resident_pairs[dev];
    }
  }
  const int units = tiles < slots ? tiles : slots;
  p.group_m = BMODE == B_TMA ? pick_group_m(p.tiles_m, p.tiles_n, BM * MT * CG, BN, p.K, units) : p.tiles_m;
  if (CG == 1) {
    kern<<<units, threads, smem, st>>>(ta, tb, p, stages);
  } else {
    cfg.gridDim = dim3(units * CG);
    NPB_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ta, tb, p, stages));
  }
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

// Tile width for the dense GEMM: minimise (waves x tile cost) with a mild preference for
// wide tiles (fewer shared-memory bytes per flop).
int pick_bn(int64_t M, int64_t N, int cg) {
  static const int forced = [] {
    const char* e = getenv("NEUROPRESS_B200_GEMM_BN");
    const int v = e ? atoi(e) : 0;
    return (v == 256 || v == 224 || v == 192 || v == 128 || v == 64) ? v : 0;
  }();
  if (forced) return forced;
  const int cands[5] = {256, 224, 192, 128, 64};
  const int sms = sm_count() / cg;
  const int64_t tm = (M + BM * cg - 1) / (BM * cg);
  double best = 1e30;
  int best_bn = 256;
  for (int bn : cands) {
    const int64_t tiles = tm * ((N + bn - 1) / bn);
    const int64_t waves = (tiles + sms - 1) / sms;
    // cost per column of a tile: narrower tiles move more operand bytes from L2 per flop, which is what
    // bounds the kernel (on CTA pairs 224 columns measured 10 % slower per flop than 256)
    double eff = bn >= 192 ? 1.0 : bn == 128 ? 1.12 : 1.5;
    if (cg == 2) eff = bn == 256 ? 1.0 : bn == 224 ? 1.07 : bn == 192 ? 1.12 : bn == 128 ? 1.25 : 1.6;
    const double cost = (double)waves * bn * eff;
    if (cost < best - 1e-9) { best = cost; best_bn = bn; }
  }
  return best_bn;
}

// CTA pairs pay when the rows fill 256-row tiles (at most 1/8 of the pair rows empty) and there
// are enough tiles to keep every pair busy.
bool use_pairs(int64_t M, int64_t N) {
  const int mode = gemm_pair_mode();
  if (mode == 0 || M <= BM) return false;
  if (mode == 2) return true;
  const int64_t rows1 = (M + BM - 1) / BM * BM, rows2 = (M + 2 * BM - 1) / (2 * BM) * (2 * BM);
  if (rows2 * 8 > rows1 * 9) return false;
  return (rows2 / (2 * BM)) * ((N + 255) / 256) >= sm_count() / 2;
}

template <typename T, bool GATHER>
int gemm_dense(const void* x, const void* w, GemmParams p, cudaStream_t st) {
  if (use_pairs(p.M, p.N)) {
    switch (pick_bn(p.M, p.N, 2)) {
      case 256: return launch_gemm<T, 256, 1, B_TMA, 0, GATHER, 2>(x, w, p, st);
      case 224: return launch_gemm<T, 224, 1, B_TMA, 0, GATHER, 2>(x, w, p, st);
      case 192: return launch_gemm<T, 192, 1, B_TMA, 0, GATHER, 2>(x, w, p, st);
      case 128: return launch_gemm<T, 128, 1, B_TMA, 0, GATHER, 2>(x, w, p, st);
      default: return launch_gemm<T, 64, 1, B_TMA, 0, GATHER, 2>(x, w, p, st);
    }
  }
  switch (pick_bn(p.M, p.N, 1)) {
    case 256: return launch_gemm<T, 256, 1, B_TMA, 0, GATHER>(x, w, p, st);
    case 224: return launch_gemm<T, 224, 1, B_TMA, 0, GATHER>(x, w, p, st);
    case 192: return launch_gemm<T, 192, 1, B_TMA, 0, GATHER>(x, w, p, st);
    case 128: return launch_gemm<T, 128, 1, B_TMA, 0, GATHER>(x, w, p, st);
    default: return launch_gemm<T, 64, 1, B_TMA, 0, GATHER>(x, w, p, st);
  }
}

template <typename T, int BMODE, int BITS>
int gemm_fused_mt(const void* x, GemmParams p, cudaStream_t st) {
  const int mt = p.M <= 128 ? 1 : p.M <= 256 ? 2 : 3;
  switch (mt) {
    case 1: return launch_gemm<T, 128, 1, BMODE, BITS>(x, nullptr, p, st);
    case 2: return launch_gemm<T, 128, 2, BMODE, BITS>(x, nullptr, p, st);
    default: return launch_gemm<T, 128, 3, BMODE, BITS>(x, nullptr, p, st);
  }
}

// NEUROPRESS_B200_Q_GEMM_STAGED=0 keeps npb_q_gemm_fused on the register-fetching form.
bool q_staged_enabled() {
  static const bool on = [] {
    const char* e = getenv("NEUROPRESS_B200_Q_GEMM_STAGED");
    return !(e && e[0] == '0');
  }();
  return on;
}

int check_gemm_common(const void* x, const void* y, int64_t M, int64_t N, int64_t K, int dtype) {
  if (M < 0 || N < 0 || K < 0) return NPB_ERR_INVALID_ARG;
  if (dtype != NPB_BF16 && dtype != NPB_F16) return NPB_ERR_UNSUPPORTED;
  if (M == 0 || N == 0) return NPB_OK;
  if (x == nullptr || y == nullptr) return NPB_ERR_INVALID_ARG;
  if (K == 0 || K % 8 != 0) return NPB_ERR_SHAPE;
  if (!aligned_to(x, 16)) return NPB_ERR_ALIGNMENT;
  if (M >= (int64_t)1 << 31 || N >= (int64_t)1 << 31 || K >= (int64_t)1 << 31) return NPB_ERR_UNSUPPORTED;
  return NPB_OK;
}

}  // namespace

namespace {
int gemm_impl(const void* x, const void* w, const float* bias, void* y, int64_t M, int64_t N, int64_t K,
              int dtype, const GatherSink* sink, cudaStream_t st) {
  if (int rc = check_gemm_common(x, sink ? x : y, M, N, K, dtype)) return rc;
  if (M == 0 || N == 0) return NPB_OK;
  if (w == nullptr) return NPB_ERR_INVALID_ARG;
  if (!aligned_to(w, 16)) return NPB_ERR_ALIGNMENT;
  GemmParams p{};
  p.bias = bias;
  p.y = y;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  if (sink) {
    p.sink = *sink;
    return dtype == NPB_BF16 ? gemm_dense<__nv_bfloat16, true>(x, w, p, st)
                             : gemm_dense<__half, true>(x, w, p, st);
  }
  return dtype == NPB_BF16 ? gemm_dense<__nv_bfloat16, false>(x, w, p, st)
                           : gemm_dense<__half, false>(x, w, p, st);
}
}  // namespace

int gemm(const void* x, const void* w, const float* bias, void* y, int64_t M, int64_t N, int64_t K,
         int dtype, cudaStream_t st) {
  return gemm_impl(x, w, bias, y, M, N, K, dtype, nullptr, st);
}

// Dense GEMM whose epilogue stores this rank's [M, N] result into columns [col0, col0 + N) of
// every rank's [M, ld] buffer and closes with the all-gather handshake (gather_sink.cuh).
int gemm_gather(const void* x, const void* w, const float* bias, int64_t M, int64_t N, int64_t K,
                int dtype, const GatherSink& sink, cudaStream_t st) {
  if (sink.peer_out == nullptr || sink.peer_flags == nullptr || sink.world < 1 ||
      sink.world > kMaxGatherWorld || sink.rank < 0 || sink.rank >= sink.world || sink.ld < N ||
      sink.col0 < 0 || sink.col0 + N > sink.ld)
    return NPB_ERR_INVALID_ARG;
  if (M == 0 || N == 0) return NPB_ERR_INVALID_ARG;  // every rank must run the handshake
  if (N % 8 != 0 || sink.ld % 8 != 0 || sink.col0 % 8 != 0) return NPB_ERR_ALIGNMENT;  // 16-byte row pieces
  return gemm_impl(x, w, bias, nullptr, M, N, K, dtype, &sink, st);
}

// q_gemm_staged.cu: the form whose raw codes / scales arrive by TMA (NPB_ERR_UNSUPPORTED outside its domain)
int q_gemm_staged(const npb_q_weight* w, const void* x, int x_dtype, int64_t M, int64_t N, int64_t K,
                  const float* bias, void* y, cudaStream_t st);
int q_gemm_staged_device_status(int* host_out);

int q_gemm_fused(const npb_q_weight* w, const void* x, int x_dtype, int64_t M, int64_t N, int64_t K,
                 const float* bias, void* y, cudaStream_t st) {
  if (int rc = validate_q(w, N, K)) return rc;
  if (int rc = check_gemm_common(x, y, M, N, K, x_dtype)) return rc;
  if (M == 0 || N == 0) return NPB_OK;
  if (w->nbits != 4 || K % 64 != 0 || w->group_size % 32 != 0) return NPB_ERR_UNSUPPORTED;
  if (!aligned_to(w->codes, 16)) return NPB_ERR_ALIGNMENT;
  if (q_staged_enabled()) {
    const int rc = q_gemm_staged(w, x, x_dtype, M, N, K, bias, y, st);
    if (rc != NPB_ERR_UNSUPPORTED) return rc;
  }
  GemmParams p{};
  p.bias = bias;
  p.y = y;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.q4.codes = w->codes;
  p.q4.scale = static_cast<const __half*>(w->scale);
  p.q4.has_zp = w->zero_point != nullptr;
  p.q4.zp = p.q4.has_zp ? static_cast<const __half*>(w->zero_point) : p.q4.scale;
  p.q4.group_size = w->group_size;
  return x_dtype == NPB_BF16 ? gemm_fused_mt<__nv_bfloat16, B_Q4, 0>(x, p, st)
                             : gemm_fused_mt<__half, B_Q4, 0>(x, p, st);
}

// Reads and clears the device-side give-up record of the GEMM kernels (synchronises).
int vq_gemm_fused_device_status(int* host_out);  // vq_gemm_fused.cu keeps its own record
int q_gemv_ring_device_status(int* host_out);    // and so does q_gemv_ring.cu
int vq_decode_copy_device_status(int* host_out); // and vq_decode_copy.cu

int gemm_device_status(int* host_out) {
  int v = 0;
  NPB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    NPB_CUDA_TRY(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int)));
  }
  int vf = 0;
  if (int rc = vq_gemm_fused_device_status(&vf)) return rc;
  if (v == 0) v = vf;
  int vr = 0;
  if (int rc = q_gemv_ring_device_status(&vr)) return rc;
  if (v == 0 && vr != 0) v = 20 + vr;
  int vc = 0;
  if (int rc = vq_decode_copy_device_status(&vc)) return rc;
  if (v == 0 && vc != 0) v = 30 + vc;
  int vs = 0;
  if (int rc = q_gemm_staged_device_status(&vs)) return rc;
  if (v == 0 && vs != 0) v = 40 + vs;
  if (host_out) *host_out = v;
  return v == 0 ? NPB_OK : NPB_ERR_DEVICE_TIMEOUT;
}

}  // namespace npb
