// Tile-dequant tensor-core GEMM for 4-bit group-affine weights with TMA-staged codes (the mid-batch
// band, 9..384 rows):
//
//   y[M, N] = x[M, K] . W[N, K]^T (+ bias),  W = (q - z) * s decoded on the fly.
//
// The weight is read once, in packed form.  A TMA producer brings the RAW operands of the W tile
// into a ring of its own, one slot per SUPER-BLOCK of eight 64-wide k blocks: BN rows x 256 bytes
// of codes and BN rows x 32 bytes of scales and, for asymmetric weights, zero points -- three
// strided 2-D tile loads that no thread waits for, with rows wide enough for the TMA unit (a box
// of 32-byte rows per k block costs it as many row requests as one of 256-byte rows per eight).
// The ring is independent of the operand ring (x tile + decoded W tile per k block), so the loads
// run up to sixteen k blocks ahead of the decode.  Every decode group walks ALL super-blocks in
// order (waiting for each and releasing each through a barrier of its own), so every barrier sees
// one producer and consumers on consecutive phases -- a one-bit parity wait is ambiguous
// otherwise.  Decode warps, in groups bound to operand stages,
// convert shared memory -> shared memory: nibble -> fp32 by byte-permute, (q - z) * s in packed
// fp32 with one rounding per operation (q4_math.cuh, the arithmetic of
// neuropress/nn/np_linear.py:334-351), one 16-byte store per eight weights into the 128B-swizzled
// operand tile of tcgen05.mma.  Nothing in the decode path waits on global memory, which is what
// bounded the register-fetching form (gemm_kernel<..., B_Q4>: ~2000 cycles per item).
//
//   warp 0 TMA producer of x tiles, warp 1 TMEM owner + tcgen05.mma issuer, warps 2-5 epilogue,
//   warp 6 TMA producer of raw W operands, 16 decode warps in groups of 1 / 2 / 4 (group g serves
//   operand stage g).  Tile width BN: a run-time multiple of 16 that fills one wave of SMs (112 for
//   N = 14336).  Every wait is bounded.
//
// Needs group_size in {32, 64, 128}, K % 512 == 0, (K / group_size) % 8 == 0 and 16-byte aligned
// operands; anything else goes to the register-fetching form.  Replaces q_linear for these row
// counts (neuropress/kernels/q4_linear.cu:80-131 re-reads the weight for every row).
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "q4_math.cuh"
#include "tcgen05.cuh"

namespace npb {

__device__ int g_q_staged_status = 0;  // 0 ok; 1..4: the role whose bounded wait gave up

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kAStageBytes = BM * BK * 2;
// Decode warps: warps 7..22.  With more than 128 rows (several MMAs per k step) the ones that share
// the MMA-issuing warp's scheduler (warp index = 1 mod 4) stay idle: with decode warps on its
// scheduler the issuer needs ~500 instead of ~300 cycles to get four MMAs and a commit out.
constexpr int kDecodeWarps = 16;
constexpr int kMaxGroups = kDecodeWarps;
constexpr int kSuper = 8;                            // k blocks per raw-operand slot
constexpr int kMaxRaw = 4;                           // slots of the raw-operand ring
constexpr int kRawRowBytes = 32 * kSuper + 32 + 32;  // codes + scales + zero points of one W row
constexpr int kFirstDecodeWarp = 7;
constexpr int kThreads = 32 * (kFirstDecodeWarp + 16);             // 736: 16 warp slots, 12 of them decode
constexpr int kBarrierBytes = 2048;

struct StagedParams {
  const float* bias;
  void* y;
  uint64_t wait_ns;
  int M, N, K, BN, tiles_m, tiles_n, groups, warps_per_group, raw_slots, decode_warps;
  int group_size, has_zp;
};

__device__ __forceinline__ void st_shared_v4(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t ld_shared_u16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}

template <typename T, int MT>
__global__ void __launch_bounds__(kThreads, 1)
q_gemm_staged_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_codes,
                     const __grid_constant__ CUtensorMap tmap_scale, const __grid_constant__ CUtensorMap tmap_zp,
                     const StagedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);   // [groups] x tile landed + W tile decoded
  uint64_t* empty_bar = full_bar + kMaxGroups;              // [groups] the MMAs have read the stage
  uint64_t* raw_full = empty_bar + kMaxGroups;              // [raw_slots] codes / scales / zero points landed
  uint64_t* raw_empty = raw_full + kMaxRaw;                 // [raw_slots][kMaxGroups] group g is past the slot's super-block
  uint64_t* tmem_full = raw_empty + kMaxRaw * kMaxGroups;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;                     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* stage_base = smem + kBarrierBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BN = p.BN;
  // operand stage: [x tile(s)] [W tile, bf16 / fp16, 128B swizzle]; raw slot: [codes BN x 256] [scales BN x 32]
  // [zero points BN x 32]
  const int off_w = MT * kAStageBytes;
  const int stage_bytes = off_w + BN * 128;
  // codes: two halves (k blocks 0-3, 4-7) of BN rows x 128 bytes, each loaded with the 128-byte swizzle so
  // that the lanes of a warp (one W row each) read different banks
  const int off_scale = BN * 32 * kSuper, off_zp = off_scale + BN * 32, raw_bytes_slot = BN * kRawRowBytes;
  const int G = p.groups, R = p.raw_slots;
  const int supers_per_tile = (p.K / BK) / kSuper;
  uint8_t* raw_base = stage_base + (size_t)G * stage_bytes;
  const int num_kb = p.K / BK;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int acc_cols = MT * BN;
  const int nbuf = (2 * acc_cols <= 512) ? 2 : 1;
  int tmem_cols = 32;
  while (tmem_cols < nbuf * acc_cols) tmem_cols <<= 1;
  const uint32_t idesc = umma_idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, BM, BN);
  const int gs = p.group_size;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < G; ++s) {
      mbar_init(&full_bar[s], 1 + p.warps_per_group);
      mbar_init(&empty_bar[s], 1);
    }
    for (int r = 0; r < R; ++r) {
      mbar_init(&raw_full[r], 1);
      for (int g = 0; g < G; ++g) mbar_init(&raw_empty[r * kMaxGroups + g], p.warps_per_group);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_codes);
    tma_prefetch_desc(&tmap_scale);
    if (p.has_zp) tma_prefetch_desc(&tmap_zp);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ================= TMA producer: x tiles =================
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int tm = t % p.tiles_m;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag, p.wait_ns, 64u)) {
            atomicExch(&g_q_staged_status, 1);
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
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int buf = (nbuf == 2) ? (it & 1) : 0;
        const uint32_t buf_ph = (nbuf == 2) ? ((it >> 1) & 1) : (it & 1);
        if (!mbar_wait_bounded(&tmem_empty[buf], buf_ph ^ 1, abort_flag, p.wait_ns)) {
          atomicExch(&g_q_staged_status, 2);
          break;
        }
        tc_fence_after();
        const uint32_t acc = tmem_base + buf * acc_cols;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag, p.wait_ns)) {
            atomicExch(&g_q_staged_status, 2);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t st = smem_u32(stage_base + (size_t)s * stage_bytes);
          const uint64_t bdesc = umma_desc_sw128(st + off_w);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint64_t adesc = umma_desc_sw128(st + mt * kAStageBytes);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_f16(acc + mt * BN, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
          if (++s == G) { s = 0; ph ^= 1; }
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
      const int buf = (nbuf == 2) ? (it & 1) : 0;
      const uint32_t buf_ph = (nbuf == 2) ? ((it >> 1) & 1) : (it & 1);
      const bool got = mbar_wait_bounded(&tmem_full[buf], buf_ph, abort_flag, p.wait_ns, 256u);
      if (!__all_sync(0xffffffffu, got)) {
        atomicExch(&g_q_staged_status, 3);
        break;
      }
      tc_fence_after();
      const uint32_t acc = tmem_base + buf * acc_cols + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        if ((tm * MT + mt) * BM >= p.M) break;  // whole sub-tile past M: skipped by all lanes together
        const int m = (tm * MT + mt) * BM + quad * 32 + lane;
#pragma unroll 1
        for (int c = 0; c < BN / 16; ++c) {
          uint32_t v[16];
          tmem_ld_32x32_x16(acc + mt * BN + c * 16, v);
          tmem_ld_wait();
          const int n0 = tn * BN + c * 16;
          if (m < p.M && n0 < p.N) {
            T* dst = y + (int64_t)m * p.N + n0;
            if (n0 + 16 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
              struct alignas(16) Out { T e[8]; } o[2];
#pragma unroll
              for (int q = 0; q < 2; ++q)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  float f = __uint_as_float(v[q * 8 + e]);
                  if (p.bias) f += __ldg(p.bias + n0 + q * 8 + e);
                  o[q].e[e] = from_f32<T>(f);
                }
              reinterpret_cast<Out*>(dst)[0] = o[0];
              reinterpret_cast<Out*>(dst)[1] = o[1];
            } else {
#pragma unroll
              for (int e = 0; e < 16; ++e)
                if (n0 + e < p.N) {
                  float f = __uint_as_float(v[e]);
                  if (p.bias) f += __ldg(p.bias + n0 + e);
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
  } else if (warp == 6) {
    // ================= TMA producer: raw W operands, their own ring =================
    if (lane == 0) {
      int u = 0;                                   // super-block counter over this CTA's tiles
      bool ok = true;
      const int sg = (kSuper * BK) / gs;            // groups per super-block: 16, 8 or 4
      const uint32_t scale_row_bytes = sg >= 8 ? (uint32_t)sg * 2u : 16u;
      const uint32_t raw_tx = (uint32_t)BN * (32u * kSuper + scale_row_bytes * (p.has_zp ? 2u : 1u));
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int tn = t / p.tiles_m;
        for (int sb = 0; sb < supers_per_tile && ok; ++sb, ++u) {
          const int r = u % R;
          const uint32_t ph = (uint32_t)(u / R) & 1u;
          for (int g = 0; g < G; ++g)
            if (!mbar_wait_bounded(&raw_empty[r * kMaxGroups + g], ph ^ 1, abort_flag, p.wait_ns, 64u)) {
              atomicExch(&g_q_staged_status, 1);
              ok = false;
              break;
            }
          if (!ok) break;
          uint8_t* slot = raw_base + (size_t)r * raw_bytes_slot;
          mbar_arrive_expect_tx(&raw_full[r], raw_tx);
          tma_load_2d(slot, &tmap_codes, &raw_full[r], sb * 32 * kSuper, tn * BN);
          tma_load_2d(slot + BN * 128, &tmap_codes, &raw_full[r], sb * 32 * kSuper + 128, tn * BN);
          const int g0 = (sb * sg) & ~7;             // scale chunk: max(8, sg) groups from a multiple of 8
          tma_load_2d(slot + off_scale, &tmap_scale, &raw_full[r], g0, tn * BN);
          if (p.has_zp) tma_load_2d(slot + off_zp, &tmap_zp, &raw_full[r], g0, tn * BN);
        }
      }
    }
  } else {
    // ================= decode warps: shared memory -> shared memory =================
    const int slot_w = warp - kFirstDecodeWarp;                 // 0..15
    const bool all16 = p.decode_warps == 16;
    const bool decodes = all16 || (warp & 3) != 1;
    const int dw = all16 ? slot_w : slot_w - (slot_w + 2) / 4;  // index over the decoding warps
    const int wpg = p.warps_per_group;
    const int grp = dw / wpg, part = dw - grp * wpg;
    if (decodes && grp < G) {
      const int rows_per_warp = BN / wpg;
      const int row0 = part * rows_per_warp;
      const int my_tiles = (int)blockIdx.x < num_tiles ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
      const int total = my_tiles * num_kb;    // the CTA's (tile, k block) items in ring order
      const uint32_t st = smem_u32(stage_base + (size_t)grp * stage_bytes);
      const bool asym = p.has_zp != 0;
      constexpr int RPL = 2;                  // rows per lane (the second one only when a warp has more than 32 rows)
      const int sg = (kSuper * BK) / gs;       // groups per super-block
      const int scale_pitch = sg >= 8 ? sg * 2 : 16;   // bytes per row of the scale / zero-point chunk
      const int total_supers = my_tiles * supers_per_tile;
      int u_seen = -1;                         // last super-block this warp has waited for
      bool ok = true;
      // Walk to super-block `u`: wait for every one on the way (consecutive phases for every waiter) and
      // release the ones left behind.
      auto advance_to = [&](int u) -> bool {
        while (u_seen < u) {
          if (u_seen >= 0) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&raw_empty[(u_seen % R) * kMaxGroups + grp]);
          }
          ++u_seen;
          const bool got = mbar_wait_bounded(&raw_full[u_seen % R], (uint32_t)(u_seen / R) & 1u, abort_flag,
                                             p.wait_ns, 32u);
          if (!__all_sync(0xffffffffu, got)) {
            atomicExch(&g_q_staged_status, 4);
            return false;
          }
        }
        return true;
      };
      for (int i = grp; i < total && ok; i += G) {
        const int kb = i % num_kb;
        const int u = (i / num_kb) * supers_per_tile + kb / kSuper;
        if (!advance_to(u)) break;
        const int j = kb % kSuper;              // k block inside the super-block
        const int g0 = ((kb / kSuper) * sg) & ~7;
        const int ga = (kb * BK) / gs - g0, gb = (kb * BK + 32) / gs - g0;   // groups of the two 32-column halves
        const uint32_t raw = smem_u32(raw_base + (size_t)(u % R) * raw_bytes_slot);
        uint4 c0[RPL], c1[RPL];
        float fsa[RPL], fsb[RPL], fza[RPL], fzb[RPL];
#pragma unroll
        for (int q = 0; q < RPL; ++q) {
          const int rr = lane + 32 * q;
          fza[q] = fzb[q] = 0.f;
          if (rr < rows_per_warp) {
            const int row = row0 + rr;
            const uint32_t crow = raw + (j >> 2) * (BN * 128) + row * 128;   // this row in its half
            const int ch = (j & 3) * 2;                                       // first of its two 16-byte chunks
            c0[q] = ld_shared_v4(crow + ((ch ^ (row & 7)) << 4));
            c1[q] = ld_shared_v4(crow + (((ch + 1) ^ (row & 7)) << 4));
            // rows past N arrive zero-filled (scale 0): their weights are 0 and their columns are never stored
            fsa[q] = __half2float(__ushort_as_half((unsigned short)ld_shared_u16(raw + off_scale + row * scale_pitch + ga * 2)));
            fsb[q] = __half2float(__ushort_as_half((unsigned short)ld_shared_u16(raw + off_scale + row * scale_pitch + gb * 2)));
            if (asym) {
              fza[q] = __half2float(__ushort_as_half((unsigned short)ld_shared_u16(raw + off_zp + row * scale_pitch + ga * 2)));
              fzb[q] = __half2float(__ushort_as_half((unsigned short)ld_shared_u16(raw + off_zp + row * scale_pitch + gb * 2)));
            }
          }
        }
        const bool got = mbar_wait_bounded(&empty_bar[grp], ((uint32_t)(i / G) & 1u) ^ 1u, abort_flag, p.wait_ns, 32u);
        if (!__all_sync(0xffffffffu, got)) {
          atomicExch(&g_q_staged_status, 4);
          break;
        }
#pragma unroll
        for (int q = 0; q < RPL; ++q) {
          const int rr = lane + 32 * q;
          if (rr < rows_per_warp) {
            const int row = row0 + rr;
            const uint32_t row_addr = st + off_w + row * 128;
            const int sw = row & 7;
            const uint32_t wa[4] = {c0[q].x, c0[q].y, c0[q].z, c0[q].w}, wb[4] = {c1[q].x, c1[q].y, c1[q].z, c1[q].w};
            if (asym) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                st_shared_v4(row_addr + ((j ^ sw) << 4), q4_word_to_chunk<T, true>(wa[j], fsa[q], fza[q]));
                st_shared_v4(row_addr + (((4 + j) ^ sw) << 4), q4_word_to_chunk<T, true>(wb[j], fsb[q], fzb[q]));
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                st_shared_v4(row_addr + ((j ^ sw) << 4), q4_word_to_chunk<T, false>(wa[j], fsa[q], 0.f));
                st_shared_v4(row_addr + (((4 + j) ^ sw) << 4), q4_word_to_chunk<T, false>(wb[j], fsb[q], 0.f));
              }
            }
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_bar[grp]);
      }
      // the producer may still be waiting for this group to pass the remaining super-blocks
      if (ok) advance_to(total_supers - 1);
      if (u_seen >= 0) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&raw_empty[(u_seen % R) * kMaxGroups + grp]);
      }
    }
  }

  // ---- teardown: everyone meets here, also after an abort ----
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);  // let issued TMA copies land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// Row-major [rows, cols] matrix of `elem`-byte elements, box [box_rows, box_cols].
int make_map(CUtensorMap* map, const void* base, CUtensorMapDataType type, int elem, int64_t rows, int64_t cols,
             int box_rows, int box_cols, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    set_last_cuda_error(cudaErrorSymbolNotFound, "cuTensorMapEncodeTiled lookup");
    return NPB_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * elem};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  if (fn(map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    set_last_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return NPB_ERR_CUDA;
  }
  return NPB_OK;
}

// BN: a multiple of 16 in [16, 256] such that (waves of tiles) x BN is smallest; ties go to the wider tile.
int pick_bn(int64_t N, int tiles_m, int mt, int sms) {
  int best_bn = 128;
  double best = 1e30;
  for (int bn = 256; bn >= 16; bn -= 16) {
    if (mt * bn > 512) continue;
    const int64_t tiles = (int64_t)tiles_m * ((N + bn - 1) / bn);
    const int64_t waves = (tiles + sms - 1) / sms;
    const double cost = (double)waves * bn;
    if (cost < best - 1e-9) { best = cost; best_bn = bn; }
  }
  return best_bn;
}

// 16 decode warps up to 128 rows, 12 (the MMA issuer's scheduler left alone) above;
// NEUROPRESS_B200_Q_STAGED_DECODE_WARPS (12 or 16) overrides.
int decode_warps_setting(int mt) {
  static const int forced = [] {
    const char* e = getenv("NEUROPRESS_B200_Q_STAGED_DECODE_WARPS");
    const int v = e ? atoi(e) : 0;
    return (v == 12 || v == 16) ? v : 0;
  }();
  return forced ? forced : (mt >= 2 ? 12 : 16);
}

template <typename T, int MT>
int launch(const npb_q_weight* w, const void* x, StagedParams p, cudaStream_t st) {
  constexpr bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  auto kern = q_gemm_staged_kernel<T, MT>;
  const int sms = sm_count();
  p.tiles_m = (p.M + BM * MT - 1) / (BM * MT);
  p.BN = pick_bn(p.N, p.tiles_m, MT, sms);
  p.tiles_n = (p.N + p.BN - 1) / p.BN;
  const int stage_bytes = MT * kAStageBytes + p.BN * 128;   // operand stage
  const int raw_bytes = p.BN * kRawRowBytes;                // raw-operand slot (one super-block)
  const int cap = max_dynamic_smem();
  int wpg = 4;
  if (p.BN <= 32) wpg = 1;
  else if (p.BN <= 64) wpg = 2;
  if (p.BN % wpg != 0) wpg = 4;
  p.warps_per_group = wpg;
  const int room = cap - kBarrierBytes - 1024;
  int groups = (room - 2 * raw_bytes) / stage_bytes;        // at least two raw slots
  p.decode_warps = decode_warps_setting(MT);
  if (groups > p.decode_warps / wpg) groups = p.decode_warps / wpg;
  if (groups < 2) return NPB_ERR_UNSUPPORTED;
  p.groups = groups;
  int raw_slots = (room - groups * stage_bytes) / raw_bytes;
  if (raw_slots > kMaxRaw) raw_slots = kMaxRaw;
  p.raw_slots = raw_slots;
  const int smem = kBarrierBytes + 1024 + groups * stage_bytes + raw_slots * raw_bytes;
  static int configured[64] = {0};
  int dev = 0;
  NPB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && configured[dev] < smem) {
    NPB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cap));
    configured[dev] = cap;
  }
  const int64_t groups_per_row = p.K / p.group_size;
  CUtensorMap ta, tc, ts, tz;
  if (int rc = make_map(&ta, x, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p.M, p.K,
                        BM, BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  const int sg = (kSuper * BK) / p.group_size;             // groups per super-block
  const int scale_box = sg >= 8 ? sg : 8;
  if (int rc = make_map(&tc, w->codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.N, p.K / 2, p.BN, 128,
                        CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = make_map(&ts, w->scale, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p.N, groups_per_row, p.BN, scale_box,
                        CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  tz = ts;
  if (p.has_zp)
    if (int rc = make_map(&tz, w->zero_point, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p.N, groups_per_row, p.BN,
                          scale_box, CU_TENSOR_MAP_SWIZZLE_NONE))
      return rc;
  p.wait_ns = wait_limit_ns();
  const int tiles = p.tiles_m * p.tiles_n;
  kern<<<tiles < sms ? tiles : sms, kThreads, smem, st>>>(ta, tc, ts, tz, p);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

}  // namespace

// Reads and clears this kernel's give-up record (synchronises).
int q_gemm_staged_device_status(int* host_out) {
  int v = 0;
  NPB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_q_staged_status, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    NPB_CUDA_TRY(cudaMemcpyToSymbol(g_q_staged_status, &zero, sizeof(int)));
  }
  if (host_out) *host_out = v;
  return NPB_OK;
}

// NPB_ERR_UNSUPPORTED: outside this form's domain (the caller takes the register-fetching form).
// Arguments were validated by the caller (q_gemm_fused).
int q_gemm_staged(const npb_q_weight* w, const void* x, int x_dtype, int64_t M, int64_t N, int64_t K,
                  const float* bias, void* y, cudaStream_t st) {
  const int gs = w->group_size;
  if (w->nbits != 4 || (gs != 32 && gs != 64 && gs != 128) || K % (kSuper * BK) != 0 || (K / gs) % 8 != 0 || M > 384)
    return NPB_ERR_UNSUPPORTED;
  if (!aligned_to(w->codes, 16) || !aligned_to(w->scale, 16) || (w->zero_point && !aligned_to(w->zero_point, 16)) ||
      !aligned_to(x, 16))
    return NPB_ERR_UNSUPPORTED;
  StagedParams p{};
  p.bias = bias;
  p.y = y;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.group_size = gs;
  p.has_zp = w->zero_point != nullptr;
  const bool bf = x_dtype == NPB_BF16;
  if (M <= 128) return bf ? launch<__nv_bfloat16, 1>(w, x, p, st) : launch<__half, 1>(w, x, p, st);
  if (M <= 256) return bf ? launch<__nv_bfloat16, 2>(w, x, p, st) : launch<__half, 2>(w, x, p, st);
  return bf ? launch<__nv_bfloat16, 3>(w, x, p, st) : launch<__half, 3>(w, x, p, st);
}

}  // namespace npb
