// 4-bit group-affine GEMV for 1-2 activation rows, with the weight streamed through a shared-
// memory ring by 1-D bulk async copies (cp.async.bulk + mbarrier; this GPU's memory only, no
// multicast) instead of through registers.
//
// Why: the GEMV reads every packed byte once, so HBM bandwidth is its roof, and a kernel of this
// size (33 MB, ~9 us at best) reaches that roof only with tens of KiB in flight per SM from the
// first microsecond on.  Loads held in registers cap that at (threads x registers); a producer
// thread that only issues bulk copies does not: eight stages of eight weight rows (codes, scales,
// zero-points: ~20 KiB each for K = 4096) are always in flight, whatever the consumers do.
//
// Consumers (16 warps): warp w owns the K slice [w*K/16, +K/16) of every row, exactly as in
// q4_gemv_mma_rows8_kernel (q_gemv_mma.cu): nibble pairs become bf16 / fp16 pairs by one shift and
// one logic op (OR into the mantissa of 128.0 / 1024.0), mma.sync.m16n8k16 does the dot products
// with the activations in a block-diagonal operand, and the lane that read a 32-value block
// applies that block's scale and zero-point to its partial sum: acc += s * (D - (OFFSET + zp) *
// sum_k x_k).  The only difference is where the 16-byte code words come from: the current ring
// stage (eight rows back to back, fetched by ONE bulk copy; even and odd rows read the two halves
// of a step pair in opposite order so that a quarter-warp hits eight different bank groups)
// instead of global memory.
//
// Measured on a B200, 14336 x 4096, Q4_0 group 32, one row, cold L2: 13.6 us (2.43 TB/s on the
// packed bytes) against 17.9 us for the register-fed kernel; the same ring with the arithmetic
// removed runs in 7.9 us, which is also what a plain read of those bytes takes -- the rest is the
// issue rate of mma.sync (one per 256 weights, the minimum for m16n8k16) and the nibble unpacking.
//
// Stands in for _q_linear (neuropress/kernels/q4_linear.cu:80-131) at 1-2 rows.
#include <type_traits>

#include "common.cuh"
#include "mma_sync.cuh"
#include "tcgen05.cuh"  // mbarrier helpers

namespace npb {
namespace {

using namespace sm100;

constexpr int kCW = 16;                    // consumer warps
constexpr int kThreads = (kCW + 1) * 32;   // + one producer warp
constexpr int kRows = 8;                   // weight rows per ring stage (one mma row group)
constexpr int kMaxStages = 8;

struct RingArgs {
  const uint8_t* codes;
  const __half* scale;
  const __half* zp;      // null: symmetric (zero-point 8)
  const float* bias;
  const void* x;
  void* y;
  uint64_t wait_ns;
  int M, N, K, gs_shift, stages;
  int rows_per_cta;      // multiple of 8
};

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ int perm8(int e) { return ((e & 3) << 1) | (e >> 2); }

__device__ int g_q_ring_status = 0;

template <typename T, int MR, int PAIRS>
__global__ void __launch_bounds__(kThreads, 1) q4_gemv_ring_kernel(RingArgs a) {
  constexpr uint32_t kMagic = std::is_same<T, __nv_bfloat16>::value ? 0x43004300u : 0x64006400u;
  constexpr float kOffset = std::is_same<T, __nv_bfloat16>::value ? 128.f : 1024.f;
  constexpr int kZeroElems = 8 * 16 + 8;
  extern __shared__ __align__(128) uint8_t smem[];
  const int K = a.K;
  const int KS = K / kCW;                   // K slice of a consumer warp (multiple of 256)
  constexpr int pairs = PAIRS;              // 256-wide step pairs per row group and warp (KS / 256)
  const int lds = (KS / 128) * 144;         // activation row stride per warp (elements)
  const int groups = K >> a.gs_shift;       // scale groups per weight row
  const int row_bytes = K / 2;              // code row in a stage (rows back to back: one copy per stage)
  const int sc_row = groups * 2;
  const int sc_bytes = kRows * sc_row;      // scales (and zero-points) of a stage
  const int stage_bytes = kRows * row_bytes + sc_bytes * (a.zp ? 2 : 1);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  // shared memory: barriers | ring | per-warp activations | partial sums
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kMaxStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kMaxStages);
  uint8_t* ring = smem + 256;
  const size_t warp_bytes = ((size_t)MR * lds + kZeroElems) * sizeof(T) + (size_t)MR * (KS / 32) * 4;
  uint8_t* xbase = ring + (size_t)a.stages * stage_bytes;
  float* part = reinterpret_cast<float*>(xbase + (size_t)kCW * warp_bytes);  // [kCW][rows_per_cta][MR]

  const int r0 = blockIdx.x * a.rows_per_cta;
  const int r1 = r0 + a.rows_per_cta < a.N ? r0 + a.rows_per_cta : a.N;
  const int n_rg = r1 > r0 ? (r1 - r0 + kRows - 1) / kRows : 0;

  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kCW);
    }
    fence_barrier_init();
  }
  __syncthreads();

  if (warp == kCW) {
    // ================= producer: one thread issues every copy =================
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int rg = 0; rg < n_rg; ++rg) {
        if (!mbar_wait_bounded(&empty[s], ph ^ 1, abort_flag, a.wait_ns, 32u)) {
          atomicExch(&g_q_ring_status, 1);
          break;
        }
        uint8_t* st = ring + (size_t)s * stage_bytes;
        const int row0 = r0 + rg * kRows;
        // rows past the end re-read the last row (always mapped); their sums are never stored
        const int nrows = r1 - row0 < kRows ? r1 - row0 : kRows;
        mbar_arrive_expect_tx(&full[s], (uint32_t)stage_bytes);
        uint8_t* sc = st + (size_t)kRows * row_bytes;
        if (nrows == kRows) {   // eight consecutive rows are contiguous in memory: three copies per stage
          bulk_g2s(st, a.codes + (size_t)row0 * row_bytes, (uint32_t)(kRows * row_bytes), &full[s]);
          bulk_g2s(sc, a.scale + (size_t)row0 * groups, (uint32_t)sc_bytes, &full[s]);
          if (a.zp) bulk_g2s(sc + sc_bytes, a.zp + (size_t)row0 * groups, (uint32_t)sc_bytes, &full[s]);
        } else {
          for (int r = 0; r < kRows; ++r) {
            const int row = r < nrows ? row0 + r : r1 - 1;
            bulk_g2s(st + (size_t)r * row_bytes, a.codes + (size_t)row * row_bytes, (uint32_t)row_bytes, &full[s]);
            bulk_g2s(sc + (size_t)r * sc_row, a.scale + (size_t)row * groups, (uint32_t)sc_row, &full[s]);
            if (a.zp)
              bulk_g2s(sc + sc_bytes + (size_t)r * sc_row, a.zp + (size_t)row * groups, (uint32_t)sc_row, &full[s]);
          }
        }
        if (++s == a.stages) { s = 0; ph ^= 1; }
      }
    }
  } else {
    // ================= consumers =================
    uint8_t* wbase = xbase + (size_t)warp * warp_bytes;
    T* xs = reinterpret_cast<T*>(wbase);
    T* zeros = xs + (size_t)MR * lds;
    float* xsum = reinterpret_cast<float*>(zeros + kZeroElems);
    // Stage this warp's activation slice: chunk j (8 values) of the slice = (step, block, word),
    // values permuted to the order one mask extracts them from a code word, plus block sums.
    {
      const T* x = static_cast<const T*>(a.x);
      const int blocks32 = KS >> 5;
      for (int i = lane; i < MR * blocks32; i += 32) {
        const int m = i / blocks32, j4 = i - m * blocks32;
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int j = j4 * 4 + c;
          struct alignas(16) V8 { T v[8]; } v, pv;
          if (m < a.M) {
            v = *reinterpret_cast<const V8*>(x + (size_t)m * K + warp * KS + j * 8);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v.v[e] = from_f32<T>(0.f);
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) { pv.v[perm8(e)] = v.v[e]; sum += to_f32(v.v[e]); }
          const int step = j >> 4, tb = (j >> 2) & 3, u = j & 3;
          T* dst = xs + (size_t)m * lds + step * 144 + tb * 4;
          *reinterpret_cast<uint2*>(dst + (2 * u) * 16) = *reinterpret_cast<const uint2*>(&pv.v[0]);
          *reinterpret_cast<uint2*>(dst + (2 * u + 1) * 16) = *reinterpret_cast<const uint2*>(&pv.v[4]);
        }
        xsum[i] = sum;
      }
      for (int i = lane; i < kZeroElems; i += 32) zeros[i] = from_f32<T>(0.f);
    }
    __syncwarp();
    // The activation operand of every mma and the block sums are the same for every row group:
    // they are read from shared memory once and stay in registers (block-diagonal operand: this
    // lane supplies column g = (block g/2, step g%2) and holds the k slots of block t, so it
    // contributes activations iff g/2 == t, zeros otherwise).
    const bool active = (g >> 1) == t;
    uint2 bfrag[PAIRS][MR][8];
    float xs_a[PAIRS][MR], xs_b[PAIRS][MR];
#pragma unroll
    for (int pr = 0; pr < PAIRS; ++pr)
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        const T* bp = active ? xs + (size_t)m * lds + (g & 1) * 144 + t * 4 + pr * 288 : zeros;
#pragma unroll
        for (int q = 0; q < 8; ++q) bfrag[pr][m][q] = *reinterpret_cast<const uint2*>(bp + q * 16);
        xs_a[pr][m] = xsum[m * (KS >> 5) + pr * 8 + t];
        xs_b[pr][m] = xsum[m * (KS >> 5) + pr * 8 + t + 4];
      }

    int s = 0;
    uint32_t ph = 0;
    const int k_lane = warp * KS + t * 32;  // first k of this lane's block in step A of pair 0
    for (int rg = 0; rg < n_rg; ++rg) {
      const bool got = mbar_wait_bounded(&full[s], ph, abort_flag, a.wait_ns);
      if (!__all_sync(0xffffffffu, got)) {
        atomicExch(&g_q_ring_status, 2);
        break;
      }
      const uint8_t* st = ring + (size_t)s * stage_bytes;
      const uint8_t* crow = st + (size_t)g * row_bytes;                       // this lane's weight row
      const __half* srow = reinterpret_cast<const __half*>(st + (size_t)kRows * row_bytes + (size_t)g * sc_row);
      const __half* zrow = reinterpret_cast<const __half*>(st + (size_t)kRows * row_bytes + sc_bytes + (size_t)g * sc_row);
      float acc[MR];
#pragma unroll
      for (int m = 0; m < MR; ++m) acc[m] = 0.f;
#pragma unroll
      for (int pr = 0; pr < pairs; ++pr) {
        const int kA = k_lane + pr * 256;                                      // step B is + 128
        // Rows sit back to back in the stage (stride K/2, a multiple of 128 bytes), so the lanes
        // of a quarter-warp -- rows g, g+1 x four blocks -- would collide pairwise if both rows
        // read the same 64-byte half of the step pair.  Odd rows therefore read step B into the
        // "first" operand and step A into the second; the sums are picked accordingly below.
        const int odd = g & 1;
        const uint4 ca = *reinterpret_cast<const uint4*>(crow + (kA >> 1) + odd * 64);
        const uint4 cb = *reinterpret_cast<const uint4*>(crow + (kA >> 1) + (odd ^ 1) * 64);
        // scales of the eight (four, two) groups of this warp's 256-wide slice: one wide load per
        // lane (the four lanes of a quad read the same address), each lane picks its two groups
        const int gsl = 256 >> a.gs_shift;                                     // groups per step pair
        const int gbase = (warp * KS + pr * 256) >> a.gs_shift;
        const int ia = (t * 32) >> a.gs_shift, ib = (128 + t * 32) >> a.gs_shift;
        // half `i` (0..7) of a 16-byte run held in four words, without indexing an array
        auto pick = [](const uint4& v, int i) {
          const uint32_t w = i < 4 ? (i < 2 ? v.x : v.y) : (i < 6 ? v.z : v.w);
          return __half2float(__ushort_as_half((unsigned short)(w >> ((i & 1) * 16))));
        };
        uint4 sv = make_uint4(0, 0, 0, 0), zv = make_uint4(0, 0, 0, 0);
        if (gsl == 8) {
          sv = *reinterpret_cast<const uint4*>(srow + gbase);
          if (a.zp) zv = *reinterpret_cast<const uint4*>(zrow + gbase);
        } else if (gsl == 4) {
          const uint2 s2 = *reinterpret_cast<const uint2*>(srow + gbase);
          sv.x = s2.x; sv.y = s2.y;
          if (a.zp) { const uint2 z2 = *reinterpret_cast<const uint2*>(zrow + gbase); zv.x = z2.x; zv.y = z2.y; }
        } else {
          sv.x = *reinterpret_cast<const uint32_t*>(srow + gbase);
          if (a.zp) zv.x = *reinterpret_cast<const uint32_t*>(zrow + gbase);
        }
        const float sa = pick(sv, ia), sb = pick(sv, ib);
        const float za = a.zp ? pick(zv, ia) : 8.f, zb = a.zp ? pick(zv, ib) : 8.f;
        float d[MR][4];
#pragma unroll
        for (int m = 0; m < MR; ++m)
#pragma unroll
          for (int i = 0; i < 4; ++i) d[m][i] = 0.f;
        const uint32_t wa[4] = {ca.x, ca.y, ca.z, ca.w};
        const uint32_t wb[4] = {cb.x, cb.y, cb.z, cb.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          uint32_t pa[4], pb[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            pa[i] = ((wa[u] >> (4 * i)) & 0x000f000fu) | kMagic;
            pb[i] = ((wb[u] >> (4 * i)) & 0x000f000fu) | kMagic;
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t af[4] = {pa[2 * h], pb[2 * h], pa[2 * h + 1], pb[2 * h + 1]};
#pragma unroll
            for (int m = 0; m < MR; ++m) mma16816<T>(d[m], af, bfrag[pr][m][2 * u + h].x, bfrag[pr][m][2 * u + h].y);
          }
        }
        // D[g][2t] / D[g][2t+1]: first operand against step A / step B activations; D[g+8][..]: second
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          const float dA = odd ? d[m][2] : d[m][0];   // the operand that holds step A, against step A
          const float dB = odd ? d[m][1] : d[m][3];   // the operand that holds step B, against step B
          acc[m] = fmaf(sa, dA - (kOffset + za) * xs_a[pr][m], acc[m]);
          acc[m] = fmaf(sb, dB - (kOffset + zb) * xs_b[pr][m], acc[m]);
        }
      }
      // this warp is done with the stage: hand it back before the (short) reduction
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      if (++s == a.stages) { s = 0; ph ^= 1; }
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        float v = acc[m];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        const int r = rg * kRows + g;
        if (t == 0 && r < a.rows_per_cta) part[((size_t)warp * a.rows_per_cta + r) * MR + m] = v;
      }
    }
  }
  __syncthreads();
  if (*abort_flag) return;
  for (int i = tid; i < (r1 - r0) * MR; i += kThreads) {
    const int r = MR == 1 ? i : i >> 1, m = MR == 1 ? 0 : i & 1;
    if (m < a.M) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kCW; ++w) v += part[((size_t)w * a.rows_per_cta + r) * MR + m];
      const int n = r0 + r;
      if (a.bias) v += __ldg(a.bias + n);
      static_cast<T*>(a.y)[(size_t)m * a.N + n] = from_f32<T>(v);
    }
  }
}

template <typename T, int MR, int PAIRS>
int launch_ring(RingArgs a, cudaStream_t st) {
  const int sms = sm_count();
  int rows_per_cta = (a.N + sms - 1) / sms;
  rows_per_cta = (rows_per_cta + kRows - 1) / kRows * kRows;
  a.rows_per_cta = rows_per_cta;
  const int grid = (a.N + rows_per_cta - 1) / rows_per_cta;
  const int K = a.K, KS = K / kCW, groups = K >> a.gs_shift;
  const size_t stage_bytes = (size_t)kRows * (K / 2) + (size_t)kRows * groups * 2 * (a.zp ? 2 : 1);
  const size_t warp_bytes = ((size_t)MR * (KS / 128) * 144 + 8 * 16 + 8) * sizeof(T) + (size_t)MR * (KS / 32) * 4;
  const size_t fixed = 256 + (size_t)kCW * warp_bytes + (size_t)kCW * rows_per_cta * MR * 4;
  const size_t cap = (size_t)max_dynamic_smem();
  if (fixed + 2 * stage_bytes > cap) return NPB_ERR_UNSUPPORTED;
  int stages = (int)((cap - fixed) / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  a.stages = stages;
  const size_t smem = fixed + (size_t)stages * stage_bytes;
  auto kern = q4_gemv_ring_kernel<T, MR, PAIRS>;
  int per_sm = 0;
  if (int rc = blocks_per_sm(reinterpret_cast<const void*>(kern), kThreads, smem, &per_sm)) return rc;
  if (per_sm < 1) return NPB_ERR_UNSUPPORTED;
  a.wait_ns = wait_limit_ns();
  kern<<<grid, kThreads, smem, st>>>(a);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

// ---- 3-8 activation rows ------------------------------------------------------------------------
// The same ring, with every column of the mma carrying an activation row.  A stage holds SIXTEEN
// weight rows (A rows g and g + 8), each row a bulk copy of its own at a stride of K/2 + 16 bytes,
// so that lane (g, t) can read ONE code word -- word t of the 32-block j of its rows -- without a
// bank conflict: the 16 k slots of an mma then belong to one 32-block, whose D tile (16 weight rows
// x 8 activation rows) takes that block's scale and zero-point once.  Two mmas per block, whatever
// the row count: 256 weights per mma at 8 rows, against 64 with a block-diagonal operand.
// The activation fragments and block sums of the warp's K slice (256 wide) stay in registers.
constexpr int kRows16 = 16;

template <typename T, bool ZP>
__global__ void __launch_bounds__(kThreads, 1) q4_gemv_ring8_kernel(RingArgs a) {
  constexpr uint32_t kMagic = std::is_same<T, __nv_bfloat16>::value ? 0x43004300u : 0x64006400u;
  constexpr float kOffset = std::is_same<T, __nv_bfloat16>::value ? 128.f : 1024.f;
  constexpr int STEPS = 2;                  // 128-wide steps of a warp's K slice (K = 4096)
  extern __shared__ __align__(128) uint8_t smem[];
  const int K = a.K;
  const int KS = K / kCW;                   // 256
  const int groups = K >> a.gs_shift;
  const int row_bytes = K / 2, row_stride = row_bytes + 16;
  const int sc_row = groups * 2, sc_stride = sc_row + 16;
  const int sc_off = kRows16 * row_stride;                   // scales of a stage
  const int zp_off = sc_off + kRows16 * sc_stride;           // zero points
  const int stage_bytes = zp_off + (ZP ? kRows16 * sc_stride : 0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kMaxStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kMaxStages);
  uint8_t* ring = smem + 256;
  float* part = reinterpret_cast<float*>(ring + (size_t)a.stages * stage_bytes);   // [kCW][rows_per_cta][8]

  const int r0 = blockIdx.x * a.rows_per_cta;
  const int r1 = r0 + a.rows_per_cta < a.N ? r0 + a.rows_per_cta : a.N;
  const int n_rg = r1 > r0 ? (r1 - r0 + kRows16 - 1) / kRows16 : 0;

  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kCW);
    }
    fence_barrier_init();
  }
  __syncthreads();

  if (warp == kCW) {
    // ================= producer: lane r issues the copies of row r of every stage =================
    int s = 0;
    uint32_t ph = 0;
    const uint32_t tx = (uint32_t)(kRows16 * (row_bytes + sc_row * (ZP ? 2 : 1)));
    for (int rg = 0; rg < n_rg; ++rg) {
      const bool ok = mbar_wait_bounded(&empty[s], ph ^ 1, abort_flag, a.wait_ns, 32u);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) atomicExch(&g_q_ring_status, 3);
        break;
      }
      uint8_t* st = ring + (size_t)s * stage_bytes;
      if (lane == 0) mbar_arrive_expect_tx(&full[s], tx);
      __syncwarp();   // the expectation is posted before any copy can complete
      if (lane < kRows16) {
        // rows past the end re-read the last row (always mapped); their sums are never stored
        const int row = r0 + rg * kRows16 + lane < r1 ? r0 + rg * kRows16 + lane : r1 - 1;
        bulk_g2s(st + (size_t)lane * row_stride, a.codes + (size_t)row * row_bytes, (uint32_t)row_bytes, &full[s]);
        bulk_g2s(st + sc_off + (size_t)lane * sc_stride, a.scale + (size_t)row * groups, (uint32_t)sc_row, &full[s]);
        if (ZP)
          bulk_g2s(st + zp_off + (size_t)lane * sc_stride, a.zp + (size_t)row * groups, (uint32_t)sc_row, &full[s]);
      }
      if (++s == a.stages) { s = 0; ph ^= 1; }
    }
  } else {
    // ================= consumers =================
    // Activation fragments of this warp's K slice, straight from global memory (read once): for
    // (step S, block j) the lane's chunk is word t of that block of activation row g; values
    // 0,4,1,5 feed the first mma of the block, 2,6,3,7 the second (the order one mask extracts
    // nibble pairs from a code word).  Block sums for the activation rows 2t, 2t+1 of the D tile.
    uint2 bfrag[STEPS][4][2];
    float2 xsum[STEPS][4];
    {
      const T* x = static_cast<const T*>(a.x);
#pragma unroll
      for (int S = 0; S < STEPS; ++S)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          struct alignas(16) V8 { T v[8]; } v, pv;
          if (g < a.M) {
            v = *reinterpret_cast<const V8*>(x + (size_t)g * K + warp * KS + S * 128 + j * 32 + t * 8);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v.v[e] = from_f32<T>(0.f);
          }
          float sum = 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) { pv.v[perm8(e)] = v.v[e]; sum += to_f32(v.v[e]); }
          bfrag[S][j][0] = *reinterpret_cast<const uint2*>(&pv.v[0]);
          bfrag[S][j][1] = *reinterpret_cast<const uint2*>(&pv.v[4]);
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);      // the block's sum for activation row g
          xsum[S][j].x = __shfl_sync(0xffffffffu, sum, (2 * t) * 4);
          xsum[S][j].y = __shfl_sync(0xffffffffu, sum, (2 * t + 1) * 4);
        }
    }

    int s = 0;
    uint32_t ph = 0;
    const int kbyte = (warp * KS) >> 1;               // this warp's slice inside a code row
    const int gbase = (warp * KS) >> a.gs_shift;      // first scale group of the slice
    for (int rg = 0; rg < n_rg; ++rg) {
      const bool got = mbar_wait_bounded(&full[s], ph, abort_flag, a.wait_ns);
      if (!__all_sync(0xffffffffu, got)) {
        atomicExch(&g_q_ring_status, 4);
        break;
      }
      const uint8_t* st = ring + (size_t)s * stage_bytes;
      const uint8_t* rowA = st + (size_t)g * row_stride + kbyte + t * 4;
      const uint8_t* rowB = rowA + 8 * row_stride;
      const unsigned short* sA = reinterpret_cast<const unsigned short*>(st + sc_off + (size_t)g * sc_stride) + gbase;
      const unsigned short* sB = reinterpret_cast<const unsigned short*>(st + sc_off + (size_t)(g + 8) * sc_stride) + gbase;
      const unsigned short* zA = reinterpret_cast<const unsigned short*>(st + zp_off + (size_t)g * sc_stride) + gbase;
      const unsigned short* zB = reinterpret_cast<const unsigned short*>(st + zp_off + (size_t)(g + 8) * sc_stride) + gbase;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};   // (row g, m 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)
#pragma unroll
      for (int S = 0; S < STEPS; ++S) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t wa = *reinterpret_cast<const uint32_t*>(rowA + S * 64 + j * 16);
          const uint32_t wb = *reinterpret_cast<const uint32_t*>(rowB + S * 64 + j * 16);
          uint32_t pa[4], pb[4];
          pa[0] = (wa & 0x000f000fu) | kMagic;
          pb[0] = (wb & 0x000f000fu) | kMagic;
#pragma unroll
          for (int i = 1; i < 4; ++i) {
            pa[i] = ((wa >> (4 * i)) & 0x000f000fu) | kMagic;
            pb[i] = ((wb >> (4 * i)) & 0x000f000fu) | kMagic;
          }
          float d[4];
          {
            const uint32_t af[4] = {pa[0], pb[0], pa[1], pb[1]};
            mma16816_first<T>(d, af, bfrag[S][j][0].x, bfrag[S][j][0].y);
          }
          {
            const uint32_t af[4] = {pa[2], pb[2], pa[3], pb[3]};
            mma16816<T>(d, af, bfrag[S][j][1].x, bfrag[S][j][1].y);
          }
          const int grp = (S * 128 + j * 32) >> a.gs_shift;
          const float sa = __half2float(__ushort_as_half(sA[grp])), sb = __half2float(__ushort_as_half(sB[grp]));
          float ca = kOffset + 8.f, cb = kOffset + 8.f;
          if (ZP) {
            ca = kOffset + __half2float(__ushort_as_half(zA[grp]));
            cb = kOffset + __half2float(__ushort_as_half(zB[grp]));
          }
          acc[0] = fmaf(sa, d[0] - ca * xsum[S][j].x, acc[0]);
          acc[1] = fmaf(sa, d[1] - ca * xsum[S][j].y, acc[1]);
          acc[2] = fmaf(sb, d[2] - cb * xsum[S][j].x, acc[2]);
          acc[3] = fmaf(sb, d[3] - cb * xsum[S][j].y, acc[3]);
        }
      }
      // this warp is done with the stage: hand it back before the partial sums are written
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      if (++s == a.stages) { s = 0; ph ^= 1; }
      const int r = rg * kRows16 + g;   // < rows_per_cta (a multiple of 16)
      float* pw = part + ((size_t)warp * a.rows_per_cta + r) * 8 + 2 * t;
      *reinterpret_cast<float2*>(pw) = make_float2(acc[0], acc[1]);
      *reinterpret_cast<float2*>(pw + 8 * 8) = make_float2(acc[2], acc[3]);
    }
  }
  __syncthreads();
  if (*abort_flag) return;
  for (int i = tid; i < (r1 - r0) * 8; i += kThreads) {
    const int r = i >> 3, m = i & 7;
    if (m < a.M) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kCW; ++w) v += part[((size_t)w * a.rows_per_cta + r) * 8 + m];
      const int n = r0 + r;
      if (a.bias) v += __ldg(a.bias + n);
      static_cast<T*>(a.y)[(size_t)m * a.N + n] = from_f32<T>(v);
    }
  }
}

template <typename T>
int launch_ring8(RingArgs a, cudaStream_t st) {
  const int sms = sm_count();
  int rows_per_cta = (a.N + sms - 1) / sms;
  rows_per_cta = (rows_per_cta + kRows16 - 1) / kRows16 * kRows16;
  a.rows_per_cta = rows_per_cta;
  const int grid = (a.N + rows_per_cta - 1) / rows_per_cta;
  const int K = a.K, groups = K >> a.gs_shift;
  const size_t stage_bytes = (size_t)kRows16 * (K / 2 + 16) + (size_t)kRows16 * (groups * 2 + 16) * (a.zp ? 2 : 1);
  const size_t fixed = 256 + (size_t)kCW * rows_per_cta * 8 * 4;
  const size_t cap = (size_t)max_dynamic_smem();
  if (fixed + 2 * stage_bytes > cap) return NPB_ERR_UNSUPPORTED;
  int stages = (int)((cap - fixed) / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  a.stages = stages;
  const size_t smem = fixed + (size_t)stages * stage_bytes;
  auto kern = a.zp ? q4_gemv_ring8_kernel<T, true> : q4_gemv_ring8_kernel<T, false>;
  int per_sm = 0;
  if (int rc = blocks_per_sm(reinterpret_cast<const void*>(kern), kThreads, smem, &per_sm)) return rc;
  if (per_sm < 1) return NPB_ERR_UNSUPPORTED;
  a.wait_ns = wait_limit_ns();
  kern<<<grid, kThreads, smem, st>>>(a);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

}  // namespace

// Reads and clears this kernel's give-up record (1 / 3: a producer, 2 / 4: a consumer); merged into
// npb_gemm_device_status.
int q_gemv_ring_device_status(int* host_out) {
  int v = 0;
  NPB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_q_ring_status, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    NPB_CUDA_TRY(cudaMemcpyToSymbol(g_q_ring_status, &zero, sizeof(int)));
  }
  if (host_out) *host_out = v;
  return NPB_OK;
}

// Returns NPB_ERR_UNSUPPORTED for shapes this kernel does not take (the caller then uses the
// register-fed tensor-core GEMV): 1-2 rows (3-8 rows: K = 4096), 4-bit codes, K a multiple of 4096, power-of-two
// groups of at least 32, rows and scale rows that start on 16-byte boundaries.
int q4_gemv_ring(const npb_q_weight* w, const void* x, int x_dtype, int64_t M, int64_t N, int64_t K,
                 const float* bias, void* y, cudaStream_t st) {
  if (w->nbits != 4 || (x_dtype != NPB_BF16 && x_dtype != NPB_F16)) return NPB_ERR_UNSUPPORTED;
  if (M < 1 || M > 8 || K % 4096 != 0 || K > 8192 || N < 8 || N >= (int64_t)1 << 30) return NPB_ERR_UNSUPPORTED;
  if (M > 2 && (K != 4096 || N < 16)) return NPB_ERR_UNSUPPORTED;   // the 3-8-row form keeps one 256-wide slice per warp
  int gs_shift = 0;
  while ((1 << gs_shift) < w->group_size) ++gs_shift;
  if ((1 << gs_shift) != w->group_size || w->group_size < 32 || w->group_size > 128) return NPB_ERR_UNSUPPORTED;
  const int64_t groups = K >> gs_shift;
  if ((groups * 2) % 16 != 0) return NPB_ERR_UNSUPPORTED;  // a row of scales is a bulk copy of its own at the tail
  if (!aligned_to(w->codes, 16) || !aligned_to(w->scale, 16) || (w->zero_point && !aligned_to(w->zero_point, 16)) ||
      !aligned_to(x, 16))
    return NPB_ERR_UNSUPPORTED;
  RingArgs a{};
  a.codes = w->codes;
  a.scale = static_cast<const __half*>(w->scale);
  a.zp = static_cast<const __half*>(w->zero_point);
  a.bias = bias;
  a.x = x;
  a.y = y;
  a.M = (int)M; a.N = (int)N; a.K = (int)K;
  a.gs_shift = gs_shift;
  if (M > 2) return x_dtype == NPB_BF16 ? launch_ring8<__nv_bfloat16>(a, st) : launch_ring8<__half>(a, st);
  const int pairs = (int)(K / 4096);   // 256-wide step pairs of a consumer warp's K slice
  if (pairs > 2) return NPB_ERR_UNSUPPORTED;   // the activation operand of the slice must fit the registers
#define NPB_RING(TT, MR_, P_) launch_ring<TT, MR_, P_>(a, st)
#define NPB_RING_P(TT, MR_) (pairs == 1 ? NPB_RING(TT, MR_, 1) : NPB_RING(TT, MR_, 2))
  if (x_dtype == NPB_BF16) return M == 1 ? NPB_RING_P(__nv_bfloat16, 1) : NPB_RING_P(__nv_bfloat16, 2);
  return M == 1 ? NPB_RING_P(__half, 1) : NPB_RING_P(__half, 2);
#undef NPB_RING_P
#undef NPB_RING
}

}  // namespace npb
