// 4-bit group-affine GEMV (1..8 rows) with the dot products on the tensor cores (mma.sync).
//
// The CUDA-core GEMV spends more than four instructions per weight value turning nibbles into
// fp32 and is issue bound at about 30 % of HBM bandwidth.  Here a nibble pair becomes a bf16x2
// (or fp16x2) register with one shift and one logic op -- the nibble is OR-ed into the
// mantissa of 128.0 (bf16) or 1024.0 (fp16), giving exactly 128+q / 1024+q -- and
// mma.sync.m16n8k16 does the multiply-adds with fp32 accumulation.
//
// Layout trick: a CTA of four warps owns 16 output rows; warp w owns every fourth 128-wide
// K step.  In a step, lane (g = lane/4, t = lane%4) loads 16 bytes (32 codes, one scale group
// slice) of row g and of row g+8 at k = step*128 + t*32.  The mma sums over the k slots held
// by the four lanes of a quad, which belong to four different 32-blocks (possibly four
// different scale groups); to keep them apart the activation operand is block-diagonal: its 8
// columns are (32-block j, activation row m) for j = 0..3, m = 0..1, and column (j, m) holds x
// only in the k slots of block j.  Then D[row][2t + m] is the partial dot product of lane t's
// own 32 codes with activation row m: the lane that loaded a block also receives its sum and
// applies its own scale and zero-point once per step:
//     acc += s * (D - (OFFSET + zp) * sum_k x_k).
// More than two activation rows repeat the mma with the next pair of rows (A registers reused).
//
// HBM bytes per call: N*K/2 codes + scales (+ zero-points) + activations; pure streaming.
#include <type_traits>

#include "common.cuh"
#include "mma_sync.cuh"

namespace npb {
namespace {

constexpr int kPrefetch = 4;   // K steps whose loads each warp keeps in flight

struct MmaArgs {
  const uint8_t* codes;
  const __half* scale;
  const __half* zp;
  const float* bias;
  const void* x;
  void* y;
  int M, N, K, group_size;
};

// Position of element e (0..7) inside its 8-element activation chunk in shared memory: the
// order 0,4,1,5,2,6,3,7 matches the nibble pairs (i, i+4) that one mask extracts from a word.
__device__ __forceinline__ int perm8(int e) { return ((e & 3) << 1) | (e >> 2); }

// Persistent: one CTA of WARPS warps per SM walks over 16-row blocks (block index strided by
// the grid); within a block warp w owns the K steps w, w + WARPS, ...  The load ring runs on
// across row blocks, so weight loads stay in flight for the whole kernel.
template <typename T, int MP, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1) q4_gemv_mma_kernel(MmaArgs a) {
  constexpr int MR = 2 * MP;                                   // activation rows held (padded)
  constexpr int kThreads = WARPS * 32;
  constexpr uint32_t kMagic = std::is_same<T, __nv_bfloat16>::value ? 0x43004300u : 0x64006400u;
  constexpr float kOffset = std::is_same<T, __nv_bfloat16>::value ? 128.f : 1024.f;
  extern __shared__ __align__(16) uint8_t smem[];
  const int K = a.K;
  const int ldx = K + 16;      // 32-byte row pad: the two rows of a pair hit different banks
  // xs[m][step][mma (8)][block t (4)][4 values]: for one mma the four active lanes of an
  // activation row read four consecutive 8-byte pieces.
  T* xs = reinterpret_cast<T*>(smem);
  T* zeros = xs + (size_t)MR * ldx;                             // 16 bytes of zeros
  float* xsum = reinterpret_cast<float*>(zeros + 8);            // [MR][K/32]
  float* red = xsum + (size_t)MR * (K / 32);                    // [2][WARPS][16][MR]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int gs = a.group_size, groups = K / gs;
  const int spw = K / 128 / WARPS;                              // K steps per warp and row block
  const int n_blocks = (a.N + 15) / 16;
  const int my_blocks = blockIdx.x < n_blocks ? (n_blocks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int total = my_blocks * spw;                            // this warp's flattened step list

  // Scales / zero points stay as loaded (one register per 16-bit load) until they are used: packing
  // them here would make the warp wait for the loads where they are issued.
  struct Step { uint4 ca, cb; unsigned short sA, sB, zA, zB; };
  const unsigned short* scale_u = reinterpret_cast<const unsigned short*>(a.scale);
  const unsigned short* zp_u = reinterpret_cast<const unsigned short*>(a.zp);
  auto load_step = [&](Step& st, int q) {
    const int rb = blockIdx.x + (q / spw) * gridDim.x;
    const int kb = warp + (q % spw) * WARPS;
    const int rA = rb * 16 + g < a.N ? rb * 16 + g : a.N - 1;
    const int rB = rb * 16 + g + 8 < a.N ? rb * 16 + g + 8 : a.N - 1;
    st.ca = __ldg(reinterpret_cast<const uint4*>(a.codes + (size_t)rA * (K / 2) + kb * 64 + t * 16));
    st.cb = __ldg(reinterpret_cast<const uint4*>(a.codes + (size_t)rB * (K / 2) + kb * 64 + t * 16));
    const int grp = (kb * 128 + t * 32) / gs;
    st.sA = __ldg(scale_u + (size_t)rA * groups + grp);
    st.sB = __ldg(scale_u + (size_t)rB * groups + grp);
    st.zA = st.zB = 0x4800;   // 8.0
    if (a.zp) {
      st.zA = __ldg(zp_u + (size_t)rA * groups + grp);
      st.zB = __ldg(zp_u + (size_t)rB * groups + grp);
    }
  };

  // The first kPrefetch steps are requested before the activations are staged.
  Step ring[kPrefetch];
#pragma unroll
  for (int p = 0; p < kPrefetch; ++p)
    if (p < total) load_step(ring[p], p);

  {
    const T* x = static_cast<const T*>(a.x);
    for (int i = tid; i < MR * (K / 32); i += kThreads) {
      const int m = i / (K / 32), j4 = i - m * (K / 32);
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int j = j4 * 4 + c;
        struct alignas(16) V8 { T v[8]; } v, p;
        if (m < a.M) {
          v = *reinterpret_cast<const V8*>(x + (size_t)m * K + j * 8);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) v.v[e] = from_f32<T>(0.f);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) { p.v[perm8(e)] = v.v[e]; s += to_f32(v.v[e]); }
        // chunk j = (step, block tb, word u); its two 4-value halves feed mma 2u and 2u+1
        const int step = j >> 4, tb = (j >> 2) & 3, u = j & 3;
        T* dst = xs + (size_t)m * ldx + step * 128 + tb * 4;
        *reinterpret_cast<uint2*>(dst + (2 * u) * 16) = *reinterpret_cast<const uint2*>(&p.v[0]);
        *reinterpret_cast<uint2*>(dst + (2 * u + 1) * 16) = *reinterpret_cast<const uint2*>(&p.v[4]);
      }
      xsum[i] = s;
    }
    if (tid < 8) zeros[tid] = from_f32<T>(0.f);
  }
  __syncthreads();

  // Block-diagonal activation operand: this lane supplies column g = (block j = g/2, row m = g%2)
  // and holds k slots of block t only, so it contributes x iff g/2 == t, zeros otherwise.
  const bool active = (g >> 1) == t;
  const int bmul = active ? 1 : 0;
  const T* brow[MP];
#pragma unroll
  for (int mp = 0; mp < MP; ++mp)
    brow[mp] = active ? xs + (size_t)(2 * mp + (g & 1)) * ldx + t * 4 : zeros;

  float acc[MP][4];
#pragma unroll
  for (int mp = 0; mp < MP; ++mp)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[mp][i] = 0.f;

  for (int base = 0; base < total; base += kPrefetch) {
#pragma unroll
    for (int p = 0; p < kPrefetch; ++p) {
      const int q = base + p;
      if (q >= total) break;
      const Step cur = ring[p];
      if (q + kPrefetch < total) load_step(ring[p], q + kPrefetch);
      const int kb = warp + (q % spw) * WARPS;

      float d[MP][4];
#pragma unroll
      for (int mp = 0; mp < MP; ++mp)
#pragma unroll
        for (int i = 0; i < 4; ++i) d[mp][i] = 0.f;
      const uint32_t wa[4] = {cur.ca.x, cur.ca.y, cur.ca.z, cur.ca.w};
      const uint32_t wb[4] = {cur.cb.x, cur.cb.y, cur.cb.z, cur.cb.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint32_t pa[4], pb[4];  // pair i = (nibble i, nibble i+4) of the word as OFFSET + q
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          pa[i] = ((wa[u] >> (4 * i)) & 0x000f000fu) | kMagic;
          pb[i] = ((wb[u] >> (4 * i)) & 0x000f000fu) | kMagic;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          // A fragment: a0/a2 = row g (k slots 2t..2t+1 / 2t+8..2t+9), a1/a3 = row g+8
          const uint32_t af[4] = {pa[2 * h], pb[2 * h], pa[2 * h + 1], pb[2 * h + 1]};
#pragma unroll
          for (int mp = 0; mp < MP; ++mp) {
            const uint2 bv =
                *reinterpret_cast<const uint2*>(brow[mp] + bmul * (kb * 128 + (2 * u + h) * 16));
            mma16816<T>(d[mp], af, bv.x, bv.y);
          }
        }
      }
      // D columns 2t, 2t+1 = this lane's own 32-block against activation rows (2mp, 2mp+1)
      const float2 sc = make_float2(__half2float(__ushort_as_half(cur.sA)), __half2float(__ushort_as_half(cur.sB)));
      const float ca = kOffset + __half2float(__ushort_as_half(cur.zA));
      const float cb = kOffset + __half2float(__ushort_as_half(cur.zB));
#pragma unroll
      for (int mp = 0; mp < MP; ++mp) {
        const float x0 = xsum[(2 * mp) * (K / 32) + kb * 4 + t];
        const float x1 = xsum[(2 * mp + 1) * (K / 32) + kb * 4 + t];
        acc[mp][0] = fmaf(sc.x, d[mp][0] - ca * x0, acc[mp][0]);
        acc[mp][1] = fmaf(sc.x, d[mp][1] - ca * x1, acc[mp][1]);
        acc[mp][2] = fmaf(sc.y, d[mp][2] - cb * x0, acc[mp][2]);
        acc[mp][3] = fmaf(sc.y, d[mp][3] - cb * x1, acc[mp][3]);
      }

      if ((q % spw) == spw - 1) {
        // Row block finished for this warp: sum the quad (four 32-blocks per step), hand the
        // partials to shared memory, and let the first lanes add the WARPS partials.
        const int blk = q / spw;
        float* rbuf = red + (size_t)(blk & 1) * WARPS * 16 * MR;
#pragma unroll
        for (int mp = 0; mp < MP; ++mp)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float v = acc[mp][i];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            acc[mp][i] = v;
          }
        if (t == 0) {
#pragma unroll
          for (int mp = 0; mp < MP; ++mp) {
            rbuf[(warp * 16 + g) * MR + 2 * mp] = acc[mp][0];
            rbuf[(warp * 16 + g) * MR + 2 * mp + 1] = acc[mp][1];
            rbuf[(warp * 16 + g + 8) * MR + 2 * mp] = acc[mp][2];
            rbuf[(warp * 16 + g + 8) * MR + 2 * mp + 1] = acc[mp][3];
          }
        }
#pragma unroll
        for (int mp = 0; mp < MP; ++mp)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[mp][i] = 0.f;
        __syncthreads();   // every warp reaches this once per row block (same step count)
        const int n0 = (blockIdx.x + blk * gridDim.x) * 16;
        for (int i = tid; i < 16 * MR; i += kThreads) {
          const int r = i / MR, m = i - r * MR;
          const int n = n0 + r;
          if (n < a.N && m < a.M) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) v += rbuf[(w * 16 + r) * MR + m];
            if (a.bias) v += __ldg(a.bias + n);
            static_cast<T*>(a.y)[(size_t)m * a.N + n] = from_f32<T>(v);
          }
        }
      }
    }
  }
}

// ---- 3-8 activation rows: all eight columns of the mma carry an activation row ---------------
// The block-diagonal operand above spends an mma column per (32-block, activation row) pair: eight
// rows cost four mmas per A fragment, and mma.sync issue (one m16n8k16 per ~11 clocks per SM on
// sm_100) is what bounds the kernel.  Here the four lanes of a quad first exchange code words so
// that, for each 32-block j of the step, lane t holds word t of block j (rows g and g + 8): the 16
// k slots of an mma then all belong to ONE 32-block, its D tile is that block's partial dot
// products for 16 weight rows x 8 activation rows, and scale / zero-point are applied to D once
// per block: two mmas per block whatever the row count (256 weights per mma at 8 rows).
//
// rot4(v, s)[i] = v[(i + s) & 3] for a run-time s (two conditional stages of selects).
__device__ __forceinline__ void rot4(uint32_t (&v)[4], int s) {
  uint32_t a0 = (s & 1) ? v[1] : v[0], a1 = (s & 1) ? v[2] : v[1], a2 = (s & 1) ? v[3] : v[2],
           a3 = (s & 1) ? v[0] : v[3];
  v[0] = (s & 2) ? a2 : a0;
  v[1] = (s & 2) ? a3 : a1;
  v[2] = (s & 2) ? a0 : a2;
  v[3] = (s & 2) ? a1 : a3;
}

// In: lane t of a quad holds w[u] = word u of block t.  Out: w[j] = word t of block j.
__device__ __forceinline__ void quad_transpose(uint32_t (&w)[4], int t, int lane) {
  rot4(w, t);                                  // w[r] = word (t + r) & 3: what the lane r places back reads
  const int base = lane & ~3;
  uint32_t r1 = __shfl_sync(0xffffffffu, w[1], base | ((t - 1) & 3));   // block (t-1)&3, word t
  uint32_t r2 = __shfl_sync(0xffffffffu, w[2], base | ((t - 2) & 3));
  uint32_t r3 = __shfl_sync(0xffffffffu, w[3], base | ((t - 3) & 3));
  // v[i] = word t of block (t + i) & 3; block j sits at i = (j - t) & 3
  w[1] = r3; w[2] = r2; w[3] = r1;
  rot4(w, (4 - t) & 3);
}

template <typename T, int WARPS, bool ZP>
__global__ void __launch_bounds__(WARPS * 32, 1) q4_gemv_mma_quad_kernel(MmaArgs a, int gs_shift, int chunk) {
  constexpr int MR = 8;
  constexpr int kThreads = WARPS * 32;
  constexpr uint32_t kMagic = std::is_same<T, __nv_bfloat16>::value ? 0x43004300u : 0x64006400u;
  constexpr float kOffset = std::is_same<T, __nv_bfloat16>::value ? 128.f : 1024.f;
  extern __shared__ __align__(16) uint8_t smem[];
  const int K = a.K;
  // xs[step][h][block j][word t][activation row g][4 values]: the 32 lanes of an mma read 256
  // consecutive bytes.  xsum[32-block][activation row].  red[WARPS][chunk][16][MR]: the warps' partial
  // tiles of `chunk` row blocks meet at one barrier, not one per row block.
  T* xs = reinterpret_cast<T*>(smem);
  float* xsum = reinterpret_cast<float*>(xs + (size_t)MR * K);
  float* red = xsum + (size_t)MR * (K / 32);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int groups = K >> gs_shift;
  const int spw = K / 128 / WARPS;
  const int n_blocks = (a.N + 15) / 16;
  const int my_blocks = blockIdx.x < n_blocks ? (n_blocks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int total = my_blocks * spw;

  // Load cursor: (row block, step of this warp) of the next request; the row offsets (32-bit: the
  // host checks the sizes) change once per row block, nothing is divided per step.  Scales and zero
  // points stay as loaded (one register per 16-bit load): packing them where they are loaded would
  // make the warp wait for the loads right there instead of kPrefetch steps later.
  struct Step { uint4 ca, cb; unsigned short sA, sB, zA, zB; };
  const unsigned short* scale_u = reinterpret_cast<const unsigned short*>(a.scale);
  const unsigned short* zp_u = reinterpret_cast<const unsigned short*>(a.zp);
  int l_rb = blockIdx.x, l_si = 0;
  uint32_t l_codeA = 0, l_codeB = 0, l_grpA = 0, l_grpB = 0;
  auto load_next = [&](Step& st) {
    if (l_si == 0) {
      const int rA = l_rb * 16 + g < a.N ? l_rb * 16 + g : a.N - 1;
      const int rB = l_rb * 16 + g + 8 < a.N ? l_rb * 16 + g + 8 : a.N - 1;
      l_codeA = (uint32_t)rA * (uint32_t)(K >> 1) + (uint32_t)t * 16u;
      l_codeB = (uint32_t)rB * (uint32_t)(K >> 1) + (uint32_t)t * 16u;
      l_grpA = (uint32_t)rA * (uint32_t)groups;
      l_grpB = (uint32_t)rB * (uint32_t)groups;
    }
    const int kb = warp + l_si * WARPS;
    st.ca = __ldg(reinterpret_cast<const uint4*>(a.codes + l_codeA + kb * 64));
    st.cb = __ldg(reinterpret_cast<const uint4*>(a.codes + l_codeB + kb * 64));
    const uint32_t grp = (uint32_t)(kb * 128 + t * 32) >> gs_shift;
    st.sA = __ldg(scale_u + l_grpA + grp);
    st.sB = __ldg(scale_u + l_grpB + grp);
    if constexpr (ZP) {
      st.zA = __ldg(zp_u + l_grpA + grp);
      st.zB = __ldg(zp_u + l_grpB + grp);
    }
    if (++l_si == spw) { l_si = 0; l_rb += (int)gridDim.x; }
  };

  Step ring[kPrefetch];
#pragma unroll
  for (int p = 0; p < kPrefetch; ++p)
    if (p < total) load_next(ring[p]);

  {
    const T* x = static_cast<const T*>(a.x);
    for (int i = tid; i < MR * (K / 32); i += kThreads) {
      const int m = i % MR, blk = i / MR;     // 32-block blk = (step, block tb)
      const int step = blk >> 2, tb = blk & 3;
      float s = 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        struct alignas(16) V8 { T v[8]; } v, p;
        if (m < a.M) {
          v = *reinterpret_cast<const V8*>(x + (size_t)m * K + blk * 32 + u * 8);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) v.v[e] = from_f32<T>(0.f);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) { p.v[perm8(e)] = v.v[e]; s += to_f32(v.v[e]); }
#pragma unroll
        for (int h = 0; h < 2; ++h)
          *reinterpret_cast<uint2*>(xs + (((((size_t)step * 2 + h) * 4 + tb) * 4 + u) * 8 + m) * 4) =
              *reinterpret_cast<const uint2*>(&p.v[4 * h]);
      }
      xsum[i] = s;
    }
  }
  __syncthreads();

  float acc[4] = {0.f, 0.f, 0.f, 0.f};   // (row g, m 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)
  const int quad = lane & ~3;
  const T* xs_lane = xs + (t * 8 + g) * 4;            // + step * 1024 + (h * 4 + j) * 128
  const float* xsum_lane = xsum + 2 * t;              // + (step * 4 + j) * MR
  int c_rb = blockIdx.x, c_si = 0, c_blk = 0;         // compute cursor
  for (int base = 0; base < total; base += kPrefetch) {
#pragma unroll
    for (int p = 0; p < kPrefetch; ++p) {
      const int q = base + p;
      if (q >= total) break;
      const Step cur = ring[p];
      if (q + kPrefetch < total) load_next(ring[p]);
      const int kb = warp + c_si * WARPS;
      uint32_t wa[4] = {cur.ca.x, cur.ca.y, cur.ca.z, cur.ca.w};
      uint32_t wb[4] = {cur.cb.x, cur.cb.y, cur.cb.z, cur.cb.w};
      quad_transpose(wa, t, lane);
      quad_transpose(wb, t, lane);
      const uint32_t s2 = (uint32_t)cur.sA | ((uint32_t)cur.sB << 16);
      const uint32_t z2 = ZP ? ((uint32_t)cur.zA | ((uint32_t)cur.zB << 16)) : 0x48004800u;   // 8.0, 8.0
      const T* xb = xs_lane + (size_t)kb * 1024;
      const float* xsb = xsum_lane + kb * (4 * MR);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float d[4];
        uint32_t pa[4], pb[4];
        pa[0] = (wa[j] & 0x000f000fu) | kMagic;
        pb[0] = (wb[j] & 0x000f000fu) | kMagic;
#pragma unroll
        for (int i = 1; i < 4; ++i) {
          pa[i] = ((wa[j] >> (4 * i)) & 0x000f000fu) | kMagic;
          pb[i] = ((wb[j] >> (4 * i)) & 0x000f000fu) | kMagic;
        }
        {
          const uint32_t af[4] = {pa[0], pb[0], pa[1], pb[1]};
          const uint2 bv = *reinterpret_cast<const uint2*>(xb + j * 128);
          mma16816_first<T>(d, af, bv.x, bv.y);
        }
        {
          const uint32_t af[4] = {pa[2], pb[2], pa[3], pb[3]};
          const uint2 bv = *reinterpret_cast<const uint2*>(xb + (4 + j) * 128);
          mma16816<T>(d, af, bv.x, bv.y);
        }
        const uint32_t sj = __shfl_sync(0xffffffffu, s2, quad | j);
        const uint32_t zj = ZP ? __shfl_sync(0xffffffffu, z2, quad | j) : z2;
        const float2 sc = __half22float2(*reinterpret_cast<const __half2*>(&sj));
        const float2 zc = __half22float2(*reinterpret_cast<const __half2*>(&zj));
        const float2 xsm = *reinterpret_cast<const float2*>(xsb + j * MR);
        const float ca = kOffset + zc.x, cb = kOffset + zc.y;
        acc[0] = fmaf(sc.x, d[0] - ca * xsm.x, acc[0]);
        acc[1] = fmaf(sc.x, d[1] - ca * xsm.y, acc[1]);
        acc[2] = fmaf(sc.y, d[2] - cb * xsm.x, acc[2]);
        acc[3] = fmaf(sc.y, d[3] - cb * xsm.y, acc[3]);
      }

      if (++c_si == spw) {
        // Row block finished for this warp: every lane holds four distinct outputs.
        c_si = 0;
        float* rbuf = red + ((size_t)warp * chunk + c_blk) * 16 * MR;
        *reinterpret_cast<float2*>(rbuf + g * MR + 2 * t) = make_float2(acc[0], acc[1]);
        *reinterpret_cast<float2*>(rbuf + (g + 8) * MR + 2 * t) = make_float2(acc[2], acc[3]);
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        ++c_blk;
        if (c_blk == chunk || q + 1 == total) {
          // Every warp reaches this after the same steps.  Sum the warps' tiles of the chunk's row blocks.
          __syncthreads();
          for (int i = tid; i < c_blk * 16 * MR; i += kThreads) {
            const int b = i / (16 * MR), rm = i - b * (16 * MR);
            const int r = rm / MR, m = rm - r * MR;
            const int n = (c_rb + b * (int)gridDim.x) * 16 + r;
            if (n < a.N && m < a.M) {
              float v = 0.f;
#pragma unroll
              for (int w = 0; w < WARPS; ++w) v += red[((size_t)w * chunk + b) * 16 * MR + rm];
              if (a.bias) v += __ldg(a.bias + n);
              static_cast<T*>(a.y)[(size_t)m * a.N + n] = from_f32<T>(v);
            }
          }
          c_rb += c_blk * (int)gridDim.x;
          c_blk = 0;
          if (q + 1 < total) __syncthreads();   // the next chunk overwrites red
        }
      }
    }
  }
}

// ---- 1-2 activation rows: the decode band proper ---------------------------------------------
// One persistent CTA per SM owns a contiguous range of output rows; warp w owns the K slice
// [w*K/WARPS, (w+1)*K/WARPS) for all of them, so it stages only its own slice of the
// activations (no CTA barrier before the first mma) and keeps a ring of weight loads in
// flight across the whole row range.  An mma covers 8 output rows and TWO consecutive 128-wide
// K steps: A rows 0-7 hold step A of the 8 rows, A rows 8-15 hold step B of the same rows.
// The activation operand is block-diagonal over (32-block j, step): column 2j holds step A's
// activations in the k slots of block j, column 2j+1 step B's, so D[g][2t] and D[g+8][2t+1]
// are lane t's own partial sums for row g (the other two D values are cross terms, ignored).
// A second activation row repeats the mma.  Partial sums of the WARPS slices meet in shared
// memory once, at the end.
template <typename T, int MR, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1)
q4_gemv_mma_rows8_kernel(MmaArgs a, int rows_per_cta, int gs_shift) {
  constexpr uint32_t kMagic = std::is_same<T, __nv_bfloat16>::value ? 0x43004300u : 0x64006400u;
  constexpr float kOffset = std::is_same<T, __nv_bfloat16>::value ? 128.f : 1024.f;
  constexpr int PF = 4;
  constexpr int kZeroElems = 8 * 16 + 8;    // inactive lanes read the same offsets inside zeros
  extern __shared__ __align__(16) uint8_t smem[];
  const int K = a.K;
  const int KS = K / WARPS;                 // this warp's K slice (multiple of 256)
  const int pairs = KS / 256;               // step pairs per row group
  // 288-byte step stride: the lanes feeding step A and step B of one mma hit different banks
  const int lds = (KS / 128) * 144;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  // per-warp shared memory: xs[MR][lds] (permuted), zeros, xsum[MR][KS/32]
  const size_t warp_bytes = ((size_t)MR * lds + kZeroElems) * sizeof(T) + (size_t)MR * (KS / 32) * 4;
  uint8_t* wbase = smem + (size_t)warp * warp_bytes;
  T* xs = reinterpret_cast<T*>(wbase);
  T* zeros = xs + (size_t)MR * lds;
  float* xsum = reinterpret_cast<float*>(zeros + kZeroElems);
  float* part = reinterpret_cast<float*>(smem + (size_t)WARPS * warp_bytes);  // [WARPS][rows_per_cta][MR]

  const int r0 = blockIdx.x * rows_per_cta;
  const int r1 = r0 + rows_per_cta < a.N ? r0 + rows_per_cta : a.N;
  const int n_rg = r1 > r0 ? (r1 - r0 + 7) / 8 : 0;
  const int total = n_rg * pairs;
  const int groups = K >> gs_shift;
  const int k_lane = warp * KS + t * 32;    // first k of this lane's block in step A of pair 0

  // Scales / zero points stay as loaded (one register per 16-bit load): packing them here would make
  // the warp wait for the loads where they are issued instead of PF steps later.
  struct Step { uint4 ca, cb; unsigned short sa, sb, za, zb; };
  const unsigned short* scale_u = reinterpret_cast<const unsigned short*>(a.scale);
  const unsigned short* zp_u = reinterpret_cast<const unsigned short*>(a.zp);
  const bool has_zp = a.zp != nullptr;
  // load cursor: (row group, pair) of the next step to request
  int l_rg = 0, l_pr = 0;
  auto load_next = [&](Step& st) {
    int row = r0 + l_rg * 8 + g;
    row = row < r1 ? row : r1 - 1;
    const int kA = k_lane + l_pr * 256;                 // step B is +128
    const uint8_t* p = a.codes + (size_t)row * (K >> 1) + (kA >> 1);
    st.ca = __ldg(reinterpret_cast<const uint4*>(p));
    st.cb = __ldg(reinterpret_cast<const uint4*>(p + 64));
    const size_t sidx = (size_t)row * groups;
    const int ga = kA >> gs_shift, gb = (kA + 128) >> gs_shift;
    st.sa = __ldg(scale_u + sidx + ga);
    st.sb = __ldg(scale_u + sidx + gb);
    if (has_zp) {
      st.za = __ldg(zp_u + sidx + ga);
      st.zb = __ldg(zp_u + sidx + gb);
    } else {
      st.za = st.zb = 0x4800;   // 8.0
    }
    if (++l_pr == pairs) { l_pr = 0; ++l_rg; }
  };

  Step ring[PF];
#pragma unroll
  for (int p = 0; p < PF; ++p)
    if (p < total) load_next(ring[p]);

  // Stage this warp's activation slice: chunk j (8 values) of the slice = (step, block, word).
  {
    const T* x = static_cast<const T*>(a.x);
    const int blocks32 = KS >> 5;
    for (int i = lane; i < MR * blocks32; i += 32) {
      const int m = i / blocks32, j4 = i - m * blocks32;
      float s = 0.f;
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
        for (int e = 0; e < 8; ++e) { pv.v[perm8(e)] = v.v[e]; s += to_f32(v.v[e]); }
        const int step = j >> 4, tb = (j >> 2) & 3, u = j & 3;
        T* dst = xs + (size_t)m * lds + step * 144 + tb * 4;
        *reinterpret_cast<uint2*>(dst + (2 * u) * 16) = *reinterpret_cast<const uint2*>(&pv.v[0]);
        *reinterpret_cast<uint2*>(dst + (2 * u + 1) * 16) = *reinterpret_cast<const uint2*>(&pv.v[4]);
      }
      xsum[i] = s;
    }
    for (int i = lane; i < kZeroElems; i += 32) zeros[i] = from_f32<T>(0.f);
  }
  __syncwarp();

  // Column g of the activation operand = (block j = g/2, step = g%2); this lane holds the k
  // slots of block t, so it supplies x iff g/2 == t.
  const bool active = (g >> 1) == t;
  const T* brow[MR];
#pragma unroll
  for (int m = 0; m < MR; ++m) brow[m] = xs + (size_t)m * lds + (g & 1) * 144 + t * 4;

  float acc[MR];
#pragma unroll
  for (int m = 0; m < MR; ++m) acc[m] = 0.f;

  int c_rg = 0, c_pr = 0;   // compute cursor
  for (int base = 0; base < total; base += PF) {
#pragma unroll
    for (int p = 0; p < PF; ++p) {
      const int q = base + p;
      if (q >= total) break;
      const Step cur = ring[p];
      if (q + PF < total) load_next(ring[p]);

      float d[MR][4];
#pragma unroll
      for (int m = 0; m < MR; ++m)
#pragma unroll
        for (int i = 0; i < 4; ++i) d[m][i] = 0.f;
      const T* bp[MR];
#pragma unroll
      for (int m = 0; m < MR; ++m) bp[m] = active ? brow[m] + c_pr * 288 : zeros;
      const uint32_t wa[4] = {cur.ca.x, cur.ca.y, cur.ca.z, cur.ca.w};
      const uint32_t wb[4] = {cur.cb.x, cur.cb.y, cur.cb.z, cur.cb.w};
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
          for (int m = 0; m < MR; ++m) {
            const uint2 bv = *reinterpret_cast<const uint2*>(bp[m] + (2 * u + h) * 16);
            mma16816<T>(d[m], af, bv.x, bv.y);
          }
        }
      }
      const float2 sc = make_float2(__half2float(__ushort_as_half(cur.sa)), __half2float(__ushort_as_half(cur.sb)));
      const float2 zc = make_float2(__half2float(__ushort_as_half(cur.za)), __half2float(__ushort_as_half(cur.zb)));
      const int xb = c_pr * 8 + t;   // 32-block index of step A inside the slice; step B is +4
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        const float xa = xsum[m * (KS >> 5) + xb];
        const float xbv = xsum[m * (KS >> 5) + xb + 4];
        acc[m] = fmaf(sc.x, d[m][0] - (kOffset + zc.x) * xa, acc[m]);
        acc[m] = fmaf(sc.y, d[m][3] - (kOffset + zc.y) * xbv, acc[m]);
      }
      if (++c_pr == pairs) {
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          float v = acc[m];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          const int r = c_rg * 8 + g;
          if (t == 0 && r < rows_per_cta) part[((size_t)warp * rows_per_cta + r) * MR + m] = v;
          acc[m] = 0.f;
        }
        c_pr = 0;
        ++c_rg;
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < (r1 - r0) * MR; i += WARPS * 32) {
    const int r = MR == 1 ? i : i >> 1, m = MR == 1 ? 0 : i & 1;
    if (m < a.M) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += part[((size_t)w * rows_per_cta + r) * MR + m];
      const int n = r0 + r;
      if (a.bias) v += __ldg(a.bias + n);
      static_cast<T*>(a.y)[(size_t)m * a.N + n] = from_f32<T>(v);
    }
  }
}

template <typename T, int MR, int WARPS>
int launch_rows8(const MmaArgs& a, cudaStream_t st) {
  const int sms = sm_count();
  int rows_per_cta = (a.N + sms - 1) / sms;
  rows_per_cta = (rows_per_cta + 7) / 8 * 8 > 8 ? rows_per_cta : 8;
  const int grid = (a.N + rows_per_cta - 1) / rows_per_cta;
  const int KS = a.K / WARPS;
  const size_t warp_bytes = ((size_t)MR * (KS / 128) * 144 + 8 * 16 + 8) * sizeof(T) + (size_t)MR * (KS / 32) * 4;
  const size_t smem = (size_t)WARPS * warp_bytes + (size_t)WARPS * rows_per_cta * MR * 4;
  if (smem > (size_t)max_dynamic_smem()) return NPB_ERR_UNSUPPORTED;
  auto kern = q4_gemv_mma_rows8_kernel<T, MR, WARPS>;
  int per_sm = 0;
  if (int rc = blocks_per_sm(reinterpret_cast<const void*>(kern), WARPS * 32, smem, &per_sm)) return rc;
  if (per_sm < 1) return NPB_ERR_UNSUPPORTED;
  int gs_shift = 0;
  while ((1 << gs_shift) < a.group_size) ++gs_shift;
  if ((1 << gs_shift) != a.group_size) return NPB_ERR_UNSUPPORTED;  // power-of-two groups only
  kern<<<grid, WARPS * 32, smem, st>>>(a, rows_per_cta, gs_shift);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

template <typename T>
int run_rows8(const MmaArgs& a, cudaStream_t st) {
  // K slice per warp must be a multiple of 256 (two 128-wide steps per mma).
  if (a.K % 4096 == 0) return a.M == 1 ? launch_rows8<T, 1, 16>(a, st) : launch_rows8<T, 2, 16>(a, st);
  if (a.K % 2048 == 0) return a.M == 1 ? launch_rows8<T, 1, 8>(a, st) : launch_rows8<T, 2, 8>(a, st);
  if (a.K % 1024 == 0) return a.M == 1 ? launch_rows8<T, 1, 4>(a, st) : launch_rows8<T, 2, 4>(a, st);
  return NPB_ERR_UNSUPPORTED;
}

template <typename T, int MP, int WARPS>
int launch_mma(const MmaArgs& a, cudaStream_t st) {
  constexpr int MR = 2 * MP;
  const size_t smem = ((size_t)MR * (a.K + 16) + 8) * sizeof(T) + (size_t)MR * (a.K / 32) * 4 +
                      (size_t)2 * WARPS * 16 * MR * 4;
  if (smem > (size_t)max_dynamic_smem()) return NPB_ERR_TOO_LARGE;
  auto kern = q4_gemv_mma_kernel<T, MP, WARPS>;
  int per_sm = 0;
  if (int rc = blocks_per_sm(reinterpret_cast<const void*>(kern), WARPS * 32, smem, &per_sm)) return rc;
  if (per_sm < 1) return NPB_ERR_UNSUPPORTED;
  const int n_blocks = (a.N + 15) / 16;
  const int cap = sm_count() * per_sm;
  kern<<<n_blocks < cap ? n_blocks : cap, WARPS * 32, smem, st>>>(a);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

template <typename T, int MP>
int launch_warps(const MmaArgs& a, cudaStream_t st) {
  if (a.K % 2048 == 0) return launch_mma<T, MP, 16>(a, st);
  if (a.K % 1024 == 0) return launch_mma<T, MP, 8>(a, st);
  return launch_mma<T, MP, 4>(a, st);
}

template <typename T, int WARPS>
int launch_quad(const MmaArgs& a, cudaStream_t st) {
  const size_t fixed = (size_t)8 * a.K * sizeof(T) + (size_t)8 * (a.K / 32) * 4;
  const size_t per_block = (size_t)WARPS * 16 * 8 * 4;    // the warps' partial tiles of one row block
  const size_t cap_smem = (size_t)max_dynamic_smem();
  if (fixed + per_block > cap_smem) return NPB_ERR_UNSUPPORTED;
  const int n_blocks_all = (a.N + 15) / 16;
  int chunk = (n_blocks_all + sm_count() - 1) / sm_count();   // row blocks per CTA
  const size_t room = (cap_smem - fixed) / per_block;
  if ((size_t)chunk > room) chunk = (int)room;
  if (chunk > 16) chunk = 16;
  const size_t smem = fixed + per_block * chunk;
  auto kern = a.zp ? q4_gemv_mma_quad_kernel<T, WARPS, true> : q4_gemv_mma_quad_kernel<T, WARPS, false>;
  int per_sm = 0;
  if (int rc = blocks_per_sm(reinterpret_cast<const void*>(kern), WARPS * 32, smem, &per_sm)) return rc;
  if (per_sm < 1) return NPB_ERR_UNSUPPORTED;
  int gs_shift = 0;
  while ((1 << gs_shift) < a.group_size) ++gs_shift;
  if ((1 << gs_shift) != a.group_size) return NPB_ERR_UNSUPPORTED;      // power-of-two groups only
  if ((int64_t)a.N * (a.K >> 1) >= ((int64_t)1 << 31)) return NPB_ERR_UNSUPPORTED;   // 32-bit row offsets
  const int n_blocks = (a.N + 15) / 16;
  const int cap = sm_count() * per_sm;
  kern<<<n_blocks < cap ? n_blocks : cap, WARPS * 32, smem, st>>>(a, gs_shift, chunk);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

template <typename T>
int run_quad(const MmaArgs& a, cudaStream_t st) {
  if (a.K % 2048 == 0) return launch_quad<T, 16>(a, st);
  if (a.K % 1024 == 0) return launch_quad<T, 8>(a, st);
  return launch_quad<T, 4>(a, st);
}

template <typename T>
int run_mma(const MmaArgs& a, cudaStream_t st) {
  if (a.M >= 3) {   // every mma column carries a row: a quarter of the mmas at 8 rows
    const int rc = run_quad<T>(a, st);
    if (rc != NPB_ERR_UNSUPPORTED) return rc;
  }
  const int mp = (a.M + 1) / 2;
  switch (mp) {
    case 1: return launch_warps<T, 1>(a, st);
    case 2: return launch_warps<T, 2>(a, st);
    case 3: return launch_warps<T, 3>(a, st);
    default: return launch_warps<T, 4>(a, st);
  }
}

}  // namespace

// Returns NPB_ERR_UNSUPPORTED when the shape / dtype is not one this kernel takes; the caller
// then uses the CUDA-core GEMV.
int q4_gemv_mma(const npb_q_weight* w, const void* x, int x_dtype, int64_t M, int64_t N, int64_t K,
                const float* bias, void* y, cudaStream_t st) {
  if (w->nbits != 4 || (x_dtype != NPB_BF16 && x_dtype != NPB_F16)) return NPB_ERR_UNSUPPORTED;
  if (K % 512 != 0 || w->group_size % 32 != 0 || M < 1 || M > 8) return NPB_ERR_UNSUPPORTED;
  if (!aligned_to(w->codes, 16) || !aligned_to(x, 16)) return NPB_ERR_UNSUPPORTED;
  MmaArgs a{};
  a.codes = w->codes;
  a.scale = static_cast<const __half*>(w->scale);
  a.zp = static_cast<const __half*>(w->zero_point);
  a.bias = bias;
  a.x = x;
  a.y = y;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.group_size = w->group_size;
  if (M <= 2) {
    const int rc = x_dtype == NPB_BF16 ? run_rows8<__nv_bfloat16>(a, st) : run_rows8<__half>(a, st);
    if (rc != NPB_ERR_UNSUPPORTED) return rc;
  }
  return x_dtype == NPB_BF16 ? run_mma<__nv_bfloat16>(a, st) : run_mma<__half>(a, st);
}

}  // namespace npb
