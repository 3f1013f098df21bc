// Entropy-coded index streams -> the plain 16-bit index table.
//
// The reference offers three prefix codes for frequency-sorted codebooks
// (neuropress/transforms/vq_packing.py: TieredIndexPacking :298-610, NTieredIndexPacking :612-1034,
// ZeroEscapePacking :1037-1384) with a GEMV kernel each (neuropress/kernels/vq_linear_tiered.cu,
// vq_linear_ntier.cu, vq_linear_zero_escape.cu).  All three are "a tier id per index from a prefix
// stream + a payload of bits[tier] bits at the index's rank inside its tier's stream":
//
//   kind 1  cascaded one-bit prefixes (two-tier and N-tier): prefix stream k holds one bit for
//           every index that is not in a tier < k (0 = tier k, 1 = a later tier);
//   kind 2  one flat two-bit prefix per index = its tier (zero escape; tier 0 has no payload).
//
// A rank is a global prefix sum, so the packers also provide, per tier, the number of its
// indices before every row (row offsets); with those a row decodes independently.  This kernel
// gives one warp a row: a lane takes 32 (kind 2: 16) consecutive indices = one 32-bit prefix
// word, tier counts are exclusive-scanned across the warp, and every index's payload is read
// straight from its bit position.  The output is the plain little-endian uint16 index table
// [N, G] every other kernel of the library takes (bits = 16), so all row-count bands work on
// entropy-coded layers: expand, then the band's kernel.  HBM traffic: coded bytes in, 2 bytes per
// index out.  Integer work only; bit-exact against the packers' unpack().
#include "common.cuh"

namespace npb {
namespace {

struct EntropyDev {
  const uint8_t* buf;
  int64_t buf_bytes;
  int kind, n_tiers;
  int64_t prefix_bit[3];   // bit position of prefix stream k's first bit in buf
  int64_t tier_bit[4];     // bit position of tier k's payload stream
  int tier_bits[4];        // payload width (0: none)
  int tier_lo[4];          // value added to a payload
  const int32_t* row_off[4];
};

// 32-bit word i of the buffer; bytes past the end read as zero (buf is 4-byte aligned).
__device__ __forceinline__ uint32_t load_word(const EntropyDev& e, int64_t i) {
  const int64_t b = i * 4;
  if (b + 4 <= e.buf_bytes) return __ldg(reinterpret_cast<const uint32_t*>(e.buf) + i);
  uint32_t v = 0;
  for (int k = 0; k < 4; ++k)
    if (b + k < e.buf_bytes) v |= (uint32_t)__ldg(e.buf + b + k) << (8 * k);
  return v;
}

// The 32 stream bits that start at bit position `pos` (LSB first).
__device__ __forceinline__ uint32_t read_bits32(const EntropyDev& e, int64_t pos) {
  const int64_t w = pos >> 5;
  const uint32_t sh = (uint32_t)pos & 31u;
  const uint32_t lo = load_word(e, w);
  if (sh == 0) return lo;
  return __funnelshift_r(lo, load_word(e, w + 1), sh);
}

__device__ __forceinline__ uint32_t low_mask(int n) { return n >= 32 ? 0xffffffffu : ((1u << n) - 1u); }

__device__ __forceinline__ int warp_excl_scan(int v, int lane, int& total) {
  int incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += t;
  }
  total = __shfl_sync(0xffffffffu, incl, 31);
  return incl - v;
}

constexpr int kWarps = 8;

template <typename V>
__device__ __forceinline__ V pick4(const V (&a)[4], int k) {
  return k == 0 ? a[0] : k == 1 ? a[1] : k == 2 ? a[2] : a[3];
}

// KIND 1: D tiers behind D - 1 cascaded one-bit prefix streams.  KIND 2: four tiers, flat prefix.
template <int KIND, int D>
__global__ void __launch_bounds__(kWarps * 32)
entropy_expand_kernel(const EntropyDev e, int64_t N, int G, uint16_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (row >= N) return;
  constexpr int PER_LANE = KIND == 1 ? 32 : 16;   // indices per lane and chunk = one 32-bit prefix word
  int64_t tier_rank0[4] = {0, 0, 0, 0};  // rank, inside its tier's stream, of the row's first index of the tier
  int64_t rest_pos0[3] = {0, 0, 0};      // KIND 1: position in prefix stream k of the row's first unplaced index
  {
    int64_t placed = 0;
#pragma unroll
    for (int k = 0; k < D; ++k) {
      tier_rank0[k] = (int64_t)__ldg(e.row_off[k] + row);
      if (k < 3) rest_pos0[k] = row * G - placed;
      placed += tier_rank0[k];
    }
  }
  int tier_seen[4] = {0, 0, 0, 0};       // indices of each tier in the row's chunks so far
  uint16_t* dst_row = out + row * G;

  for (int c0 = 0; c0 < G; c0 += 32 * PER_LANE) {
    const int first = c0 + lane * PER_LANE;   // this lane's first index in the row
    const int valid = max(0, min(PER_LANE, G - first));
    uint32_t w[3] = {0, 0, 0};
    int cnt[4] = {0, 0, 0, 0};                // this lane's indices per tier
    if (KIND == 1) {
      int population = valid;                 // this lane's indices not placed in a tier < k
      int unplaced_before_chunk = c0;         // of the row, before this chunk
      int before = first - c0;                // of this chunk, before this lane
#pragma unroll
      for (int k = 0; k < D - 1; ++k) {
        if (k > 0) {
          int tot;
          before = warp_excl_scan(population, lane, tot);
          unplaced_before_chunk -= tier_seen[k - 1];
        }
        const int64_t pos = rest_pos0[k] + unplaced_before_chunk + before;
        w[k] = population > 0 ? (read_bits32(e, e.prefix_bit[k] + pos) & low_mask(population)) : 0u;
        const int rest = __popc(w[k]);
        cnt[k] = population - rest;
        population = rest;
      }
      cnt[D - 1] = population;
    } else {
      const uint32_t p =
          valid > 0 ? (read_bits32(e, e.prefix_bit[0] + 2 * (row * G + first)) & low_mask(2 * valid)) : 0u;
      w[0] = p;
      const uint32_t lo = p & 0x55555555u, hi = (p >> 1) & 0x55555555u;
      cnt[1] = __popc(lo & ~hi);
      cnt[2] = __popc(hi & ~lo);
      cnt[3] = __popc(lo & hi);
      cnt[0] = valid - cnt[1] - cnt[2] - cnt[3];
    }
    int64_t rank_base[4] = {0, 0, 0, 0};      // rank of this lane's first index of each tier
    int tot[4] = {0, 0, 0, 0};
#pragma unroll
    for (int k = 0; k < D; ++k)
      rank_base[k] = tier_rank0[k] + tier_seen[k] + warp_excl_scan(cnt[k], lane, tot[k]);

    // whole groups of eight indices at 16-byte aligned places take vector stores
    const bool vec_ok = (valid & 7) == 0 && ((reinterpret_cast<uintptr_t>(dst_row + first) & 15u) == 0);
    uint32_t acc[4] = {0, 0, 0, 0};
    for (int j = 0; j < valid; ++j) {
      int k = 0, r = 0;
      if (KIND == 1) {
        int p = j;          // position inside the current population (this lane's part of it)
        bool placed = false;
#pragma unroll
        for (int t = 0; t < D - 1; ++t) {
          if (!placed) {
            const int ones_before = __popc(w[t] & low_mask(p));
            if ((w[t] >> p) & 1u) { p = ones_before; k = t + 1; }
            else { r = p - ones_before; placed = true; }
          }
        }
        if (!placed) r = p;
      } else {
        const uint32_t lo = w[0] & 0x55555555u, hi = (w[0] >> 1) & 0x55555555u;
        k = (int)((w[0] >> (2 * j)) & 3u);
        const uint32_t sel = k == 1 ? (lo & ~hi) : k == 2 ? (hi & ~lo) : k == 3 ? (lo & hi) : (~(lo | hi) & 0x55555555u);
        r = __popc(sel & low_mask(2 * j));
      }
      uint32_t v = (uint32_t)e.tier_lo[k];
      const int nb = e.tier_bits[k];
      if (nb > 0) v += read_bits32(e, e.tier_bit[k] + (pick4(rank_base, k) + r) * nb) & low_mask(nb);
      v = min(v, 65535u);
      if (vec_ok) {
        // eight indices per 16-byte store (a lane's run of 2-byte stores would touch a sector each)
        const int q = j & 7;
        if (q & 1) acc[q >> 1] |= v << 16; else acc[q >> 1] = v;
        if (q == 7) *reinterpret_cast<uint4*>(dst_row + first + j - 7) = make_uint4(acc[0], acc[1], acc[2], acc[3]);
      } else {
        dst_row[first + j] = (uint16_t)v;
      }
    }
#pragma unroll
    for (int k = 0; k < D; ++k) tier_seen[k] += tot[k];
  }
}

}  // namespace

int vq_entropy_expand(const npb_vq_entropy_stream* s, int64_t N, int64_t G, void* out_u16, cudaStream_t st) {
  if (s == nullptr || N < 0 || G < 0) return NPB_ERR_INVALID_ARG;
  if (N == 0 || G == 0) return NPB_OK;
  if (s->buf == nullptr || out_u16 == nullptr || s->buf_bytes <= 0) return NPB_ERR_INVALID_ARG;
  if (s->kind != 1 && s->kind != 2) return NPB_ERR_INVALID_ARG;
  if (s->n_tiers < 2 || s->n_tiers > 4 || (s->kind == 2 && s->n_tiers != 4)) return NPB_ERR_INVALID_ARG;
  if (G >= (int64_t)1 << 30 || N * G >= (int64_t)1 << 40) return NPB_ERR_UNSUPPORTED;
  if (!aligned_to(s->buf, 4) || !aligned_to(out_u16, 2)) return NPB_ERR_ALIGNMENT;
  EntropyDev e{};
  e.buf = s->buf;
  e.buf_bytes = s->buf_bytes;
  e.kind = s->kind;
  e.n_tiers = s->n_tiers;
  const int n_prefix = s->kind == 1 ? s->n_tiers - 1 : 1;
  for (int k = 0; k < 3; ++k) {
    if (k < n_prefix && (s->prefix_off[k] < 0 || s->prefix_off[k] > s->buf_bytes)) return NPB_ERR_SHAPE;
    e.prefix_bit[k] = k < n_prefix ? s->prefix_off[k] * 8 : 0;
  }
  for (int k = 0; k < 4; ++k) {
    const bool used = k < s->n_tiers;
    if (used) {
      if (s->tier_bits[k] < 0 || s->tier_bits[k] > 20 || s->tier_lo[k] < 0) return NPB_ERR_INVALID_ARG;
      if (s->tier_off[k] < 0 || s->tier_off[k] > s->buf_bytes) return NPB_ERR_SHAPE;
      if (s->row_off[k] == nullptr) return NPB_ERR_INVALID_ARG;
      if (!aligned_to(s->row_off[k], 4)) return NPB_ERR_ALIGNMENT;
    }
    e.tier_bit[k] = used ? s->tier_off[k] * 8 : 0;
    e.tier_bits[k] = used ? s->tier_bits[k] : 0;
    e.tier_lo[k] = used ? s->tier_lo[k] : 0;
    e.row_off[k] = used ? s->row_off[k] : s->row_off[0];
  }
  const unsigned blocks = (unsigned)((N + kWarps - 1) / kWarps);
  uint16_t* out = static_cast<uint16_t*>(out_u16);
  if (s->kind == 2) entropy_expand_kernel<2, 4><<<blocks, kWarps * 32, 0, st>>>(e, N, (int)G, out);
  else if (s->n_tiers == 2) entropy_expand_kernel<1, 2><<<blocks, kWarps * 32, 0, st>>>(e, N, (int)G, out);
  else if (s->n_tiers == 3) entropy_expand_kernel<1, 3><<<blocks, kWarps * 32, 0, st>>>(e, N, (int)G, out);
  else entropy_expand_kernel<1, 4><<<blocks, kWarps * 32, 0, st>>>(e, N, (int)G, out);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

}  // namespace npb
