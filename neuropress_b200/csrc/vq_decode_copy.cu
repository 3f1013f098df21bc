// One-pass decode of a plain vector-quantized weight as a pipelined gather-copy.
//
// For a weight without residual codebook and row scale, the decoded matrix in a 16-bit type T is
//     W[n, 8g .. 8g+7] = T(C[idx[n, g]])            (neuropress/kernels/vq_dequant.cu:60-83)
// and both W (row-major) and the index stream are flat in v = n*G + g.  With the codebook already
// cast to T (npb_vq_codebook_cast) the whole decode is  out16[v] = table16[idx[v]]  on 16-byte
// units: no arithmetic at all.  The kernel therefore never brings a codebook entry into a
// register:
//
//   * eight producer warps turn index words into cp.async.cg copies (global -> shared, 16 bytes,
//     L2 only: a 1 MiB codebook does not live in L1 anyway) that land in a linear staging chunk
//     of 2048 vectors = 32 KiB, and count their completion on the chunk's mbarrier
//     (cp.async.mbarrier.arrive.noinc);
//   * one thread of a ninth warp waits for a chunk, makes it visible to the async proxy and
//     writes it out with ONE 1-D bulk copy (cp.async.bulk, shared -> global, 32 KiB), then hands
//     the stage back once the previous store has read its shared memory.
//
// Six stages = 12 288 gathers in flight per SM, bounded by shared memory instead of registers
// (the thread-per-vector decode in vq_decode.cu keeps ~2 per thread).  Bound: L2 gather rate for
// a 65536-entry codebook, HBM write for small ones.  Algorithmic bytes: index bytes + 16 bytes
// per vector out.  Bit-exact against the thread-per-vector decode.  Every wait is bounded.
#include "common.cuh"
#include "tcgen05.cuh"

namespace npb {

__device__ int g_vq_copy_status = 0;  // 0 ok; 1 a producer's wait gave up, 2 the store thread's

namespace {

using namespace sm100;

constexpr int kProducerWarps = 8;
constexpr int kThreads = (kProducerWarps + 1) * 32;     // + the store warp
constexpr int kChunkVectors = kProducerWarps * 32 * 8;   // 2048: eight vectors per producer thread
constexpr int kChunkBytes = kChunkVectors * 16;          // 32 KiB
constexpr int kStages = 6;
constexpr int kSmemBytes = 1024 + kStages * kChunkBytes;

struct CopyArgs {
  const uint8_t* packed;
  const uint8_t* table;      // codebook in the output type, 16 bytes per entry
  uint8_t* out;
  uint64_t wait_ns;
  int64_t n_vectors;         // multiple of 8
  uint32_t G;                // vectors per row
  uint32_t groups_per_codebook, num_centroids, table_rows;
  int clamp;
};

__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 1-D bulk copy shared -> global (bytes: multiple of 16, both addresses 16-byte aligned).
__device__ __forceinline__ void bulk_store(void* gmem_dst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_src),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns once all but the newest `N` committed bulk stores have finished reading shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int BITS>
struct IndexWords {
  uint32_t w[BITS / 4];
};

template <int BITS>
__device__ __forceinline__ void load_words(IndexWords<BITS>& it, const uint8_t* packed, int64_t item) {
  const uint8_t* q = packed + item * BITS;   // eight indices = BITS bytes
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
}

template <int BITS>
__device__ __forceinline__ uint32_t index_of(const IndexWords<BITS>& it, int i) {
  if constexpr (BITS == 16) return (i & 1) ? it.w[i >> 1] >> 16 : it.w[i >> 1] & 0xffffu;
  if constexpr (BITS == 8) return (it.w[i >> 2] >> (8 * (i & 3))) & 0xffu;
  const int bit = i * BITS;
  const uint32_t lo = it.w[bit / 32];
  const uint32_t hi = (bit / 32 + 1 < BITS / 4) ? it.w[bit / 32 + 1] : 0u;
  return (uint32_t)((((uint64_t)hi << 32) | lo) >> (bit % 32)) & ((1u << BITS) - 1u);
}

template <int BITS>
__global__ void __launch_bounds__(kThreads, 1)
vq_decode_copy_kernel(const CopyArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);    // [kStages] all of a chunk's copies have landed
  uint64_t* empty_bar = full_bar + kStages;                  // [kStages] the chunk's store has read the stage
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kStages);
  uint8_t* stage0 = smem + 896;                              // 16-byte aligned

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n_chunks = (a.n_vectors + kChunkVectors - 1) / kChunkVectors;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], kProducerWarps * 32);
      mbar_init(&empty_bar[s], 1);
    }
    fence_barrier_init();
  }
  __syncthreads();

  if (warp < kProducerWarps) {
    const int t = warp * 32 + lane;                          // this thread's item inside a chunk
    const uint32_t dst0 = smem_u32(stage0) + (uint32_t)t * 128u;
    IndexWords<BITS> cur, nxt;
    int64_t c = blockIdx.x;
    auto item_of = [&](int64_t chunk) { return chunk * (kChunkVectors / 8) + t; };   // 8-vector items
    const int64_t n_items = a.n_vectors >> 3;
    if (c < n_chunks && item_of(c) < n_items) load_words<BITS>(cur, a.packed, item_of(c));
    int s = 0;
    uint32_t ph = 0;
    for (; c < n_chunks; c += gridDim.x) {
      const int64_t cn = c + gridDim.x;
      if (cn < n_chunks && item_of(cn) < n_items) load_words<BITS>(nxt, a.packed, item_of(cn));
      if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, abort_flag, a.wait_ns, 32u)) {
        atomicExch(&g_vq_copy_status, 1);
        break;
      }
      const int64_t item = item_of(c);
      if (item < n_items) {
        uint32_t off = 0;
        if (a.groups_per_codebook) off = (uint32_t)(((item << 3) % a.G) / a.groups_per_codebook) * a.num_centroids;
        const uint32_t dst = dst0 + (uint32_t)s * kChunkBytes;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint32_t e = index_of<BITS>(cur, i);
          if (a.clamp) e = min(e + off, a.table_rows - 1u);   // an index past the codebook reads its last entry
          cp_async_16(dst + 16u * i, a.table + ((size_t)e << 4));
        }
      }
      cp_async_arrive(&full_bar[s]);   // every producer thread, also one without an item in a ragged last chunk
      cur = nxt;
      if (++s == kStages) { s = 0; ph ^= 1; }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (lane == 0) {
    // ---- store thread ----
    int s = 0;
    uint32_t ph = 0;
    int prev = -1;
    for (int64_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
      if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag, a.wait_ns)) {
        atomicExch(&g_vq_copy_status, 2);
        break;
      }
      fence_proxy_async_smem();   // the chunk was written through the generic proxy (cp.async)
      const int64_t v0 = c * kChunkVectors;
      const int64_t left = a.n_vectors - v0;
      const uint32_t bytes = (uint32_t)(left < kChunkVectors ? left : kChunkVectors) * 16u;
      bulk_store(a.out + (v0 << 4), smem_u32(stage0) + (uint32_t)s * kChunkBytes, bytes);
      bulk_commit();
      if (prev >= 0) {              // the store before this one has read its stage: hand it back
        bulk_wait_read<1>();
        mbar_arrive(&empty_bar[prev]);
      }
      prev = s;
      if (++s == kStages) { s = 0; ph ^= 1; }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // all stores complete before the CTA's memory goes
  }
  __syncthreads();
}

template <int BITS>
int launch(const CopyArgs& a, cudaStream_t st) {
  auto kern = vq_decode_copy_kernel<BITS>;
  static int configured[64] = {0};
  int dev = 0;
  NPB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    NPB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    configured[dev] = 1;
  }
  const int64_t n_chunks = (a.n_vectors + kChunkVectors - 1) / kChunkVectors;
  const int sms = sm_count();
  const unsigned grid = (unsigned)(n_chunks < sms ? n_chunks : sms);
  kern<<<grid, kThreads, kSmemBytes, st>>>(a);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

}  // namespace

// Reads and clears the give-up record of the copy-form decode (synchronises).
int vq_decode_copy_device_status(int* host_out) {
  int v = 0;
  NPB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_vq_copy_status, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    NPB_CUDA_TRY(cudaMemcpyToSymbol(g_vq_copy_status, &zero, sizeof(int)));
  }
  if (host_out) *host_out = v;
  return NPB_OK;
}

// table_x: the codebook in the output type (vq_codebook_cast).  NPB_ERR_UNSUPPORTED when the weight
// or the sizes are outside the copy form's domain: the caller then runs vq_decode.
int vq_decode_copy(const npb_vq_weight* w, const void* table_x, int64_t N, int64_t K, void* out, int out_dtype,
                   cudaStream_t st) {
  if (int rc = validate_vq(w, N, K)) return rc;
  if (table_x == nullptr || (out == nullptr && N * K > 0)) return NPB_ERR_INVALID_ARG;
  if (out_dtype != NPB_BF16 && out_dtype != NPB_F16) return NPB_ERR_UNSUPPORTED;
  if (N * K == 0) return NPB_OK;
  if (w->res_packed != nullptr || w->row_scale != nullptr || w->vector_len != 8) return NPB_ERR_UNSUPPORTED;
  if (w->bits != 16 && w->bits != 12 && w->bits != 8) return NPB_ERR_UNSUPPORTED;
  if (K % 64 != 0 || (w->cols_per_codebook > 0 && w->cols_per_codebook % 64 != 0)) return NPB_ERR_UNSUPPORTED;
  if (!aligned_to(out, 16) || !aligned_to(table_x, 16) || !aligned_to(w->packed, w->bits == 12 ? 4 : w->bits))
    return NPB_ERR_ALIGNMENT;
  CopyArgs a{};
  a.packed = w->packed;
  a.table = static_cast<const uint8_t*>(table_x);
  a.out = static_cast<uint8_t*>(out);
  a.wait_ns = wait_limit_ns();
  a.G = (uint32_t)(K / 8);
  a.n_vectors = N * (K / 8);
  a.groups_per_codebook = w->cols_per_codebook > 0 ? (uint32_t)(w->cols_per_codebook / 8) : 0u;
  a.num_centroids = (uint32_t)w->num_centroids;
  a.table_rows = (uint32_t)w->num_centroids *
                 (w->cols_per_codebook > 0 ? (uint32_t)((K + w->cols_per_codebook - 1) / w->cols_per_codebook) : 1u);
  a.clamp = (w->num_centroids != (1 << w->bits)) || a.groups_per_codebook > 0;
  switch (w->bits) {
    case 16: return launch<16>(a, st);
    case 12: return launch<12>(a, st);
    default: return launch<8>(a, st);
  }
}

}  // namespace npb
