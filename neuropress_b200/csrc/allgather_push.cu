// All-gather of out-feature shards by pushing: every rank stores its [M, N/P] slice straight
// into every rank's [M, N] output buffer (peer stores over NVLink into symmetric memory), then
// tells every peer "my slice has landed" with one flag store and waits, bounded, for the same
// flag from every peer.  One small kernel per forward instead of a collective plus a re-layout
// copy; no multicast, no TMA, plain st.global to peer addresses.
//
// Ordering: every CTA fences its stores system-wide and bumps a local counter; the CTA that
// sees the counter complete knows all stores of this rank are fenced, publishes the flags with
// release semantics and then polls its own flags with acquire semantics.  The kernel ends only
// when all peers' slices are visible here, so later kernels on the stream can read the buffer.
// The wait gives up after 2 s and records it in the status word (no trap, no endless spin).
// Ranks must run on different GPUs: two ranks waiting on each other on one GPU may never be
// resident together.
#include "common.cuh"

namespace npb {
namespace {

struct PushArgs {
  const uint8_t* src;            // [M, row_local] bytes, contiguous
  uint8_t* const* peer_out;      // device array [world]: base of each rank's [M, row_full] buffer
  uint32_t* const* peer_flags;   // device array [world]: each rank's flag words
  int64_t M, row_local, row_full;
  int rank, world;
  uint32_t epoch;
};

// Flag words of one rank: [0, world) = "slice of rank q has landed here" epochs,
// [world] = CTA completion counter, [world + 1] = status (0 ok, 1 = a wait gave up).
__global__ void __launch_bounds__(256) allgather_push_kernel(PushArgs a) {
  const int64_t chunks_per_row = a.row_local / 16;
  const int64_t per_peer = a.M * chunks_per_row;
  const int64_t total = per_peer * a.world;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int p = (int)(i / per_peer);
    const int64_t r = i - (int64_t)p * per_peer;
    const int64_t m = r / chunks_per_row, c = r - m * chunks_per_row;
    const uint4 v = *reinterpret_cast<const uint4*>(a.src + m * a.row_local + c * 16);
    // start with the next rank so that the peers' links are loaded evenly
    const int dst_rank = (a.rank + 1 + p) % a.world;
    uint8_t* dst = a.peer_out[dst_rank] + m * a.row_full + (int64_t)a.rank * a.row_local + c * 16;
    *reinterpret_cast<uint4*>(dst) = v;
  }
  __shared__ int is_last;
  __threadfence_system();
  __syncthreads();
  uint32_t* mine = a.peer_flags[a.rank];
  if (threadIdx.x == 0) {
    const unsigned old = atomicAdd(mine + a.world, 1u);
    is_last = (old == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  if (threadIdx.x == 0) mine[a.world] = 0;   // counter ready for the next launch
  if (threadIdx.x < a.world) {
    const int q = threadIdx.x;
    uint32_t* theirs = a.peer_flags[q] + a.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(a.epoch) : "memory");
    const uint32_t* wait_on = mine + q;
    uint64_t t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(wait_on) : "memory");
      if ((int32_t)(v - a.epoch) >= 0) break;
      if ((spin & 63u) == 63u) {
        uint64_t now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        if (t0 == 0) t0 = now;
        else if (now - t0 > 2000000000ull) { atomicExch(reinterpret_cast<int*>(mine + a.world + 1), 1); break; }
        __nanosleep(200);
      }
    }
  }
}

}  // namespace

int allgather_push(const void* src, int64_t M, int64_t n_local, int64_t elem_bytes,
                   const void* peer_out, const void* peer_flags, int rank, int world,
                   uint32_t epoch, cudaStream_t st) {
  if (src == nullptr || peer_out == nullptr || peer_flags == nullptr) return NPB_ERR_INVALID_ARG;
  if (world < 1 || world > 64 || rank < 0 || rank >= world || M < 0 || n_local <= 0) return NPB_ERR_INVALID_ARG;
  if (M == 0) return NPB_OK;
  const int64_t row_local = n_local * elem_bytes;
  if (row_local % 16 != 0 || !aligned_to(src, 16)) return NPB_ERR_ALIGNMENT;
  PushArgs a;
  a.src = static_cast<const uint8_t*>(src);
  a.peer_out = static_cast<uint8_t* const*>(peer_out);
  a.peer_flags = static_cast<uint32_t* const*>(peer_flags);
  a.M = M;
  a.row_local = row_local;
  a.row_full = row_local * world;
  a.rank = rank;
  a.world = world;
  a.epoch = epoch;
  const int64_t total = M * (row_local / 16) * world;
  int64_t blocks = (total + 255) / 256;
  const int cap = sm_count() * 2;
  if (blocks > cap) blocks = cap;
  allgather_push_kernel<<<(unsigned)blocks, 256, 0, st>>>(a);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

}  // namespace npb
