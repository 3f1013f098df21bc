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
// The wait gives up after the wait limit (2 s unless npb_set_wait_limit_ns changed it) and records it in the status word (no trap, no endless spin).
// Ranks must run on different GPUs: two ranks waiting on each other on one GPU may never be
// resident together.
#include "common.cuh"
#include "gather_sink.cuh"

namespace npb {
namespace {

struct PushArgs {
  const uint8_t* src;            // [M, row_local] bytes, contiguous
  uint8_t* const* peer_out;      // device array [world]: base of each rank's [M, row_full] buffer
  uint32_t* const* peer_flags;   // device array [world]: each rank's flag words
  int64_t M, row_local, row_full;
  int rank, world;
  uint32_t epoch;
  uint64_t wait_ns;
};

// The flag words and the closing handshake are those of gather_sink.cuh; epoch 0 takes the
// epoch from the call counter there, which keeps the launch arguments constant and so lets
// the call be replayed from a CUDA graph.
constexpr int kPushUnroll = 4;

__global__ void __launch_bounds__(256) allgather_push_kernel(PushArgs a) {
  const int64_t chunks_per_row = a.row_local / 16;
  const int64_t per_peer = a.M * chunks_per_row;
  const int64_t total = per_peer * a.world;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // kPushUnroll independent 16-byte loads, then the stores: more bytes in flight per thread.
  for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += stride * kPushUnroll) {
    uint4 v[kPushUnroll];
    uint8_t* dst[kPushUnroll];
#pragma unroll
    for (int u = 0; u < kPushUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      dst[u] = nullptr;
      if (i < total) {
        const int p = (int)(i / per_peer);
        const int64_t r = i - (int64_t)p * per_peer;
        const int64_t m = r / chunks_per_row, c = r - m * chunks_per_row;
        v[u] = *reinterpret_cast<const uint4*>(a.src + m * a.row_local + c * 16);
        // start with the next rank so that the peers' links are loaded evenly
        const int dst_rank = (a.rank + 1 + p) % a.world;
        dst[u] = a.peer_out[dst_rank] + m * a.row_full + (int64_t)a.rank * a.row_local + c * 16;
      }
    }
#pragma unroll
    for (int u = 0; u < kPushUnroll; ++u)
      if (dst[u] != nullptr) *reinterpret_cast<uint4*>(dst[u]) = v[u];
  }
  __shared__ int is_last;
  __threadfence_system();
  __syncthreads();
  GatherSink g;
  g.peer_out = nullptr;
  g.peer_flags = a.peer_flags;
  g.ld = 0; g.col0 = 0;
  g.rank = a.rank; g.world = a.world; g.epoch = a.epoch; g.wait_ns = a.wait_ns;
  if (threadIdx.x == 0) is_last = gather_cta_arrive(g, gridDim.x);
  __syncthreads();
  if (!is_last) return;
  if (threadIdx.x < 32) gather_signal_and_wait(g, threadIdx.x);
}

}  // namespace

int allgather_push(const void* src, int64_t M, int64_t n_local, int64_t elem_bytes,
                   const void* peer_out, const void* peer_flags, int rank, int world,
                   uint32_t epoch, cudaStream_t st) {
  if (src == nullptr || peer_out == nullptr || peer_flags == nullptr) return NPB_ERR_INVALID_ARG;
  if (world < 1 || world > 32 || rank < 0 || rank >= world || M < 0 || n_local <= 0) return NPB_ERR_INVALID_ARG;
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
  a.wait_ns = wait_limit_ns();
  const int64_t total = M * (row_local / 16) * world;
  int64_t blocks = (total + 255) / 256;
  const int cap = sm_count() * 2;
  if (blocks > cap) blocks = cap;
  allgather_push_kernel<<<(unsigned)blocks, 256, 0, st>>>(a);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

}  // namespace npb
