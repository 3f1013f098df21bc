// Device-side half of the fused "compute, then all-gather" epilogues: a kernel that produced
// this rank's [M, N/P] slice stores it straight into every rank's [M, N] buffer (peer stores
// over NVLink into symmetric memory) and finishes with the same handshake as the stand-alone
// push kernel: each CTA fences its stores system-wide and bumps a counter; the CTA that
// completes the counter publishes "my slice has landed" to every peer (release) and waits,
// bounded, until every peer's flag for this call is visible (acquire).  The kernel therefore
// ends only when the local [M, N] buffer is complete.  No multicast, no TMA: plain stores.
//
// Flag words of one rank (uint32, zero-initialised): [0, world) = epoch of the last call whose
// slice from rank q has landed here, [world] = CTA counter, [world + 1] = status (1 = a wait
// gave up after the wait limit, 2 s by default), [world + 2] = call counter (epoch source when the caller passes 0).
#pragma once

#include <stdint.h>

namespace npb {

constexpr int kMaxGatherWorld = 32;  // one lane of the signalling warp per rank

struct GatherSink {
  void* const* peer_out;        // device array [world]: base of each rank's [M, ld] buffer; null = none
  uint32_t* const* peer_flags;  // device array [world]: each rank's flag words
  int64_t ld;                   // row stride of the destination buffers, in elements
  int64_t col0;                 // first destination column of this rank's slice
  int rank, world;
  uint32_t epoch;               // 0: use the call counter in the flag words
  uint64_t wait_ns;             // limit of the wait for the peers' flags (set on the host side)
};

// Called by ONE thread of a CTA after that CTA's stores were fenced (__threadfence_system by
// the storing threads, then a CTA-level barrier).  Returns true in the last CTA to arrive.
__device__ __forceinline__ bool gather_cta_arrive(const GatherSink& g, unsigned n_ctas) {
  uint32_t* mine = g.peer_flags[g.rank];
  const unsigned old = atomicAdd(mine + g.world, 1u);
  return old == n_ctas - 1;
}

// Called by one whole warp of the last CTA.  Lane q < world signals rank q and waits for it.
__device__ __forceinline__ void gather_signal_and_wait(const GatherSink& g, int lane) {
  uint32_t* mine = g.peer_flags[g.rank];
  uint32_t epoch = g.epoch;
  if (lane == 0) {
    mine[g.world] = 0;  // counter ready for the next launch
    if (epoch == 0) {   // device-side epochs: every rank makes the same sequence of calls
      epoch = mine[g.world + 2] + 1;
      mine[g.world + 2] = epoch;
    }
  }
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  if (lane < g.world) {
    uint32_t* theirs = g.peer_flags[lane] + g.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
    const uint32_t* wait_on = mine + lane;
    uint64_t t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(wait_on) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      if ((spin & 63u) == 63u) {
        uint64_t now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        if (t0 == 0) t0 = now;
        else if (now - t0 > g.wait_ns) {
          atomicExch(reinterpret_cast<int*>(mine + g.world + 1), 1);
          break;
        }
        __nanosleep(200);
      }
    }
  }
  __syncwarp();
}

// Tail of a kernel whose CTAs have written this rank's [M, n_cols] result (a few KiB: the GEMV
// and small-batch kernels) into the rank's OWN buffer: every thread of every CTA calls it once
// its stores are issued.  The last CTA to arrive copies the slice to every peer with
// row-contiguous 16-byte stores and runs the handshake.  n_cols * sizeof(T), ld * sizeof(T) and
// col0 * sizeof(T) must be multiples of 16.
template <typename T>
__device__ __forceinline__ void gather_tail_small(const GatherSink& g, int M, int n_cols) {
  __shared__ int is_last;
  const int tid = threadIdx.x;
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = gather_cta_arrive(g, gridDim.x) ? 1 : 0;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const T* mine = static_cast<const T*>(g.peer_out[g.rank]);
  constexpr int EPC = 16 / (int)sizeof(T);  // elements per 16-byte chunk
  const int cpr = n_cols / EPC;
  for (int i = tid; i < M * cpr; i += blockDim.x) {
    const int m = i / cpr, c = i - m * cpr;
    const size_t off = (size_t)m * g.ld + g.col0 + (size_t)c * EPC;
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(mine + off));
    for (int d = 1; d < g.world; ++d) {
      T* peer = static_cast<T*>(g.peer_out[(g.rank + d) % g.world]);
      *reinterpret_cast<uint4*>(peer + off) = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < 32) gather_signal_and_wait(g, tid);
}

}  // namespace npb
