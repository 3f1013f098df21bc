// Decode + dense GEMM for callers that cannot allocate device memory.
//
// The large-batch band needs a temporary dense weight [N, K] between its two kernels.  The
// regular entry points leave that buffer to the caller (the Python layer takes it from torch's
// caching allocator).  Some callers have no allocator to ask: a C or C++ host that was handed a
// fixed set of buffers, a serving loop that must not call cudaMalloc because it synchronises the
// whole device and can fail under memory pressure, code running where the framework's allocator
// is not reachable.  For them this file keeps one fixed scratch array inside the library image.
//
// Cost: NPB_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the library, held
// until the process exits.  Every call uses the same array, so two calls that run on the GPU at
// the same time (different streams, or different host threads) overwrite each other's weight;
// calls must be ordered on one stream.  Nothing in the array has to start at zero: the decode
// writes every element that the GEMM of the same call reads, and what an earlier call left
// behind is never read.
#include <mutex>

#include "common.cuh"

namespace npb {

int vq_decode(const npb_vq_weight*, int64_t, int64_t, void*, int, cudaStream_t);
int gemm(const void*, const void*, const float*, void*, int64_t, int64_t, int64_t, int,
         cudaStream_t);

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[NPB_STATIC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address;
// the address of each device's copy is looked up once, with that device current.  The cache is
// guarded, so host threads that make their first call on a device together do not race.
void* g_scratch_addr[64] = {nullptr};
std::mutex g_scratch_mutex;

int scratch_address(void** out) {
  int dev = 0;
  NPB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return NPB_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    NPB_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
    if (p == nullptr || !aligned_to(p, 256)) return NPB_ERR_ALIGNMENT;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return NPB_OK;
}

}  // namespace

int vq_linear_static_scratch(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M,
                             int64_t N, int64_t K, const float* bias, void* y, cudaStream_t st) {
  if (x_dtype != NPB_BF16 && x_dtype != NPB_F16) return NPB_ERR_UNSUPPORTED;
  if (M < 0 || N < 0 || K < 0) return NPB_ERR_INVALID_ARG;
  // 2 bytes per decoded element; checked before anything is launched.
  if (N > 0 && K > 0 && (uint64_t)N * (uint64_t)K > (uint64_t)NPB_STATIC_SCRATCH_BYTES / 2)
    return NPB_ERR_TOO_LARGE;
  if (M == 0 || N == 0) return NPB_OK;
  // Everything the GEMM would reject is rejected here, before the decode is launched.
  if (x == nullptr || y == nullptr) return NPB_ERR_INVALID_ARG;
  if (K == 0 || K % 8 != 0) return NPB_ERR_SHAPE;
  if (!aligned_to(x, 16)) return NPB_ERR_ALIGNMENT;
  if (M >= (int64_t)1 << 31 || N >= (int64_t)1 << 31 || K >= (int64_t)1 << 31) return NPB_ERR_UNSUPPORTED;
  if (int rc = validate_vq(w, N, K)) return rc;
  void* scratch = nullptr;
  if (int rc = scratch_address(&scratch)) return rc;
  if (int rc = vq_decode(w, N, K, scratch, x_dtype, st)) return rc;
  return gemm(x, scratch, bias, y, M, N, K, x_dtype, st);
}

}  // namespace npb
