// extern "C" surface of libneuropress_b200.so: argument validation, status strings and the
// thin forwarding layer onto the kernels.  No torch types, no allocation, no host sync.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <tuple>
#include <map>

#include "common.cuh"
#include "gather_sink.cuh"

namespace npb {

// kernels (one translation unit each)
int vq_decode(const npb_vq_weight*, int64_t, int64_t, void*, int, cudaStream_t);
int vq_gemv(const npb_vq_weight*, const void*, int, int64_t, int64_t, int64_t, const float*,
            void*, cudaStream_t);
int q_decode(const npb_q_weight*, int64_t, int64_t, void*, int, cudaStream_t);
int q_gemv(const npb_q_weight*, const void*, int, int64_t, int64_t, int64_t, const float*, void*,
           cudaStream_t);
int gemm(const void*, const void*, const float*, void*, int64_t, int64_t, int64_t, int,
         cudaStream_t);
int vq_codebook_cast(const void*, int64_t, void*, int, cudaStream_t);
int vq_gemm_fused_grouped(const npb_vq_weight*, int, const void* const*, const int64_t*, const float* const*,
                          const void*, int, int64_t, int64_t, void*, cudaStream_t);
int vq_lut_gather(const float*, int64_t, int64_t, int64_t, const uint8_t*, int64_t, int, int64_t, float*, cudaStream_t);
int vq_decode_copy(const npb_vq_weight*, const void*, int64_t, int64_t, void*, int, cudaStream_t);
int vq_entropy_expand(const npb_vq_entropy_stream*, int64_t, int64_t, void*, cudaStream_t);
int vq_gemm_fused(const npb_vq_weight*, const void*, const void*, int, int64_t, int64_t, int64_t,
                  const float*, void*, cudaStream_t);
int q_gemm_fused(const npb_q_weight*, const void*, int, int64_t, int64_t, int64_t, const float*,
                 void*, cudaStream_t);

int gemm_device_status(int*);
int vq_gemv_mma(const npb_vq_weight*, const void*, int, int64_t, int64_t, int64_t, const float*, void*,
                const GatherSink*, cudaStream_t);
int rms_norm(const void*, const void*, void*, int64_t, int64_t, float, int, cudaStream_t);
int vq_gemv_grouped(const npb_vq_weight*, int, const int64_t*, const float* const*, const void*, int, int64_t,
                    int64_t, const void*, float, void*, cudaStream_t);
int vq_embedding(const int64_t*, int64_t, const uint16_t*, int64_t, int64_t, const void*, int, int, const int64_t*,
                 float, void*, int, cudaStream_t);
int q_embedding(const int64_t*, int64_t, const npb_q_weight*, int64_t, int64_t, int64_t, float, void*, int,
                cudaStream_t);
int gemm_gather(const void*, const void*, const float*, int64_t, int64_t, int64_t, int, const GatherSink&,
                cudaStream_t);
int vq_gemv_gather(const npb_vq_weight*, const void*, int, int64_t, int64_t, int64_t, const float*,
                   const GatherSink&, cudaStream_t);
int allgather_push(const void*, int64_t, int64_t, int64_t, const void*, const void*, int, int, uint32_t,
                   cudaStream_t);
int vq_linear_static_scratch(const npb_vq_weight*, const void*, int, int64_t, int64_t, int64_t,
                             const float*, void*, cudaStream_t);

static thread_local char g_last_error[256] = "";

static std::atomic<uint64_t> g_wait_limit_ns{2000000000ull};
uint64_t wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }

// 0 never, 1 where the shape fills pair tiles (default), 2 for every dense GEMM of more than
// 128 rows.  NEUROPRESS_B200_GEMM_PAIRS gives the initial value.
static std::atomic<int> g_gemm_pair_mode{[] {
  const char* e = getenv("NEUROPRESS_B200_GEMM_PAIRS");
  return (e && e[0] >= '0' && e[0] <= '2' && e[1] == 0) ? e[0] - '0' : 1;
}()};
int gemm_pair_mode() { return g_gemm_pair_mode.load(std::memory_order_relaxed); }

void set_last_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", where, cudaGetErrorName(e),
           cudaGetErrorString(e));
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int max_dynamic_smem() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 48 * 1024;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess ||
        n <= 0)
      n = 48 * 1024;
    cached[dev] = n;
  }
  return cached[dev];
}

int blocks_per_sm(const void* kernel, int threads, size_t smem, int* per_sm) {
  static std::mutex mu;
  static std::map<std::tuple<int, const void*, size_t>, int> cache;
  // Largest dynamic shared-memory size opted into so far, per device and kernel: the attribute
  // is a maximum, so it is only ever raised (lowering it would break a later, larger launch).
  static std::map<std::pair<int, const void*>, size_t> opted;
  int dev = 0;
  NPB_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  const auto key = std::make_tuple(dev, kernel, smem);
  auto it = cache.find(key);
  if (it == cache.end()) {
    // opt in as soon as dynamic + (small) static shared memory can pass the 48 KiB default
    size_t& have = opted[std::make_pair(dev, kernel)];
    if (smem + 1024 > 48 * 1024 && smem > have) {
      NPB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      have = smem;
    }
    int n = 0;
    NPB_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem));
    it = cache.emplace(key, n).first;
  }
  *per_sm = it->second;
  return NPB_OK;
}

int validate_vq(const npb_vq_weight* w, int64_t N, int64_t K) {
  if (w == nullptr || N < 0 || K < 0) return NPB_ERR_INVALID_ARG;
  if (w->vector_len != 4 && w->vector_len != 8) return NPB_ERR_UNSUPPORTED;
  if (w->bits < 4 || w->bits > 16) return NPB_ERR_UNSUPPORTED;
  if (K % w->vector_len != 0) return NPB_ERR_SHAPE;
  const int64_t n_vectors = N * (K / w->vector_len);
  if (n_vectors == 0) return NPB_OK;
  if (w->packed == nullptr || w->centroids == nullptr) return NPB_ERR_INVALID_ARG;
  if (w->num_centroids <= 0 || w->num_centroids > (1 << w->bits)) {
    // A codebook larger than the index range is legal (unused rows); smaller than 1 is not.
    if (w->num_centroids <= 0) return NPB_ERR_INVALID_ARG;
  }
  if ((n_vectors * w->bits + 7) / 8 > w->packed_bytes) return NPB_ERR_SHAPE;
  if (w->cols_per_codebook < 0 || (w->cols_per_codebook % w->vector_len) != 0)
    return NPB_ERR_SHAPE;
  if (w->res_packed != nullptr) {
    if (w->res_centroids == nullptr || w->res_num_centroids <= 0) return NPB_ERR_INVALID_ARG;
    if (w->res_bits < 4 || w->res_bits > 16) return NPB_ERR_UNSUPPORTED;
    if ((n_vectors * w->res_bits + 7) / 8 > w->res_packed_bytes) return NPB_ERR_SHAPE;
  }
  const size_t cb_align = (size_t)w->vector_len * 2;
  if (!aligned_to(w->centroids, cb_align)) return NPB_ERR_ALIGNMENT;
  if (w->res_centroids && !aligned_to(w->res_centroids, cb_align)) return NPB_ERR_ALIGNMENT;
  if (w->row_scale && !aligned_to(w->row_scale, 2)) return NPB_ERR_ALIGNMENT;
  return NPB_OK;
}

int validate_q(const npb_q_weight* w, int64_t N, int64_t K) {
  if (w == nullptr || N < 0 || K < 0) return NPB_ERR_INVALID_ARG;
  if (w->nbits != 4 && w->nbits != 8) return NPB_ERR_UNSUPPORTED;
  if (w->group_size <= 0 || w->group_size % 8 != 0) return NPB_ERR_UNSUPPORTED;
  if (K % w->group_size != 0) return NPB_ERR_SHAPE;
  if (N * K == 0) return NPB_OK;
  if (w->codes == nullptr || w->scale == nullptr) return NPB_ERR_INVALID_ARG;
  if (!aligned_to(w->scale, 2) || (w->zero_point && !aligned_to(w->zero_point, 2)))
    return NPB_ERR_ALIGNMENT;
  if (!aligned_to(w->codes, 4)) return NPB_ERR_ALIGNMENT;
  return NPB_OK;
}

}  // namespace npb

extern "C" {

const char* npb_status_string(int status) {
  switch (status) {
    case NPB_OK: return "ok";
    case NPB_ERR_INVALID_ARG: return "invalid argument (null pointer, negative size or bad enum)";
    case NPB_ERR_UNSUPPORTED: return "unsupported bits / vector_len / dtype / shape";
    case NPB_ERR_SHAPE: return "inconsistent shape (K % vector_len, group size, or packed buffer too short)";
    case NPB_ERR_ALIGNMENT: return "pointer not aligned as required";
    case NPB_ERR_CUDA: return "CUDA call failed (see npb_last_cuda_error)";
    case NPB_ERR_TOO_LARGE: return "size exceeds a fixed capacity (the built-in scratch array or shared memory)";
    case NPB_ERR_DEVICE_TIMEOUT: return "a bounded in-kernel wait gave up";
    default: return "unknown status";
  }
}

const char* npb_last_cuda_error(void) { return npb::g_last_error; }

int npb_version(void) { return 100; }

int npb_vq_decode(const npb_vq_weight* w, int64_t N, int64_t K, void* out, int out_dtype,
                  npb_stream_t stream) {
  return npb::vq_decode(w, N, K, out, out_dtype, static_cast<cudaStream_t>(stream));
}

int npb_q_decode(const npb_q_weight* w, int64_t N, int64_t K, void* out, int out_dtype,
                 npb_stream_t stream) {
  return npb::q_decode(w, N, K, out, out_dtype, static_cast<cudaStream_t>(stream));
}

int npb_vq_gemv(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M, int64_t N,
                int64_t K, const float* bias, void* y, npb_stream_t stream) {
  // The tensor-core kernel where the weight form allows it (it is as fast at 16 rows as the
  // CUDA-core GEMV at one); else the CUDA-core GEMV, which takes up to NPB_GEMV_MAX_ROWS rows.
  if (M >= 1 && M <= NPB_VQ_SMALL_BATCH_MAX_ROWS && N > 0) {
    const int rc = npb::vq_gemv_mma(w, x, x_dtype, M, N, K, bias, y, nullptr, static_cast<cudaStream_t>(stream));
    if (rc != NPB_ERR_UNSUPPORTED) return rc;
  }
  return npb::vq_gemv(w, x, x_dtype, M, N, K, bias, y, static_cast<cudaStream_t>(stream));
}

int npb_vq_gemv_grouped(const npb_vq_weight* weights, int n_weights, const int64_t* Ns,
                        const float* const* biases, const void* x, int x_dtype, int64_t M, int64_t K,
                        const void* norm_weight, float norm_eps, void* y, npb_stream_t stream) {
  return npb::vq_gemv_grouped(weights, n_weights, Ns, biases, x, x_dtype, M, K, norm_weight, norm_eps, y,
                              static_cast<cudaStream_t>(stream));
}

int npb_q_gemv(const npb_q_weight* w, const void* x, int x_dtype, int64_t M, int64_t N,
               int64_t K, const float* bias, void* y, npb_stream_t stream) {
  return npb::q_gemv(w, x, x_dtype, M, N, K, bias, y, static_cast<cudaStream_t>(stream));
}

int npb_gemm(const void* x, const void* w, const float* bias, void* y, int64_t M, int64_t N,
             int64_t K, int dtype, npb_stream_t stream) {
  return npb::gemm(x, w, bias, y, M, N, K, dtype, static_cast<cudaStream_t>(stream));
}

int npb_vq_gemm_fused(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M,
                      int64_t N, int64_t K, const float* bias, void* y, npb_stream_t stream) {
  return npb::vq_gemm_fused(w, nullptr, x, x_dtype, M, N, K, bias, y, static_cast<cudaStream_t>(stream));
}

int npb_vq_entropy_expand(const npb_vq_entropy_stream* s, int64_t N, int64_t G, void* out_u16,
                          npb_stream_t stream) {
  return npb::vq_entropy_expand(s, N, G, out_u16, static_cast<cudaStream_t>(stream));
}

int npb_vq_decode_cb(const npb_vq_weight* w, const void* codebook_x, int64_t N, int64_t K, void* out,
                     int out_dtype, npb_stream_t stream) {
  return npb::vq_decode_copy(w, codebook_x, N, K, out, out_dtype, static_cast<cudaStream_t>(stream));
}

int npb_vq_lut_gather(const float* lut, int64_t M, int64_t G, int64_t NC, const uint8_t* packed,
                      int64_t packed_bytes, int bits, int64_t N, float* out, npb_stream_t stream) {
  return npb::vq_lut_gather(lut, M, G, NC, packed, packed_bytes, bits, N, out, static_cast<cudaStream_t>(stream));
}

int npb_vq_gemm_fused_grouped(const npb_vq_weight* weights, int n_weights, const void* const* codebooks_x,
                              const int64_t* Ns, const float* const* biases, const void* x, int x_dtype, int64_t M,
                              int64_t K, void* y, npb_stream_t stream) {
  return npb::vq_gemm_fused_grouped(weights, n_weights, codebooks_x, Ns, biases, x, x_dtype, M, K, y,
                                    static_cast<cudaStream_t>(stream));
}

int npb_vq_codebook_cast(const void* centroids, int64_t n_values, void* out, int out_dtype, npb_stream_t stream) {
  return npb::vq_codebook_cast(centroids, n_values, out, out_dtype, static_cast<cudaStream_t>(stream));
}

int npb_vq_gemm_fused_cb(const npb_vq_weight* w, const void* codebook_x, const void* x, int x_dtype, int64_t M,
                         int64_t N, int64_t K, const float* bias, void* y, npb_stream_t stream) {
  if (codebook_x == nullptr) return NPB_ERR_INVALID_ARG;
  return npb::vq_gemm_fused(w, codebook_x, x, x_dtype, M, N, K, bias, y, static_cast<cudaStream_t>(stream));
}

int npb_q_gemm_fused(const npb_q_weight* w, const void* x, int x_dtype, int64_t M, int64_t N,
                     int64_t K, const float* bias, void* y, npb_stream_t stream) {
  return npb::q_gemm_fused(w, x, x_dtype, M, N, K, bias, y, static_cast<cudaStream_t>(stream));
}

int npb_vq_linear_static_scratch(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M,
                                 int64_t N, int64_t K, const float* bias, void* y,
                                 npb_stream_t stream) {
  return npb::vq_linear_static_scratch(w, x, x_dtype, M, N, K, bias, y,
                                       static_cast<cudaStream_t>(stream));
}

int npb_allgather_push(const void* src, int64_t M, int64_t n_local, int64_t elem_bytes,
                       const void* peer_out, const void* peer_flags, int rank, int world,
                       uint32_t epoch, npb_stream_t stream) {
  return npb::allgather_push(src, M, n_local, elem_bytes, peer_out, peer_flags, rank, world, epoch,
                             static_cast<cudaStream_t>(stream));
}

static int to_sink(const npb_gather_sink* in, npb::GatherSink* out) {
  if (in == nullptr) return NPB_ERR_INVALID_ARG;
  out->peer_out = static_cast<void* const*>(in->peer_out);
  out->peer_flags = static_cast<uint32_t* const*>(in->peer_flags);
  out->ld = in->ld;
  out->col0 = in->col0;
  out->rank = in->rank;
  out->world = in->world;
  out->epoch = in->epoch;
  out->wait_ns = npb::wait_limit_ns();
  return NPB_OK;
}

int npb_gemm_allgather(const void* x, const void* w, const float* bias, int64_t M, int64_t N_local,
                       int64_t K, int dtype, const npb_gather_sink* sink, npb_stream_t stream) {
  npb::GatherSink s;
  if (int rc = to_sink(sink, &s)) return rc;
  return npb::gemm_gather(x, w, bias, M, N_local, K, dtype, s, static_cast<cudaStream_t>(stream));
}

int npb_vq_gemv_allgather(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M,
                          int64_t N_local, int64_t K, const float* bias,
                          const npb_gather_sink* sink, npb_stream_t stream) {
  npb::GatherSink s;
  if (int rc = to_sink(sink, &s)) return rc;
  return npb::vq_gemv_gather(w, x, x_dtype, M, N_local, K, bias, s, static_cast<cudaStream_t>(stream));
}

int npb_rms_norm(const void* x, const void* weight, void* out, int64_t M, int64_t H, float eps,
                 int dtype, npb_stream_t stream) {
  return npb::rms_norm(x, weight, out, M, H, eps, dtype, static_cast<cudaStream_t>(stream));
}

int npb_vq_embedding(const int64_t* ids, int64_t T, const uint16_t* all_indices, int64_t V, int64_t G,
                     const void* centroids, int32_t num_centroids, int32_t vector_len, const int64_t* inv_perm,
                     float scale, void* out, int out_dtype, npb_stream_t stream) {
  return npb::vq_embedding(ids, T, all_indices, V, G, centroids, num_centroids, vector_len, inv_perm, scale, out,
                           out_dtype, static_cast<cudaStream_t>(stream));
}

int npb_q_embedding(const int64_t* ids, int64_t T, const npb_q_weight* w, int64_t V, int64_t D,
                    int64_t padding_idx, float embed_scale, void* out, int out_dtype, npb_stream_t stream) {
  return npb::q_embedding(ids, T, w, V, D, padding_idx, embed_scale, out, out_dtype,
                          static_cast<cudaStream_t>(stream));
}

int npb_gemm_device_status(int* host_out) { return npb::gemm_device_status(host_out); }

int npb_set_wait_limit_ns(uint64_t ns) {
  if (ns < 1000ull || ns > 60000000000ull) return NPB_ERR_INVALID_ARG;  // 1 us .. 60 s
  npb::g_wait_limit_ns.store(ns, std::memory_order_relaxed);
  return NPB_OK;
}

uint64_t npb_get_wait_limit_ns(void) { return npb::wait_limit_ns(); }

int npb_set_gemm_pair_mode(int mode) {
  if (mode < 0 || mode > 2) return NPB_ERR_INVALID_ARG;
  npb::g_gemm_pair_mode.store(mode, std::memory_order_relaxed);
  return NPB_OK;
}

int npb_get_gemm_pair_mode(void) { return npb::gemm_pair_mode(); }

}  // extern "C"
