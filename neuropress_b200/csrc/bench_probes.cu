// Measurement probes for bench.py, built into their own library (libneuropress_b200_bench.so):
// they are not part of the product's C ABI and nothing in the package calls them.
//
// Each probe isolates one hardware rate that bounds a kernel of the forward path, so that the
// benchmark can state, next to the HBM roofline, the rate the access pattern itself allows:
//
//   npbb_stream_read    a plain coalesced read of `bytes` (what a GEMV over the same number of
//                       packed bytes could reach if it did nothing but load them);
//   npbb_l2_gather      random 16-byte gathers from a table in global memory (a 65536-entry
//                       codebook: every gather misses L1 and fetches one L2 sector);
//   npbb_smem_lookup    random shared-memory reads: 16-byte gathers from a 4096-entry table
//                       (a codebook staged in shared memory) or 4-byte lookups from a 16384-entry
//                       table (a per-group dot-product table).
//
// All read their indices as a stream of uint16 (eight per 16-byte load, like the index streams
// of the product kernels) and fold the loaded values into a checksum nobody reads back.
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

__device__ __forceinline__ void fold(uint4& a, const uint4 v) { a.x ^= v.x; a.y += v.y; a.z ^= v.z; a.w += v.w; }

__global__ void __launch_bounds__(512) stream_read_kernel(const uint4* __restrict__ src, size_t n16, uint4* out) {
  const int lane = threadIdx.x & 31;
  const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  uint4 a = make_uint4(0, 0, 0, 0);
  for (size_t base = warp * 256; base < n16; base += nwarps * 256) {
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const size_t j = base + i * 32 + lane;
      v[i] = j < n16 ? __ldg(src + j) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) fold(a, v[i]);
  }
  if (a.x == 0x12345u && a.y == 77u) out[0] = a;
}

__global__ void __launch_bounds__(256) l2_gather_kernel(const uint4* __restrict__ table, uint32_t mask,
                                                         const uint4* __restrict__ idx, size_t n_chunks, uint4* out) {
  uint4 a = make_uint4(0, 0, 0, 0);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t c = blockIdx.x * (size_t)blockDim.x + threadIdx.x; c < n_chunks; c += stride) {
    const uint4 iv = __ldg(idx + c);  // eight 16-bit indices, consecutive threads read consecutive chunks
    const uint32_t w[4] = {iv.x, iv.y, iv.z, iv.w};
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __ldg(table + (((w[j >> 1] >> (16 * (j & 1))) & 0xffffu) & mask));
#pragma unroll
    for (int j = 0; j < 8; ++j) fold(a, v[j]);
  }
  if (a.x == 0x12345u && a.y == 77u) out[0] = a;
}

template <int MODE>  // 0: 16-byte gathers, 4096 entries; 1: 4-byte lookups, 16384 entries (both 64 KiB)
__global__ void __launch_bounds__(512, 1) smem_lookup_kernel(const uint4* __restrict__ idx, size_t n_chunks, uint4* out) {
  extern __shared__ __align__(16) uint8_t tab[];
  for (int i = threadIdx.x; i < 65536 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(tab)[i] = i * 2654435761u;
  __syncthreads();
  uint4 a = make_uint4(0, 0, 0, 0);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t c = blockIdx.x * (size_t)blockDim.x + threadIdx.x; c < n_chunks; c += stride) {
    const uint4 iv = __ldg(idx + c);
    const uint32_t w[4] = {iv.x, iv.y, iv.z, iv.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t id = (w[j >> 1] >> (16 * (j & 1))) & 0xffffu;
      if (MODE == 0) fold(a, reinterpret_cast<const uint4*>(tab)[id & 4095u]);
      else a.x += reinterpret_cast<const uint32_t*>(tab)[id & 16383u];
    }
  }
  if (a.x == 0x12345u && a.y == 77u) out[0] = a;
}

}  // namespace

extern "C" {

// Each returns a cudaError_t as int (0 = ok).  `out` is 16 bytes of device memory.
int npbb_stream_read(const void* src, int64_t bytes, void* out, void* stream) {
  stream_read_kernel<<<148 * 4, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), (size_t)bytes / 16, static_cast<uint4*>(out));
  return (int)cudaGetLastError();
}

// table: 16-byte entries, entries = power of two <= 65536; idx: n_indices uint16 (multiple of 8).
int npbb_l2_gather(const void* table, int entries, const void* idx, int64_t n_indices, void* out, void* stream) {
  l2_gather_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(table), (uint32_t)entries - 1u, static_cast<const uint4*>(idx),
      (size_t)n_indices / 8, static_cast<uint4*>(out));
  return (int)cudaGetLastError();
}

int npbb_smem_lookup(int mode, const void* idx, int64_t n_indices, void* out, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (mode == 0) {
    e = cudaFuncSetAttribute(smem_lookup_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    if (e != cudaSuccess) return (int)e;
    smem_lookup_kernel<0><<<148, 512, 65536, st>>>(static_cast<const uint4*>(idx), (size_t)n_indices / 8,
                                                   static_cast<uint4*>(out));
  } else {
    e = cudaFuncSetAttribute(smem_lookup_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    if (e != cudaSuccess) return (int)e;
    smem_lookup_kernel<1><<<148, 512, 65536, st>>>(static_cast<const uint4*>(idx), (size_t)n_indices / 8,
                                                   static_cast<uint4*>(out));
  }
  return (int)cudaGetLastError();
}

}  // extern "C"
