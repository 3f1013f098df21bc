// LUT gather: y[m, n] = sum_g lut[m, g, idx[n, g]] with a caller-built table
// lut[m, g, e] = dot(x[m, VL*g .. VL*g + VL), C[e])  (fp32 [M, G, NC]).
//
// The gather phase of the reference's cuda_lut path (neuropress/kernels/vq_linear_lut.cu:121-206,
// wrapper kernels/__init__.py:405-426; the caller builds the table with one matmul,
// neuropress/nn/np_vq_linear.py:1189-1248).  The reference gives a thread one output and walks its
// G groups in order; here a warp takes one output, lanes take groups g = lane, lane + 32, ... (so
// the index reads of a warp are contiguous) and the partial sums meet in a shuffle tree: same
// terms, fp32, another summation order.  Any index width 4..16.  Bound by the random 4-byte
// table reads (G of them per output through L2: the table is M * G * NC * 4 bytes, 128 MiB per
// row for G = 512, NC = 65536), which is why neither library routes a layer here by default.
#include "common.cuh"

namespace npb {
namespace {

constexpr int kWarps = 8;

__global__ void __launch_bounds__(kWarps * 32)
vq_lut_gather_kernel(const float* __restrict__ lut, const uint8_t* __restrict__ packed, int64_t packed_bytes,
                     float* __restrict__ out, int64_t N, int G, int NC, int bits) {
  const int lane = threadIdx.x & 31;
  const int64_t n = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int64_t m = blockIdx.y;
  if (n >= N) return;
  const float* lut_m = lut + m * (int64_t)G * NC;
  float acc = 0.f;
  for (int g = lane; g < G; g += 32) {
    uint32_t e = read_index_generic(packed, packed_bytes, n * G + g, bits);
    e = e < (uint32_t)NC ? e : (uint32_t)NC - 1u;   // an index past the table reads its last entry
    acc += __ldg(lut_m + (int64_t)g * NC + e);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (lane == 0) out[m * N + n] = acc;
}

}  // namespace

int vq_lut_gather(const float* lut, int64_t M, int64_t G, int64_t NC, const uint8_t* packed, int64_t packed_bytes,
                  int bits, int64_t N, float* out, cudaStream_t st) {
  if (M < 0 || N < 0 || G <= 0 || NC <= 0) return NPB_ERR_INVALID_ARG;
  if (bits < 4 || bits > 16) return NPB_ERR_UNSUPPORTED;
  if (M == 0 || N == 0) return NPB_OK;
  if (lut == nullptr || packed == nullptr || out == nullptr) return NPB_ERR_INVALID_ARG;
  if (packed_bytes < (N * G * bits + 7) / 8) return NPB_ERR_SHAPE;
  if (M > 65535 || G >= (int64_t)1 << 30 || NC >= (int64_t)1 << 30) return NPB_ERR_UNSUPPORTED;
  if (!aligned_to(lut, 4) || !aligned_to(out, 4)) return NPB_ERR_ALIGNMENT;
  const dim3 grid((unsigned)((N + kWarps - 1) / kWarps), (unsigned)M);
  vq_lut_gather_kernel<<<grid, kWarps * 32, 0, st>>>(lut, packed, packed_bytes, out, N, (int)G, (int)NC, bits);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

}  // namespace npb
