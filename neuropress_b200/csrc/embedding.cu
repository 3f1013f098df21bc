// Embedding lookups for quantized tables: only the rows a batch of token ids selects are decoded.
//
//   vq_embedding : out[t, VL*g + j] = C[idx[ids[t], g]][j]   (pure indexing, fp16 codebook), then
//                  an optional column permutation, an optional scalar multiply rounded to fp16,
//                  and one conversion to the output type -- the arithmetic of
//                  NPVQEmbedding.forward (neuropress/nn/np_vq_embedding.py:119-141).  The index
//                  table is the reference's pre-unpacked [vocab, n_groups] 16-bit table (:88).
//   q_embedding  : out[t, k] = fp16((q - zp) * s) for the selected rows of a group-affine table
//                  (fp32 arithmetic, one rounding per operation), padding row zeroed, converted to
//                  the output type, then multiplied by embed_scale -- _emb_dequant and
//                  NPEmbedding.forward (neuropress/nn/np_embedding.py:120-183, 449-473).
//
// One warp per token; lanes take consecutive vectors / code words, so index loads and output
// stores are contiguous.  Bound by the output write (tokens x dim x sizeof(T)); a token id outside
// the table yields a zero row instead of an out-of-bounds read.
#include "common.cuh"

namespace npb {
namespace {

constexpr int kWarps = 8;

template <typename T>
__device__ __forceinline__ T finish_half(__half h, float scale, bool scaled) {
  if (scaled) h = __float2half_rn(__half2float(h) * scale);  // fp16 tensor x python scalar: fp32 product, fp16 result
  return from_half<T>(h);
}

template <typename T, int VL>
__global__ void __launch_bounds__(kWarps * 32)
vq_embedding_kernel(const int64_t* __restrict__ ids, int64_t T_, const uint16_t* __restrict__ table, int64_t V,
                    int G, const __half* __restrict__ cent, int NC, const int64_t* __restrict__ inv_perm,
                    float scale, int scaled, T* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (t >= T_) return;
  const int64_t id = ids[t];
  const int D = G * VL;
  T* o = out + t * D;
  if (id < 0 || id >= V) {
    for (int c = lane; c < D; c += 32) o[c] = from_f32<T>(0.f);
    return;
  }
  const uint16_t* row = table + id * G;
  if (inv_perm == nullptr) {
    for (int g = lane; g < G; g += 32) {
      uint32_t e = row[g];
      e = e < (uint32_t)NC ? e : (uint32_t)NC - 1u;
      const __half* c = cent + (size_t)e * VL;
#pragma unroll
      for (int j = 0; j < VL; ++j) o[g * VL + j] = finish_half<T>(c[j], scale, scaled != 0);
    }
  } else {
    for (int c = lane; c < D; c += 32) {   // output column c takes decoded column inv_perm[c]
      const int64_t src = inv_perm[c];
      const int g = (int)(src / VL), j = (int)(src % VL);
      uint32_t e = row[g];
      e = e < (uint32_t)NC ? e : (uint32_t)NC - 1u;
      o[c] = finish_half<T>(cent[(size_t)e * VL + j], scale, scaled != 0);
    }
  }
}

template <typename T>
__device__ __forceinline__ T finish_q(float w, float embed_scale, bool scaled) {
  const __half h = __float2half_rn(w);                // the table decodes in the fp16 scale dtype
  T v = from_half<T>(h);
  if (scaled) v = from_f32<T>(to_f32(v) * embed_scale);  // tensor of T x python scalar
  return v;
}

template <typename T, int NBITS>
__global__ void __launch_bounds__(kWarps * 32)
q_embedding_kernel(const int64_t* __restrict__ ids, int64_t T_, const uint8_t* __restrict__ codes,
                   const __half* __restrict__ scale, const __half* __restrict__ zp, int64_t V, int D,
                   int group_size, int64_t padding_idx, float embed_scale, int scaled, T* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (t >= T_) return;
  const int64_t id = ids[t];
  T* o = out + t * D;
  if (id < 0 || id >= V || id == padding_idx) {
    for (int c = lane; c < D; c += 32) o[c] = from_f32<T>(0.f);
    return;
  }
  constexpr int VPB = 8 / NBITS;          // values per byte
  const uint8_t* row = codes + id * (D / VPB);
  const int groups = D / group_size;
  const float zsym = (float)(1 << (NBITS - 1));
  for (int b = lane; b < D / VPB; b += 32) {   // one code byte per lane and step
    const uint32_t byte = row[b];
    const int k0 = b * VPB;
    const int g = k0 / group_size;           // group_size is a multiple of 8 >= VPB
    const float s = __half2float(scale[id * groups + g]);
    const float z = zp ? __half2float(zp[id * groups + g]) : zsym;
#pragma unroll
    for (int j = 0; j < VPB; ++j) {
      const float q = (float)((byte >> (j * NBITS)) & ((1u << NBITS) - 1u));
      o[k0 + j] = finish_q<T>(__fmul_rn(__fsub_rn(q, z), s), embed_scale, scaled != 0);
    }
  }
}

template <typename T>
int launch_vq(const int64_t* ids, int64_t T_, const uint16_t* table, int64_t V, int G, const __half* cent, int NC,
              int VL, const int64_t* inv_perm, float scale, T* out, cudaStream_t st) {
  const unsigned blocks = (unsigned)((T_ + kWarps - 1) / kWarps);
  const int scaled = scale != 1.0f;
  if (VL == 8)
    vq_embedding_kernel<T, 8><<<blocks, kWarps * 32, 0, st>>>(ids, T_, table, V, G, cent, NC, inv_perm, scale, scaled, out);
  else
    vq_embedding_kernel<T, 4><<<blocks, kWarps * 32, 0, st>>>(ids, T_, table, V, G, cent, NC, inv_perm, scale, scaled, out);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

template <typename T>
int launch_q(const int64_t* ids, int64_t T_, const npb_q_weight* w, int64_t V, int D, int64_t padding_idx,
             float embed_scale, T* out, cudaStream_t st) {
  const unsigned blocks = (unsigned)((T_ + kWarps - 1) / kWarps);
  const int scaled = embed_scale != 1.0f;
  const __half* s = static_cast<const __half*>(w->scale);
  const __half* z = static_cast<const __half*>(w->zero_point);
  if (w->nbits == 4)
    q_embedding_kernel<T, 4><<<blocks, kWarps * 32, 0, st>>>(ids, T_, w->codes, s, z, V, D, w->group_size,
                                                             padding_idx, embed_scale, scaled, out);
  else
    q_embedding_kernel<T, 8><<<blocks, kWarps * 32, 0, st>>>(ids, T_, w->codes, s, z, V, D, w->group_size,
                                                             padding_idx, embed_scale, scaled, out);
  NPB_LAUNCH_CHECK();
  return NPB_OK;
}

}  // namespace

int vq_embedding(const int64_t* ids, int64_t T_, const uint16_t* table, int64_t V, int64_t G, const void* centroids,
                 int NC, int VL, const int64_t* inv_perm, float scale, void* out, int out_dtype, cudaStream_t st) {
  if (T_ < 0 || V <= 0 || G <= 0 || NC <= 0) return NPB_ERR_INVALID_ARG;
  if (VL != 4 && VL != 8) return NPB_ERR_UNSUPPORTED;
  if (T_ == 0) return NPB_OK;
  if (ids == nullptr || table == nullptr || centroids == nullptr || out == nullptr) return NPB_ERR_INVALID_ARG;
  if (G * VL >= (int64_t)1 << 30) return NPB_ERR_UNSUPPORTED;
  if (!aligned_to(table, 2) || !aligned_to(centroids, 2) || !aligned_to(ids, 8)) return NPB_ERR_ALIGNMENT;
  const __half* c = static_cast<const __half*>(centroids);
  switch (out_dtype) {
    case NPB_F16: return launch_vq<__half>(ids, T_, table, V, (int)G, c, NC, VL, inv_perm, scale, static_cast<__half*>(out), st);
    case NPB_BF16: return launch_vq<__nv_bfloat16>(ids, T_, table, V, (int)G, c, NC, VL, inv_perm, scale, static_cast<__nv_bfloat16*>(out), st);
    case NPB_F32: return launch_vq<float>(ids, T_, table, V, (int)G, c, NC, VL, inv_perm, scale, static_cast<float*>(out), st);
    default: return NPB_ERR_UNSUPPORTED;
  }
}

int q_embedding(const int64_t* ids, int64_t T_, const npb_q_weight* w, int64_t V, int64_t D, int64_t padding_idx,
                float embed_scale, void* out, int out_dtype, cudaStream_t st) {
  if (int rc = validate_q(w, V, D)) return rc;
  if (T_ < 0 || V <= 0 || D <= 0) return NPB_ERR_INVALID_ARG;
  if (T_ == 0) return NPB_OK;
  if (ids == nullptr || out == nullptr) return NPB_ERR_INVALID_ARG;
  if (D >= (int64_t)1 << 30 || D % (8 / w->nbits) != 0) return NPB_ERR_UNSUPPORTED;
  switch (out_dtype) {
    case NPB_F16: return launch_q<__half>(ids, T_, w, V, (int)D, padding_idx, embed_scale, static_cast<__half*>(out), st);
    case NPB_BF16: return launch_q<__nv_bfloat16>(ids, T_, w, V, (int)D, padding_idx, embed_scale, static_cast<__nv_bfloat16*>(out), st);
    case NPB_F32: return launch_q<float>(ids, T_, w, V, (int)D, padding_idx, embed_scale, static_cast<float*>(out), st);
    default: return NPB_ERR_UNSUPPORTED;
  }
}

}  // namespace npb
