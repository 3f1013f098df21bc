/*
 * neuropress_b200.h — C ABI of the B200 (sm_100a) quantized-linear kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, launches
 * asynchronously on that stream, never allocates, never synchronises, and returns an
 * npb_status.  The caller owns every buffer (inputs, outputs, scratch).  Pointers are
 * device pointers unless stated otherwise.
 *
 * Weight formats (identical to the reference's wire formats):
 *   - VQ index stream: 1-D uint8, LSB-first bit-stream, index i occupies bits
 *     [i*bits, (i+1)*bits); flat order n*G + g with G = K / vector_len
 *     (neuropress/transforms/vq_packing.py:210-252, IndexPacking._pack_bitstream).
 *   - Codebook: fp16 [num_centroids, vector_len] (neuropress/nn/np_vq_linear.py:421-427).
 *   - Group-affine codes: uint8 [N, K*nbits/8], value j of a byte at bits
 *     [j*nbits, (j+1)*nbits) (neuropress/nn/np_linear.py:78-117), fp16 scale / zero-point
 *     flat [N * K/group_size].
 */
#ifndef NEUROPRESS_B200_H_
#define NEUROPRESS_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque CUDA stream handle (a cudaStream_t / CUstream passed as a pointer). */
typedef void* npb_stream_t;

typedef enum {
  NPB_OK = 0,
  NPB_ERR_INVALID_ARG = 1,     /* null pointer, negative size, bad enum          */
  NPB_ERR_UNSUPPORTED = 2,     /* bits / vector_len / dtype / shape not handled  */
  NPB_ERR_SHAPE = 3,           /* K % vector_len, packed buffer too short, ...   */
  NPB_ERR_ALIGNMENT = 4,       /* pointer not aligned as the kernel requires     */
  NPB_ERR_CUDA = 5,            /* a CUDA runtime / driver call failed            */
  NPB_ERR_TOO_LARGE = 6,       /* exceeds a fixed capacity (no-alloc entry point)*/
  NPB_ERR_DEVICE_TIMEOUT = 7   /* a bounded in-kernel wait gave up               */
} npb_status;

typedef enum { NPB_F16 = 0, NPB_BF16 = 1, NPB_F32 = 2 } npb_dtype;

/* Largest row count the fused GEMV kernels accept (the decode band is 1-2 rows by
 * default; up to this many rows are supported for tuning the band edge). */
#define NPB_GEMV_MAX_ROWS 8
#define NPB_VQ_SMALL_BATCH_MAX_ROWS 16 /* npb_vq_gemv, tensor-core form (see there) */

/*
 * One vector-quantized weight matrix W[N, K].
 *   W16[n, VL*g + j] = hmul(hadd(C[cb(g)][idx[n,g]][j], R[ridx[n,g]][j]), s[n])   (fp16, RN)
 * with the residual term and the row scale optional, cb(g) = (g*VL) / cols_per_codebook.
 * Without residual / scale this is exactly the reference decode
 * (neuropress/kernels/vq_dequant.cu:1-18, neuropress/nn/np_vq_linear.py:1091-1095).
 */
typedef struct {
  const uint8_t* packed;        /* main index stream                                  */
  int64_t packed_bytes;
  int32_t bits;                 /* 4..16                                              */
  int32_t vector_len;           /* 4 or 8                                             */
  const void* centroids;        /* fp16 [n_codebooks * num_centroids, vector_len]     */
  int32_t num_centroids;        /* entries per codebook                               */
  int32_t cols_per_codebook;    /* 0: one codebook for all columns                    */
  const uint8_t* res_packed;    /* residual index stream or NULL                      */
  int64_t res_packed_bytes;
  int32_t res_bits;
  int32_t res_num_centroids;
  const void* res_centroids;    /* fp16 [res_num_centroids, vector_len] or NULL       */
  const void* row_scale;        /* fp16 [N] or NULL                                   */
} npb_vq_weight;

/*
 * An entropy-coded index stream in one of the reference's three wire formats
 * (neuropress/transforms/vq_packing.py: TieredIndexPacking :298-610, NTieredIndexPacking
 * :612-1034, ZeroEscapePacking :1037-1384), described by where its sub-streams sit:
 *   kind 1: n_tiers - 1 cascaded one-bit prefix streams (prefix k has one bit per index not in a
 *           tier < k: 0 = tier k, 1 = later); two-tier and N-tier buffers.
 *   kind 2: one two-bit prefix per index = its tier (zero escape: n_tiers = 4, tier 0 = centroid
 *           0 without payload).
 * Index value = tier_lo[t] + the tier_bits[t]-bit payload at the index's rank in tier t's stream.
 * row_off[t][n] = number of tier-t indices in rows < n (device int32 [N + 1], the packers'
 * compute_row_offsets).  Offsets are bytes from buf.
 */
typedef struct {
  const uint8_t* buf;           /* the whole coded buffer (header included), 4-byte aligned   */
  int64_t buf_bytes;
  int32_t kind;                 /* 1 or 2                                                     */
  int32_t n_tiers;              /* 2..4                                                       */
  int64_t prefix_off[3];        /* kind 1: prefix stream k, k < n_tiers - 1; kind 2: [0]      */
  int64_t tier_off[4];          /* payload stream of tier t                                   */
  int32_t tier_bits[4];         /* 0..20 (0: no payload)                                      */
  int32_t tier_lo[4];
  const int32_t* row_off[4];
} npb_vq_entropy_stream;

/*
 * One group-affine weight matrix W[N, K] = (q - zp) * scale, fp32 arithmetic, cast to the
 * activation dtype (neuropress/nn/np_linear.py:298-353; kernel q4_linear.cu:80-131).
 * zero_point == NULL means the symmetric scheme with zp = 2^(nbits-1).
 */
typedef struct {
  const uint8_t* codes;         /* uint8 [N, K*nbits/8]                               */
  const void* scale;            /* fp16 [N * K/group_size]                            */
  const void* zero_point;       /* fp16 [N * K/group_size] or NULL                    */
  int32_t nbits;                /* 4 (8 also accepted by decode / GEMV)               */
  int32_t group_size;           /* multiple of 8, divides K                           */
} npb_q_weight;

const char* npb_status_string(int status);
/* Text of the most recent CUDA error seen by this library on the calling thread. */
const char* npb_last_cuda_error(void);
int npb_version(void);

/* ---- one-pass decode (large-batch band, and the bit-exact parity anchor) ---------- */

/* out[N, K] in out_dtype.  Replaces vq_dequant (neuropress/kernels/vq_dequant.cu:105-146;
 * Python wrapper neuropress/kernels/__init__.py:497-529). */
int npb_vq_decode(const npb_vq_weight* w, int64_t N, int64_t K, void* out, int out_dtype,
                  npb_stream_t stream);

/* out[N, K] in out_dtype.  GPU form of the dequantisation inside _q_dequant_linear
 * (neuropress/nn/np_linear.py:334-351). */
int npb_q_decode(const npb_q_weight* w, int64_t N, int64_t K, void* out, int out_dtype,
                 npb_stream_t stream);

/* ---- fused index-decode GEMV (1..NPB_GEMV_MAX_ROWS rows) --------------------------- */

/* y[M, N] = x[M, K] . W^T (+ bias), x / y in x_dtype, bias fp32 [N] or NULL.
 * Replaces vq_linear / vq_linear_wmma's GEMV branch / vq_lut_gather
 * (neuropress/kernels/vq_linear.cu:344-424, vq_linear_wmma.cu:187-240,468-540,
 * vq_linear_lut.cu:121-206).  Up to NPB_GEMV_MAX_ROWS rows for every weight form and fp16 /
 * bf16 / fp32 activations; up to NPB_VQ_SMALL_BATCH_MAX_ROWS rows when the tensor-core kernel
 * applies (vector_len 8, 8 / 12 / 16-bit indices, K % 1024 == 0, fp16 / bf16 activations,
 * 8-bit residual indices, codebook groups of a multiple of 256 columns), else
 * NPB_ERR_UNSUPPORTED for more than NPB_GEMV_MAX_ROWS rows. */
int npb_vq_gemv(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M, int64_t N,
                int64_t K, const float* bias, void* y, npb_stream_t stream);

/* Grouped launch: n_weights (1..4) weights that are applied to the SAME activations -- the q / k / v
 * or the gate / up projections of a decoder layer -- in one kernel, as if their rows were
 * stacked: y is [M, sum N_i] with weight i at columns [sum_{j<i} N_j, +N_i).  Ns and biases are
 * HOST arrays (biases NULL, or device pointers / NULL per weight).  Optionally the activations
 * are RMS-normalised on their way into shared memory: norm_weight [K] in x_dtype (NULL: none),
 * x' = T(x * rsqrt(mean(x^2) + norm_eps) * norm_weight) in fp32, the arithmetic of npb_rms_norm, so
 * the norm before q / k / v or gate / up costs no launch and no HBM round trip.  1..16 rows, the
 * weight forms of the tensor-core path of npb_vq_gemv without residual codebook / row scale, all
 * weights with the same index width and codebook layout; otherwise NPB_ERR_UNSUPPORTED (call
 * npb_rms_norm and npb_vq_gemv per weight instead).  No reference counterpart: the reference
 * launches one kernel per linear and one per norm (neuropress/nn/np_vq_linear.py:1250-1267,
 * neuropress/nn/np_rms_norm.py:86-99). */
int npb_vq_gemv_grouped(const npb_vq_weight* weights, int n_weights, const int64_t* Ns,
                        const float* const* biases, const void* x, int x_dtype, int64_t M, int64_t K,
                        const void* norm_weight, float norm_eps, void* y, npb_stream_t stream);

/* Same contract for group-affine weights.  Replaces q_linear
 * (neuropress/kernels/q4_linear.cu:179-253). */
int npb_q_gemv(const npb_q_weight* w, const void* x, int x_dtype, int64_t M, int64_t N,
               int64_t K, const float* bias, void* y, npb_stream_t stream);

/* ---- tensor-core GEMMs (tcgen05 / TMEM) --------------------------------------------- */

/* y[M, N] = x[M, K] . w[N, K]^T (+ bias); x, w, y in dtype (NPB_BF16 or NPB_F16), fp32
 * accumulation, bias fp32 [N] or NULL.  Stands in for the cuBLAS call after the decode
 * (F.linear at neuropress/nn/np_vq_linear.py:1148).  K % 8 == 0 and 16-byte aligned
 * pointers are required (TMA). */
int npb_gemm(const void* x, const void* w, const float* bias, void* y, int64_t M, int64_t N,
             int64_t K, int dtype, npb_stream_t stream);

/* Tile-decode GEMM: B tiles are decoded from the index stream straight into the swizzled
 * shared-memory stage, never written to HBM.  Replaces vq_gemm_triton
 * (neuropress/kernels/vq_triton.py:37-179) and vq_linear_wmma's GEMM branch
 * (vq_linear_wmma.cu:261-394).  vector_len 8, K % 64 == 0. */
int npb_vq_gemm_fused(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M,
                      int64_t N, int64_t K, const float* bias, void* y, npb_stream_t stream);

/* The copy form of the tile-decode GEMM for plain weights (no residual codebook, no row scale).
 * A decoded vector of such a weight is its codebook entry cast to the activation type, so with
 * the codebook already in that type the decode is a 16-byte copy, which the kernel issues as
 * asynchronous global -> shared copies (no register destination, nothing waits for a gather).
 *   npb_vq_codebook_cast: out[i] = dtype(centroids[i]) for n_values = entries * vector_len fp16
 *     values (NPB_F16 copies).  Done once per codebook and activation type by the caller.
 *   npb_vq_gemm_fused_cb: npb_vq_gemm_fused with codebook_x = that table ([n_codebooks *
 *     num_centroids, 8] of x_dtype, 16-byte aligned; for NPB_F16 w->centroids itself will do).
 *     Same results bit for bit.  NPB_ERR_UNSUPPORTED for weights with a residual or a row scale
 *     and for index streams that do not allow wide reads (bits other than 8 / 12 / 16,
 *     unaligned stream): call npb_vq_gemm_fused for those.
 * Replaces the same reference code as npb_vq_gemm_fused. */
int npb_vq_codebook_cast(const void* centroids, int64_t n_values, void* out, int out_dtype,
                         npb_stream_t stream);
/* The one-pass decode of a plain weight as a gather-copy from the same table: asynchronous 16-byte
 * copies into a shared-memory chunk, written out by bulk copies; the decoded matrix is bit for bit
 * npb_vq_decode's.  out_dtype NPB_F16 / NPB_BF16 (= the table's type), vector_len 8, bits 8 / 12 /
 * 16, K % 64 == 0; NPB_ERR_UNSUPPORTED otherwise (call npb_vq_decode).  Replaces vq_dequant
 * (neuropress/kernels/vq_dequant.cu:105-146) like npb_vq_decode. */
int npb_vq_decode_cb(const npb_vq_weight* w, const void* codebook_x, int64_t N, int64_t K, void* out,
                     int out_dtype, npb_stream_t stream);
int npb_vq_gemm_fused_cb(const npb_vq_weight* w, const void* codebook_x, const void* x, int x_dtype,
                         int64_t M, int64_t N, int64_t K, const float* bias, void* y,
                         npb_stream_t stream);

/* Expands an entropy-coded index stream of N rows x G indices into the plain little-endian
 * uint16 index table [N, G] (= an IndexPacking stream with bits = 16) that every other entry
 * point takes, so each row-count band serves entropy-coded layers: expand, then the band's
 * kernel.  One warp per row; bit-exact against the packers' unpack().  Values above 65535 are
 * stored as 65535.  Stands in for the index decoding inside the reference's tiered GEMV kernels
 * (neuropress/kernels/vq_linear_tiered.cu, vq_linear_ntier.cu, vq_linear_zero_escape.cu). */
int npb_vq_entropy_expand(const npb_vq_entropy_stream* s, int64_t N, int64_t G, void* out_u16,
                          npb_stream_t stream);

/* npb_vq_gemm_fused_cb for up to four plain weights that share the activations (q / k / v, gate / up)
 * in one launch: y is [M, sum of Ns], weight i's outputs in the columns after those of the weights
 * before it; codebooks_x[i] is weight i's codebook in x_dtype; biases may be NULL or hold NULLs.  The
 * weights must agree in bits, num_centroids and cols_per_codebook.  Same bits out as n_weights
 * separate calls.  No reference counterpart (the reference launches each linear by itself). */
int npb_vq_gemm_fused_grouped(const npb_vq_weight* weights, int n_weights, const void* const* codebooks_x,
                              const int64_t* Ns, const float* const* biases, const void* x, int x_dtype,
                              int64_t M, int64_t K, void* y, npb_stream_t stream);

/* LUT gather: out[m, n] = sum over g of lut[m, g, idx[n, g]], lut fp32 [M, G, NC] built by the
 * caller (one matmul of the activations with the codebook), idx the packed index stream of N * G
 * indices of `bits` bits, out fp32 [M, N].  Replaces vq_lut_gather
 * (neuropress/kernels/vq_linear_lut.cu:121-206, pybind :208-211).  M <= 65535. */
int npb_vq_lut_gather(const float* lut, int64_t M, int64_t G, int64_t NC, const uint8_t* packed,
                      int64_t packed_bytes, int bits, int64_t N, float* out, npb_stream_t stream);

/* Same for group-affine weights (no reference counterpart beyond q_linear, which re-reads
 * the weight per row: neuropress/kernels/q4_linear.cu:80-131). nbits 4, K % 64 == 0,
 * group_size % 32 == 0 (NPB_ERR_UNSUPPORTED otherwise: decode, then npb_gemm). */
int npb_q_gemm_fused(const npb_q_weight* w, const void* x, int x_dtype, int64_t M, int64_t N,
                     int64_t K, const float* bias, void* y, npb_stream_t stream);

/* Size of the scratch array built into the library for npb_vq_linear_static_scratch: 32 MiB,
 * i.e. weights of up to 16,777,216 elements (4096 x 4096) in bf16 / fp16. */
#define NPB_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)

/*
 * y[M, N] = x[M, K] . W^T (+ bias) by one-pass decode + dense tensor-core GEMM, for callers
 * that cannot allocate device memory.  It has no counterpart in the reference, which always
 * takes its temporary weight from torch's allocator.
 *
 * Who needs it: a host that only owns the buffers it was given (a plain C / C++ service with a
 * fixed memory budget, a plugin loaded into someone else's process), or a latency-critical
 * loop where cudaMalloc is off limits because it synchronises the device and may fail when
 * memory is tight.  The dense temporary weight lives in an array of NPB_STATIC_SCRATCH_BYTES
 * inside the library, so the call allocates nothing - not with cudaMalloc, not through any
 * library.  The price is that every GPU that loads the library gives up that much memory
 * until the process ends.
 *
 * Rules:  N * K * 2 bytes must fit in the array, otherwise NPB_ERR_TOO_LARGE is returned and
 * nothing is launched.  x / y are NPB_BF16 or NPB_F16, K % 8 == 0, bias fp32 or NULL; inputs
 * and outputs are still the caller's.  All calls share the one array: order them on a single
 * stream - calls that overlap on the GPU corrupt each other's weights.  The array never needs
 * clearing (each call overwrites the part it reads).  The first call on each device looks up
 * the array's device address (cudaGetSymbolAddress) and sets kernel attributes; make that
 * first call outside of any stream capture.
 */
int npb_vq_linear_static_scratch(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M,
                                 int64_t N, int64_t K, const float* bias, void* y,
                                 npb_stream_t stream);

/* Fused RMSNorm over the last dimension, the step on the input side of the q/k/v and gate/up
 * linears: out[m, i] = T(x[m, i] * rsqrt(mean(x[m, :]^2) + eps) * weight[i]), fp32 arithmetic.
 * Replaces rms_norm (neuropress/kernels/rms_norm.cu:27-123; wrapper kernels/__init__.py:1091-1110).
 * x, out [M, H] contiguous, weight [H], all of `dtype` (NPB_BF16 / NPB_F16 / NPB_F32). */
int npb_rms_norm(const void* x, const void* weight, void* out, int64_t M, int64_t H, float eps,
                 int dtype, npb_stream_t stream);

/* ---- embedding lookups (only the rows the token ids select are decoded) ------------- */

/* out[t, :] = decode(row ids[t]) of a VQ-compressed embedding table, t < T.  all_indices is the
 * pre-unpacked [V, G] table of 16-bit codebook indices the reference keeps
 * (neuropress/nn/np_vq_embedding.py:88, read as unsigned), centroids fp16 [num_centroids,
 * vector_len] with vector_len 4 or 8, inv_perm int64 [G * vector_len] or NULL (output column c
 * takes decoded column inv_perm[c]), scale applied to the fp16 value and rounded to fp16, then one
 * conversion to out_dtype: the arithmetic of NPVQEmbedding.forward (:119-141).  ids int64; an id
 * outside [0, V) yields a zero row. */
int npb_vq_embedding(const int64_t* ids, int64_t T, const uint16_t* all_indices, int64_t V, int64_t G,
                     const void* centroids, int32_t num_centroids, int32_t vector_len,
                     const int64_t* inv_perm, float scale, void* out, int out_dtype,
                     npb_stream_t stream);

/* out[t, :] = embed_scale * T(fp16((q - zp) * s)) for the rows ids[t] of a group-affine table
 * w (codes [V, D * nbits / 8], fp16 scale / zero-point [V * D / group_size]); the row
 * padding_idx (-1: none) and ids outside [0, V) yield zeros.  Replaces _emb_dequant and
 * NPEmbedding.forward (neuropress/nn/np_embedding.py:120-183, 449-473). */
int npb_q_embedding(const int64_t* ids, int64_t T, const npb_q_weight* w, int64_t V, int64_t D,
                    int64_t padding_idx, float embed_scale, void* out, int out_dtype,
                    npb_stream_t stream);

/*
 * Multi-GPU (new; the reference has no distributed code): all-gather of out-feature shards by
 * pushing.  This rank's src[M, n_local] (elem_bytes per element) is stored into columns
 * [rank*n_local, (rank+1)*n_local) of EVERY rank's [M, n_local*world] buffer; then each rank
 * flags every peer and waits (bounded: npb_set_wait_limit_ns, 2 s by default) for all peers' flags, so when the kernel ends the
 * local buffer holds the full [M, N].  peer_out / peer_flags are DEVICE arrays of `world`
 * pointers (symmetric-memory buffer addresses of ranks 0..world-1); each rank's flag buffer
 * holds world + 3 zero-initialised uint32 words (per-peer epochs, a counter, a status word
 * that becomes 1 if a wait gave up, a call counter).  epoch must increase by one per call on
 * all ranks; epoch 0 means "use the call counter kept in the flag words", which keeps the
 * arguments constant from call to call (CUDA-graph replay).  Do not mix the two on one flag
 * buffer.  n_local * elem_bytes must be a multiple of 16.  One rank per GPU.
 */
int npb_allgather_push(const void* src, int64_t M, int64_t n_local, int64_t elem_bytes,
                       const void* peer_out, const void* peer_flags, int rank, int world,
                       uint32_t epoch, npb_stream_t stream);

/*
 * Fused compute + all-gather: the producing kernel stores this rank's [M, N_local] result
 * straight into columns [col0, col0 + N_local) of every rank's [M, ld] buffer (peer stores
 * from the GEMM epilogue / the GEMV's final store) and ends with the handshake of
 * npb_allgather_push, so no separate gather pass runs.  Same flag words, epochs and rules as
 * npb_allgather_push; all buffers 16-byte aligned, ld and col0 in elements of the activation
 * dtype.  Every rank must make the call (M > 0).  npb_vq_gemv_allgather takes the row counts
 * of npb_vq_gemv.
 */
typedef struct npb_gather_sink {
  const void* peer_out;    /* device array [world] of buffer base pointers */
  const void* peer_flags;  /* device array [world] of flag-word pointers */
  int64_t ld;
  int64_t col0;
  int32_t rank;
  int32_t world;
  uint32_t epoch;          /* 0: epochs kept in the flag words (CUDA-graph friendly) */
  uint32_t reserved;
} npb_gather_sink;

int npb_gemm_allgather(const void* x, const void* w, const float* bias, int64_t M,
                       int64_t N_local, int64_t K, int dtype, const npb_gather_sink* sink,
                       npb_stream_t stream);
int npb_vq_gemv_allgather(const npb_vq_weight* w, const void* x, int x_dtype, int64_t M,
                          int64_t N_local, int64_t K, const float* bias,
                          const npb_gather_sink* sink, npb_stream_t stream);


/* Every wait inside the tensor-core GEMMs (on an mbarrier) is bounded; a kernel that gives up
 * records which role did so, frees its tensor memory and returns.  This call synchronises the
 * device, copies that record to *host_out (0 = no give-up since the last call), clears it, and
 * returns NPB_ERR_DEVICE_TIMEOUT if it was set.  No reference counterpart. */
int npb_gemm_device_status(int* host_out);

/* Limit of every bounded in-kernel wait of this library (the mbarrier waits of the GEMMs, the
 * wait for the peers' flags in the all-gather kernels), in nanoseconds; 2 s by default,
 * accepted range 1 us .. 60 s.  Process-wide, read when a kernel is launched.  A wait that
 * runs out does not fault: the kernel records it (npb_gemm_device_status, the status word of
 * the flag buffer) and returns.  Tests lower it to exercise exactly that path.  No reference
 * counterpart. */
int npb_set_wait_limit_ns(uint64_t ns);
uint64_t npb_get_wait_limit_ns(void);

/* Tile policy of the dense GEMM (npb_gemm, npb_gemm_allgather, the large-batch band of the
 * linears): 0 = every tile by one CTA (tcgen05 cta_group::1); 1 = automatic (default): CTA
 * pairs (cta_group::2, 256-row tiles, each CTA stages half of the W tile) where the row count
 * fills pair tiles and there is a tile for every pair; 2 = pairs for every launch of more than
 * 128 rows.  Every mode accumulates the same products in fp32 in the same order along K.
 * Process-wide, read at launch; the environment variable NEUROPRESS_B200_GEMM_PAIRS
 * gives the initial value.  No reference counterpart (the reference calls cuBLAS). */
int npb_set_gemm_pair_mode(int mode);
int npb_get_gemm_pair_mode(void);

#ifdef __cplusplus
}
#endif
#endif /* NEUROPRESS_B200_H_ */
