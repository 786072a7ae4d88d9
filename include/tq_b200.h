/*
 * libtq_b200 — C ABI of the TurboQuant hot paths for NVIDIA B200 (sm_100a).
 *
 * Conventions (the launcher style of the reference's native library,
 * turboquant/kernels/fp4_pa_v9.hip:177-197 as called from
 * turboquant/integration/tq_fp4_backend.py:274-295): C linkage, raw device
 * pointers, plain ints and floats, the stream last.  Unlike the reference's
 * `void` launchers every function returns a status: 0 on success, a negative
 * TQ_ERR_* otherwise.  Nothing here allocates, synchronises or keeps global
 * state unless its comment says so; the caller owns every buffer, including
 * the split-K workspace, so the calls can be captured in CUDA graphs.
 *
 * All tensors are contiguous in their last dimension; head_dim is 128.
 * "rotated space" means multiplied by the normalised 128x128 Walsh-Hadamard
 * matrix of turboquant/core/rotation.py:28-44.
 */
#ifndef TQ_B200_H_
#define TQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* tq_stream_t; /* same type as cudaStream_t */

#define TQ_OK 0
#define TQ_ERR_ARG (-1)         /* null pointer, negative size, bad stride or alignment */
#define TQ_ERR_UNSUPPORTED (-2) /* bit width / block size / group size outside what is built */
#define TQ_ERR_LAUNCH (-3)      /* the CUDA runtime rejected the launch */
#define TQ_ERR_WORKSPACE (-4)   /* caller-provided workspace too small */

#define TQ_DTYPE_F16 0
#define TQ_DTYPE_BF16 1
#define TQ_DTYPE_F32 2

/* Flags that may be OR-ed into the io_dtype argument of tq_decode_paged / tq_decode_paged_static. */
#define TQ_IO_ROTATE_Q 0x100     /* q_rot is given in ORIGINAL space: the kernel rotates it (q' = q H) while loading;
                                    q_proj must be NULL */
#define TQ_IO_DEROTATE_OUT 0x200 /* write out in original space (out H), as the reference's rotate_output does */
#define TQ_IO_TCGEN05 0x400      /* run the tensor-memory (tcgen05) variant of the decode kernel where it exists: 2- and
                                    3-bit codebooks without Sparse-V; other formats ignore the flag.  Slower than the
                                    default kernel on this hardware and held to the same output tolerance. */

/* Bits set by kernels in the optional device-side status word. */
#define TQ_COMPRESS_TCGEN05 2 /* flag in tq_compress_paged's `prerotated` argument, see there */

#define TQ_STATUS_BAD_BLOCK 1 /* a block-table entry was outside [0, num_blocks) and was clamped */
#define TQ_STATUS_TIMEOUT 2   /* a bounded wait on an async copy ran out */
#define TQ_STATUS_BAD_SLOT 4  /* a slot index was >= num_blocks * block_size and was skipped */

/* Library version, (major << 16) | minor.  Host only. */
int tq_version(void);

/* Bytes of one 16-token page of the paged cache for a format, or a negative
 * status.  The cache tensor is uint8 [num_blocks, num_kv_heads,
 * block_size / 16 * page_bytes]; this replaces the fixed 68-byte slot of
 * TurboQuantFP4Backend.get_kv_cache_shape
 * (turboquant/integration/tq_fp4_backend.py:699-722).  Host only. */
int tq_page_bytes(int k_bits, int v_bits, int use_qjl);

/* KV compression into the paged cache: rotation (fast WHT, skipped when
 * `prerotated`), norm, Lloyd-Max bucketize, residual signs and norm (K only,
 * when use_qjl), bit-packing, scatter by slot.  One launch handles K and V.
 *
 * Replaces the cache-update step the reference does with torch ops,
 * turbo4_fp8_compress_and_scatter (turboquant/integration/vllm_backend.py:
 * 179-230) / TurboQuantFP4Impl.do_kv_cache_update
 * (turboquant/integration/tq_fp4_backend.py:456-484), with the arithmetic of
 * polarquant_compress (turboquant/core/quantizer.py:141-173) and the packed
 * fields of compress_k / compress_v (turboquant/kernels/packed_compress.py:
 * 157-177, 226-240).
 *
 * key, value: [n_tokens, n_kv_heads, 128] of in_dtype with element strides
 * (stride_token, stride_head); the 128 values of a head are contiguous and
 * 16-byte aligned.  slot_mapping: int64 [n_tokens]; negative slots are
 * clamped to 0 as the reference does (vllm_backend.py:224); slots beyond the
 * cache are skipped and flagged in *status.  centroids: fp32 [2^bits],
 * boundaries: fp32 [2^bits - 1], ascending, on the device.  status: optional
 * device int32, OR-ed with TQ_STATUS_* bits; may be NULL.
 *
 * The fast path (tensor-core rotation, table-driven bucketize) needs
 * neighbouring boundaries to be more than 1/64 apart - true of the Lloyd-Max
 * codebooks for 128 dims at 2, 3 and 4 bits; other codebooks are handled by a
 * slower generic path with the same results.  A vector that contains a NaN or
 * an infinity gets the indices of a zero vector and a non-finite norm.  The
 * first call on a device sets a function attribute (shared-memory size) and
 * should be made before any stream capture.
 *
 * prerotated: 0 = rotate here, 1 = the rows are already rotated; OR-ed with
 * TQ_COMPRESS_TCGEN05 the rotation of fp16 / bf16 rows of a large launch runs as
 * one 128 x 128 x 128 tcgen05 product per 128 rows with one thread per vector
 * afterwards (an opt-in variant: same results within the rotation allowance,
 * about 15 % slower than the default kernel on this hardware). */
int tq_compress_paged(const void* key, const void* value, int in_dtype,
                      int64_t k_stride_token, int64_t k_stride_head,
                      int64_t v_stride_token, int64_t v_stride_head,
                      void* cache, int64_t num_blocks, int block_size,
                      const int64_t* slot_mapping,
                      const float* k_centroids, const float* k_boundaries,
                      const float* v_centroids, const float* v_boundaries,
                      int n_tokens, int n_kv_heads, int k_bits, int v_bits,
                      int use_qjl, int prerotated, int32_t* status, tq_stream_t stream);

/* Pages of one (sequence, kv head) that a split-K chunk covers when the
 * caller passes chunk_pages = 0 to tq_decode_paged.  Host only. */
int tq_decode_auto_chunk_pages(int num_seqs, int num_kv_heads, int num_q_heads, int max_pages_per_seq);

/* Bytes of split-K workspace tq_decode_paged needs.  Host only. */
int64_t tq_decode_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads,
                                  int max_pages_per_seq, int chunk_pages);

/* Asymmetric packed paged decode attention with GQA and split-K, one query
 * token per sequence.  Replaces _tq_v12_sparse_v_kernel / _tq_v11_single_kernel
 * (turboquant/kernels/sparse_v.py:26-159, 164-261) and, for the score
 * estimator with the QJL sign term, _packed_attn_v7 + _splitk_reduce
 * (turboquant/kernels/packed_attention.py:76-227); it is called where the
 * reference calls launch_fp4_pa_v9 (turboquant/integration/tq_fp4_backend.py:
 * 274-295).
 *
 * out, q_rot, q_proj: [num_seqs, num_q_heads, 128] of io_dtype (fp16 or
 * bf16, optionally OR-ed with TQ_IO_ROTATE_Q / TQ_IO_DEROTATE_OUT to fuse the two
 * rotations of TurboQuantFP8State.rotate_query / rotate_output,
 * turboquant/integration/vllm_backend.py:158-176, into this call); q_rot is the query in rotated space, q_proj = S q_rot (pass q_rot,
 * or NULL, when S = I).  score = sm_scale * (k_norm <q_rot, c[k_idx]> +
 * corr_scale * k_rnorm <q_proj, signs>); out = softmax(score) applied to
 * v_norm * c_v[v_idx], in rotated space.  Query head h reads kv head
 * h / (num_q_heads / num_kv_heads).  sparse_thresh > 0 enables the Sparse-V
 * rule (a 16-token V page is not fetched when every softmax weight in it, for
 * every query head of the group, is <= sparse_thresh relative to the running
 * maximum); <= 0 disables it.  block_tables: int32 [num_seqs, bt_stride];
 * seq_lens: int32 [num_seqs].  workspace: at least
 * tq_decode_workspace_bytes(...) bytes, 16-byte aligned.  skip_stats:
 * optional device uint32[2] = {V pages visited, V pages skipped}, accumulated
 * with atomics when non-NULL.  Sequences of length 0 produce zeros. */
int tq_decode_paged(void* out, const void* q_rot, const void* q_proj, int io_dtype,
                    const void* cache, int64_t num_blocks, int block_size,
                    const int32_t* block_tables, int64_t bt_stride, const int32_t* seq_lens,
                    const float* k_centroids, const float* v_centroids,
                    float sm_scale, float corr_scale, float sparse_thresh,
                    void* workspace, int64_t workspace_bytes,
                    int32_t* status, uint32_t* skip_stats,
                    int num_seqs, int num_q_heads, int num_kv_heads, int max_pages_per_seq,
                    int k_bits, int v_bits, int use_qjl, int chunk_pages, tq_stream_t stream);

#define TQ_DECODE_STATIC_SCRATCH_BYTES (16 * 1024 * 1024)

/* tq_decode_paged for callers that cannot provide a workspace.  It has no
 * counterpart in the reference.  Meant for hosts that cannot allocate device
 * memory themselves: a server that gave all free HBM to its KV-cache pool at
 * start-up, so any later allocation fails, or a foreign-language binding that
 * only passes on pointers it received.  Same arguments as tq_decode_paged
 * without workspace / workspace_bytes; the split-K partials go to a fixed
 * 16 MiB array that is part of the library image (every GPU that loads the
 * library holds those 16 MiB until the process exits).  Problems that need
 * more (tq_decode_workspace_bytes(...) > TQ_DECODE_STATIC_SCRATCH_BYTES)
 * are refused with TQ_ERR_WORKSPACE before anything is launched: pass a
 * larger chunk_pages or use tq_decode_paged.  The function calls no
 * allocation routine.  The first call on each device looks up the device
 * address of the array (cudaGetSymbolAddress) and remembers it; make that
 * first call during set-up, before any stream capture begins.  All calls on
 * a device share the one array, which keeps whatever the last call left in it
 * (nothing in it needs clearing: each call writes every partial it later
 * reads); two calls whose kernels overlap on the GPU, e.g. on different
 * streams, race on it and must be serialised by the caller. */
int tq_decode_paged_static(void* out, const void* q_rot, const void* q_proj, int io_dtype,
                           const void* cache, int64_t num_blocks, int block_size,
                           const int32_t* block_tables, int64_t bt_stride, const int32_t* seq_lens,
                           const float* k_centroids, const float* v_centroids,
                           float sm_scale, float corr_scale, float sparse_thresh,
                           int32_t* status, uint32_t* skip_stats,
                           int num_seqs, int num_q_heads, int num_kv_heads, int max_pages_per_seq,
                           int k_bits, int v_bits, int use_qjl, int chunk_pages, tq_stream_t stream);

/* Fast Walsh-Hadamard rotation of n rows of 128 values: out = scale * (in @ H).
 * Used for q' = q H before decode and out = o H after it, the two matmuls of
 * TurboQuantFP8State.rotate_query / rotate_output
 * (turboquant/integration/vllm_backend.py:158-176).  in and out may alias. */
int tq_wht_rows(const void* in, void* out, int dtype, int64_t n_rows, float scale, tq_stream_t stream);

/* Contiguous packed K compression, the output format of compress_k /
 * compress_k_permuted (turboquant/kernels/packed_compress.py:157-177,
 * 219-223): k_idx uint8 [n, 16*bits] (2-bit: 4 per byte LSB first; 4-bit: low
 * nibble first; 3-bit: little-endian bit stream as decoded at
 * turboquant/kernels/sparse_v.py:57-60), k_signs uint8 [n, 16] (sequential,
 * or in the stride-4 order of permute_signs_for_chunked,
 * packed_compress.py:180-216, when permute_signs), k_rnorm and k_norm fp16 [n].
 * Arithmetic as turboquant/core/quantizer.py:141-173.  More than 32768 rows
 * take the persistent table-driven kernel (as tq_compress_paged: on already
 * rotated rows the indices and signs are the reference's bit for bit, with
 * the rotation done here at most 1e-4 of the coordinates differ by one
 * centroid); smaller launches take the binary-search kernel. */
int tq_compress_k(const void* K, int in_dtype, int64_t n, const float* centroids, const float* boundaries,
                  int bits, int prerotated, int permute_signs,
                  uint8_t* k_idx, uint8_t* k_signs, void* k_rnorm, void* k_norm, tq_stream_t stream);

/* Contiguous packed V compression, compress_v (packed_compress.py:226-240):
 * v_idx uint8 [n, 16*bits], v_norm fp16 [n]. */
int tq_compress_v(const void* V, int in_dtype, int64_t n, const float* boundaries, int bits, int prerotated,
                  uint8_t* v_idx, void* v_norm, tq_stream_t stream);

/* polarquant_compress (turboquant/core/quantizer.py:111-183) with unpacked
 * outputs: indices int64 [n,128], norms fp32 [n], k_mse_rot fp32 [n,128] and,
 * when use_qjl, signs fp32 (+-1) [n,128] and rnorm fp32 [n]. */
int tq_polarquant_compress(const void* x, int in_dtype, int64_t n, const float* centroids,
                           const float* boundaries, int bits, int use_qjl, int prerotated,
                           int64_t* indices, float* norms, float* k_mse_rot, float* signs, float* rnorm,
                           tq_stream_t stream);

/* Bytes of workspace tq_packed_attention needs for a split count.  Host only. */
int64_t tq_packed_attention_workspace_bytes(int BH, int num_splits);

/* Split count tq_packed_attention picks when num_splits = 0; replaces the
 * MI355X tuning table of _get_config (packed_attention.py:236-267).  Host only. */
int tq_packed_attention_auto_splits(int BH, int Sk);

/* packed_attention (turboquant/kernels/packed_attention.py:290-344):
 * contiguous [BH, Sk, ...] packed K/V, one query row per BH, split-K partial
 * kernel plus merge.  Q, Q_proj fp16 [BH,128]; k_idx/v_idx uint8
 * [BH,Sk,16*bits]; k_signs_perm uint8 [BH,Sk,16] in stride-4 order; norms fp16
 * [BH,Sk]; centroids fp32 [2^bits]; out fp16 [BH,128] in rotated space. */
int tq_packed_attention(const void* Q, const void* Q_proj, const uint8_t* k_idx, const uint8_t* k_signs_perm,
                        const void* k_rnorm, const void* k_norm, const uint8_t* v_idx, const void* v_norm,
                        const float* centroids, float corr_scale, int BH, int Sk, int bits, int num_splits,
                        void* workspace, int64_t workspace_bytes, void* out, tq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TQ_B200_H_ */
