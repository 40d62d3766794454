/*
 * C ABI of libfa_b200.so: FlashAttention forward / backward for NVIDIA B200 (sm_100a).
 *
 * The entry points replace the host functions of the reference extension
 * (csrc/flash_attn/fmha_api.cpp): the same argument contract, expressed as plain pointers and
 * sizes so that any binding (pybind11, ctypes, cgo, JNI ...) can call it.  Nothing here
 * allocates output tensors: the caller owns every buffer.  All launches are asynchronous on the
 * stream that is passed in; no entry point synchronises.
 *
 * Tensor layouts (identical to the reference, fmha_api.cpp:173-186):
 *   q            [total_q, heads, head_dim]   16-bit (fp16 or bf16), last dim contiguous,
 *   k, v         [total_k, heads, head_dim]   row / head strides given in elements
 *   cu_seqlens_* [batch + 1] int32            cumulative sequence lengths (varlen packing)
 *   o            [total_q, heads, head_dim]
 *   softmax_lse  [batch, heads, lse_stride]   fp32, natural-log LSE of the scaled scores
 *
 * Every function returns FA_OK (0) or a negative FA_ERR_* code; fa_status_string() names it and
 * fa_last_error() returns a thread-local detail message.
 */
#ifndef FA_B200_H_
#define FA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA_OK 0
#define FA_ERR_INVALID_ARGUMENT (-1) /* shape / stride / dtype / alignment the kernels cannot take */
#define FA_ERR_CUDA (-2)             /* a CUDA runtime or driver call failed                        */
#define FA_ERR_UNSUPPORTED (-3)      /* valid in the reference but not built here                    */
#define FA_ERR_WORKSPACE (-4)        /* workspace missing or too small                               */

/* Forward arguments: replaces FMHA_fprop_params (csrc/flash_attn/src/fmha.h:50-139) as filled by
 * set_params_fprop (csrc/flash_attn/fmha_api.cpp:37-117). */
typedef struct fa_fwd_params {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* softmax_lse;
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;
  /* Block-sparse only (fmha_api.cpp:451-573): converted block mask, int32
   * [blockmask_rows, blockmask_cols] as produced by convert_blockmask, with
   * blockmask_rows >= ceil(max_seqlen_k / 256) key blocks and
   * blockmask_cols >= ceil(max_seqlen_q / 16) list slots; NULL for dense attention. */
  const int32_t* blockmask;
  /* Optional [batch, heads, s_rows, s_cols] 16-bit output (return_softmax, a test aid): the softmax
   * probability of every (query, key) pair with the sign bit set where dropout dropped it, in
   * plain row-major order (the reference writes un-normalised values in its MMA fragment order,
   * csrc/flash_attn/src/fmha/gmem_tile.h:289-405).  Entries outside the sequences are not written.
   * Recomputed on the CUDA cores after the attention kernel: O(seqlen^2 * d), for tests.  NULL to skip. */
  void* s_dmask;
  int64_t s_rows, s_cols;
  /* strides in elements */
  int64_t q_row_stride, q_head_stride;
  int64_t k_row_stride, k_head_stride;
  int64_t v_row_stride, v_head_stride;
  int64_t o_row_stride, o_head_stride;
  int64_t lse_stride; /* row length of softmax_lse, >= max_seqlen_q */
  int32_t batch, heads, head_dim;
  int32_t total_q, total_k;
  int32_t max_seqlen_q, max_seqlen_k; /* as passed by the caller, un-rounded */
  float p_dropout;                    /* probability of dropping, in [0, 1) */
  float softmax_scale;
  int32_t is_causal;
  int32_t is_bf16; /* 0 = fp16, 1 = bf16 */
  /* Philox state (seed, offset) exactly as at::cuda::philox::unpack returns it in the reference
   * (fmha_fprop_kernel_1xN.h:653-656); ignored when p_dropout == 0. */
  uint64_t philox_seed, philox_offset;
  /* Head count / first head used in the Philox subsequence, for callers that shard heads across
   * devices and want the mask of the unsharded call.  0 / 0 means (heads, 0). */
  int32_t mask_heads_total, mask_head_offset;
  /* Optional device int32[4].  A CTA that abandons a bounded wait writes the (non-zero) serial
   * number of its launch into word 0, which keeps the CTAs of that launch that have not started
   * from starting; words 2 (forward) and 3 (backward) are set to 1 at the same time and never
   * cleared by the library. */
  int32_t* status;
  /* Block-sparse only: device scratch of fa_blocksparse_workspace_bytes() for the per-sequence
   * block-visit table the call derives from blockmask and cu_seqlens. */
  void* bs_workspace;
  size_t bs_workspace_bytes;
  int32_t blockmask_rows, blockmask_cols;
} fa_fwd_params;

/* Backward arguments: replaces FMHA_dgrad_params (csrc/flash_attn/src/fmha.h:141-163) as filled
 * by set_params_dgrad (csrc/flash_attn/fmha_api.cpp:119-171). */
typedef struct fa_bwd_params {
  fa_fwd_params fwd; /* q, k, v, o (read), softmax_lse (read), strides, sizes, flags, philox */
  const void* dout;  /* [total_q, heads, head_dim], contiguous */
  void* dq;          /* written in place, caller owned, strides below */
  void* dk;
  void* dv;
  float* softmax_d; /* [batch, heads, lse_stride] fp32 out: p_keep * rowsum(dO * O) */
  int64_t dq_row_stride, dq_head_stride;
  int64_t dk_row_stride, dk_head_stride;
  int64_t dv_row_stride, dv_head_stride;
  /* Scratch of at least fa_bwd_workspace_bytes(): fp32 dQ accumulator.  Contents on entry are
   * ignored; the call clears what it needs. */
  void* workspace;
  size_t workspace_bytes;
  /* Profiling aid: which of the three backward launches to run.  0 = all; otherwise a bit mask,
   * 1 = preprocess (softmax_d, accumulator clear), 2 = main kernel, 4 = postprocess (dq write). */
  int32_t stage_mask;
  /* Non-zero: dq is bit-for-bit reproducible from run to run, like the reference's, which adds the
   * key blocks into dq_tmp one after the other (csrc/flash_attn/src/fmha_dgrad_kernel_1xN_loop.h:
   * 523-595).  The key-tile CTAs then add their dQ tiles into the accumulator in ascending key-tile
   * order through one ticket word per (batch, head, 128-row query tile) instead of in arrival
   * order; the workspace must hold fa_bwd_workspace_bytes_ex(..., 1).  Slower: see the bench. */
  int32_t deterministic;
} fa_bwd_params;

/* mha_fwd (csrc/flash_attn/fmha_api.cpp:173-299) and, with blockmask != NULL, mha_fwd_block
 * (:451-573).  Writes o and softmax_lse. */
int fa_fwd(const fa_fwd_params* params, void* cuda_stream);

/* mha_bwd (csrc/flash_attn/fmha_api.cpp:302-449) and, with blockmask != NULL, mha_bwd_block
 * (:575-718).  Writes dq, dk, dv and softmax_d. */
int fa_bwd(const fa_bwd_params* params, void* cuda_stream);

/* Capacity of the dQ accumulator built into the library for fa_bwd_static_scratch. */
#define FA_STATIC_SCRATCH_BYTES (8u << 20)

/* No counterpart in the reference.  Same computation and arguments as fa_bwd, for callers that
 * cannot allocate device memory when they call (a serving process whose memory was partitioned at
 * start-up and must not enter the CUDA allocator again, or a C / Go / Java binding with no caching
 * allocator to borrow scratch from): `workspace` and `workspace_bytes` are ignored and the fp32 dQ
 * accumulator is a fixed array inside the library image instead, FA_STATIC_SCRATCH_BYTES per GPU
 * that loads the library, held until the process exits.
 *   - Limit: total_q * heads * (head_dim <= 64 ? 64 : 128) * 4 <= FA_STATIC_SCRATCH_BYTES; larger
 *     calls return FA_ERR_WORKSPACE and launch nothing.
 *   - The call allocates and frees nothing (no cudaMalloc / cudaFree, no allocating library call).
 *   - The first call on each device looks up the device address of the array and caches it; make
 *     that first call before starting any stream capture on that device.
 *   - All calls on a device share the one array.  Each call clears the rows it is about to use,
 *     so the previous call's contents never leak into a result, but two calls that overlap on the
 *     GPU (different streams, or different host threads on the same device) race on it: order them
 *     on one stream or with events.  Block-sparse calls still need fwd.bs_workspace. */
int fa_bwd_static_scratch(const fa_bwd_params* params, void* cuda_stream);

/* Size of the scratch fa_bwd needs: replaces the dq_tmp allocation of mha_bwd
 * (csrc/flash_attn/fmha_api.cpp:402-404). */
size_t fa_bwd_workspace_bytes(int32_t total_q, int32_t heads, int32_t head_dim);

/* The same with the ticket words of the deterministic mode behind the accumulator when
 * `deterministic` is non-zero (equal to fa_bwd_workspace_bytes otherwise). */
size_t fa_bwd_workspace_bytes_ex(int32_t total_q, int32_t heads, int32_t head_dim, int32_t batch,
                                 int32_t max_seqlen_q, int32_t deterministic);

/* Scratch a block-sparse call needs (fa_fwd_params.bs_workspace): one int32 per (batch entry,
 * blockmask row, blockmask column).  The reference keeps this walk implicit in its kernels
 * (csrc/flash_attn/src/fmha_block_fprop_kernel_1xN.h:205-232). */
size_t fa_blocksparse_workspace_bytes(int32_t batch, int32_t blockmask_rows, int32_t blockmask_cols);

/* Generator increment the caller must apply after a forward with dropout: replaces the
 * counter_offset computed in run_fmha_fp16_sm80_loop_ (fmha_fprop_fp16_kernel.sm80.cu:44-54). */
uint64_t fa_philox_increment(int32_t head_dim, int32_t max_seqlen_q, int32_t max_seqlen_k,
                             int32_t is_blocksparse);

/* Key-block size N that fixes the dropout-mask layout: the block-size rule of mha_fwd for an
 * sm80 device (csrc/flash_attn/fmha_api.cpp:232-239 with fmha_fprop_fp16_kernel.sm80.cu:84-146). */
int32_t fa_mask_block_n(int32_t head_dim, int32_t max_seqlen_k, int32_t is_blocksparse);

/* Writes the dropout keep-mask (1 = kept) of one (batch, head) pair into a device uint8
 * [seqlen_q, seqlen_k] buffer using the same device code as the attention kernels; test hook
 * standing in for the sign bits of the reference's S_dmask output
 * (csrc/flash_attn/src/fmha/gmem_tile.h:289-405). */
int fa_debug_dropout_mask(uint8_t* mask_out, int32_t batch_idx, int32_t head_idx,
                          const fa_fwd_params* params, int32_t seqlen_q, int32_t seqlen_k,
                          void* cuda_stream);

/* Test hook for the Philox generator of the dropout mask (csrc/flash_attn/src/philox.cuh:7-136):
 * writes out[4*i .. 4*i+3] = the four output words for key `seed`, subsequence i, counter
 * offset/4, for i < n.  use_curand = 0 runs this library's round function `rounds` times (the
 * attention kernels use 7); use_curand = 1 runs cuRAND's Philox4_32_10 device generator instead,
 * an independent implementation of the same generator at 10 rounds. */
int fa_debug_philox(uint32_t* out, int32_t n, uint64_t seed, uint64_t offset, int32_t rounds,
                    int32_t use_curand, void* cuda_stream);

/* Row gather for the padding helpers: dst[r, :] = src[indices[r], :] for r < n_rows, rows of
 * `row_bytes` bytes (a multiple of 16; src and dst 16-byte aligned, rows contiguous).  Replaces the
 * framework indexing in flash_attn/bert_padding.py:14-19 (IndexFirstAxis.forward, used by
 * unpad_input :60-80) and :50-54 (IndexPutFirstAxis.backward).  An index outside [0, src_rows)
 * yields a zero row. */
int fa_gather_rows(const void* src, const int64_t* indices, void* dst, int64_t n_rows,
                   int64_t src_rows, int64_t row_bytes, void* cuda_stream);

/* Row scatter over zeros: dst (n_dst_rows rows) = 0 except dst[indices[r], :] = src[r, :] for
 * r < n_src_rows, written in one pass.  Replaces flash_attn/bert_padding.py:40-45
 * (IndexPutFirstAxis.forward, used by pad_input :83-95) and :22-29 (IndexFirstAxis.backward).
 * `workspace` holds n_dst_rows int32 (the inverse index map).  Indices outside [0, n_dst_rows) are
 * skipped; with duplicate indices one of the source rows wins. */
int fa_scatter_rows(const void* src, const int64_t* indices, void* dst, int64_t n_src_rows,
                    int64_t n_dst_rows, int64_t row_bytes, int32_t* workspace, void* cuda_stream);

/* Rotary position embedding on a packed qkv tensor (rows, 3, heads, head_dim), rows = batch *
 * seqlen with the token position = row % seqlen: q and k are rotated pairwise (channels 2i, 2i+1 by
 * the angle with cosine cos_table[pos][i] and sine sin_table[pos][i], fp32 tables of head_dim / 2
 * entries per position), v is copied; `out` has the layout of `qkv` and may not alias it.
 * Replaces flash_attn/rotary.py:33-43 (apply_rotary_pos_emb on q and k) plus the re-stack in
 * flash_attn/flash_attention.py:102-105.  conjugate != 0 rotates by the negative angles (the
 * gradient).  head_dim must be a multiple of 8; qkv and out 16-byte aligned and contiguous. */
int fa_rotary_qkv(const void* qkv, void* out, const float* cos_table, const float* sin_table,
                  int64_t rows, int32_t seqlen, int32_t heads, int32_t head_dim, int32_t is_bf16,
                  int32_t conjugate, void* cuda_stream);

const char* fa_status_string(int status);
const char* fa_last_error(void);

/* 0 when the current device is an sm_100 part and the library can run on it. */
int fa_device_supported(void);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H_ */
