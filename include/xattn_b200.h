/*
 * xattn_b200 -- C ABI of the B200 (sm_100a) XAttention prefill hot path.
 *
 * Every entry point takes plain pointers and sizes, launches on the CUDA stream it is given and
 * returns an int status (0 = ok, see xattn_b200_error_string).  Nothing here synchronises the
 * stream or throws.  Unless stated otherwise every pointer is a device pointer on the current
 * device; the library allocates no device memory: scratch is passed in by the caller, sized by the
 * *_workspace_bytes functions.  No entry point keeps state between calls, except
 * xattn_b200_estimate_static, whose scratch is a fixed array inside the library that all of its
 * calls share (see there), and the diagnostic launch counter.
 *
 * File:line citations name the reference interface (mit-han-lab/x-attention) each entry replaces.
 *
 * Tensor conventions: q is [batch, hq, q_len, head_dim], k/v are [batch, hkv, k_len, head_dim],
 * addressed through element strides (stride_b, stride_h, stride_l) with a unit stride along
 * head_dim; base pointers and all strides must keep 16-byte alignment.  hq must be a multiple of
 * hkv (query head h reads kv head h / (hq/hkv)); the reference requires hq == hkv
 * (xattn/src/Xattention.py:31) and callers repeat K/V beforehand -- passing un-repeated K/V here
 * gives the same result without the copy.
 *
 * `status` arguments: optional pointer to ONE int32 that kernels can write from the device --
 * device memory or pinned host memory mapped into the device (zero it before the call).  A kernel
 * whose bounded wait ran out stores a non-zero code there instead of hanging.
 */
#ifndef XATTN_B200_H_
#define XATTN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
#define XATTN_B200_BF16 0
#define XATTN_B200_F16 1

/* estimate semantics: which of the reference's two code paths to reproduce */
#define XATTN_B200_SEMANTICS_TORCH 0  /* torch branch, xattn/src/Xattention.py:174-252 (what the reference runs on a B200) */
#define XATTN_B200_SEMANTICS_TRITON 1 /* Triton kernels, xattn/src/kernels.py:5-156,197-235 */
/* The torch branch with attn_sums in CHUNK-BAND layout [batch, hq, q_blocks_pad, chunk_size/block_size]: when the
 * keys are not padded the torch branch leaves every column outside the row's own chunk at zero, so only the
 * chunk's own key blocks (columns current_index .. current_index + blocks_per_chunk) are written.  Causal and
 * k_len % chunk_size == 0 only (XATTN_B200_ERR_ARG otherwise).  Feed the result to xattn_b200_select_band. */
#define XATTN_B200_SEMANTICS_TORCH_BAND 2

/* status codes */
#define XATTN_B200_OK 0
#define XATTN_B200_ERR_ARG 1        /* bad shape / stride / alignment / unsupported value */
#define XATTN_B200_ERR_WORKSPACE 2  /* workspace too small or NULL */
#define XATTN_B200_ERR_CUDA 3       /* a CUDA runtime / driver call failed */
#define XATTN_B200_ERR_ARCH 4       /* current device is not sm_100 */
#define XATTN_B200_ERR_LIMIT 5      /* size beyond a stated maximum */
#define XATTN_B200_ERR_DEVICE_WAIT 101 /* written to *status by a kernel whose bounded wait ran out */

int xattn_b200_version(void);
const char* xattn_b200_error_string(int code);

/* Number of kernel launches the library has issued in this process so far (all entry points, all devices).
 * A diagnostic counter for benchmarks and tests; no counterpart in the reference.  Host function. */
unsigned long long xattn_b200_launch_count(void);

/* Default estimate chunk of Xattention_prefill (xattn/src/Xattention.py:322-331). */
int xattn_b200_default_chunk_size(int k_len);

/*
 * Padded geometry of xattn_estimate (xattn/src/Xattention.py:33-40,65-70):
 * out[0]=q_len_pad out[1]=k_len_pad out[2]=q_blocks_pad out[3]=k_blocks_pad
 * out[4]=q_chunks  out[5]=k_chunks  out[6]=blocks_per_chunk out[7]=k_blocks_pad-q_blocks_pad
 * Host function, no CUDA call.
 */
int xattn_b200_estimate_geometry(int q_len, int k_len, int chunk_size, int stride, int block_size, int out[8]);

/* Scratch needed by xattn_b200_estimate (bytes), enough for any mask and semantics.  0: unsupported geometry.
 * Host function, no CUDA call. */
size_t xattn_b200_estimate_workspace_bytes(int batch, int hq, int q_len, int k_len, int stride, int block_size,
                                           int chunk_size);
/* The same for one call's `causal` and `semantics` arguments.  Much smaller when the torch branch blanks every
 * column left of a row's chunk (causal, keys not padded, XATTN_B200_SEMANTICS_TORCH or _TORCH_BAND): a row then
 * keeps partial sums for its own chunk only (131072 tokens, stride 16, 32 heads: 20 MiB instead of 1 GiB). */
size_t xattn_b200_estimate_workspace_bytes_ex(int batch, int hq, int q_len, int k_len, int stride, int block_size,
                                              int chunk_size, int causal, int semantics);

/*
 * Phase 1 -- antidiagonal block-importance estimate.
 * Replaces flat_group_gemm_fuse_reshape + softmax_fuse_block_sum (xattn/src/kernels.py:325-363,
 * 238-289) and the torch estimate body (xattn/src/Xattention.py:71-136,174-252).
 *
 * For every head: S'[i,j] = scale * sum_{t<stride} Q[stride*i + stride-1-t] . K[stride*j + t];
 * row softmax over the visible columns; sums over (block_size/stride)^2 cells.  The S' matrix is
 * never written to memory: a tcgen05 GEMM keeps 128x256 tiles in tensor memory and its epilogue
 * emits per-row, per-key-block partial sums (into `workspace`), which a second small kernel
 * normalises into `attn_sums`.
 *
 * q_len / k_len need not be multiples of `stride`: the tokens a ragged last stride group lacks count as the
 * zeros the reference pads with (xattn/src/Xattention.py:42-51); the library stages a zero-padded copy of the
 * one 128-row tile of Q (128- or 256-row tile of K) that holds that group in `workspace` -- a few MB instead
 * of a padded copy of the tensors (workspace sizes assume head_dim 128 for it).  head_dim is the
 * length of a row in elements, a multiple of 64 (it may exceed the model's head dimension when
 * rows carry split-precision terms, see xattn_b200_split_f32);  `scale` = 1/(sqrt(D)*stride*norm).
 * attn_sums: float32 [batch, hq, q_blocks_pad, k_blocks_pad] (fully written).
 */
int xattn_b200_estimate(const void* q, const void* k, int dtype, int batch, int hq, int hkv, int q_len, int k_len,
                        int head_dim, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_l, int64_t k_stride_b,
                        int64_t k_stride_h, int64_t k_stride_l, int stride, int block_size, int chunk_size,
                        float scale, int causal, int semantics, float* attn_sums, void* workspace,
                        size_t workspace_bytes, int* status, void* cuda_stream);

/*
 * The estimate without a caller-supplied workspace.  No counterpart in the reference.
 *
 * Meant for callers that cannot allocate device memory where they call the estimate: a process whose
 * GPU memory was handed out at start-up to a pool that this caller does not own, a plugin host that
 * forbids allocation after initialisation, or a latency-critical section where an allocation (and the
 * device synchronisation it can imply) is not acceptable.  The scratch that xattn_b200_estimate takes
 * from the caller lives here in a fixed array inside the library image, XATTN_B200_STATIC_SCRATCH_BYTES
 * large, resident on every GPU that loads the library until the process exits.  The call itself
 * allocates and frees nothing; the caller still provides q, k and attn_sums.
 *
 * Arguments and results are those of xattn_b200_estimate (minus workspace/workspace_bytes).
 * Returns XATTN_B200_ERR_LIMIT when xattn_b200_estimate_workspace_bytes_ex(...) for the call exceeds
 * XATTN_B200_STATIC_SCRATCH_BYTES -- use xattn_b200_estimate with your own workspace then.
 *
 * The first call on each device looks up the array's device address (the device must be current, as
 * for every call); make that first call outside any CUDA stream capture.  All calls on a device share
 * the one array, which simply keeps whatever the last call left in it (no call relies on its previous
 * contents): two calls whose kernels can overlap on the GPU -- different streams without an ordering
 * between them, or several host threads -- race on it and give wrong sums.  Order them on one stream
 * or with events.
 */
#define XATTN_B200_STATIC_SCRATCH_BYTES (32u << 20)
int xattn_b200_estimate_static(const void* q, const void* k, int dtype, int batch, int hq, int hkv, int q_len,
                               int k_len, int head_dim, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_l,
                               int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_l, int stride,
                               int block_size, int chunk_size, float scale, int causal, int semantics,
                               float* attn_sums, int* status, void* cuda_stream);

/*
 * Split fp32 rows into three bf16 terms (x = hi + mid + lo) laid out as rows of 6*head_dim so that
 * a bf16 GEMM over the widened rows reproduces the fp32 product to ~2^-24:
 *   role 0 (query side): [hi, hi, mid, hi, lo, mid]     role 1 (key side): [hi, mid, hi, lo, hi, mid]
 * x is [batch, heads, len_valid, head_dim] fp32 with element strides; out is contiguous
 * [batch, heads, len, 6*head_dim] bf16 with len >= len_valid, the rows past len_valid zero (the reference's
 * zero padding, xattn/src/Xattention.py:42-51).  No counterpart in the reference (its torch branch multiplies
 * fp32 directly, xattn/src/Xattention.py:183).
 */
int xattn_b200_split_f32(const float* x, int batch, int heads, int len, int len_valid, int head_dim, int64_t stride_b,
                         int64_t stride_h, int64_t stride_l, int role, void* out, void* cuda_stream);

/*
 * Rotary position embedding, applied in place to the query and key projections in one launch.
 * Replaces apply_rotary_pos_emb (xattn/src/load_llama.py:34-65, called at :142 and :356):
 *   x' = x*cos + rotate_half(x)*sin, with each product and the sum rounded to the 16-bit storage type exactly
 *   as the reference's three tensor operations round them (results are bit-identical).
 * q: [batch, hq, len, head_dim], k: [batch, hkv, len, head_dim], element strides, unit stride on head_dim --
 * typically the [batch, len, heads*head_dim] projection outputs seen through strides, so that no transposed
 * copy is made before the estimate and attention kernels (which take the same strided views).
 * cos, sin: [batch, len, head_dim] in the same dtype (stride_b may be 0 for one table shared by the batch).
 * head_dim a multiple of 16; bases 16-byte aligned; strides multiples of 8 elements.
 */
int xattn_b200_rope_qk(void* q, void* k, int dtype, int batch, int hq, int hkv, int len, int head_dim,
                       int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_l, int64_t k_stride_b,
                       int64_t k_stride_h, int64_t k_stride_l, const void* cos, const void* sin,
                       int64_t cs_stride_b, int64_t cs_stride_l, void* cuda_stream);

/*
 * Phase 2 -- threshold block selection for all query chunks at once.
 * Replaces find_blocks_chunked (xattn/src/utils.py:44-191, prefill branch :87-172) as called per
 * chunk by xattn_estimate (xattn/src/Xattention.py:255-263), plus the mask post-processing of
 * xattn/src/Xattention.py:275-297 (causal clean-up, keep_sink, keep_recent).
 *
 * attn_sums: float32 [batch, heads, q_blocks, k_blocks].  Row R belongs to chunk R/blocks_per_chunk
 * whose current_index is block_offset + (R/blocks_per_chunk)*blocks_per_chunk.
 * diagonal_cleanup: 1 = also clear columns right of each row's diagonal block, as xattn_estimate does
 * after concatenating the chunks (xattn/src/Xattention.py:275-285); 0 = find_blocks_chunked alone.
 * threshold_per_head: optional device float32[heads] (overrides `threshold`).
 * Outputs (any may be NULL):
 *   mask       uint8 [batch, heads, q_blocks, k_blocks]           (the reference's simple_masks)
 *   block_idx  int32 [batch, heads, list_q_blocks, list_k_blocks] ascending kept key blocks per row,
 *   block_cnt  int32 [batch, heads, list_q_blocks]                restricted to rows < list_q_blocks,
 *              columns < list_k_blocks and, when causal, to blocks that hold at least one key visible
 *              to the row's last token (query end aligned to key end, list_q_len/list_k_len tokens).
 * k_blocks <= 8192.
 */
int xattn_b200_select(const float* attn_sums, int batch, int heads, int q_blocks, int k_blocks,
                      int blocks_per_chunk, int block_offset, int causal, int diagonal_cleanup, double threshold,
                      const float* threshold_per_head, int keep_sink, int keep_recent, uint8_t* mask,
                      int32_t* block_idx, int32_t* block_cnt, int list_q_blocks, int list_k_blocks, int list_q_len,
                      int list_k_len, int* status, void* cuda_stream);

/*
 * xattn_b200_select for attn_sums in chunk-band layout (XATTN_B200_SEMANTICS_TORCH_BAND): attn_sums is
 * [batch, heads, q_blocks, blocks_per_chunk]; entry c of row R is the score of key block current_index + c, every
 * other key block has score zero.  Same rule, same outputs (mask and lists are over all k_blocks columns), but a
 * row is blocks_per_chunk values instead of k_blocks.  Causal only.
 */
int xattn_b200_select_band(const float* attn_sums, int batch, int heads, int q_blocks, int k_blocks,
                           int blocks_per_chunk, int block_offset, int causal, int diagonal_cleanup, double threshold,
                           const float* threshold_per_head, int keep_sink, int keep_recent, uint8_t* mask,
                           int32_t* block_idx, int32_t* block_cnt, int list_q_blocks, int list_k_blocks,
                           int list_q_len, int list_k_len, int* status, void* cuda_stream);

/*
 * Block mask -> per-row block lists, for callers that bring their own mask (the `base_blockmask`
 * argument of block_sparse_attn_func, call site xattn/src/Xattention.py:377-391).
 * mask: uint8/bool [batch, heads, mask_q_blocks, mask_k_blocks]; only the first ceil(q_len/128) rows
 * and ceil(k_len/128) columns are read.  Lists have the layout described above with
 * list_q_blocks = ceil(q_len/128), list_k_blocks = ceil(k_len/128).
 */
int xattn_b200_mask_to_lists(const uint8_t* mask, int batch, int heads, int mask_q_blocks, int mask_k_blocks,
                             int q_len, int k_len, int causal, int32_t* block_idx, int32_t* block_cnt,
                             void* cuda_stream);

/*
 * Phase 3 -- block-sparse FlashAttention forward over 128x128 blocks.
 * Replaces block_sparse_attn.block_sparse_attn_func (third-party; call site
 * xattn/src/Xattention.py:377-391) for one sequence per batch entry, head_mask_type 1 on every
 * head, no dropout.
 *
 * out[b,h,i,:] = softmax_j(scale * q_i.k_j) v_j over keys j in kept blocks, and j <= i + (k_len-q_len)
 * when causal.  head_dim must be 128.  Rows with no visible key give zeros.
 * out has element strides (o_stride_b, o_stride_h, o_stride_l), unit stride along head_dim, same
 * dtype as the inputs.
 */
int xattn_b200_block_sparse_attn(const void* q, const void* k, const void* v, int dtype, int batch, int hq, int hkv,
                                 int q_len, int k_len, int head_dim, int64_t q_stride_b, int64_t q_stride_h,
                                 int64_t q_stride_l, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_l,
                                 int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_l, const int32_t* block_idx,
                                 const int32_t* block_cnt, int causal, float scale, void* out, int64_t o_stride_b,
                                 int64_t o_stride_h, int64_t o_stride_l, int* status, void* cuda_stream);

/*
 * The same operation with scratch memory, which lets the library treat the lists that long-context prefill
 * produces most -- one or two blocks (attention sink + diagonal), identical for all query heads of a kv head --
 * in a kernel of their own: K/V tiles loaded once per kv head and query block and shared by its query heads
 * (GQA head sharing), both Q.K^T products and both P.V products issued back to back, one softmax pass without
 * online rescaling.  Which rows qualify is decided on the device (no synchronisation); all other rows run through
 * the general kernel of xattn_b200_block_sparse_attn.  Because two kernels in a row cost a second tail, the split is
 * also only made, again decided on the device, when the qualifying rows list at least 92 % of the call's blocks
 * (Llama-3.1-8B at 128K tokens: 95 %, 8 % faster; at 64K: 89 %, no gain; at 32K: 66 %, a loss); below that the
 * general kernel computes everything and the attempt has cost 30-45 microseconds (so callers with short sequences
 * should use xattn_b200_block_sparse_attn; the Python layer offers the workspace from 96K tokens on).
 * xattn_b200_block_sparse_attn_split_share(percent) replaces the 92 for the calls enqueued after it (0: split
 * whenever anything qualifies, 101: never) and returns the previous value; a negative argument only reads it.
 * Same call-site contract (xattn/src/Xattention.py:377-391), same results up to the summation order.
 * A non-causal call uses the scratch memory differently: its work items (batch, query head, query block) are sorted
 * by list length, longest first, by one small kernel, and dealt to the SMs in that order; masks whose rows differ
 * widely in length (video diffusion: 5 to 891 blocks per row) otherwise leave the most loaded SM 16 % above the mean.
 * workspace: device memory of xattn_b200_block_sparse_attn_workspace_bytes() bytes, 16-byte aligned, contents
 * irrelevant on entry; the call's kernels use it until they finish.  With workspace == NULL the call equals
 * xattn_b200_block_sparse_attn.
 */
size_t xattn_b200_block_sparse_attn_workspace_bytes(int batch, int hq, int hkv, int q_len, int k_len);
int xattn_b200_block_sparse_attn_split_share(int percent);
int xattn_b200_block_sparse_attn_ws(const void* q, const void* k, const void* v, int dtype, int batch, int hq, int hkv,
                                    int q_len, int k_len, int head_dim, int64_t q_stride_b, int64_t q_stride_h,
                                    int64_t q_stride_l, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_l,
                                    int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_l,
                                    const int32_t* block_idx, const int32_t* block_cnt, int causal, float scale,
                                    void* out, int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_l,
                                    void* workspace, size_t workspace_bytes, int* status, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* XATTN_B200_H_ */
