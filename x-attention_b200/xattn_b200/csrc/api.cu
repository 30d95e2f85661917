// extern "C" surface of libxattn_b200.so (declared in include/xattn_b200.h): argument plumbing only.
#include "host_common.cuh"

namespace xb {
size_t estimate_workspace_bytes(int batch, int hq, int q_len, int k_len, int stride, int block_size, int chunk_size,
                                int causal, int semantics);
int estimate_launch(const void* q, const void* k, int dtype, int batch, int hq, int hkv, int q_len, int k_len,
                    int head_dim, int64_t qsb, int64_t qsh, int64_t qsl, int64_t ksb, int64_t ksh, int64_t ksl,
                    int stride, int block_size, int chunk_size, float scale, int causal, int semantics,
                    float* attn_sums, void* workspace, size_t workspace_bytes, int* status, cudaStream_t stream);
int split_f32_launch(const float* x, int batch, int heads, int len, int len_valid, int head_dim, int64_t sb, int64_t sh,
                     int64_t sl, int role, void* out, cudaStream_t stream);
int rope_qk_launch(void* q, void* k, int dtype, int batch, int hq, int hkv, int len, int head_dim, int64_t qsb,
                   int64_t qsh, int64_t qsl, int64_t ksb, int64_t ksh, int64_t ksl, const void* cos, const void* sin,
                   int64_t cs_stride_b, int64_t cs_stride_l, cudaStream_t stream);
int select_launch(const float* attn_sums, int batch, int heads, int q_blocks, int k_blocks, int bpc, int block_offset,
                  int causal, int diagonal_cleanup, double threshold, const float* thr_per_head, int keep_sink,
                  int keep_recent, uint8_t* mask, int32_t* block_idx, int32_t* block_cnt, int list_q_blocks,
                  int list_k_blocks, int list_q_len, int list_k_len, int band, int* status, cudaStream_t stream);
int mask_to_lists_launch(const uint8_t* mask, int batch, int heads, int mask_q_blocks, int mask_k_blocks, int q_len,
                         int k_len, int causal, int32_t* block_idx, int32_t* block_cnt, cudaStream_t stream);
int block_sparse_attn_launch(const void* q, const void* k, const void* v, int dtype, int batch, int hq, int hkv,
                             int q_len, int k_len, int head_dim, int64_t qsb, int64_t qsh, int64_t qsl, int64_t ksb,
                             int64_t ksh, int64_t ksl, int64_t vsb, int64_t vsh, int64_t vsl,
                             const int32_t* block_idx, const int32_t* block_cnt, int causal, float scale, void* out,
                             int64_t osb, int64_t osh, int64_t osl, void* workspace, size_t workspace_bytes,
                             int* status, cudaStream_t stream);
size_t block_sparse_attn_workspace_bytes(int batch, int hq, int hkv, int q_len, int k_len);
int pair_min_share_pct(int set_to);
}  // namespace xb

extern "C" {

int xattn_b200_version(void) { return 101; }

unsigned long long xattn_b200_launch_count(void) { return xb::launch_counter().load(std::memory_order_relaxed); }

const char* xattn_b200_error_string(int code) {
  switch (code) {
    case XATTN_B200_OK: return "ok";
    case XATTN_B200_ERR_ARG: return "invalid argument (shape, stride, alignment or unsupported value)";
    case XATTN_B200_ERR_WORKSPACE: return "workspace missing or too small";
    case XATTN_B200_ERR_CUDA: return "a CUDA runtime or driver call failed";
    case XATTN_B200_ERR_ARCH: return "the current device is not sm_100";
    case XATTN_B200_ERR_LIMIT: return "size beyond a stated maximum";
    case XATTN_B200_ERR_DEVICE_WAIT: return "a device-side bounded wait ran out";
    default: return "unknown status";
  }
}

int xattn_b200_default_chunk_size(int k_len) {
  if (k_len < 1) return 2048;
  long long p = 1;
  while (p < k_len) p <<= 1;
  long long a = p > 2048 ? p : 2048;
  const long long b = 128LL * 1024 * 2048 / p;
  if (b < a) a = b;
  return static_cast<int>(a > 2048 ? a : 2048);
}

int xattn_b200_estimate_geometry(int q_len, int k_len, int chunk_size, int stride, int block_size, int out[8]) {
  if (!out || q_len < 1 || k_len < 1 || chunk_size < 1 || stride < 1 || block_size < 1) return XATTN_B200_ERR_ARG;
  if (chunk_size % block_size != 0 || block_size % stride != 0) return XATTN_B200_ERR_ARG;
  const int lq = (q_len + chunk_size - 1) / chunk_size * chunk_size;
  const int lk = (k_len + chunk_size - 1) / chunk_size * chunk_size;
  if (lk / chunk_size < lq / chunk_size) return XATTN_B200_ERR_ARG;
  out[0] = lq; out[1] = lk; out[2] = lq / block_size; out[3] = lk / block_size;
  out[4] = lq / chunk_size; out[5] = lk / chunk_size; out[6] = chunk_size / block_size;
  out[7] = out[3] - out[2];
  return XATTN_B200_OK;
}

size_t xattn_b200_estimate_workspace_bytes(int batch, int hq, int q_len, int k_len, int stride, int block_size,
                                           int chunk_size) {
  return xb::estimate_workspace_bytes(batch, hq, q_len, k_len, stride, block_size, chunk_size, -1, 0);
}

size_t xattn_b200_estimate_workspace_bytes_ex(int batch, int hq, int q_len, int k_len, int stride, int block_size,
                                              int chunk_size, int causal, int semantics) {
  if (causal < 0) return 0;
  return xb::estimate_workspace_bytes(batch, hq, q_len, k_len, stride, block_size, chunk_size, causal ? 1 : 0, semantics);
}

int xattn_b200_estimate(const void* q, const void* k, int dtype, int batch, int hq, int hkv, int q_len, int k_len,
                        int head_dim, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_l, int64_t k_stride_b,
                        int64_t k_stride_h, int64_t k_stride_l, int stride, int block_size, int chunk_size,
                        float scale, int causal, int semantics, float* attn_sums, void* workspace,
                        size_t workspace_bytes, int* status, void* cuda_stream) {
  return xb::estimate_launch(q, k, dtype, batch, hq, hkv, q_len, k_len, head_dim, q_stride_b, q_stride_h, q_stride_l,
                             k_stride_b, k_stride_h, k_stride_l, stride, block_size, chunk_size, scale, causal,
                             semantics, attn_sums, workspace, workspace_bytes, status,
                             static_cast<cudaStream_t>(cuda_stream));
}

int xattn_b200_split_f32(const float* x, int batch, int heads, int len, int len_valid, int head_dim, int64_t stride_b,
                         int64_t stride_h, int64_t stride_l, int role, void* out, void* cuda_stream) {
  return xb::split_f32_launch(x, batch, heads, len, len_valid, head_dim, stride_b, stride_h, stride_l, role, out,
                              static_cast<cudaStream_t>(cuda_stream));
}

int xattn_b200_rope_qk(void* q, void* k, int dtype, int batch, int hq, int hkv, int len, int head_dim,
                       int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_l, int64_t k_stride_b,
                       int64_t k_stride_h, int64_t k_stride_l, const void* cos, const void* sin,
                       int64_t cs_stride_b, int64_t cs_stride_l, void* cuda_stream) {
  return xb::rope_qk_launch(q, k, dtype, batch, hq, hkv, len, head_dim, q_stride_b, q_stride_h, q_stride_l,
                            k_stride_b, k_stride_h, k_stride_l, cos, sin, cs_stride_b, cs_stride_l,
                            static_cast<cudaStream_t>(cuda_stream));
}

int xattn_b200_select(const float* attn_sums, int batch, int heads, int q_blocks, int k_blocks,
                      int blocks_per_chunk, int block_offset, int causal, int diagonal_cleanup, double threshold,
                      const float* threshold_per_head, int keep_sink, int keep_recent, uint8_t* mask,
                      int32_t* block_idx, int32_t* block_cnt, int list_q_blocks, int list_k_blocks, int list_q_len,
                      int list_k_len, int* status, void* cuda_stream) {
  return xb::select_launch(attn_sums, batch, heads, q_blocks, k_blocks, blocks_per_chunk, block_offset, causal,
                           diagonal_cleanup, threshold, threshold_per_head, keep_sink, keep_recent, mask, block_idx,
                           block_cnt, list_q_blocks, list_k_blocks, list_q_len, list_k_len, 0, status,
                           static_cast<cudaStream_t>(cuda_stream));
}

int xattn_b200_select_band(const float* attn_sums, int batch, int heads, int q_blocks, int k_blocks,
                           int blocks_per_chunk, int block_offset, int causal, int diagonal_cleanup, double threshold,
                           const float* threshold_per_head, int keep_sink, int keep_recent, uint8_t* mask,
                           int32_t* block_idx, int32_t* block_cnt, int list_q_blocks, int list_k_blocks,
                           int list_q_len, int list_k_len, int* status, void* cuda_stream) {
  return xb::select_launch(attn_sums, batch, heads, q_blocks, k_blocks, blocks_per_chunk, block_offset, causal,
                           diagonal_cleanup, threshold, threshold_per_head, keep_sink, keep_recent, mask, block_idx,
                           block_cnt, list_q_blocks, list_k_blocks, list_q_len, list_k_len, 1, status,
                           static_cast<cudaStream_t>(cuda_stream));
}

int xattn_b200_mask_to_lists(const uint8_t* mask, int batch, int heads, int mask_q_blocks, int mask_k_blocks,
                             int q_len, int k_len, int causal, int32_t* block_idx, int32_t* block_cnt,
                             void* cuda_stream) {
  return xb::mask_to_lists_launch(mask, batch, heads, mask_q_blocks, mask_k_blocks, q_len, k_len, causal, block_idx,
                                  block_cnt, static_cast<cudaStream_t>(cuda_stream));
}

int xattn_b200_block_sparse_attn(const void* q, const void* k, const void* v, int dtype, int batch, int hq, int hkv,
                                 int q_len, int k_len, int head_dim, int64_t q_stride_b, int64_t q_stride_h,
                                 int64_t q_stride_l, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_l,
                                 int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_l, const int32_t* block_idx,
                                 const int32_t* block_cnt, int causal, float scale, void* out, int64_t o_stride_b,
                                 int64_t o_stride_h, int64_t o_stride_l, int* status, void* cuda_stream) {
  return xb::block_sparse_attn_launch(q, k, v, dtype, batch, hq, hkv, q_len, k_len, head_dim, q_stride_b, q_stride_h,
                                      q_stride_l, k_stride_b, k_stride_h, k_stride_l, v_stride_b, v_stride_h,
                                      v_stride_l, block_idx, block_cnt, causal, scale, out, o_stride_b, o_stride_h,
                                      o_stride_l, nullptr, 0, status, static_cast<cudaStream_t>(cuda_stream));
}

int xattn_b200_block_sparse_attn_split_share(int percent) { return xb::pair_min_share_pct(percent); }

size_t xattn_b200_block_sparse_attn_workspace_bytes(int batch, int hq, int hkv, int q_len, int k_len) {
  return xb::block_sparse_attn_workspace_bytes(batch, hq, hkv, q_len, k_len);
}

int xattn_b200_block_sparse_attn_ws(const void* q, const void* k, const void* v, int dtype, int batch, int hq, int hkv,
                                    int q_len, int k_len, int head_dim, int64_t q_stride_b, int64_t q_stride_h,
                                    int64_t q_stride_l, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_l,
                                    int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_l,
                                    const int32_t* block_idx, const int32_t* block_cnt, int causal, float scale,
                                    void* out, int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_l,
                                    void* workspace, size_t workspace_bytes, int* status, void* cuda_stream) {
  return xb::block_sparse_attn_launch(q, k, v, dtype, batch, hq, hkv, q_len, k_len, head_dim, q_stride_b, q_stride_h,
                                      q_stride_l, k_stride_b, k_stride_h, k_stride_l, v_stride_b, v_stride_h,
                                      v_stride_l, block_idx, block_cnt, causal, scale, out, o_stride_b, o_stride_h,
                                      o_stride_l, workspace, workspace_bytes, status,
                                      static_cast<cudaStream_t>(cuda_stream));
}

}  // extern "C"
