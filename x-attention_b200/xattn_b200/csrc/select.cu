// Phase 2 of the XAttention prefill path: threshold block selection.
//
// Reference: find_blocks_chunked, xattn/src/utils.py:87-172 (+ :176-180), called per query chunk by
// xattn_estimate (xattn/src/Xattention.py:255-263), and the post-processing at
// xattn/src/Xattention.py:275-297.  The reference sorts every row twice in fp64 with torch.sort,
// builds cumulative sums with cat/cumsum and scatters; here one thread block owns one
// (head, query-block) row: a bitonic sort of (score, index) keys in shared memory, an fp64 prefix
// scan, the take/skip decision per rank, then the mask row and the compacted ascending block list
// that the attention kernel walks.
//
// Rule per row R (chunk c = R / bpc, current_index cur = block_offset + c*bpc, diagonal d = cur + R%bpc),
// scores x[0..N) taken as fp64, req = sum(x) * threshold:
//   causal    : d is forced; block 0 is forced unless cur == 0.  The other blocks are ranked by score
//               (descending, lower index first on ties); the i-th (1-based) is taken iff c_i < req,
//               c_i = forced + (sum of the first i-1-lag ranked scores), c_i = 0 when i-lag <= 0,
//               lag = 1 when a single block is forced.
//   non-causal: nothing forced, c_i = sum of the first i-1 ranked scores.
//   block 0 is set when at least one rank position was not taken; causal clears columns >= cur + bpc
//   and columns right of the diagonal; keep_sink sets query-block row 0; keep_recent sets the diagonal.
#include "host_common.cuh"

namespace xb {

constexpr int kSelThreads = 256;

struct SelParams {
  int batch, heads, q_blocks, k_blocks;
  int bpc, block_offset, causal, diagonal_cleanup;
  double threshold;
  int keep_sink, keep_recent;
  int list_q_blocks, list_k_blocks, list_q_len, list_k_len;
  int np2;   // k_blocks rounded up to a power of two
};

__device__ __forceinline__ bool list_keeps(int causal, int R, int j, int list_q_len, int list_k_len) {
  if (!causal) return true;
  // last token of query block R sees keys up to this position (query end aligned to key end)
  int last_q = R * 128 + 127;
  if (last_q > list_q_len - 1) last_q = list_q_len - 1;
  return static_cast<long long>(j) * 128 <= static_cast<long long>(last_q) + (list_k_len - list_q_len);
}

__global__ void __launch_bounds__(kSelThreads)
select_kernel(const float* __restrict__ sums, const SelParams p, const float* __restrict__ thr_per_head,
              uint8_t* __restrict__ mask_out, int32_t* __restrict__ idx_out, int32_t* __restrict__ cnt_out) {
  extern __shared__ __align__(16) uint8_t sel_smem[];
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(sel_smem);       // [np2]
  double* scan = reinterpret_cast<double*>(sel_smem + sizeof(unsigned long long) * p.np2);  // [np2]
  uint8_t* mrow = reinterpret_cast<uint8_t*>(scan + p.np2);                          // [k_blocks]
  __shared__ double s_red[kSelThreads / 32];
  __shared__ double s_total, s_forced;
  __shared__ int s_untaken, s_count;
  __shared__ int s_wsum[kSelThreads / 32];

  const int R = blockIdx.x;
  const int bh = blockIdx.y;
  const int h = bh % p.heads;
  const int N = p.k_blocks;
  const int tid = threadIdx.x;
  const float* x = sums + (static_cast<size_t>(bh) * p.q_blocks + R) * N;

  const int cur = p.block_offset + (R / p.bpc) * p.bpc;
  const int d = cur + R % p.bpc;
  const bool f0 = p.causal && cur != 0;            // block 0 forced
  const int n_forced = p.causal ? (f0 ? 2 : 1) : 0;
  const int lag = n_forced == 1 ? 1 : 0;

  // keys + total
  double part = 0.0, fpart = 0.0;
  for (int j = tid; j < p.np2; j += kSelThreads) {
    unsigned long long key = 0ull;
    if (j < N) {
      const float v = x[j];
      part += static_cast<double>(v);
      const bool forced = p.causal && (j == d || (f0 && j == 0));
      if (forced) fpart += static_cast<double>(v);
      else {
        const float vc = v > 0.f ? v : 0.f;
        key = (static_cast<unsigned long long>(__float_as_uint(vc)) << 32) | (0xFFFFFFFFull - static_cast<unsigned>(j));
      }
      mrow[j] = forced ? 1 : 0;
    }
    keys[j] = key;
  }
  // block reductions (fp64)
  for (int pass = 0; pass < 2; ++pass) {
    double v = pass == 0 ? part : fpart;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((tid & 31) == 0) s_red[tid >> 5] = v;
    __syncthreads();
    if (tid == 0) {
      double t = 0.0;
      for (int w = 0; w < kSelThreads / 32; ++w) t += s_red[w];
      if (pass == 0) s_total = t; else s_forced = t;
      s_untaken = 0;
    }
    __syncthreads();
  }
  const double thr = thr_per_head ? static_cast<double>(thr_per_head[h]) : p.threshold;
  const double req = s_total * thr;
  const double fsum = s_forced;

  // bitonic sort, descending
  for (int k = 2; k <= p.np2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = tid; t < p.np2; t += kSelThreads) {
        const int ixj = t ^ j;
        if (ixj > t) {
          const unsigned long long a = keys[t], b = keys[ixj];
          const bool desc = (t & k) == 0;
          if (desc ? (a < b) : (a > b)) { keys[t] = b; keys[ixj] = a; }
        }
      }
      __syncthreads();
    }
  }

  // inclusive fp64 scan of the ranked scores
  for (int t = tid; t < p.np2; t += kSelThreads)
    scan[t] = static_cast<double>(__uint_as_float(static_cast<unsigned>(keys[t] >> 32)));
  __syncthreads();
  for (int off = 1; off < p.np2; off <<= 1) {
    double tmp[32];   // np2 <= 8192 -> at most 32 elements per thread
    int c = 0;
    for (int t = tid; t < p.np2; t += kSelThreads, ++c) tmp[c] = t >= off ? scan[t - off] : 0.0;
    __syncthreads();
    c = 0;
    for (int t = tid; t < p.np2; t += kSelThreads, ++c) scan[t] += tmp[c];
    __syncthreads();
  }

  // decisions per rank position
  const int n_others = N - n_forced;
  int untaken = 0;
  for (int t = tid; t < n_others; t += kSelThreads) {
    const int i = t + 1;
    double c;
    if (i - lag <= 0) c = 0.0;
    else {
      const int m = i - lag - 1;           // number of ranked scores summed
      c = fsum + (m >= 1 ? scan[m - 1] : 0.0);
    }
    if (c < req) {
      const unsigned j = 0xFFFFFFFFu - static_cast<unsigned>(keys[t] & 0xFFFFFFFFull);
      mrow[j] = 1;
    } else {
      untaken = 1;
    }
  }
  if (!(req > 0.0)) untaken = 1;           // the forced slots of the reference compare 0 < req too
  if (untaken) s_untaken = 1;
  __syncthreads();
  if (tid == 0 && s_untaken) mrow[0] = 1;
  __syncthreads();

  // post-processing + outputs
  const bool want_list = idx_out && cnt_out && R < p.list_q_blocks;
  int32_t* lrow = want_list ? idx_out + (static_cast<size_t>(bh) * p.list_q_blocks + R) * p.list_k_blocks : nullptr;
  uint8_t* mo = mask_out ? mask_out + (static_cast<size_t>(bh) * p.q_blocks + R) * N : nullptr;
  int base = 0;
  for (int j0 = 0; j0 < N; j0 += kSelThreads) {
    const int j = j0 + tid;
    int m = 0;
    if (j < N) {
      m = mrow[j];
      if (p.causal && (j >= cur + p.bpc || (p.diagonal_cleanup && j > p.block_offset + R))) m = 0;
      if (p.keep_sink && R == 0) m = 1;
      if (p.keep_recent && j == p.block_offset + R) m = 1;
      if (mo) mo[j] = static_cast<uint8_t>(m);
    }
    if (want_list) {
      const int keep = (m && j < p.list_k_blocks && list_keeps(p.causal, R, j, p.list_q_len, p.list_k_len)) ? 1 : 0;
      const unsigned bal = __ballot_sync(0xffffffffu, keep);
      const int wpre = __popc(bal & ((1u << (tid & 31)) - 1u));
      if ((tid & 31) == 0) s_wsum[tid >> 5] = __popc(bal);
      __syncthreads();
      int woff = 0, tot = 0;
      for (int w = 0; w < kSelThreads / 32; ++w) {
        if (w < (tid >> 5)) woff += s_wsum[w];
        tot += s_wsum[w];
      }
      if (keep) lrow[base + woff + wpre] = j;
      base += tot;
      __syncthreads();
    }
  }
  if (want_list && tid == 0) cnt_out[static_cast<size_t>(bh) * p.list_q_blocks + R] = base;
  (void)s_count;
}

// One warp per (head, query-block) row of a caller-supplied mask.
__global__ void mask_to_lists_kernel(const uint8_t* __restrict__ mask, int rows_total, int mask_q_blocks,
                                     int mask_k_blocks, int list_q_blocks, int list_k_blocks, int q_len, int k_len,
                                     int causal, int32_t* __restrict__ idx_out, int32_t* __restrict__ cnt_out) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= rows_total) return;
  const int bh = w / list_q_blocks, R = w - bh * list_q_blocks;
  const uint8_t* mrow = mask + (static_cast<size_t>(bh) * mask_q_blocks + R) * mask_k_blocks;
  int32_t* lrow = idx_out + static_cast<size_t>(w) * list_k_blocks;
  int base = 0;
  for (int j0 = 0; j0 < list_k_blocks; j0 += 32) {
    const int j = j0 + lane;
    const int keep = (j < list_k_blocks && mrow[j] && list_keeps(causal, R, j, q_len, k_len)) ? 1 : 0;
    const unsigned bal = __ballot_sync(0xffffffffu, keep);
    if (keep) lrow[base + __popc(bal & ((1u << lane) - 1u))] = j;
    base += __popc(bal);
  }
  if (lane == 0) cnt_out[w] = base;
}

int select_launch(const float* attn_sums, int batch, int heads, int q_blocks, int k_blocks, int bpc, int block_offset,
                  int causal, int diagonal_cleanup, double threshold, const float* thr_per_head, int keep_sink, int keep_recent,
                  uint8_t* mask, int32_t* block_idx, int32_t* block_cnt, int list_q_blocks, int list_k_blocks,
                  int list_q_len, int list_k_len, int* status, cudaStream_t stream) {
  (void)status;
  if (!attn_sums || batch < 1 || heads < 1 || q_blocks < 1 || k_blocks < 1 || bpc < 1 || block_offset < 0)
    return XATTN_B200_ERR_ARG;
  if (k_blocks > 8192) return XATTN_B200_ERR_LIMIT;
  if (q_blocks % bpc != 0) return XATTN_B200_ERR_ARG;
  if (causal && block_offset + q_blocks > k_blocks) return XATTN_B200_ERR_ARG;
  if ((block_idx == nullptr) != (block_cnt == nullptr)) return XATTN_B200_ERR_ARG;
  if (block_idx && (list_q_blocks < 1 || list_k_blocks < 1 || list_q_blocks > q_blocks || list_k_blocks > k_blocks ||
                    list_q_len < 1 || list_k_len < 1))
    return XATTN_B200_ERR_ARG;
  SelParams p;
  p.batch = batch; p.heads = heads; p.q_blocks = q_blocks; p.k_blocks = k_blocks;
  p.bpc = bpc; p.block_offset = block_offset; p.causal = causal ? 1 : 0;
  p.diagonal_cleanup = diagonal_cleanup ? 1 : 0;
  p.threshold = threshold; p.keep_sink = keep_sink ? 1 : 0; p.keep_recent = keep_recent ? 1 : 0;
  p.list_q_blocks = list_q_blocks; p.list_k_blocks = list_k_blocks;
  p.list_q_len = list_q_len; p.list_k_len = list_k_len;
  int np2 = 32;
  while (np2 < k_blocks) np2 <<= 1;
  p.np2 = np2;
  const size_t smem = static_cast<size_t>(np2) * 16 + ((k_blocks + 15) & ~15);
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
          cudaSuccess)
    return XATTN_B200_ERR_CUDA;
  select_kernel<<<dim3(q_blocks, batch * heads), kSelThreads, smem, stream>>>(attn_sums, p, thr_per_head, mask,
                                                                               block_idx, block_cnt);
  return launch_status();
}

int mask_to_lists_launch(const uint8_t* mask, int batch, int heads, int mask_q_blocks, int mask_k_blocks, int q_len,
                         int k_len, int causal, int32_t* block_idx, int32_t* block_cnt, cudaStream_t stream) {
  if (!mask || !block_idx || !block_cnt || batch < 1 || heads < 1 || q_len < 1 || k_len < 1) return XATTN_B200_ERR_ARG;
  const int lq = (q_len + 127) / 128, lk = (k_len + 127) / 128;
  if (mask_q_blocks < lq || mask_k_blocks < lk) return XATTN_B200_ERR_ARG;
  const int rows = batch * heads * lq;
  const int wpb = 8;
  mask_to_lists_kernel<<<(rows + wpb - 1) / wpb, wpb * 32, 0, stream>>>(mask, rows, mask_q_blocks, mask_k_blocks, lq,
                                                                        lk, q_len, k_len, causal ? 1 : 0, block_idx,
                                                                        block_cnt);
  return launch_status();
}

}  // namespace xb
