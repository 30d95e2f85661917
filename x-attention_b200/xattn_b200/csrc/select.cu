// Phase 2 of the XAttention prefill path: threshold block selection.
//
// Reference: find_blocks_chunked, xattn/src/utils.py:87-172 (+ :176-180), called per query chunk by
// xattn_estimate (xattn/src/Xattention.py:255-263), and the post-processing at
// xattn/src/Xattention.py:275-297.  The reference sorts every row twice in fp64 with torch.sort,
// builds cumulative sums with cat/cumsum and scatters, once per chunk with two host syncs.  Here one
// launch covers all chunks and one WARP owns one (head, query-block) row, staged in shared memory.
// Attention rows are peaked, so the kept set is small: the warp extracts the largest remaining score
// (lowest index on ties) one at a time, accumulating the prefix in fp64 exactly as the rule is
// stated, and stops at the first rank that is not taken.  Rows that are still going after
// kPeelMax extractions (flat score rows) switch to a warp-level bitonic sort of what is left (every warp
// has its own sort buffer) plus an fp64 prefix scan.  Both routes apply the same rule, so the result does not depend on the route.
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

constexpr int kPeelMax = 24;
constexpr int kPeelProbe = 8;

struct SelParams {
  int batch, heads, q_blocks, k_blocks;
  int bpc, block_offset, causal, diagonal_cleanup;
  double threshold;
  int keep_sink, keep_recent;
  int list_q_blocks, list_k_blocks, list_q_len, list_k_len;
  int np2;            // k_blocks rounded up to a power of two (>= 32)
  int warps_per_cta;
  int words;          // 32-column words per row
  int vals_bytes, idx_bytes, keys_bytes, per_warp_bytes;   // keys: one sort buffer per CTA, taken in turn by its warps
  int rows_total;
  int vec_in;         // score rows can be read as float4
  int vec_mask;       // mask rows can be written as 16-byte vectors
  int band;           // score rows hold only the chunk's own key blocks [cur, cur + bpc)
};

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// bits of 32-column word t whose column is <= hi
__device__ __forceinline__ uint32_t bits_le(int hi, int t) {
  const int r = hi - 32 * t;
  return r < 0 ? 0u : (r >= 31 ? 0xffffffffu : (2u << r) - 1u);
}

// Bitonic sort, descending, of the np2 = 32 * SEG keys of a row by one warp, in registers: lane l holds the
// positions [l * SEG, (l + 1) * SEG).  Compare-exchanges between positions of one lane are register moves, those
// between lanes one 64-bit shuffle; nothing goes through shared memory until the sorted keys are written out
// (the same network run on a shared-memory array costs a warp barrier and two round trips per stage: 150 us for
// a 1024-key row, most of the selection time on non-causal masks whose rows are flat).
template <int SEG>
__device__ __forceinline__ void warp_sort_desc(unsigned long long* __restrict__ keys, const float* __restrict__ cval,
                                               const uint16_t* __restrict__ cidx, int M, int lane) {
  unsigned long long kr[SEG];
#pragma unroll
  for (int r = 0; r < SEG; ++r) {
    const int t = lane * SEG + r;
    unsigned long long key = 0ull;
    if (t < M && cval[t] > 0.f)
      key = (static_cast<unsigned long long>(__float_as_uint(cval[t])) << 32) | (0xFFFFFFFFull - cidx[t]);
    kr[r] = key;
  }
  constexpr int np2 = 32 * SEG;
#pragma unroll 1
  for (int k = 2; k <= np2; k <<= 1) {
    // partners in other lanes (distance j >= SEG): the lower position keeps the larger key where the run descends
#pragma unroll 1
    for (int j = k >> 1; j >= SEG; j >>= 1) {
      const int lane_bit = j / SEG;
      const bool lower = (lane & lane_bit) == 0;
#pragma unroll
      for (int r = 0; r < SEG; ++r) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, kr[r], lane_bit);
        const bool desc = ((lane * SEG + r) & k) == 0;
        const unsigned long long hi = kr[r] > other ? kr[r] : other, lo = kr[r] > other ? other : kr[r];
        kr[r] = (lower == desc) ? hi : lo;
      }
    }
    // partners inside the lane (distance jj < SEG)
#pragma unroll
    for (int jj = SEG / 2; jj > 0; jj >>= 1) {
      if (jj < k) {
#pragma unroll
        for (int r = 0; r < SEG; ++r) {
          if ((r & jj) == 0) {
            const bool desc = ((lane * SEG + r) & k) == 0;
            const unsigned long long a = kr[r], b = kr[r | jj];
            const bool swap = desc ? (a < b) : (a > b);
            kr[r] = swap ? b : a;
            kr[r | jj] = swap ? a : b;
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < SEG; ++r) keys[lane * SEG + r] = kr[r];
  __syncwarp();
}

// One warp per row.  The row is read once (16-byte loads): fp64 total, the forced blocks, and the positive
// scores compacted in column order into shared memory (score rows are sparse: most blocks hold no mass).
// Zero-score columns are not stored: all of them rank after the positive ones, in column order, and the rule
// can only take the first of them or all of them (see below).  Taken columns are a bitmap, so the mask row and
// the ascending block list are produced word by word.
// kMaxSeg: the longest row the register sort is compiled for, in keys per lane (4 / 16 / 32: rows of up to 128 /
// 512 / 1024 key blocks; the kernel's register count, and with it the warps per SM, follows the largest one).
template <int kMaxSeg>
__global__ void __launch_bounds__(256) select_kernel(const float* __restrict__ sums, const SelParams p,
                              const float* __restrict__ thr_per_head, uint8_t* __restrict__ mask_out,
                              int32_t* __restrict__ idx_out, int32_t* __restrict__ cnt_out, int* status) {
  extern __shared__ __align__(16) uint8_t sel_smem[];
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int w = blockIdx.x * p.warps_per_cta + wib;
  if (w >= p.rows_total) return;                         // whole warps leave; no block-wide barrier below
  uint8_t* base_ptr = sel_smem + static_cast<size_t>(wib) * p.per_warp_bytes;
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(base_ptr);        // [np2] sort buffer of this warp
  float* cval = reinterpret_cast<float*>(base_ptr + p.keys_bytes);                   // [M] positive scores (-1 = taken)
  uint16_t* cidx = reinterpret_cast<uint16_t*>(base_ptr + p.keys_bytes + p.vals_bytes);   // [M] their columns, ascending
  uint32_t* taken = reinterpret_cast<uint32_t*>(base_ptr + p.keys_bytes + p.vals_bytes + p.idx_bytes);   // [words]
  uint32_t* cand = taken + p.words;                                                  // [words] columns with a positive score

  const int bh = w / p.q_blocks;
  const int R = w - bh * p.q_blocks;
  const int h = bh % p.heads;
  const int N = p.k_blocks;
  const int W = p.words;
  auto valid = [&](int t) -> uint32_t { return bits_le(N - 1, t); };

  const int cur = p.block_offset + (R / p.bpc) * p.bpc;
  const int d = cur + R % p.bpc;
  const bool f0 = p.causal && cur != 0;            // block 0 forced
  const int n_forced = p.causal ? (f0 ? 2 : 1) : 0;
  const int lag = n_forced == 1 ? 1 : 0;
  const int n_others = N - n_forced;
  // stored part of the row: `n_read` scores, the first of them belongs to column `col0`; the rest are zero
  const int n_read = p.band ? p.bpc : N;
  const int col0 = p.band ? cur : 0;
  const float* x = sums + static_cast<size_t>(w) * n_read;

  for (int t = lane; t < W; t += 32) { taken[t] = 0u; cand[t] = 0u; }
  __syncwarp();

  // ---- the row, once
  double part = 0.0, fpart = 0.0;
  int M = 0;                                       // positive non-forced scores so far (warp-uniform)
  // 1024 columns at a time: all loads of the piece are issued before any of it is processed, so a row costs one
  // memory round trip per 1024 columns instead of one per 128
  for (int j1 = 0; j1 < n_read; j1 += 1024) {
    float vv[8][4];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int j = j1 + u * 128 + 4 * lane;
#pragma unroll
      for (int e = 0; e < 4; ++e) vv[u][e] = 0.f;
      if (p.vec_in) {
        if (j < n_read) {
          const float4 q = __ldg(reinterpret_cast<const float4*>(x + j));
          vv[u][0] = q.x; vv[u][1] = q.y; vv[u][2] = q.z; vv[u][3] = q.w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (j + e < n_read) vv[u][e] = __ldg(x + j + e);
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int j0 = j1 + u * 128;
      if (j0 >= n_read) break;
      const int j = j0 + 4 * lane;
      const float (&v)[4] = vv[u];
      uint32_t nib = 0u;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int jj = col0 + j + e;              // column
        if (j + e < n_read) {
          part += static_cast<double>(v[e]);
          const bool forced = p.causal && (jj == d || (f0 && jj == 0));
          if (forced) fpart += static_cast<double>(v[e]);
          else if (v[e] > 0.f) nib |= 1u << e;
        }
      }
      // candidate bitmap (col0 and j are multiples of 4, so the four bits stay inside one word)
      if (nib) atomicOr(&cand[(col0 + j) >> 5], nib << ((col0 + j) & 31));
      // compaction in column order (rows are sparse: skip the scan when the piece holds no positive score)
      if (__any_sync(0xffffffffu, nib != 0u)) {
        const int c = __popc(nib);
        int incl = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += up;
        }
        int pos = M + incl - c;
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if ((nib >> e) & 1u) {
            cval[pos] = v[e];
            cidx[pos] = static_cast<uint16_t>(col0 + j + e);
            ++pos;
          }
        M += __shfl_sync(0xffffffffu, incl, 31);
      }
    }
  }
  const double total = warp_sum(part);
  const double fsum = warp_sum(fpart);
  const double thr = thr_per_head ? static_cast<double>(thr_per_head[h]) : p.threshold;
  const double req = total * thr;
  if (lane == 0 && p.causal) {
    taken[d >> 5] |= 1u << (d & 31);
    if (f0) taken[0] |= 1u;
  }
  __syncwarp();

  bool untaken = !(req > 0.0);                     // the leading slots of the reference compare 0 < req too
  if (req > 0.0) {
    int i = 1;                                     // rank being decided
    int live = M;                                  // positive scores not ranked yet
    double s_cur = 0.0, s_lag = 0.0;               // prefix[i-1], prefix[max(i-2,0)] of the ranked scores
    bool stop = false;                             // a rank was refused: every later rank is refused too
    // ---- ranks that hold a positive score: the largest remaining one (lowest column on ties) at a time
    while (live > 0 && i <= kPeelMax) {
      const double c = lag ? (i == 1 ? 0.0 : fsum + s_lag) : fsum + s_cur;
      if (!(c < req)) { untaken = true; stop = true; break; }
      // a flat row (the eight largest scores hold less than a third of the mass wanted) will need far more ranks
      // than this loop is meant for: sort the rest right away (the sort continues from any state of this loop)
      if (i == kPeelProbe + 1 && (fsum + s_cur) * 3.0 < req) break;
      float bv = -1.f;
      int bp = 0x7fffffff;
      for (int t = lane; t < M; t += 32) {
        const float v = cval[t];
        if (v > bv) { bv = v; bp = t; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int op = __shfl_xor_sync(0xffffffffu, bp, o);
        if (ov > bv || (ov == bv && op < bp)) { bv = ov; bp = op; }
      }
      if (lane == 0) {
        const int col = cidx[bp];
        cval[bp] = -1.f;
        taken[col >> 5] |= 1u << (col & 31);
      }
      __syncwarp();
      s_lag = s_cur;
      s_cur += static_cast<double>(bv);
      ++i;
      --live;
    }
    // ---- flat rows: sort what is left of the positive scores, fp64 prefix, decide per rank
    if (!stop && live > 0) {
      {
        int np2 = 32;
        while (np2 < M) np2 <<= 1;
        if (np2 <= 32 * kMaxSeg) {
          if (np2 == 32) warp_sort_desc<1>(keys, cval, cidx, M, lane);
          else if (np2 == 64) warp_sort_desc<2>(keys, cval, cidx, M, lane);
          else if (np2 == 128) warp_sort_desc<4>(keys, cval, cidx, M, lane);
          if constexpr (kMaxSeg >= 16) {
            if (np2 == 256) warp_sort_desc<8>(keys, cval, cidx, M, lane);
            else if (np2 == 512) warp_sort_desc<16>(keys, cval, cidx, M, lane);
          }
          if constexpr (kMaxSeg >= 32) {
            if (np2 == 1024) warp_sort_desc<32>(keys, cval, cidx, M, lane);
          }
        } else {
          // longer rows: the same network on the shared-memory array
          for (int t = lane; t < np2; t += 32) {
            unsigned long long key = 0ull;
            if (t < M && cval[t] > 0.f)
              key = (static_cast<unsigned long long>(__float_as_uint(cval[t])) << 32) | (0xFFFFFFFFull - cidx[t]);
            keys[t] = key;
          }
          __syncwarp();
          for (int k = 2; k <= np2; k <<= 1) {
            for (int j = k >> 1; j > 0; j >>= 1) {
              for (int t = lane; t < np2; t += 32) {
                const int ixj = t ^ j;
                if (ixj > t) {
                  const unsigned long long a = keys[t], b = keys[ixj];
                  const bool desc = (t & k) == 0;
                  if (desc ? (a < b) : (a > b)) { keys[t] = b; keys[ixj] = a; }
                }
              }
              __syncwarp();
            }
          }
        }
        const int seg = np2 / 32;                  // contiguous positions per lane
        const int t0 = lane * seg;
        double local = 0.0;
        for (int t = t0; t < t0 + seg; ++t) local += static_cast<double>(__uint_as_float(static_cast<unsigned>(keys[t] >> 32)));
        double incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const double up = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += up;
        }
        double running = incl - local;             // sum of the sorted scores before position t0
        int ut = 0;
        for (int t = t0; t < t0 + seg && t < live; ++t) {
          const unsigned long long key = keys[t];
          const double v = static_cast<double>(__uint_as_float(static_cast<unsigned>(key >> 32)));
          double c;
          if (!lag) c = fsum + s_cur + running;                       // prefix[rank-1]
          else if (t == 0) c = (i == 1) ? 0.0 : fsum + s_lag;         // prefix[rank-2], rank = i
          else c = fsum + s_cur + (running - static_cast<double>(__uint_as_float(static_cast<unsigned>(keys[t - 1] >> 32))));
          if (c < req) {
            const unsigned col = 0xFFFFFFFFu - static_cast<unsigned>(key & 0xFFFFFFFFull);
            atomicOr(&taken[col >> 5], 1u << (col & 31));
          } else {
            ut = 1;
          }
          running += v;
        }
        if (__any_sync(0xffffffffu, ut)) { untaken = true; stop = true; }
        // the prefix after all positive scores, and the one before the last of them
        const double sorted_total = __shfl_sync(0xffffffffu, incl, 31);
        const double last_v = static_cast<double>(__uint_as_float(static_cast<unsigned>(keys[live - 1] >> 32)));
        s_lag = s_cur + (sorted_total - last_v);
        s_cur += sorted_total;
        i += live;
        live = 0;
        __syncwarp();
      }
    }
    // ---- ranks that hold a zero score (column order).  The prefix no longer moves, so after the first of
    // them the decision value is fsum + s_cur for all: either every remaining rank is taken, or (only when a
    // single block is forced, whose decision values lag one rank behind) just the first one.
    if (!stop && i <= n_others) {
      const double c = lag ? (i == 1 ? 0.0 : fsum + s_lag) : fsum + s_cur;
      if (!(c < req)) {
        untaken = true;
      } else if (fsum + s_cur < req) {
        for (int t = lane; t < W; t += 32) taken[t] |= ~cand[t] & valid(t);
      } else {
        // lowest zero-score column that is not forced
        int best = 0x7fffffff;
        for (int t = lane; t < W; t += 32) {
          const uint32_t z = ~(cand[t] | taken[t]) & valid(t);
          if (z && best == 0x7fffffff) best = 32 * t + __ffs(z) - 1;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const int ob = __shfl_xor_sync(0xffffffffu, best, o);
          best = ob < best ? ob : best;
        }
        if (lane == 0 && best != 0x7fffffff) taken[best >> 5] |= 1u << (best & 31);
        if (i < n_others) untaken = true;          // the next rank compares fsum + s_cur >= req
      }
    }
  }
  __syncwarp();
  if (untaken && lane == 0) taken[0] |= 1u;
  __syncwarp();

  // ---- post-processing + outputs, one 32-column word per lane
  const bool want_list = idx_out && cnt_out && R < p.list_q_blocks;
  int32_t* lrow = want_list ? idx_out + (static_cast<size_t>(bh) * p.list_q_blocks + R) * p.list_k_blocks : nullptr;
  uint8_t* mo = mask_out ? mask_out + static_cast<size_t>(w) * N : nullptr;
  int hi_keep = N - 1;                             // causal clean-up: columns above are cleared
  if (p.causal) {
    hi_keep = cur + p.bpc - 1;
    if (p.diagonal_cleanup && p.block_offset + R < hi_keep) hi_keep = p.block_offset + R;
  }
  int hi_list = p.list_k_blocks - 1;               // columns the block list may hold
  if (p.causal) {
    // last token of query block R sees keys up to this position (query end aligned to key end)
    int last_q = R * 128 + 127;
    if (last_q > p.list_q_len - 1) last_q = p.list_q_len - 1;
    const long long lim = static_cast<long long>(last_q) + (p.list_k_len - p.list_q_len);
    const int jm = lim < 0 ? -1 : static_cast<int>(lim / 128);
    if (jm < hi_list) hi_list = jm;
  }
  const int recent = p.block_offset + R;
  int base = 0;
  for (int t0 = 0; t0 < W; t0 += 32) {
    const int t = t0 + lane;
    uint32_t word = 0u;
    if (t < W) {
      word = taken[t] & valid(t) & bits_le(hi_keep, t);
      if (p.keep_sink && R == 0) word = valid(t);
      if (p.keep_recent && recent < N && (recent >> 5) == t) word |= 1u << (recent & 31);
      if (mo) {
        if (p.vec_mask && 32 * t + 32 <= N) {
          uint32_t b[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) b[q] = (((word >> (4 * q)) & 15u) * 0x00204081u) & 0x01010101u;
          uint4* dst = reinterpret_cast<uint4*>(mo + 32 * t);
          dst[0] = make_uint4(b[0], b[1], b[2], b[3]);
          dst[1] = make_uint4(b[4], b[5], b[6], b[7]);
        } else {
          for (int q = 0; q < 32 && 32 * t + q < N; ++q) mo[32 * t + q] = static_cast<uint8_t>((word >> q) & 1u);
        }
      }
    }
    if (want_list) {
      uint32_t lw = t < W ? word & bits_le(hi_list, t) : 0u;
      const int c = __popc(lw);
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      int pos = base + incl - c;
      while (lw) {
        lrow[pos++] = 32 * t + __ffs(lw) - 1;
        lw &= lw - 1;
      }
      base += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  if (want_list && lane == 0) cnt_out[static_cast<size_t>(bh) * p.list_q_blocks + R] = base;
}

__device__ __forceinline__ bool list_keeps(int causal, int R, int j, int list_q_len, int list_k_len) {
  if (!causal) return true;
  // last token of query block R sees keys up to this position (query end aligned to key end)
  int last_q = R * 128 + 127;
  if (last_q > list_q_len - 1) last_q = list_q_len - 1;
  return static_cast<long long>(j) * 128 <= static_cast<long long>(last_q) + (list_k_len - list_q_len);
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
                  int list_q_len, int list_k_len, int band, int* status, cudaStream_t stream) {
  if (!attn_sums || batch < 1 || heads < 1 || q_blocks < 1 || k_blocks < 1 || bpc < 1 || block_offset < 0)
    return XATTN_B200_ERR_ARG;
  if (k_blocks > 8192) return XATTN_B200_ERR_LIMIT;
  // band layout: the stored columns are the chunk's own ones, which needs the causal chunk structure and a
  // column origin that keeps groups of four inside a 32-column word
  if (band && (!causal || bpc % 4 != 0 || block_offset % 4 != 0)) return XATTN_B200_ERR_ARG;
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
  p.band = band ? 1 : 0;
  const int n_read = band ? bpc : k_blocks;        // scores stored per row = most candidates a row can have
  int np2 = 32;
  while (np2 < n_read) np2 <<= 1;
  p.np2 = np2;
  p.words = (k_blocks + 31) / 32;
  p.vals_bytes = (n_read * 4 + 15) & ~15;
  p.idx_bytes = (n_read * 2 + 15) & ~15;
  p.keys_bytes = np2 * 8;                           // every warp has its own sort buffer: flat rows do not queue
  p.per_warp_bytes = p.keys_bytes + p.vals_bytes + p.idx_bytes + ((2 * p.words * 4 + 15) & ~15);
  // 16-byte accesses to the rows of the scores and of the mask
  p.vec_in = (n_read % 4 == 0 && (reinterpret_cast<uintptr_t>(attn_sums) & 15) == 0) ? 1 : 0;
  p.vec_mask = (k_blocks % 16 == 0 && mask != nullptr && (reinterpret_cast<uintptr_t>(mask) & 15) == 0) ? 1 : 0;
  int wpc = (72 * 1024) / p.per_warp_bytes;        // three CTAs per SM when rows are long
  wpc = wpc < 1 ? 1 : (wpc > 8 ? 8 : wpc);
  p.warps_per_cta = wpc;
  const long long rows = static_cast<long long>(batch) * heads * q_blocks;
  if (rows > 0x7fffffffLL) return XATTN_B200_ERR_LIMIT;
  p.rows_total = static_cast<int>(rows);
  const size_t smem = static_cast<size_t>(wpc) * p.per_warp_bytes;
  const int grid = static_cast<int>((rows + wpc - 1) / wpc);
  auto launch = [&](auto kern) -> int {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return XATTN_B200_ERR_CUDA;
    kern<<<grid, wpc * 32, smem, stream>>>(attn_sums, p, thr_per_head, mask, block_idx, block_cnt, status);
    return launch_status();
  };
  // the instantiation whose flat-row sort holds just enough keys per lane in registers for this row length
  return np2 > 512 ? launch(select_kernel<32>) : (np2 > 128 ? launch(select_kernel<16>) : launch(select_kernel<4>));
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
