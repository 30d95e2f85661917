// Phase 3 of the XAttention prefill path: block-sparse FlashAttention forward over 128x128 blocks.
//
// Replaces block_sparse_attn.block_sparse_attn_func (third-party CUDA package; call site
// xattn/src/Xattention.py:377-391).  A work item is one (batch, head, 128-row query block) with its list
// of kept key blocks.  Mask rows are short (often 2-10 blocks), so per-item latency chains
// (Q load -> QK^T -> softmax -> PV -> store) matter as much as the inner loop.  The kernel is persistent
// (one CTA per SM) and runs TWO independent item streams per CTA: the CTA's non-empty items alternate
// between stream 0 and stream 1, each stream has its own Q / K / V tiles in shared memory, its own
// score/probability buffer S and output accumulator O in tensor memory and its own softmax warpgroup,
// so the bubbles of one stream's dependency chain are filled by the other stream's work.
//
//   warps 0-3   softmax of stream 0  } one thread per query row.  Two passes over S in TMEM: row max
//   warps 4-7   softmax of stream 1  } (8 independent chains), then exp2 in 32-column chunks, P packed to
//                                      16-bit back into the S columns; lazy rescale of O only when the max
//                                      grew by more than 2^8; the row sum of the item's last block goes to
//                                      shared memory for the epilogue
//   warps 8-11  epilogue of both streams: O / l from TMEM -> global memory, hands the O buffer back
//   warps 12,14 TMA loader of stream 0 / 1 (lane 0 issues): Q, then K_j, V_j in list order, one TMA
//               instruction per 128x128 tile
//   warps 13,15 (1 thread each) tcgen05 issuer of stream 0 / 1: S = Q K^T (operands in shared memory), then
//               O += P V (P from TMEM, V from shared memory as an MN-major operand)
//
// Lists are walked from the last entry (the diagonal block when causal, which usually holds the row
// maximum) to the first, so the running maximum settles at the first block and O is rarely rescaled.
// TMEM columns: [0,128) S of stream 0, [128,256) S of stream 1, [256,384) O of stream 0, [384,512) O of stream 1.
#include <math.h>

#include "host_common.cuh"
#include "sm100_primitives.cuh"

namespace xb {

constexpr int kAttnThreads = 512;
constexpr int kTile16 = 128 * 128 * 2;     // one 128x128 16-bit tile = two 64-column TMA boxes
constexpr int kHalf16 = kTile16 / 2;
constexpr int kAttnSmemTiles = kTile16 * 6;                   // Q, K, V per stream
constexpr int kSchedCap = 2048;                               // work items one CTA can schedule
constexpr int kStageBytes = 4 * 32 * 128;                     // per epilogue warp: 32 rows x 64 16-bit columns
constexpr int kAttnSmem = kAttnSmemTiles + 2 * 2 * 128 * 4 /*row sums*/ + 256 /*barriers*/ +
                          3 * kSchedCap * 2 /*schedule*/ + 16 + kStageBytes;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct AttnParams {
  int batch, hq, hkv, q_len, k_len;
  int q_blocks, list_k_blocks;
  int causal, is_bf16;
  int total_items;
  float scale_log2;
  int64_t osb, osh, osl;
};

__device__ __forceinline__ uint32_t pack16(float lo, float hi, int is_bf16) {
  if (is_bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Development aid, compiled only with -DXB_TRACE: per-role timestamps of the first CTAs, written behind the
// status word (which must then point to a device buffer of at least 64 + 16*7*2*XB_TRACE_CAP bytes).
#ifdef XB_TRACE
#ifndef XB_TRACE_CAP
#define XB_TRACE_CAP 4096          // records per (CTA, role); 7 roles, first 2 CTAs
#endif
__device__ __forceinline__ void xb_trace(int* status, uint32_t& n, int role, uint32_t tag, uint32_t val) {
  if (blockIdx.x >= 2 || !status || n >= XB_TRACE_CAP) return;
  unsigned long long* buf = reinterpret_cast<unsigned long long*>(status) + 8 +
                            2ull * XB_TRACE_CAP * (blockIdx.x * 7 + role);
  buf[2 * n] = (static_cast<unsigned long long>(tag) << 32) | val;
  buf[2 * n + 1] = static_cast<unsigned long long>(clock64());
  ++n;
}
#define XB_TRACE_EV(tag, val) xb_trace(status, trace_n, trace_role, (tag), (val))
#else
#define XB_TRACE_EV(tag, val) ((void)0)
#endif

template <int N> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// Work item t -> (b, h, qb): heaviest query blocks (largest index) first, the heads of a kv group adjacent.
struct Item {
  int b, h, qb;
  size_t row;
};
__device__ __forceinline__ Item decode_item(const AttnParams& p, int t) {
  Item it;
  it.h = t % p.hq;
  const int rest = t / p.hq;
  it.b = rest % p.batch;
  it.qb = p.q_blocks - 1 - rest / p.batch;
  it.row = (static_cast<size_t>(it.b) * p.hq + it.h) * p.q_blocks + it.qb;
  return it;
}
__device__ __forceinline__ int item_count(const AttnParams& p, const int32_t* __restrict__ cnt, int t) {
  return t < p.total_items ? __ldg(cnt + decode_item(p, t).row) : 0;
}
// lane's entry of the 32-wide window at walk position j0: walk position j maps to list[n-1-j]
__device__ __forceinline__ int list_window(const AttnParams& p, const int32_t* __restrict__ block_idx, size_t row,
                                           int n, int j0, int lane) {
  const int e = n - 1 - (j0 + lane);
  if (e < 0) return 0;
  // volatile asm pins the issue point: a plain read-only load would be sunk by the compiler to its first use,
  // which turns the intended prefetch into an exposed memory latency
  int v;
  asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(v) : "l"(block_idx + row * p.list_k_blocks + e));
  return v;
}

// Per-CTA schedule, built once in shared memory by the prologue: the block count of every item of this CTA
// (item i is work item t = blockIdx.x + i * gridDim.x) and, per stream, the order of its items (the k-th
// non-empty item of the CTA runs on stream k & 1).  Roles then walk their items without touching global memory.
struct Sched {
  const uint16_t* cnt;      // [n_local]
  const uint16_t* seq[2];   // [n_seq[s]] CTA-local item indices of stream s
  int n_local, n_seq[2];
};

__global__ void __launch_bounds__(kAttnThreads, 1)
block_sparse_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const AttnParams p,
                         const int32_t* __restrict__ block_idx, const int32_t* __restrict__ block_cnt,
                         void* __restrict__ out, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  // tiles: [stream][Q, K, V]
  float* s_l = reinterpret_cast<float*>(smem + kAttnSmemTiles);          // [stream][2][128] final row sums
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kAttnSmemTiles + 2 * 2 * 128 * 4);
  // per stream s: 10 barriers at bars[10*s + ...]
  enum { Q_FULL = 0, Q_EMPTY, K_FULL, K_EMPTY, V_FULL, V_EMPTY, S_FULL, P_READY, O_FULL, O_EMPTY, NBAR };
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int s, int which) -> uint32_t { return bar0 + 8u * (NBAR * s + which); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
#ifdef XB_TRACE
  uint32_t trace_n = 0;
  const int trace_role = warp < 4 ? 2 : (warp < 8 ? 3 : (warp < 12 ? 4 : (warp == 12 ? 0 : (warp == 13 ? 1 : (warp == 14 ? 5 : 6)))));
#endif

  if ((smem_u32(smem) & 1023u) != 0) {              // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && status) atomicExch(status, static_cast<int>(kDevBadSmemAlign));
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s)
      for (int w = 0; w < NBAR; ++w) mbar_init(bar(s, w), (w == P_READY || w == O_EMPTY) ? 128 : 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 13) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  // schedule table
  uint16_t* sch_cnt = reinterpret_cast<uint16_t*>(smem + kAttnSmemTiles + 2 * 2 * 128 * 4 + 256);
  uint16_t* sch_seq0 = sch_cnt + kSchedCap;
  uint16_t* sch_seq1 = sch_seq0 + kSchedCap;
  int* sch_total = reinterpret_cast<int*>(sch_seq1 + kSchedCap);
  uint8_t* stage_base = reinterpret_cast<uint8_t*>(sch_total) + 16;     // 16-byte aligned
  const int G = gridDim.x;
  const int n_local = (p.total_items - static_cast<int>(blockIdx.x) + G - 1) / G;     // host guarantees <= kSchedCap
  for (int i = threadIdx.x; i < n_local; i += kAttnThreads) {
    const int c = __ldg(block_cnt + decode_item(p, blockIdx.x + i * G).row);
    sch_cnt[i] = static_cast<uint16_t>(c > 65535 ? 65535 : c);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) {
    int running = 0;
    for (int base = 0; base < n_local; base += 32) {
      const int i = base + lane;
      const bool ne = i < n_local && sch_cnt[i] > 0;
      const unsigned bal = __ballot_sync(0xffffffffu, ne);
      const int k = running + __popc(bal & ((1u << lane) - 1u));
      if (ne) ((k & 1) ? sch_seq1 : sch_seq0)[k >> 1] = static_cast<uint16_t>(i);
      running += __popc(bal);
    }
    if (lane == 0) *sch_total = running;
  }
  __syncthreads();
  Sched sch;
  sch.cnt = sch_cnt;
  sch.seq[0] = sch_seq0;
  sch.seq[1] = sch_seq1;
  sch.n_local = n_local;
  sch.n_seq[0] = (*sch_total + 1) >> 1;
  sch.n_seq[1] = *sch_total >> 1;
  const uint32_t tmem_base = *tmem_slot;
  const int group = p.hq / p.hkv;

  if (warp >= 12) {
    reg_dec<80>();
    const int s = (warp - 12) >> 1;                   // stream of this warp
    uint8_t* tiles = smem + s * 3 * kTile16;          // Q, K, V tiles of the stream
    if ((warp & 1) == 0) {
      // ---------------------------------------------------------------- TMA loader of stream s (lane 0 issues)
      const int n_items = sch.n_seq[s];
      uint32_t bc = 0;
      int ok = 1;
      // list window of the first item; the next item's window is fetched while the current one is loaded
      Item it = decode_item(p, n_items > 0 ? blockIdx.x + sch.seq[s][0] * G : 0);
      int n = n_items > 0 ? sch.cnt[sch.seq[s][0]] : 0;
      int win = n_items > 0 ? list_window(p, block_idx, it.row, n, 0, lane) : 0;
      for (int m = 0; m < n_items && ok; ++m) {
        Item nit = it;
        int nn = 0, nwin = 0;
        if (m + 1 < n_items) {
          const int i2 = sch.seq[s][m + 1];
          nit = decode_item(p, blockIdx.x + i2 * G);
          nn = sch.cnt[i2];
          nwin = list_window(p, block_idx, nit.row, nn, 0, lane);
        }
        const int hkv = it.h / group;
        if (lane == 0) {
          if (mbar_wait(bar(s, Q_EMPTY), (m & 1) ^ 1, abort_flag)) {
            XB_TRACE_EV(0x10, m);
            mbar_expect_tx(bar(s, Q_FULL), kTile16);
            tma_load_5d(smem_u32(tiles), &tmQ, bar(s, Q_FULL), 0, it.qb * 128, 0, it.h, it.b);
          } else {
            ok = 0;
          }
        }
        int w = win, w_next = list_window(p, block_idx, it.row, n, 32, lane);
        for (int j = 0; j < n; ++j, ++bc) {
          if (j > 0 && (j & 31) == 0) {
            w = w_next;
            w_next = list_window(p, block_idx, it.row, n, j + 32, lane);
          }
          const int k0 = __shfl_sync(0xffffffffu, w, j & 31) * 128;
          if (lane == 0 && ok) {
            if (mbar_wait(bar(s, K_EMPTY), (bc & 1) ^ 1, abort_flag)) {
              XB_TRACE_EV(0x12, bc);
              mbar_expect_tx(bar(s, K_FULL), kTile16);
              tma_load_5d(smem_u32(tiles + kTile16), &tmK, bar(s, K_FULL), 0, k0, 0, hkv, it.b);
            } else {
              ok = 0;
            }
            if (ok && mbar_wait(bar(s, V_EMPTY), (bc & 1) ^ 1, abort_flag)) {
              XB_TRACE_EV(0x13, bc);
              mbar_expect_tx(bar(s, V_FULL), kTile16);
              tma_load_5d(smem_u32(tiles + 2 * kTile16), &tmV, bar(s, V_FULL), 0, k0, 0, hkv, it.b);
            } else {
              ok = 0;
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        it = nit; n = nn; win = nwin;
      }
    } else if (lane == 0) {
      // ---------------------------------------------------------------- MMA issuer of stream s
      const uint32_t idesc_qk = make_idesc_f16(128, 128, p.is_bf16 != 0, false, false);
      const uint32_t idesc_pv = make_idesc_f16(128, 128, p.is_bf16 != 0, false, true);
      const uint32_t qa = smem_u32(tiles), ka = smem_u32(tiles + kTile16), va = smem_u32(tiles + 2 * kTile16);
      const uint32_t sd = tmem_base + s * 128;          // S / P
      const uint32_t od = tmem_base + 256 + s * 128;    // O
      // operand descriptors never change (one Q, K and V slot per stream): build them once
      uint64_t dq[8], dk[8], dv[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t o = (k >> 2) * kHalf16 + (k & 3) * 32;
        dq[k] = smem_desc_sw128(qa + o, 16, 1024);
        dk[k] = smem_desc_sw128(ka + o, 16, 1024);
        // 16 keys per step: V rows advance by 16 x 128 B (P columns by 8: two 16-bit values per column)
        dv[k] = smem_desc_sw128(va + k * 2048, kHalf16, 1024);
      }
      const int n_items = sch.n_seq[s];
      uint32_t bc = 0;
      bool ok = true;
      for (int m = 0; m < n_items && ok; ++m) {
        const int n = sch.cnt[sch.seq[s][m]];
        for (int j = 0; j < n && ok; ++j, ++bc) {
          // S = Q K^T
          if (j == 0 && !mbar_wait(bar(s, Q_FULL), m & 1, abort_flag)) { ok = false; break; }
          if (!mbar_wait(bar(s, K_FULL), bc & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          XB_TRACE_EV(0x20, bc);
          mma_ss(sd, dq[0], dk[0], idesc_qk, 0u);
#pragma unroll
          for (int k = 1; k < 8; ++k) mma_ss(sd, dq[k], dk[k], idesc_qk, 1u);
          mma_commit(bar(s, K_EMPTY));
          mma_commit(bar(s, S_FULL));
          if (j == n - 1) mma_commit(bar(s, Q_EMPTY));
          // O += P V
          if (!mbar_wait(bar(s, P_READY), bc & 1, abort_flag)) { ok = false; break; }
          if (!mbar_wait(bar(s, V_FULL), bc & 1, abort_flag)) { ok = false; break; }
          if (j == 0 && !mbar_wait(bar(s, O_EMPTY), (m & 1) ^ 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          XB_TRACE_EV(0x22, bc);
          mma_ts(od, sd, dv[0], idesc_pv, j > 0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < 8; ++k) mma_ts(od, sd + k * 8, dv[k], idesc_pv, 1u);
          mma_commit(bar(s, V_EMPTY));
          if (j == n - 1) mma_commit(bar(s, O_FULL));
        }
      }
    }
  } else if (warp < 8) {
    // -------------------------------------------------------------------- softmax of stream (warp >> 2)
    reg_inc<168>();
    const int s = warp >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t ts = tmem_base + s * 128 + lane_bits;          // S / P of this stream, this row
    const uint32_t tmem_o = tmem_base + 256 + s * 128 + lane_bits;
    const int k_off = p.k_len - p.q_len;
    const uint32_t s_full = bar(s, S_FULL), p_ready = bar(s, P_READY);
    const int n_items = sch.n_seq[s];
    uint32_t bc = 0;
    bool ok = true;
    Item it = decode_item(p, n_items > 0 ? blockIdx.x + sch.seq[s][0] * G : 0);
    int n = n_items > 0 ? sch.cnt[sch.seq[s][0]] : 0;
    int win = n_items > 0 ? list_window(p, block_idx, it.row, n, 0, lane) : 0;
    for (int m = 0; m < n_items && ok; ++m) {
      if (threadIdx.x == (s << 7)) XB_TRACE_EV(0x36, m);
      // the stream's next item: fetch its first list window while this one is processed
      Item nit = it;
      int nn = 0, nwin = 0;
      if (m + 1 < n_items) {
        const int i2 = sch.seq[s][m + 1];
        nit = decode_item(p, blockIdx.x + i2 * G);
        nn = sch.cnt[i2];
        nwin = list_window(p, block_idx, nit.row, nn, 0, lane);
      }
      const size_t row = it.row;
      const int q_pos = it.qb * 128 + r;
      int row_last = p.k_len - 1;                       // last key position this row may see
      if (p.causal && q_pos + k_off < row_last) row_last = q_pos + k_off;
      float m_used = -INFINITY, l = 0.f;
      int w = win, w_next = list_window(p, block_idx, row, n, 32, lane);
      if (threadIdx.x == (s << 7)) XB_TRACE_EV(0x37, m);
      for (int j = 0; j < n; ++j, ++bc) {
        if (j > 0 && (j & 31) == 0) {
          w = w_next;
          w_next = list_window(p, block_idx, row, n, j + 32, lane);
        }
        const int k0 = __shfl_sync(0xffffffffu, w, j & 31) * 128;
        if (threadIdx.x == (s << 7)) XB_TRACE_EV(0x38, bc);
        const int limit = row_last - k0;                // columns c <= limit are visible
        const bool masked = __any_sync(0xffffffffu, limit < 127);
        if (threadIdx.x == (s << 7)) XB_TRACE_EV(0x30, bc);
        // waits are made warp-uniform: the tensor-memory loads/stores below are warp-collective
        if (!__all_sync(0xffffffffu, mbar_wait(s_full, bc & 1, abort_flag))) { ok = false; break; }
        tc_fence_after();
        if (threadIdx.x == (s << 7)) XB_TRACE_EV(0x31, bc);
        // ---- pass 1: row maximum, 8 independent chains of 3-input max.  In a masked block (diagonal / tail)
        // each 32-column chunk is classified per warp: all visible, none visible, or mixed (per-element
        // select).  The chunk loops are kept rolled: the kernel is bound by instruction issue and a small
        // loop body measured faster than a fully unrolled one.
        float mx8[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) mx8[q] = -INFINITY;
        uint32_t cls_mixed = 0u, cls_none = 0u;        // bit c4
        if (masked) {
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            const bool all_vis = __all_sync(0xffffffffu, limit - 32 * c4 >= 31);
            const bool none_vis = __all_sync(0xffffffffu, limit - 32 * c4 < 0);
            if (none_vis) cls_none |= 1u << c4;
            else if (!all_vis) cls_mixed |= 1u << c4;
          }
        }
        if (!masked) {
          // two tensor-memory loads in flight per wait
#pragma unroll 1
          for (int c2 = 0; c2 < 2; ++c2) {
            uint32_t v0[32], v1[32];
            tmem_ld32(ts + c2 * 64, v0);
            tmem_ld32(ts + c2 * 64 + 32, v1);
            tc_wait_ld();
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              mx8[k & 7] = max3(mx8[k & 7], __uint_as_float(v0[2 * k]), __uint_as_float(v0[2 * k + 1]));
              mx8[(k + 4) & 7] = max3(mx8[(k + 4) & 7], __uint_as_float(v1[2 * k]), __uint_as_float(v1[2 * k + 1]));
            }
          }
        }
#pragma unroll 1
        for (int c4 = masked ? 0 : 4; c4 < 4; ++c4) {
          if ((cls_none >> c4) & 1u) continue;
          uint32_t v[32];
          tmem_ld32(ts + c4 * 32, v);
          tc_wait_ld();
          if (!((cls_mixed >> c4) & 1u)) {
#pragma unroll
            for (int k = 0; k < 16; ++k)
              mx8[k & 7] = max3(mx8[k & 7], __uint_as_float(v[2 * k]), __uint_as_float(v[2 * k + 1]));
          } else {
            const int lim4 = limit - 32 * c4;
#pragma unroll
            for (int k = 0; k < 16; ++k)
              mx8[k & 7] = max3(mx8[k & 7], 2 * k <= lim4 ? __uint_as_float(v[2 * k]) : -INFINITY,
                                2 * k + 1 <= lim4 ? __uint_as_float(v[2 * k + 1]) : -INFINITY);
          }
        }
        const float mx = fmaxf(max3(mx8[0], mx8[1], mx8[2]), max3(max3(mx8[3], mx8[4], mx8[5]), mx8[6], mx8[7]));
        const float m_new = fmaxf(m_used, mx * p.scale_log2);
        const bool need = m_new > m_used + kRescaleThreshold || (j == 0) || (m_used == -INFINITY && m_new > -INFINITY);
        if (__any_sync(0xffffffffu, need)) {
          const float alpha = !need ? 1.f : (m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_new));
          if (j > 0) {
            // S of block j is complete, and the tensor pipe runs in order, so the P.V of block j-1 of this
            // stream has completed too: O may be touched
            if (threadIdx.x == (s << 7)) XB_TRACE_EV(0x32, bc);
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              uint32_t v[32];
              tmem_ld32(tmem_o + c4 * 32, v);
              tc_wait_ld();
#pragma unroll
              for (int k = 0; k < 32; ++k) v[k] = __float_as_uint(__uint_as_float(v[k]) * alpha);
              tmem_st32(tmem_o + c4 * 32, v);
            }
          }
          l *= alpha;
          if (need) m_used = m_new;
        }
        const float m_ref = m_used == -INFINITY ? 0.f : m_used;
        if (threadIdx.x == (s << 7)) XB_TRACE_EV(0x35, bc);
        // ---- pass 2: exp2 in 32-column chunks; P chunk c4 (16 packed columns) overwrites S columns that were
        // read already (packed column c/2 <= c)
        const unsigned long long scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
        const unsigned long long nmref2 = pack_f32x2(-m_ref, -m_ref);
        unsigned long long ls2[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) ls2[q] = 0ull;     // (+0.f, +0.f)
        if (!masked) {
          // the load of the next 32 columns is in flight while the current ones are exponentiated
          auto chunk = [&](const uint32_t (&v)[32], int c4) {
            uint32_t pk[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              float y0, y1;
              unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(v[2 * k]), __uint_as_float(v[2 * k + 1])), scale2, nmref2),
                           y0, y1);
              const float p0 = fast_exp2(y0), p1 = fast_exp2(y1);
              ls2[k & 3] = add_f32x2(ls2[k & 3], pack_f32x2(p0, p1));
              pk[k] = pack16(p0, p1, p.is_bf16);
            }
            tmem_st16(ts + c4 * 16, pk);
          };
          uint32_t va[32], vb[32];
          tmem_ld32(ts, va);
#pragma unroll 1
          for (int c2 = 0; c2 < 2; ++c2) {
            tc_wait_ld();
            tmem_ld32(ts + (2 * c2 + 1) * 32, vb);
            chunk(va, 2 * c2);
            tc_wait_ld();
            if (c2 == 0) tmem_ld32(ts + 64, va);
            chunk(vb, 2 * c2 + 1);
          }
        }
#pragma unroll 1
        for (int c4 = masked ? 0 : 4; c4 < 4; ++c4) {
          uint32_t pk[16];
          if ((cls_none >> c4) & 1u) {
#pragma unroll
            for (int k = 0; k < 16; ++k) pk[k] = 0u;
            tmem_st16(ts + c4 * 16, pk);
            continue;
          }
          uint32_t v[32];
          tmem_ld32(ts + c4 * 32, v);
          tc_wait_ld();
          if (!((cls_mixed >> c4) & 1u)) {
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              float y0, y1;
              unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(v[2 * k]), __uint_as_float(v[2 * k + 1])), scale2, nmref2),
                           y0, y1);
              const float p0 = fast_exp2(y0), p1 = fast_exp2(y1);
              ls2[k & 3] = add_f32x2(ls2[k & 3], pack_f32x2(p0, p1));
              pk[k] = pack16(p0, p1, p.is_bf16);
            }
          } else {
            const int lim4 = limit - 32 * c4;
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const float x0 = 2 * k <= lim4 ? __uint_as_float(v[2 * k]) : -INFINITY;
              const float x1 = 2 * k + 1 <= lim4 ? __uint_as_float(v[2 * k + 1]) : -INFINITY;
              float y0, y1;
              unpack_f32x2(fma_f32x2(pack_f32x2(x0, x1), scale2, nmref2), y0, y1);
              const float p0 = fast_exp2(y0), p1 = fast_exp2(y1);
              ls2[k & 3] = add_f32x2(ls2[k & 3], pack_f32x2(p0, p1));
              pk[k] = pack16(p0, p1, p.is_bf16);
            }
          }
          tmem_st16(ts + c4 * 16, pk);
        }
        {
          float a0, a1, b0, b1;
          unpack_f32x2(add_f32x2(add_f32x2(ls2[0], ls2[1]), add_f32x2(ls2[2], ls2[3])), a0, a1);
          (void)b0; (void)b1;
          l += a0 + a1;
        }
        if (j == n - 1) s_l[(s * 2 + (m & 1)) * 128 + r] = l;   // read by the epilogue once this item's last P.V is done
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(p_ready);
        if (threadIdx.x == (s << 7)) XB_TRACE_EV(0x33, bc);
      }
      it = nit; n = nn; win = nwin;
    }
  } else {
    // -------------------------------------------------------------------- epilogue (warps 8-11), both streams
    reg_dec<96>();
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t seen = 0;                 // non-empty items so far: item `seen` runs on stream seen & 1
    bool ok = true;
    for (int i = 0; i < sch.n_local && ok; ++i) {
      const int t = blockIdx.x + i * G;
      const int n = sch.cnt[i];
      const Item it = decode_item(p, t);
      const int q_pos = it.qb * 128 + r;
      const bool store = q_pos < p.q_len;
      uint8_t* orow = static_cast<uint8_t*>(out) +
                      2 * (static_cast<int64_t>(it.b) * p.osb + static_cast<int64_t>(it.h) * p.osh +
                           static_cast<int64_t>(store ? q_pos : 0) * p.osl);
      if (n == 0) {
        if (store) {
          uint4* dst = reinterpret_cast<uint4*>(orow);
#pragma unroll
          for (int q4 = 0; q4 < 16; ++q4) dst[q4] = make_uint4(0u, 0u, 0u, 0u);
        }
        continue;
      }
      const int s = seen & 1;
      const uint32_t m = seen >> 1;
      ++seen;
      if (threadIdx.x == 256) XB_TRACE_EV(0x40 + s, m);
      if (!__all_sync(0xffffffffu, mbar_wait(bar(s, O_FULL), m & 1, abort_flag))) { ok = false; break; }
      tc_fence_after();
      if (threadIdx.x == 256) XB_TRACE_EV(0x42 + s, m);
      const float l = s_l[(s * 2 + (m & 1)) * 128 + r];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const uint32_t tmem_o = tmem_base + 256 + s * 128 + lane_bits;
      // A thread owns one output row, but a store instruction should write whole cache lines: each 64-column
      // half of the warp's 32 rows goes through a 4 KiB shared-memory buffer (16-byte chunks XOR-swizzled by
      // row against bank conflicts) and leaves as 8 instructions of 4 rows x 128 contiguous bytes.
      uint8_t* stg = stage_base + quad * (32 * 128);
      const int q_row0 = it.qb * 128 + quad * 32;                     // first row of this warp
      uint8_t* obase = static_cast<uint8_t*>(out) +
                       2 * (static_cast<int64_t>(it.b) * p.osb + static_cast<int64_t>(it.h) * p.osh);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t v[32];
          tmem_ld32(tmem_o + half * 64 + c2 * 32, v);
          tc_wait_ld();
          if (half == 1 && c2 == 1) {
            // every read of this O buffer is done: the stream's next item may accumulate into it
            tc_fence_before();
            mbar_arrive(bar(s, O_EMPTY));
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 wv;
            wv.x = pack16(__uint_as_float(v[q4 * 8 + 0]) * inv, __uint_as_float(v[q4 * 8 + 1]) * inv, p.is_bf16);
            wv.y = pack16(__uint_as_float(v[q4 * 8 + 2]) * inv, __uint_as_float(v[q4 * 8 + 3]) * inv, p.is_bf16);
            wv.z = pack16(__uint_as_float(v[q4 * 8 + 4]) * inv, __uint_as_float(v[q4 * 8 + 5]) * inv, p.is_bf16);
            wv.w = pack16(__uint_as_float(v[q4 * 8 + 6]) * inv, __uint_as_float(v[q4 * 8 + 7]) * inv, p.is_bf16);
            const int chunk = c2 * 4 + q4;                            // 16-byte chunk within the 128-byte half row
            *reinterpret_cast<uint4*>(stg + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = wv;
          }
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = 4 * i + (lane >> 3);                         // row within the warp's 32
          const int chunk = lane & 7;
          const uint4 wv = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((chunk ^ (rr & 7)) << 4));
          const int q_pos_r = q_row0 + rr;
          if (q_pos_r < p.q_len)
            *reinterpret_cast<uint4*>(obase + 2 * static_cast<int64_t>(q_pos_r) * p.osl + half * 128 + chunk * 16) = wv;
        }
        __syncwarp();
      }
      if (threadIdx.x == 256) XB_TRACE_EV(0x44 + s, m);
    }
  }

  // -------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) { __nanosleep(1000); }
    if (threadIdx.x == 0 && status) atomicExch(status, static_cast<int>(kDevWaitTimeout));
    __syncthreads();
  }
  if (warp == 13) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// [64 columns, rows, 2 column halves, heads, batch]: one box {64, 128, 2, 1, 1} brings a whole 128x128 tile
// with a single TMA instruction, laid out as two 64-column swizzled halves one after the other.
static int make_qkv_map(CUtensorMap* m, const void* base, int len, int heads, int batch, int64_t sb, int64_t sh,
                        int64_t sl) {
  const uint64_t dims[5] = {64, (uint64_t)len, 2, (uint64_t)heads, (uint64_t)batch};
  // a dimension of extent 1 never moves: give it a harmless valid stride
  const uint64_t s_h = heads > 1 ? (uint64_t)sh * 2 : 256, s_b = batch > 1 ? (uint64_t)sb * 2 : 256;
  const uint64_t str[4] = {(uint64_t)sl * 2, 128, s_h, s_b};
  const uint32_t box[5] = {64, 128, 2, 1, 1};
  return make_tmap_16bit(m, base, 5, dims, str, box);
}

int block_sparse_attn_launch(const void* q, const void* k, const void* v, int dtype, int batch, int hq, int hkv,
                             int q_len, int k_len, int head_dim, int64_t qsb, int64_t qsh, int64_t qsl, int64_t ksb,
                             int64_t ksh, int64_t ksl, int64_t vsb, int64_t vsh, int64_t vsl,
                             const int32_t* block_idx, const int32_t* block_cnt, int causal, float scale, void* out,
                             int64_t osb, int64_t osh, int64_t osl, int* status, cudaStream_t stream) {
  if (!q || !k || !v || !out || !block_idx || !block_cnt) return XATTN_B200_ERR_ARG;
  if (dtype != XATTN_B200_BF16 && dtype != XATTN_B200_F16) return XATTN_B200_ERR_ARG;
  if (head_dim != 128 || batch < 1 || hq < 1 || hkv < 1 || hq % hkv != 0 || q_len < 1 || k_len < 1)
    return XATTN_B200_ERR_ARG;
  if (causal && k_len < q_len) return XATTN_B200_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (osl % 8) || (osh % 8) || (osb % 8)) return XATTN_B200_ERR_ARG;
  if (!(scale > 0.f)) return XATTN_B200_ERR_ARG;
  int rc;
  if ((rc = check_sm100())) return rc;
  CUtensorMap tmQ, tmK, tmV;
  if ((rc = make_qkv_map(&tmQ, q, q_len, hq, batch, qsb, qsh, qsl))) return rc;
  if ((rc = make_qkv_map(&tmK, k, k_len, hkv, batch, ksb, ksh, ksl))) return rc;
  if ((rc = make_qkv_map(&tmV, v, k_len, hkv, batch, vsb, vsh, vsl))) return rc;
  AttnParams p;
  p.batch = batch; p.hq = hq; p.hkv = hkv; p.q_len = q_len; p.k_len = k_len;
  p.q_blocks = (q_len + 127) / 128; p.list_k_blocks = (k_len + 127) / 128;
  p.causal = causal ? 1 : 0; p.is_bf16 = dtype == XATTN_B200_BF16 ? 1 : 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.osb = osb; p.osh = osh; p.osl = osl;
  if (cudaFuncSetAttribute(block_sparse_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem) !=
      cudaSuccess)
    return XATTN_B200_ERR_CUDA;
  const long long items = static_cast<long long>(batch) * hq * p.q_blocks;
  if (items > 0x7fffffffLL) return XATTN_B200_ERR_LIMIT;
  p.total_items = static_cast<int>(items);
  const int sms = sm_count();
  const int grid = items < sms ? static_cast<int>(items) : sms;
  if ((items + grid - 1) / grid > kSchedCap || p.list_k_blocks > 65535) return XATTN_B200_ERR_LIMIT;
  block_sparse_attn_kernel<<<grid, kAttnThreads, kAttnSmem, stream>>>(tmQ, tmK, tmV, p, block_idx, block_cnt, out,
                                                                      status);
  return launch_status();
}

}  // namespace xb
