// Block-sparse attention for the lists long-context prefill produces most: one or two key blocks per query
// block (the attention sink and the diagonal), the same for every query head of a kv group.
//
// Same operation as attention.cu (replaces block_sparse_attn.block_sparse_attn_func, call site
// xattn/src/Xattention.py:377-391), restricted to work the general kernel handles worst.  With two blocks per
// item that kernel is all prologue and epilogue: every (head, query block) loads its own Q, K and V tiles and
// walks QK^T -> softmax -> P.V twice with an online-softmax dependency between the blocks.  Here a work unit is
// a GROUP item: one (batch, kv head, query block) with all hq/hkv query heads that read that kv head.
//
//   * K and V tiles of the (at most two) listed blocks are loaded ONCE per group item and serve every query head
//     of the group (GQA head sharing): with 4 heads per group, tile traffic into shared memory drops from
//     160 KiB to 64 KiB per (head, query block).
//   * The heads of the group run two at a time, one per stream.  A stream issues BOTH Q.K^T products back to
//     back into two score buffers in tensor memory (S_a, S_b), takes ONE row maximum over all their columns,
//     exponentiates once (no online rescale, no second MMA round trip), and issues both P.V products back to
//     back.  O has no buffer of its own.  A stream owns 256 columns of tensor memory: S_a in [0,128), S_b in
//     [128,256).  P_a (16 bit) overwrites columns [0,64) of S_a in ascending chunk order and P_b columns
//     [192,256) of S_b in descending chunk order (each P chunk lands on S columns that are in registers
//     already), which leaves the 128 columns [64,192) in the middle for O once the softmax has read them.
//   * A stream has TWO softmax warpgroups, one per block: each thread owns one row of ONE block (128 columns), the
//     row maxima of the two blocks are exchanged through shared memory, and the second warpgroup (the diagonal
//     block, which has less to exponentiate) also normalises the output and hands it to TMA stores.  Four softmax
//     warps per scheduler instead of two: a softmax warp runs at the instruction rate of a single warp (dependent
//     chains behind tensor-memory loads), so the schedulers were two thirds idle.
//   * The two streams run half a round apart on purpose: stream 1 issues its Q.K^T when stream 0 has finished
//     its first softmax pass, and stream 0 issues its next Q.K^T when that one has completed.  Left alone both streams fall into
//     lockstep (both in their MMA phase, then both exponentiating on the same special-function units, each at
//     half speed); kept apart, one stream's MMAs run under the other's softmax.
//
//   warps 0-3 / 4-7     stream 0: softmax of block a / softmax of block b + output   } one thread per query row
//   warps 8-11 / 12-15  stream 1: the same                                            } and block
//   warp  16            TMA loader (lane 0): K_a, K_b, V_a, V_b per group item, Q per (round, stream)
//   warp  17/19         tcgen05 issuer of stream 0 / 1 (lane 0)
//
// Which group items qualify is decided on the device by pair_classify_kernel (no host synchronisation): it
// compacts them into a list and marks their items as taken in a copy of the block counts, which the general
// kernel then skips.
#include "attention_common.cuh"

namespace xb {

constexpr int kPairThreads = 640;
constexpr int kPairLaunchRegs = 96;                       // 65536 / 640, rounded down to a multiple of 8
constexpr int kPairSchedCap = 64;                         // group items one CTA handles per launch
constexpr int kPairSmemTiles = kTile16 * 6;               // Q0, Q1, K_a, K_b, V_a, V_b
constexpr int kPairStage = 8 * 32 * 128;                  // per output warp: 32 rows x 64 16-bit columns
constexpr int kPairXchg = 2 * 2 * 128 * 4;                // [stream][block][row] floats exchanged between warpgroups
constexpr int kPairSmem = kPairSmemTiles + kPairStage + kPairXchg + kPairSchedCap * 8 + 256;
static_assert(kPairSmem <= 232448, "shared memory of one CTA");
constexpr uint32_t kNoBlock = 0xFFFFu;

struct PairEntry {
  int32_t unit;        // (b * hkv + g) * q_blocks + qb
  uint32_t blocks;     // first block | second block << 16 (kNoBlock: the list has one entry)
};

// ------------------------------------------------------------------------------------------------ classify
// One thread per group item: it qualifies when every query head of the group lists the same one or two blocks.
// Qualifying items go to `list`, the work items (batch, query head, query block) of all others to `rest_list` in
// the general kernel's numbering (order: as the atomics fall; every item is computed independently, so the order
// changes nothing in the result).  The general kernel then takes its items from that list, evenly over its CTAs.
__global__ void pair_classify_kernel(const int32_t* __restrict__ block_idx, const int32_t* __restrict__ block_cnt,
                                     int batch, int hq, int hkv, int q_blocks, int list_k_blocks,
                                     PairEntry* __restrict__ list, int* __restrict__ counter,
                                     int32_t* __restrict__ rest_list) {
  pdl_launch_dependents();          // the pair kernel's CTAs may take their places; they wait for this grid to end
  const int units = batch * hkv * q_blocks;
  const int u = blockIdx.x * blockDim.x + threadIdx.x;
  int total = 0, taken = 0;
  if (u < units) {
    const int group = hq / hkv;
    const int qb = u % q_blocks;
    const int bg = u / q_blocks;
    const int g = bg % hkv, b = bg / hkv;
    const size_t row0 = (static_cast<size_t>(b) * hq + static_cast<size_t>(g) * group) * q_blocks + qb;
    // The loads of the heads do not depend on each other (no early exit): a unit costs two memory round trips,
    // counts then list heads, whatever the number of heads.  The first two list entries are read even when the
    // list is shorter (they exist: a row of the index array has list_k_blocks >= 1 entries, and the second is
    // only read when list_k_blocks >= 2); they are ignored then.
    const int c0 = __ldg(block_cnt + row0);
    bool same_cnt = true;
#pragma unroll 4
    for (int j = 0; j < group; ++j) {
      const int c = __ldg(block_cnt + row0 + static_cast<size_t>(j) * q_blocks);
      same_cnt &= c == c0;
      total += c;
    }
    bool ok = same_cnt && (c0 == 1 || c0 == 2);
    const bool two = list_k_blocks >= 2;
    const int i0 = __ldg(block_idx + row0 * list_k_blocks);
    const int i1 = two ? __ldg(block_idx + row0 * list_k_blocks + 1) : 0;
    bool same_idx = true;
#pragma unroll 4
    for (int j = 1; j < group; ++j) {
      const size_t row = row0 + static_cast<size_t>(j) * q_blocks;
      const int a = __ldg(block_idx + row * list_k_blocks);
      const int b2 = two ? __ldg(block_idx + row * list_k_blocks + 1) : 0;
      same_idx &= a == i0 && (c0 == 1 || b2 == i1);
    }
    ok = ok && same_idx;
    if (ok) {
      const int pos = atomicAdd(counter, 1);
      list[pos].unit = u;
      list[pos].blocks = static_cast<uint32_t>(i0) | ((c0 == 2 ? static_cast<uint32_t>(i1) : kNoBlock) << 16);
    }
    taken = ok ? total : 0;
    if (!ok) {
      // work item t of the general kernel: t = ((q_blocks - 1 - qb) * batch + b) * hq + h
      const int pos = atomicAdd(counter + kPairRestCount, group);
      const int t0 = ((q_blocks - 1 - qb) * batch + b) * hq + g * group;
      for (int j = 0; j < group; ++j) rest_list[pos + j] = t0 + j;
    }
  }
  // block totals for pair_path_chosen(): one atomic per warp and word
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    total += __shfl_xor_sync(0xffffffffu, total, o);
    taken += __shfl_xor_sync(0xffffffffu, taken, o);
  }
  if ((threadIdx.x & 31) == 0 && total > 0) {
    atomicAdd(reinterpret_cast<unsigned long long*>(counter + kPairTotalAll), static_cast<unsigned long long>(total));
    atomicAdd(reinterpret_cast<unsigned long long*>(counter + kPairTotalTaken), static_cast<unsigned long long>(taken));
  }
}

// ------------------------------------------------------------------------------------------------ the kernel
// columns > lim of a 32-column chunk become -inf
__device__ __forceinline__ void mask_chunk(uint32_t (&v)[32], int lim) {
#pragma unroll
  for (int k = 0; k < 32; ++k) v[k] = k <= lim ? v[k] : 0xff800000u;
}

__global__ void __launch_bounds__(kPairThreads, 1)
block_sparse_attn_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                              const AttnParams p,
                              const PairEntry* __restrict__ list, const int* __restrict__ counter, int list_offset,
                              int min_share_pct, void* __restrict__ out, int* status) {
  constexpr int kRegSoftmax = 104, kRegOther = 64;                  // 16 x 104 + 4 x 64 = 1920 = 20 x 96
  static_assert(16 * kRegSoftmax + 4 * kRegOther <= 20 * kPairLaunchRegs, "register budget of the roles");
  extern __shared__ __align__(1024) uint8_t smem[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if ((smem_u32(smem) & 1023u) != 0) {              // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && status) atomicExch(status, static_cast<int>(kDevBadSmemAlign));
    return;
  }
  // launched while the classify kernel (or this kernel's previous window) may still run: let the next kernel of the
  // stream queue up behind this one in the same way, then wait for what the earlier ones wrote
  pdl_launch_dependents();
  pdl_wait();
  if (!pair_path_chosen(counter, min_share_pct)) return;           // the general kernel computes everything (same test there)
  // tiles: Q0, Q1, K_a, K_b, V_a, V_b
  uint8_t* stage_base = smem + kPairSmemTiles;
  float* xchg = reinterpret_cast<float*>(smem + kPairSmemTiles + kPairStage);          // [stream][block][row]
  PairEntry* sch = reinterpret_cast<PairEntry*>(smem + kPairSmemTiles + kPairStage + kPairXchg);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPairSmemTiles + kPairStage + kPairXchg + kPairSchedCap * 8);
  // GO0: stream 1's Q.K^T of a round has completed (stream 0 may issue its next one); GO1: stream 0 has the row
  // maxima of a round (stream 1 may issue its Q.K^T of that round)
  // XCH1: both warpgroups of a stream have written their block's row maxima; XCH2: both have read them (the slot of
  // block a then carries block a's row sums to the output warpgroup)
  enum { K_FULL = 0, K_EMPTY, V_FULL, V_EMPTY, GO0, GO1, PER_STREAM,
         Q_FULL = 0, Q_EMPTY, S_FULL, P_READY, O_FULL, TMEM_FREE, XCH1, XCH2, NSTREAM };
  const uint32_t bar0 = smem_u32(bars);
  auto gbar = [&](int which) -> uint32_t { return bar0 + 8u * which; };
  auto sbar = [&](int s, int which) -> uint32_t { return bar0 + 8u * (PER_STREAM + NSTREAM * s + which); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + PER_STREAM + 2 * NSTREAM);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
#ifdef XB_TRACE
  uint32_t trace_n = 0;
  // softmax warps: quad 0 of (stream, block) -> 2..5, quad 3 -> 7..10, the others share 13
  const int trace_role = warp < 16 ? ((warp & 3) == 0 ? 2 + (warp >> 2) : ((warp & 3) == 3 ? 7 + (warp >> 2) : 13))
                                   : (warp == 16 ? 0 : (warp == 17 ? 1 : (warp == 19 ? 6 : 11)));
#endif

  // this launch's share of the list: entries list_offset + blockIdx.x + i * gridDim.x, at most kPairSchedCap
  const int total = __ldg(counter);
  const int G = gridDim.x;
  int n_local = 0;
  {
    const long long first = static_cast<long long>(list_offset) + blockIdx.x;
    if (first < total) {
      const long long avail = (total - first + G - 1) / G;
      n_local = static_cast<int>(avail < kPairSchedCap ? avail : kPairSchedCap);
    }
  }
  for (int i = threadIdx.x; i < n_local; i += kPairThreads) sch[i] = list[list_offset + blockIdx.x + i * G];
  if (threadIdx.x == 0) {
    mbar_init(gbar(K_FULL), 1);
    mbar_init(gbar(K_EMPTY), 2);
    mbar_init(gbar(V_FULL), 1);
    mbar_init(gbar(V_EMPTY), 2);
    mbar_init(gbar(GO0), 1);
    mbar_init(gbar(GO1), 256);
    for (int s = 0; s < 2; ++s) {
      mbar_init(sbar(s, Q_FULL), 1);
      mbar_init(sbar(s, Q_EMPTY), 1);
      mbar_init(sbar(s, S_FULL), 1);
      mbar_init(sbar(s, P_READY), 256);
      mbar_init(sbar(s, O_FULL), 1);
      mbar_init(sbar(s, TMEM_FREE), 128);
      mbar_init(sbar(s, XCH1), 256);
      mbar_init(sbar(s, XCH2), 256);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO);
  }
  if (warp == 17) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int group = p.hq / p.hkv;
  const int rounds = group >> 1;                     // two heads per round, one per stream
  auto decode = [&](const PairEntry& e, int& b, int& g, int& qb) {
    qb = e.unit % p.q_blocks;
    const int bg = e.unit / p.q_blocks;
    g = bg % p.hkv;
    b = bg / p.hkv;
  };

  if (warp >= 16) {
    reg_set_from<kRegOther, kPairLaunchRegs>();
    if (warp == 16) {
      // ------------------------------------------------------------------------------------- TMA loader
      if (lane == 0) {
        uint32_t rc = 0;                             // rounds so far (both streams advance together here)
        bool ok = true;
        for (int i = 0; i < n_local && ok; ++i) {
          const PairEntry e = sch[i];
          int b, g, qb;
          decode(e, b, g, qb);
          const int ka = static_cast<int>(e.blocks & 0xFFFFu), kb = static_cast<int>(e.blocks >> 16);
          const int n = kb == static_cast<int>(kNoBlock) ? 1 : 2;
          for (int r = 0; r < rounds && ok; ++r, ++rc) {
            // In the order the barriers open at a group-item boundary: stream 0's Q buffer (its last Q.K^T is
            // the earlier one), then the K tiles (both streams' last Q.K^T), then stream 1's Q buffer.
            for (int s = 0; s < 2 && ok; ++s) {
              if (!mbar_wait(sbar(s, Q_EMPTY), (rc & 1) ^ 1, abort_flag)) { ok = false; break; }
              XB_TRACE_EV(0x10, rc * 2 + s);
              mbar_expect_tx(sbar(s, Q_FULL), kTile16);
              tma_load_5d(smem_u32(smem + s * kTile16), &tmQ, sbar(s, Q_FULL), 0, qb * 128, 0,
                          g * group + 2 * r + s, b);
              if (r == 0 && s == 0) {
                if (!mbar_wait(gbar(K_EMPTY), (i & 1) ^ 1, abort_flag)) { ok = false; break; }
                XB_TRACE_EV(0x12, i);
                mbar_expect_tx(gbar(K_FULL), n * kTile16);
                tma_load_5d(smem_u32(smem + 2 * kTile16), &tmK, gbar(K_FULL), 0, ka * 128, 0, g, b);
                if (n == 2) tma_load_5d(smem_u32(smem + 3 * kTile16), &tmK, gbar(K_FULL), 0, kb * 128, 0, g, b);
              }
            }
            if (r == 0 && ok) {
              if (!mbar_wait(gbar(V_EMPTY), (i & 1) ^ 1, abort_flag)) { ok = false; break; }
              XB_TRACE_EV(0x13, i);
              mbar_expect_tx(gbar(V_FULL), n * kTile16);
              tma_load_5d(smem_u32(smem + 4 * kTile16), &tmV, gbar(V_FULL), 0, ka * 128, 0, g, b);
              if (n == 2) tma_load_5d(smem_u32(smem + 5 * kTile16), &tmV, gbar(V_FULL), 0, kb * 128, 0, g, b);
              // the next group item's tiles start their way from HBM to L2 a whole item ahead
              if (i + 1 < n_local) {
                const PairEntry e2 = sch[i + 1];
                int b2, g2, qb2;
                decode(e2, b2, g2, qb2);
                const int ka2 = static_cast<int>(e2.blocks & 0xFFFFu), kb2 = static_cast<int>(e2.blocks >> 16);
                tma_prefetch_l2_5d(&tmK, 0, ka2 * 128, 0, g2, b2);
                tma_prefetch_l2_5d(&tmV, 0, ka2 * 128, 0, g2, b2);
                if (kb2 != static_cast<int>(kNoBlock)) {
                  tma_prefetch_l2_5d(&tmK, 0, kb2 * 128, 0, g2, b2);
                  tma_prefetch_l2_5d(&tmV, 0, kb2 * 128, 0, g2, b2);
                }
                for (int h2 = 0; h2 < group; ++h2) tma_prefetch_l2_5d(&tmQ, 0, qb2 * 128, 0, g2 * group + h2, b2);
              }
            }
          }
        }
      }
    } else if ((warp == 17 || warp == 19) && lane == 0) {
      // ------------------------------------------------------------------------------------- MMA issuer of stream s
      const int s = warp == 17 ? 0 : 1;
      const uint32_t idesc_qk = make_idesc_f16(128, 128, p.is_bf16 != 0, false, false);
      const uint32_t idesc_pv = make_idesc_f16(128, 128, p.is_bf16 != 0, false, true);
      const uint32_t sa = tmem_base + s * 256, sb2 = sa + 128;             // S_a / S_b
      const uint32_t pa = sa, pb = sa + 192, od = sa + 64;                 // P_a, P_b, O
      const uint32_t qa = smem_u32(smem + s * kTile16);
      const uint32_t kt = smem_u32(smem + 2 * kTile16), vt = smem_u32(smem + 4 * kTile16);
      // K-major operand, k-step k: 16 columns = 32 B inside the 64-column half (k & 3), second half 16 KiB on
      const uint64_t dq0 = smem_desc_sw128(qa, 16, 1024);
      const uint64_t dk0 = smem_desc_sw128(kt, 16, 1024);
      // V as MN-major operand: 16 keys per step = 16 x 128 B rows, the second 64 columns 16 KiB on
      const uint64_t dv0 = smem_desc_sw128(vt, kHalf16, 1024);
      uint32_t rc = 0;
      bool ok = true;
      for (int i = 0; i < n_local && ok; ++i) {
        const PairEntry e = sch[i];
        const int n = (e.blocks >> 16) == kNoBlock ? 1 : 2;
        for (int r = 0; r < rounds && ok; ++r, ++rc) {
          if (r == 0 && !mbar_wait(gbar(K_FULL), i & 1, abort_flag)) { ok = false; break; }
          if (!mbar_wait(sbar(s, Q_FULL), rc & 1, abort_flag)) { ok = false; break; }
          if (!mbar_wait(sbar(s, TMEM_FREE), (rc & 1) ^ 1, abort_flag)) { ok = false; break; }
          // half a round apart: stream 0 waits for stream 1's Q.K^T of the round before, stream 1 for the end of
          // stream 0's first softmax pass of this round
          if (!mbar_wait(gbar(s == 0 ? GO0 : GO1), s == 0 ? (rc & 1) ^ 1 : (rc & 1), abort_flag)) { ok = false; break; }
          tc_fence_after();
          XB_TRACE_EV(0x20, rc);
          for (int blk = 0; blk < n; ++blk) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint32_t o = (k >> 2) * kHalf16 + (k & 3) * 32;
              mma_ss(blk == 0 ? sa : sb2, dq0 + (o >> 4), dk0 + ((blk * kTile16 + o) >> 4), idesc_qk, k > 0 ? 1u : 0u);
            }
          }
          mma_commit(sbar(s, S_FULL));
          mma_commit(sbar(s, Q_EMPTY));
          if (s == 1) mma_commit(gbar(GO0));
          if (r == rounds - 1) mma_commit(gbar(K_EMPTY));
          if (!mbar_wait(sbar(s, P_READY), rc & 1, abort_flag)) { ok = false; break; }
          if (r == 0 && !mbar_wait(gbar(V_FULL), i & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          XB_TRACE_EV(0x22, rc);
          for (int blk = 0; blk < n; ++blk) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
              mma_ts(od, (blk == 0 ? pa : pb) + k * 8, dv0 + ((blk * kTile16 + k * 2048) >> 4), idesc_pv,
                     (blk > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit(sbar(s, O_FULL));
          if (r == rounds - 1) mma_commit(gbar(V_EMPTY));
        }
      }
    }
  } else {
    // --------------------------------------------------------------------------------------- softmax (+ output)
    reg_set_from<kRegSoftmax, kPairLaunchRegs>();
    const int s = warp >> 3;                                           // stream
    const int blk = (warp >> 2) & 1;                                   // this warpgroup's block: 0 = a, 1 = b
    const int quad = warp & 3;
    const int rr = quad * 32 + lane;                                   // query row inside the block
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t ts = tmem_base + s * 256 + lane_bits;               // the stream's 256 columns, this row
    const uint32_t tS = ts + blk * 128;                                // S of this warpgroup's block
    const uint32_t tP = ts + blk * 192;                                // its P: [0,64) for a, [192,256) for b
    const int k_off = p.k_len - p.q_len;
    const unsigned long long scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
    float* x_own = xchg + (s * 2 + blk) * 128 + rr;
    float* x_other = xchg + (s * 2 + (blk ^ 1)) * 128 + rr;
    float* x_a = xchg + (s * 2) * 128 + rr;                            // after XCH2: block a's row sum
    uint8_t* stg = stage_base + (s * 4 + quad) * (32 * 128);           // output warps only
    uint32_t rc = 0;
    bool ok = true;
    for (int i = 0; i < n_local && ok; ++i) {
      const PairEntry e = sch[i];
      int b, g, qb;
      decode(e, b, g, qb);
      const int n = (e.blocks >> 16) == kNoBlock ? 1 : 2;
      const int k0 = static_cast<int>(blk == 0 ? (e.blocks & 0xFFFFu) : (e.blocks >> 16)) * 128;
      const int q_pos = qb * 128 + rr;
      int row_last = p.k_len - 1;                       // last key position this row may see
      if (p.causal && q_pos + k_off < row_last) row_last = q_pos + k_off;
      // the visible chunks of the block are a prefix [0, nv) (visibility only ever ends towards higher columns);
      // bit c of `mixed` = some row of the warp sees only part of chunk c.  No second block: nothing visible.
      const int lim = row_last - k0;
      int nv = 0;
      uint32_t mixed = 0u;
      if (blk < n) {
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          const bool all_v = __all_sync(0xffffffffu, lim - 32 * c4 >= 31);
          const bool none_v = __all_sync(0xffffffffu, lim - 32 * c4 < 0);
          if (!none_v) {
            nv = c4 + 1;
            if (!all_v) mixed |= 1u << c4;
          }
        }
      }
      for (int r = 0; r < rounds && ok; ++r, ++rc) {
        const int h = g * group + 2 * r + s;
        if (lane == 0) XB_TRACE_EV(0x30, rc);
        if (!__all_sync(0xffffffffu, mbar_wait(sbar(s, S_FULL), rc & 1, abort_flag))) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) XB_TRACE_EV(0x31, rc);
        // ---- pass 1: row maximum over the visible columns of this block (8 chains of 3-input max), two
        // tensor-memory loads in flight per wait
        float mx8[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) mx8[q] = -INFINITY;
#pragma unroll 1
        for (int c2 = 0; c2 < 2 && 2 * c2 < nv; ++c2) {
          uint32_t v0[32], v1[32];
          const bool two = 2 * c2 + 1 < nv;
          tmem_ld32(tS + c2 * 64, v0);
          if (two) tmem_ld32(tS + c2 * 64 + 32, v1);
          tc_wait_ld();
          if ((mixed >> (2 * c2)) & 1u) mask_chunk(v0, lim - 64 * c2);
#pragma unroll
          for (int k = 0; k < 16; ++k)
            mx8[k & 7] = max3(mx8[k & 7], __uint_as_float(v0[2 * k]), __uint_as_float(v0[2 * k + 1]));
          if (two) {
            if ((mixed >> (2 * c2 + 1)) & 1u) mask_chunk(v1, lim - 64 * c2 - 32);
#pragma unroll
            for (int k = 0; k < 16; ++k)
              mx8[(k + 4) & 7] = max3(mx8[(k + 4) & 7], __uint_as_float(v1[2 * k]), __uint_as_float(v1[2 * k + 1]));
          }
        }
        float mx = fmaxf(max3(mx8[0], mx8[1], mx8[2]), max3(max3(mx8[3], mx8[4], mx8[5]), mx8[6], mx8[7]));
        // the row's maximum over both blocks: through shared memory, with the other warpgroup of the stream
        *x_own = mx;
        mbar_arrive(sbar(s, XCH1));
        if (!__all_sync(0xffffffffu, mbar_wait(sbar(s, XCH1), rc & 1, abort_flag))) { ok = false; break; }
        mx = fmaxf(mx, *x_other);
        mbar_arrive(sbar(s, XCH2));                                    // this thread has read the other's maximum
        if (s == 0) mbar_arrive(gbar(GO1));            // stream 1 may issue its Q.K^T: it runs under this stream's pass 2
        const float m_ref = mx == -INFINITY ? 0.f : mx * p.scale_log2;
        if (lane == 0) XB_TRACE_EV(0x35, rc);
        // ---- pass 2: P = exp2(S * scale - m) in 32-column chunks.  Block a ascending, P chunk c to columns
        // [16 c, 16 c + 16) of S_a; block b descending, P chunk c to columns [64 + 16 c, 64 + 16 c + 16) of S_b:
        // either way a P chunk overwrites only S columns that have been read (or are invisible).
        const unsigned long long nmref2 = pack_f32x2(-m_ref, -m_ref);
        unsigned long long ls2[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) ls2[q] = 0ull;     // (+0.f, +0.f)
        if (blk < n) {
#pragma unroll 1
          for (int kk = 0; kk < 4; ++kk) {
            const int c4 = blk == 0 ? kk : 3 - kk;
            uint32_t pk[16];
            if (c4 < nv) {
              uint32_t v[32];
              tmem_ld32(tS + c4 * 32, v);
              tc_wait_ld();
              if ((mixed >> c4) & 1u) mask_chunk(v, lim - 32 * c4);
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
#pragma unroll
              for (int k = 0; k < 16; ++k) pk[k] = 0u;
            }
            tmem_st16(tP + c4 * 16, pk);
          }
        }
        float l;
        {
          float l0, l1;
          unpack_f32x2(add_f32x2(add_f32x2(ls2[0], ls2[1]), add_f32x2(ls2[2], ls2[3])), l0, l1);
          l = l0 + l1;
        }
        if (blk == 0) {
          // block a's row sum travels to the output warpgroup in this warpgroup's exchange slot, once both
          // warpgroups have read the maxima out of the slots
          if (!__all_sync(0xffffffffu, mbar_wait(sbar(s, XCH2), rc & 1, abort_flag))) { ok = false; break; }
          *x_a = l;
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(sbar(s, P_READY));
        if (lane == 0) XB_TRACE_EV(0x33, rc);
        if (blk == 0) continue;                        // the warpgroup of block a goes on to the next head's scores
        // ---- output (warpgroup of block b): O / l from columns [64, 192) of the stream
        if (!__all_sync(0xffffffffu, mbar_wait(sbar(s, O_FULL), rc & 1, abort_flag))) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) XB_TRACE_EV(0x42, rc);
        l += *x_a;                                     // (read before the tensor memory is handed back: the other
                                                       // warpgroup reuses the slot in the next round)
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int q_row0 = qb * 128 + quad * 32;
        auto load_half = [&](int half, uint4 (&pk)[8]) {   // O columns [64 half, 64 half + 64), normalised, 16 bit
          uint32_t v0[32], v1[32];
          tmem_ld32(ts + 64 + half * 64, v0);
          tmem_ld32(ts + 96 + half * 64, v1);
          tc_wait_ld();
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            pk[q4] = make_uint4(
                pack16(__uint_as_float(v0[q4 * 8 + 0]) * inv, __uint_as_float(v0[q4 * 8 + 1]) * inv, p.is_bf16),
                pack16(__uint_as_float(v0[q4 * 8 + 2]) * inv, __uint_as_float(v0[q4 * 8 + 3]) * inv, p.is_bf16),
                pack16(__uint_as_float(v0[q4 * 8 + 4]) * inv, __uint_as_float(v0[q4 * 8 + 5]) * inv, p.is_bf16),
                pack16(__uint_as_float(v0[q4 * 8 + 6]) * inv, __uint_as_float(v0[q4 * 8 + 7]) * inv, p.is_bf16));
            pk[4 + q4] = make_uint4(
                pack16(__uint_as_float(v1[q4 * 8 + 0]) * inv, __uint_as_float(v1[q4 * 8 + 1]) * inv, p.is_bf16),
                pack16(__uint_as_float(v1[q4 * 8 + 2]) * inv, __uint_as_float(v1[q4 * 8 + 3]) * inv, p.is_bf16),
                pack16(__uint_as_float(v1[q4 * 8 + 4]) * inv, __uint_as_float(v1[q4 * 8 + 5]) * inv, p.is_bf16),
                pack16(__uint_as_float(v1[q4 * 8 + 6]) * inv, __uint_as_float(v1[q4 * 8 + 7]) * inv, p.is_bf16));
          }
        };
        // A 64-column half of the warp's 32 rows is written to the warp's 4 KiB staging tile in the 128-byte
        // swizzle pattern (16-byte chunk c of row r at chunk c ^ (r & 7)) and leaves as ONE TMA store, which
        // also clips the rows past q_len.  The staging tile may be rewritten once the store has read it.
        auto stage_and_store = [&](const uint4 (&pk)[8], int half) {
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
#pragma unroll
          for (int chunk = 0; chunk < 8; ++chunk)
            *reinterpret_cast<uint4*>(stg + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = pk[chunk];
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_5d(&tmO, smem_u32(stg), 0, q_row0, half, h, b);
            tma_store_commit();
          }
        };
        {
          uint4 pk0[8];
          load_half(0, pk0);
          stage_and_store(pk0, 0);
          load_half(1, pk0);
          // the stream's tensor memory is free for the next head's Q.K^T as soon as O has left it
          tc_fence_before();
          mbar_arrive(sbar(s, TMEM_FREE));
          if (lane == 0) XB_TRACE_EV(0x43, rc);
          stage_and_store(pk0, 1);
        }
        if (lane == 0) XB_TRACE_EV(0x44, rc);
      }
    }
    if (lane == 0) tma_store_wait_all();                 // the staging tiles must outlive the stores that read them
  }

  // ------------------------------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) { __nanosleep(1000); }      // let copies in flight land
    if (threadIdx.x == 0 && status) atomicExch(status, static_cast<int>(kDevWaitTimeout));
    __syncthreads();
  }
  if (warp == 17) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------ host side
size_t pair_workspace_bytes(int batch, int hq, int hkv, int q_len) {
  const size_t q_blocks = (static_cast<size_t>(q_len) + 127) / 128;
  const size_t units = static_cast<size_t>(batch) * hkv * q_blocks, items = static_cast<size_t>(batch) * hq * q_blocks;
  return 256 + units * sizeof(PairEntry) + items * sizeof(int32_t);
}

bool pair_path_applies(int hq, int hkv, int k_len) {
  const int group = hq / hkv;
  return group >= 2 && group % 2 == 0 && (k_len + 127) / 128 < static_cast<int>(kNoBlock);
}

// Classifies the group items, runs the pair kernel on those that qualify and leaves in *rest_list the work items
// the general kernel has to compute (their number in the header) provided pair_path_chosen(*header) holds on the
// device; otherwise the pair kernel has done nothing.  The workspace is laid out as
// [header, padding to 256 B][PairEntry x group items][int32 x items].

int block_sparse_attn_pair_launch(const CUtensorMap& tmQ, const CUtensorMap& tmKf, const CUtensorMap& tmVf,
                                  const AttnParams& p, const int32_t* block_idx, const int32_t* block_cnt, void* out,
                                  void* workspace, size_t workspace_bytes, const int32_t** rest_list,
                                  const int** header, int min_share_pct, int* status, cudaStream_t stream) {
  if (workspace_bytes < pair_workspace_bytes(p.batch, p.hq, p.hkv, p.q_len)) return XATTN_B200_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0) return XATTN_B200_ERR_ARG;
  const long long units_ll = static_cast<long long>(p.batch) * p.hkv * p.q_blocks;
  if (units_ll > 0x7fffffffLL) return XATTN_B200_ERR_LIMIT;
  const int units = static_cast<int>(units_ll);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int* counter = reinterpret_cast<int*>(ws);
  PairEntry* list = reinterpret_cast<PairEntry*>(ws + 256);
  int32_t* rest = reinterpret_cast<int32_t*>(ws + 256 + static_cast<size_t>(units) * sizeof(PairEntry));
  // the output as [64 columns, rows, 2 column halves, heads, batch]: a store box is 32 rows of one 64-column half
  CUtensorMap tmO;
  int rc;
  if ((rc = make_qkv_map(&tmO, out, p.q_len, p.hq, p.batch, p.osb, p.osh, p.osl, 32, 1))) return rc;
  if (cudaMemsetAsync(counter, 0, 32, stream) != cudaSuccess) return XATTN_B200_ERR_CUDA;
  pair_classify_kernel<<<(units + 255) / 256, 256, 0, stream>>>(block_idx, block_cnt, p.batch, p.hq, p.hkv, p.q_blocks,
                                                               p.list_k_blocks, list, counter, rest);
  if ((rc = launch_status())) return rc;
  if (cudaFuncSetAttribute(block_sparse_attn_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem) !=
      cudaSuccess)
    return XATTN_B200_ERR_CUDA;
  const int sms = sm_count();
  const int grid = units < sms ? units : sms;
  // the number of qualifying items is known on the device only: launch for the worst case, a launch whose share
  // of the list is empty ends at once
  for (long long off = 0; off < units; off += static_cast<long long>(grid) * kPairSchedCap) {
    if ((rc = launch_dependent(block_sparse_attn_pair_kernel, dim3(grid), dim3(kPairThreads), kPairSmem, stream, tmQ,
                               tmKf, tmVf, tmO, p, static_cast<const PairEntry*>(list),
                               static_cast<const int*>(counter), static_cast<int>(off), min_share_pct, out, status)))
      return rc;
  }
  *rest_list = rest;
  *header = counter;
  return XATTN_B200_OK;
}

}  // namespace xb
