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
//   warps 0-3   softmax of stream 0  } one thread per query row.  A block is taken as two halves of 64 keys, each
//   warps 4-7   softmax of stream 1  } an online-softmax step: the half's scores come out of TMEM once (two
//                                      32-column loads in flight) and stay in registers for the row max (8
//                                      independent chains) and the exp2; P packed to 16-bit goes back into S
//                                      columns already read; lazy rescale of O only when the max grew by more
//                                      than 2^8; the row sum of the item's last block goes to shared memory for
//                                      the epilogue
//   warps 8-11  epilogue of both streams: O / l from TMEM -> global memory, hands the O buffer back
//   warps 12,14 TMA loader of stream 0 / 1 (lane 0 issues): Q, then K_j, V_j in list order, one TMA
//               instruction per 128x128 tile
//   warps 13,15 (1 thread each) tcgen05 issuer of stream 0 / 1: S = Q K^T (operands in shared memory), then
//               O += P V (P from TMEM, V from shared memory as an MN-major operand)
//
// Lists are walked from the last entry (the diagonal block when causal, which usually holds the row
// maximum) to the first, so the running maximum settles at the first block and O is rarely rescaled.
// The kernel is a template over how a stream walks a 128-key block (see kHalfModeMinBlocksX2): as one block
// (K and V as 32 KiB tiles, one Q.K^T per block: the shortest chain per item, for short lists), or as two
// 64-key halves (S of half h in its own 64-column TMEM buffer, so while the softmax warpgroup works on one half
// the tensor pipe computes the other half's S and the previous half's P.V; K and V as four 16 KiB half-tiles
// per block: for long lists).  Every CTA picks one of the two from its own list lengths.
// TMEM columns: [0,128) S of stream 0 (two 64-column halves in half mode), [128,256) S of stream 1,
// [256,384) O of stream 0, [384,512) O of stream 1.
#include <math.h>

#include <atomic>

#include "attention_common.cuh"

namespace xb {

constexpr int kAttnThreads = 512;
constexpr int kHalfTile = 64 * 128 * 2;    // 64 keys x 128 columns: [2 column halves][64 rows][64 columns]
constexpr int kAttnSmemTiles = kTile16 * 6;                   // Q, K, V per stream
constexpr int kSchedCap = 2048;                               // work items one CTA can schedule
constexpr int kStageBytes = 4 * 32 * 128;                     // per epilogue warp: 32 rows x 64 16-bit columns
constexpr int kAttnSmem = kAttnSmemTiles + 2 * 2 * 128 * 4 /*row sums*/ + 512 /*barriers*/ +
                          3 * kSchedCap * 2 /*schedule*/ + 16 + kStageBytes;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

// Register budget of a role.  The kernel is launched with 512 threads x 128 registers; setmaxnreg moves registers
// between warpgroups inside that allocation (8 x softmax + 4 x epilogue + 4 x load/MMA warps = 2048 per lane).
template <int N> __device__ __forceinline__ void reg_set() {
  if constexpr (N > 128) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
  if constexpr (N < 128) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// Work item t -> (b, h, qb): heaviest query blocks (largest index) first, the heads of a kv group adjacent.
// (Ordering the items kv group by kv group instead, so that all CTAs work on one kv head at a time, was measured:
// +4 % on the 119K-token non-causal mask, -5 % to -15 % on causal masks, whose heavy rows then no longer all
// come first.)
struct Item {
  int b, h, qb;
  size_t row;
};
__device__ __forceinline__ Item decode_item(const AttnParams& p, int t) {
  Item it;
  if (p.item_list) t = __ldg(p.item_list + t);
  it.h = t % p.hq;
  const int rest = t / p.hq;
  it.b = rest % p.batch;
  it.qb = p.q_blocks - 1 - rest / p.batch;
  it.row = (static_cast<size_t>(it.b) * p.hq + it.h) * p.q_blocks + it.qb;
  return it;
}
// Work slot of this CTA's i-th item and the number of its items.  Plain dealing: slot i * G + blockIdx.x.  With
// `snake` (the item list is sorted by list length, longest first) odd rows of the deal run backwards, so that no
// CTA gets the longest item of every row: the loads of the CTAs then differ by about one item of the first row.
__device__ __forceinline__ int item_slot(const AttnParams& p, int i, int G) {
  const int c = (p.snake && (i & 1)) ? G - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
  return i * G + c;
}
__device__ __forceinline__ int local_item_count(const AttnParams& p, int G) {
  const int full = p.total_items / G, rem = p.total_items % G;
  const int c = (p.snake && (full & 1)) ? G - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
  return full + (c < rem ? 1 : 0);
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

// kHalf selects how a stream walks a 128-key block: as two 64-key halves with their own S buffers (softmax of
// one half overlaps the MMAs of the other: 62 % of the dense bf16 peak on long lists) or as one block (fewer
// instructions and barriers: better when a row lists only a handful of blocks).  The kernel sums the CTA's
// block counts while it builds the schedule and calls the body meant for its average list length, so the
// choice needs no host synchronisation.
// twice the average number of listed blocks per non-empty item from which the half-block body pays off
// (random masks with n blocks per row, 16 heads x 16K, full / half body in TFLOP/s: n=3 583-596 / 532-542,
// n=4 637-651 / 645-663, n=6 691-708 / 756-771, n=8 726-739 / 818-824; the 32K Llama mask with its masked diagonal
// blocks, 2.5 blocks per row: 676 / 484)
constexpr int kHalfModeMinBlocksX2 = 7;
template <bool kHalf>
__device__ __forceinline__ void attn_cta(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                                         const CUtensorMap& tmKf, const CUtensorMap& tmVf, const AttnParams& p,
                                         const int32_t* __restrict__ block_idx, void* __restrict__ out, int* status) {
  // Shared memory takes nearly the whole L1, so a register spilled to local memory costs an L2 round trip:
  // the split below is the one with the fewest spills ptxas reports for this kernel (48 bytes, in cold paths).
#ifdef XB_A_SM
  constexpr int kRegSoftmax = XB_A_SM, kRegEpilogue = XB_A_EP, kRegLoadMma = XB_A_LM;
#else
  constexpr int kRegSoftmax = 152, kRegEpilogue = 112, kRegLoadMma = 96;
#endif
  static_assert(8 * kRegSoftmax + 4 * kRegEpilogue + 4 * kRegLoadMma <= 16 * 128, "register budget of the roles");
  extern __shared__ __align__(1024) uint8_t smem[];
  // tiles: [stream][Q, K, V]
  float* s_l = reinterpret_cast<float*>(smem + kAttnSmemTiles);          // [stream][2][128] final row sums
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kAttnSmemTiles + 2 * 2 * 128 * 4);
  // per stream s: NBAR barriers at bars[NBAR*s + ...].  H_* : the four half-tile slots of a block
  // (0: keys 0-63 of K, 1: keys 64-127 of K, 2: keys 0-63 of V, 3: keys 64-127 of V); S_FULL/P_READY: per half
  enum { Q_FULL = 0, Q_EMPTY, H_FULL, H_EMPTY = H_FULL + 4, S_FULL = H_EMPTY + 4, P_READY = S_FULL + 2,
         O_FULL = P_READY + 2, O_EMPTY, PV_DONE, NBAR };
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int s, int which) -> uint32_t { return bar0 + 8u * (NBAR * s + which); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
#ifdef XB_TRACE
  uint32_t trace_n = 0;
  const int trace_role = warp < 8 ? ((warp & 3) == 0 ? 2 + (warp >> 2) : 7 + 3 * (warp >> 2) + (warp & 3) - 1)
                                  : (warp < 12 ? 4 : (warp == 12 ? 0 : (warp == 13 ? 1 : (warp == 14 ? 5 : 6))));
#endif

  // schedule table, built by the kernel before it picked this instantiation
  uint16_t* sch_cnt = reinterpret_cast<uint16_t*>(smem + kAttnSmemTiles + 2 * 2 * 128 * 4 + 512);
  uint16_t* sch_seq0 = sch_cnt + kSchedCap;
  uint16_t* sch_seq1 = sch_seq0 + kSchedCap;
  int* sch_total = reinterpret_cast<int*>(sch_seq1 + kSchedCap);
  uint8_t* stage_base = reinterpret_cast<uint8_t*>(sch_total) + 16;     // 16-byte aligned (sch_total: 2 ints)
  const int G = gridDim.x;
  const int n_local = local_item_count(p, G);                       // host guarantees <= kSchedCap
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s)
      for (int w = 0; w < NBAR; ++w)
        mbar_init(bar(s, w), (w == P_READY || w == P_READY + 1 || w == O_EMPTY) ? 128 : 1);
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
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
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
    reg_set<kRegLoadMma>();
    const int s = (warp - 12) >> 1;                   // stream of this warp
    uint8_t* tiles = smem + s * 3 * kTile16;          // Q, K, V tiles of the stream
    if ((warp & 1) == 0) {
      // ---------------------------------------------------------------- TMA loader of stream s (lane 0 issues)
      const int n_items = sch.n_seq[s];
      uint32_t bc = 0;
      int ok = 1;
      // list window of the first item; the next item's window is fetched while the current one is loaded
      Item it = decode_item(p, n_items > 0 ? item_slot(p, sch.seq[s][0], G) : 0);
      int n = n_items > 0 ? sch.cnt[sch.seq[s][0]] : 0;
      int win = n_items > 0 ? list_window(p, block_idx, it.row, n, 0, lane) : 0;
      for (int m = 0; m < n_items && ok; ++m) {
        Item nit = it;
        int nn = 0, nwin = 0;
        if (m + 1 < n_items) {
          const int i2 = sch.seq[s][m + 1];
          nit = decode_item(p, item_slot(p, i2, G));
          nn = sch.cnt[i2];
          nwin = list_window(p, block_idx, nit.row, nn, 0, lane);
        }
        const int hkv = it.h / group;
        if (lane == 0) {
          if (mbar_wait(bar(s, Q_EMPTY), (m & 1) ^ 1, abort_flag)) {
            XB_TRACE_EV(0x10, m);
            mbar_expect_tx(bar(s, Q_FULL), kTile16);
            tma_load_5d(smem_u32(tiles), &tmQ, bar(s, Q_FULL), 0, it.qb * 128, 0, it.h, it.b);
            // the stream has one Q buffer, so the next item's Q can only be loaded when this item's last S is
            // done: pull it into L2 now so that load does not wait on HBM
            if (m + 1 < n_items) tma_prefetch_l2_5d(&tmQ, 0, nit.qb * 128, 0, nit.h, nit.b);
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
          if constexpr (kHalf) {
          if (lane == 0 && ok) {
#pragma unroll
            for (int slot = 0; slot < 4; ++slot) {
              if (!mbar_wait(bar(s, H_EMPTY + slot), (bc & 1) ^ 1, abort_flag)) { ok = 0; break; }
              XB_TRACE_EV(0x12 + (slot >> 1), bc * 2 + (slot & 1));
              mbar_expect_tx(bar(s, H_FULL + slot), kHalfTile);
              tma_load_5d(smem_u32(tiles + kTile16 + slot * kHalfTile), slot < 2 ? &tmK : &tmV, bar(s, H_FULL + slot), 0,
                          k0 + (slot & 1) * 64, 0, hkv, it.b);
            }
          }
          } else {
          if (lane == 0 && ok) {
            if (mbar_wait(bar(s, H_EMPTY), (bc & 1) ^ 1, abort_flag)) {
              XB_TRACE_EV(0x12, bc);
              mbar_expect_tx(bar(s, H_FULL), kTile16);
              tma_load_5d(smem_u32(tiles + kTile16), &tmKf, bar(s, H_FULL), 0, k0, 0, hkv, it.b);
            } else {
              ok = 0;
            }
            if (ok && mbar_wait(bar(s, H_EMPTY + 2), (bc & 1) ^ 1, abort_flag)) {
              XB_TRACE_EV(0x13, bc);
              mbar_expect_tx(bar(s, H_FULL + 2), kTile16);
              tma_load_5d(smem_u32(tiles + 2 * kTile16), &tmVf, bar(s, H_FULL + 2), 0, k0, 0, hkv, it.b);
            } else {
              ok = 0;
            }
          }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        it = nit; n = nn; win = nwin;
      }
    } else if (lane == 0) {
      // ---------------------------------------------------------------- MMA issuer of stream s
      const uint32_t idesc_pv = make_idesc_f16(128, 128, p.is_bf16 != 0, false, true);
      if constexpr (kHalf) {
      const uint32_t qa = smem_u32(tiles), ha = smem_u32(tiles + kTile16);      // Q tile, four half-tile slots
      const uint32_t sd = tmem_base + s * 128;          // S / P, half h at +64*h
      const uint32_t od = tmem_base + 256 + s * 128;    // O
      // operand descriptors never change: build them once.  Q: [2][128 rows][64]; K half: [2][64 keys][64];
      // V half: [2][64 keys][64], MN-major (16 keys per step = 16 x 128 B rows, next 64 columns 8 KiB away)
      uint64_t dq[8], dk[2][8], dv[2][4];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        dq[k] = smem_desc_sw128(qa + (k >> 2) * kHalf16 + (k & 3) * 32, 16, 1024);
#pragma unroll
        for (int h = 0; h < 2; ++h)
          dk[h][k] = smem_desc_sw128(ha + h * kHalfTile + (k >> 2) * (kHalfTile / 2) + (k & 3) * 32, 16, 1024);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          dv[h][k] = smem_desc_sw128(ha + (2 + h) * kHalfTile + k * 2048, kHalfTile / 2, 1024);
      const uint32_t idesc_qk64 = make_idesc_f16(128, 64, p.is_bf16 != 0, false, false);
      const int n_items = sch.n_seq[s];
      bool ok = true;
      // S of half h of block (m, j): needs Q (first block of an item) and K half h
      auto issue_qk = [&](int m, int n, int j, uint32_t bc, int h) -> bool {
        if (j == 0 && h == 0 && !mbar_wait(bar(s, Q_FULL), m & 1, abort_flag)) return false;
        if (!mbar_wait(bar(s, H_FULL + h), bc & 1, abort_flag)) return false;
        tc_fence_after();
        XB_TRACE_EV(0x20 + h, bc);
        mma_ss(sd + h * 64, dq[0], dk[h][0], idesc_qk64, 0u);
#pragma unroll
        for (int k = 1; k < 8; ++k) mma_ss(sd + h * 64, dq[k], dk[h][k], idesc_qk64, 1u);
        mma_commit(bar(s, H_EMPTY + h));
        mma_commit(bar(s, S_FULL + h));
        if (h == 1 && j == n - 1) mma_commit(bar(s, Q_EMPTY));
        return true;
      };
      // O += P V of half h: needs the softmax of that half and V half h
      auto issue_pv = [&](int m, int n, int j, uint32_t bc, int h) -> bool {
        if (j == 0 && h == 0 && !mbar_wait(bar(s, O_EMPTY), (m & 1) ^ 1, abort_flag)) return false;
        if (!mbar_wait(bar(s, P_READY + h), bc & 1, abort_flag)) return false;
        if (!mbar_wait(bar(s, H_FULL + 2 + h), bc & 1, abort_flag)) return false;
        tc_fence_after();
        XB_TRACE_EV(0x22 + h, bc);
        mma_ts(od, sd + h * 64, dv[h][0], idesc_pv, (j > 0 || h > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 1; k < 4; ++k) mma_ts(od, sd + h * 64 + k * 8, dv[h][k], idesc_pv, 1u);
        mma_commit(bar(s, H_EMPTY + 2 + h));
        mma_commit(bar(s, PV_DONE));
        if (h == 1 && j == n - 1) mma_commit(bar(s, O_FULL));
        return true;
      };
      // order inside the stream: ..., PV(b,0), QK(b+1,0), PV(b,1), QK(b+1,1), PV(b+1,0), ...
      int m = 0, j = 0;
      int n = n_items > 0 ? sch.cnt[sch.seq[s][0]] : 0;
      uint32_t bc = 0;
      if (n_items > 0) ok = issue_qk(m, n, j, bc, 0) && issue_qk(m, n, j, bc, 1);
      while (ok && m < n_items) {
        // the block after (m, j)
        int m2 = m, j2 = j + 1, n2 = n;
        if (j2 == n) { m2 = m + 1; j2 = 0; n2 = m2 < n_items ? sch.cnt[sch.seq[s][m2]] : 0; }
        const bool has_next = m2 < n_items;
        if (!issue_pv(m, n, j, bc, 0)) { ok = false; break; }
        if (has_next && !issue_qk(m2, n2, j2, bc + 1, 0)) { ok = false; break; }
        if (!issue_pv(m, n, j, bc, 1)) { ok = false; break; }
        if (has_next && !issue_qk(m2, n2, j2, bc + 1, 1)) { ok = false; break; }
        m = m2; j = j2; n = n2; ++bc;
      }
      } else {
      const uint32_t idesc_qk = make_idesc_f16(128, 128, p.is_bf16 != 0, false, false);
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
          if (!mbar_wait(bar(s, H_FULL), bc & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          XB_TRACE_EV(0x20, bc);
          mma_ss(sd, dq[0], dk[0], idesc_qk, 0u);
#pragma unroll
          for (int k = 1; k < 8; ++k) mma_ss(sd, dq[k], dk[k], idesc_qk, 1u);
          mma_commit(bar(s, H_EMPTY));
          mma_commit(bar(s, S_FULL));
          if (j == n - 1) mma_commit(bar(s, Q_EMPTY));
          // O += P V, in two steps: keys 0-63 as soon as their half of P is written, so that this half of the
          // product runs while the softmax warpgroup still exponentiates keys 64-127
          if (!mbar_wait(bar(s, P_READY), bc & 1, abort_flag)) { ok = false; break; }
          if (!mbar_wait(bar(s, H_FULL + 2), bc & 1, abort_flag)) { ok = false; break; }
          if (j == 0 && !mbar_wait(bar(s, O_EMPTY), (m & 1) ^ 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          XB_TRACE_EV(0x22, bc);
          mma_ts(od, sd, dv[0], idesc_pv, j > 0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < 4; ++k) mma_ts(od, sd + k * 8, dv[k], idesc_pv, 1u);
          mma_commit(bar(s, PV_DONE));                  // (a softmax warp that has to rescale O waits for this)
          if (!mbar_wait(bar(s, P_READY + 1), bc & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 4; k < 8; ++k) mma_ts(od, sd + k * 8, dv[k], idesc_pv, 1u);
          mma_commit(bar(s, PV_DONE));
          mma_commit(bar(s, H_EMPTY + 2));
          if (j == n - 1) mma_commit(bar(s, O_FULL));
        }
      }
      }
    }
  } else if (warp < 8) {
    // -------------------------------------------------------------------- softmax of stream (warp >> 2)
    reg_set<kRegSoftmax>();
    if constexpr (kHalf) {
    const int s = warp >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t ts0 = tmem_base + s * 128 + lane_bits;         // S / P of this stream, this row (half h at +64h)
    const uint32_t tmem_o = tmem_base + 256 + s * 128 + lane_bits;
    const int k_off = p.k_len - p.q_len;
    const unsigned long long scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
    const int n_items = sch.n_seq[s];
    uint32_t bc = 0;
    bool ok = true;
    Item it = decode_item(p, n_items > 0 ? item_slot(p, sch.seq[s][0], G) : 0);
    int n = n_items > 0 ? sch.cnt[sch.seq[s][0]] : 0;
    int win = n_items > 0 ? list_window(p, block_idx, it.row, n, 0, lane) : 0;
    for (int m = 0; m < n_items && ok; ++m) {
      if (lane == 0) XB_TRACE_EV(0x36, m);
      // the stream's next item: fetch its first list window while this one is processed
      Item nit = it;
      int nn = 0, nwin = 0;
      if (m + 1 < n_items) {
        const int i2 = sch.seq[s][m + 1];
        nit = decode_item(p, item_slot(p, i2, G));
        nn = sch.cnt[i2];
        nwin = list_window(p, block_idx, nit.row, nn, 0, lane);
      }
      const size_t row = it.row;
      const int q_pos = it.qb * 128 + r;
      int row_last = p.k_len - 1;                       // last key position this row may see
      if (p.causal && q_pos + k_off < row_last) row_last = q_pos + k_off;
      float m_used = -INFINITY, l = 0.f;
      int w = win, w_next = list_window(p, block_idx, row, n, 32, lane);
      for (int j = 0; j < n && ok; ++j, ++bc) {
        if (j > 0 && (j & 31) == 0) {
          w = w_next;
          w_next = list_window(p, block_idx, row, n, j + 32, lane);
        }
        const int k0 = __shfl_sync(0xffffffffu, w, j & 31) * 128;
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          const int limit = row_last - k0 - 64 * h;       // columns c <= limit of this half are visible
          const bool masked = __any_sync(0xffffffffu, limit < 63);
          const uint32_t ts = ts0 + h * 64;
          if (lane == 0) XB_TRACE_EV(0x30, bc * 2 + h);
          // waits are made warp-uniform: the tensor-memory loads/stores below are warp-collective
          if (!__all_sync(0xffffffffu, mbar_wait(bar(s, S_FULL + h), bc & 1, abort_flag))) { ok = false; break; }
          tc_fence_after();
          if (lane == 0) XB_TRACE_EV(0x31, bc * 2 + h);
          // ---- pass 1: row maximum over the 64 columns, 8 chains of 3-input max, both loads in flight
          float mx8[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) mx8[q] = -INFINITY;
          // the half's 64 scores stay in registers for both passes: one tensor-memory round trip per half
          uint32_t v0[32], v1[32];
          {
            tmem_ld32(ts, v0);
            tmem_ld32(ts + 32, v1);
            tc_wait_ld();
            if (!masked) {
#pragma unroll
              for (int k = 0; k < 16; ++k) {
                mx8[k & 7] = max3(mx8[k & 7], __uint_as_float(v0[2 * k]), __uint_as_float(v0[2 * k + 1]));
                mx8[(k + 4) & 7] = max3(mx8[(k + 4) & 7], __uint_as_float(v1[2 * k]), __uint_as_float(v1[2 * k + 1]));
              }
            } else {
#pragma unroll
              for (int k = 0; k < 16; ++k) {
                mx8[k & 7] = max3(mx8[k & 7], 2 * k <= limit ? __uint_as_float(v0[2 * k]) : -INFINITY,
                                  2 * k + 1 <= limit ? __uint_as_float(v0[2 * k + 1]) : -INFINITY);
                mx8[(k + 4) & 7] = max3(mx8[(k + 4) & 7], 32 + 2 * k <= limit ? __uint_as_float(v1[2 * k]) : -INFINITY,
                                        33 + 2 * k <= limit ? __uint_as_float(v1[2 * k + 1]) : -INFINITY);
              }
            }
          }
          const float mx = fmaxf(max3(mx8[0], mx8[1], mx8[2]), max3(max3(mx8[3], mx8[4], mx8[5]), mx8[6], mx8[7]));
          const float m_new = fmaxf(m_used, mx * p.scale_log2);
          const bool first = j == 0 && h == 0;
          const bool need = m_new > m_used + kRescaleThreshold || first || (m_used == -INFINITY && m_new > -INFINITY);
          if (__any_sync(0xffffffffu, need)) {
            const float alpha = !need ? 1.f : (m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_new));
            if (!first) {
              // O may be touched once every P.V issued so far for this stream has completed (the half before
              // this one is the latest: its P.V cannot have been issued before this half's P is ready)
              if (lane == 0) XB_TRACE_EV(0x32, bc * 2 + h);
              const uint32_t hq = bc * 2 + h;
              if (!__all_sync(0xffffffffu, mbar_wait(bar(s, PV_DONE), (hq - 1) & 1, abort_flag))) { ok = false; break; }
              tc_fence_after();
#pragma unroll 1
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
          if (lane == 0) XB_TRACE_EV(0x35, bc * 2 + h);
          // ---- pass 2: exp2 of the two 32-column chunks; P chunk c (16 packed columns) overwrites S columns that
          // were read already
          const unsigned long long nmref2 = pack_f32x2(-m_ref, -m_ref);
          unsigned long long ls2[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) ls2[q] = 0ull;     // (+0.f, +0.f)
          auto chunk = [&](const uint32_t (&v)[32], int c) {
            uint32_t pk[16];
            const int lim = limit - 32 * c;
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              float x0 = __uint_as_float(v[2 * k]), x1 = __uint_as_float(v[2 * k + 1]);
              if (masked) {
                x0 = 2 * k <= lim ? x0 : -INFINITY;
                x1 = 2 * k + 1 <= lim ? x1 : -INFINITY;
              }
              float y0, y1;
              unpack_f32x2(fma_f32x2(pack_f32x2(x0, x1), scale2, nmref2), y0, y1);
              const float p0 = fast_exp2(y0), p1 = fast_exp2(y1);
              ls2[k & 3] = add_f32x2(ls2[k & 3], pack_f32x2(p0, p1));
              pk[k] = pack16(p0, p1, p.is_bf16);
            }
            tmem_st16(ts + c * 16, pk);
          };
          chunk(v0, 0);
          chunk(v1, 1);
          {
            float a0, a1;
            unpack_f32x2(add_f32x2(add_f32x2(ls2[0], ls2[1]), add_f32x2(ls2[2], ls2[3])), a0, a1);
            l += a0 + a1;
          }
          if (j == n - 1 && h == 1) s_l[(s * 2 + (m & 1)) * 128 + r] = l;   // for the epilogue of this item
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(bar(s, P_READY + h));
          if (lane == 0) XB_TRACE_EV(0x33, bc * 2 + h);
        }
      }
      it = nit; n = nn; win = nwin;
    }
    } else {
    const int s = warp >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t ts = tmem_base + s * 128 + lane_bits;          // S / P of this stream, this row
    const uint32_t tmem_o = tmem_base + 256 + s * 128 + lane_bits;
    const int k_off = p.k_len - p.q_len;
    const uint32_t s_full = bar(s, S_FULL);
    const int n_items = sch.n_seq[s];
    uint32_t bc = 0;
    bool ok = true;
    Item it = decode_item(p, n_items > 0 ? item_slot(p, sch.seq[s][0], G) : 0);
    int n = n_items > 0 ? sch.cnt[sch.seq[s][0]] : 0;
    int win = n_items > 0 ? list_window(p, block_idx, it.row, n, 0, lane) : 0;
    for (int m = 0; m < n_items && ok; ++m) {
      if (lane == 0) XB_TRACE_EV(0x36, m);
      // the stream's next item: fetch its first list window while this one is processed
      Item nit = it;
      int nn = 0, nwin = 0;
      if (m + 1 < n_items) {
        const int i2 = sch.seq[s][m + 1];
        nit = decode_item(p, item_slot(p, i2, G));
        nn = sch.cnt[i2];
        nwin = list_window(p, block_idx, nit.row, nn, 0, lane);
      }
      const size_t row = it.row;
      const int q_pos = it.qb * 128 + r;
      int row_last = p.k_len - 1;                       // last key position this row may see
      if (p.causal && q_pos + k_off < row_last) row_last = q_pos + k_off;
      float m_used = -INFINITY, l = 0.f;
      int w = win, w_next = list_window(p, block_idx, row, n, 32, lane);
      if (lane == 0) XB_TRACE_EV(0x37, m);
      for (int j = 0; j < n; ++j, ++bc) {
        if (j > 0 && (j & 31) == 0) {
          w = w_next;
          w_next = list_window(p, block_idx, row, n, j + 32, lane);
        }
        const int k0 = __shfl_sync(0xffffffffu, w, j & 31) * 128;
        if (lane == 0) XB_TRACE_EV(0x38, bc);
        if (lane == 0) XB_TRACE_EV(0x30, bc);
        // waits are made warp-uniform: the tensor-memory loads/stores below are warp-collective
        if (!__all_sync(0xffffffffu, mbar_wait(s_full, bc & 1, abort_flag))) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) XB_TRACE_EV(0x31, bc);
        // The block's 128 scores are taken in two halves of 64 columns, each an online-softmax step of its own:
        // one tensor-memory round trip per half (both 32-column loads in flight), the 64 scores stay in registers
        // for the maximum and for the exponentiation, and P of keys 0-63 is handed to the tensor pipe while keys
        // 64-127 are still being worked on.  P (16-bit, two keys per column) of half h goes to columns
        // [32h, 32h + 32), which hold scores that are in registers by then.
        const unsigned long long scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          const int limit = row_last - k0 - 64 * h;       // columns c <= limit of this half are visible
          const bool none_vis = __all_sync(0xffffffffu, limit < 0);
          const bool masked = __any_sync(0xffffffffu, limit < 63);
          if (none_vis) {
            // (the upper half of the diagonal block for the first 64 rows) P = 0, nothing else changes
            uint32_t z[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) z[k] = 0u;
            tmem_st16(ts + h * 32, z);
            tmem_st16(ts + h * 32 + 16, z);
          } else {
            float mx8[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) mx8[q] = -INFINITY;
            uint32_t v0[32], v1[32];
            tmem_ld32(ts + h * 64, v0);
            tmem_ld32(ts + h * 64 + 32, v1);
            tc_wait_ld();
            if (!masked) {
#pragma unroll
              for (int k = 0; k < 16; ++k) {
                mx8[k & 7] = max3(mx8[k & 7], __uint_as_float(v0[2 * k]), __uint_as_float(v0[2 * k + 1]));
                mx8[(k + 4) & 7] = max3(mx8[(k + 4) & 7], __uint_as_float(v1[2 * k]), __uint_as_float(v1[2 * k + 1]));
              }
            } else {
#pragma unroll
              for (int k = 0; k < 16; ++k) {
                mx8[k & 7] = max3(mx8[k & 7], 2 * k <= limit ? __uint_as_float(v0[2 * k]) : -INFINITY,
                                  2 * k + 1 <= limit ? __uint_as_float(v0[2 * k + 1]) : -INFINITY);
                mx8[(k + 4) & 7] = max3(mx8[(k + 4) & 7], 32 + 2 * k <= limit ? __uint_as_float(v1[2 * k]) : -INFINITY,
                                        33 + 2 * k <= limit ? __uint_as_float(v1[2 * k + 1]) : -INFINITY);
              }
            }
            const float mx = fmaxf(max3(mx8[0], mx8[1], mx8[2]), max3(max3(mx8[3], mx8[4], mx8[5]), mx8[6], mx8[7]));
            const float m_new = fmaxf(m_used, mx * p.scale_log2);
            const bool first = j == 0 && h == 0;
            const bool need = m_new > m_used + kRescaleThreshold || first || (m_used == -INFINITY && m_new > -INFINITY);
            if (__any_sync(0xffffffffu, need)) {
              const float alpha = !need ? 1.f : (m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_new));
              if (!first) {
                // O may be touched once every P.V issued so far for this stream has completed (the half before
                // this one is the latest: its P.V cannot have been issued before this half's P is ready)
                if (lane == 0) XB_TRACE_EV(0x32, bc);
                const uint32_t hq = bc * 2 + h;
                if (!__all_sync(0xffffffffu, mbar_wait(bar(s, PV_DONE), (hq - 1) & 1, abort_flag))) { ok = false; break; }
                tc_fence_after();
#pragma unroll 1
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
            if (lane == 0) XB_TRACE_EV(0x35, bc);
            const unsigned long long nmref2 = pack_f32x2(-m_ref, -m_ref);
            unsigned long long ls2[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) ls2[q] = 0ull;     // (+0.f, +0.f)
            auto chunk = [&](const uint32_t (&v)[32], int c) {
              uint32_t pk[16];
              const int lim = limit - 32 * c;
#pragma unroll
              for (int k = 0; k < 16; ++k) {
                float x0 = __uint_as_float(v[2 * k]), x1 = __uint_as_float(v[2 * k + 1]);
                if (masked) {
                  x0 = 2 * k <= lim ? x0 : -INFINITY;
                  x1 = 2 * k + 1 <= lim ? x1 : -INFINITY;
                }
                float y0, y1;
                unpack_f32x2(fma_f32x2(pack_f32x2(x0, x1), scale2, nmref2), y0, y1);
                const float p0 = fast_exp2(y0), p1 = fast_exp2(y1);
                ls2[k & 3] = add_f32x2(ls2[k & 3], pack_f32x2(p0, p1));
                pk[k] = pack16(p0, p1, p.is_bf16);
              }
              tmem_st16(ts + h * 32 + c * 16, pk);
            };
            chunk(v0, 0);
            chunk(v1, 1);
            float a0, a1;
            unpack_f32x2(add_f32x2(add_f32x2(ls2[0], ls2[1]), add_f32x2(ls2[2], ls2[3])), a0, a1);
            l += a0 + a1;
          }
          if (j == n - 1 && h == 1) s_l[(s * 2 + (m & 1)) * 128 + r] = l;   // read by the epilogue once this item's last P.V is done
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(bar(s, P_READY + h));
          if (lane == 0) XB_TRACE_EV(0x33, bc * 2 + h);
        }
        if (!ok) break;
      }
      it = nit; n = nn; win = nwin;
    }
    }
  } else {
    // -------------------------------------------------------------------- epilogue (warps 8-11), both streams
    reg_set<kRegEpilogue>();
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t seen = 0;                 // non-empty items so far: item `seen` runs on stream seen & 1
    bool ok = true;
    for (int i = 0; i < sch.n_local && ok; ++i) {
      const int t = item_slot(p, i, G);
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
      // O leaves tensor memory first, half by half (scaled and packed to 16 bit; the first half is parked in the
      // staging buffer, the second in registers), so that the stream's next item can start accumulating while
      // this one is still being stored
      auto load_half = [&](int half, uint4 (&pk)[8]) {
        uint32_t v0[32], v1[32];
        tmem_ld32(tmem_o + half * 64, v0);
        tmem_ld32(tmem_o + half * 64 + 32, v1);
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
      auto stage = [&](const uint4 (&pk)[8]) {
#pragma unroll
        for (int chunk = 0; chunk < 8; ++chunk)
          *reinterpret_cast<uint4*>(stg + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = pk[chunk];
      };
      auto store_half = [&](int half) {
#pragma unroll
        for (int i2 = 0; i2 < 8; ++i2) {
          const int rr = 4 * i2 + (lane >> 3);                        // row within the warp's 32
          const int chunk = lane & 7;
          const uint4 wv = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((chunk ^ (rr & 7)) << 4));
          const int q_pos_r = q_row0 + rr;
          if (q_pos_r < p.q_len)
            *reinterpret_cast<uint4*>(obase + 2 * static_cast<int64_t>(q_pos_r) * p.osl + half * 128 + chunk * 16) = wv;
        }
      };
      {
        uint4 pk[8];
        load_half(0, pk);
        stage(pk);
        load_half(1, pk);
        tc_fence_before();
        mbar_arrive(bar(s, O_EMPTY));
        __syncwarp();
        store_half(0);
        __syncwarp();
        stage(pk);
        __syncwarp();
        store_half(1);
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

// The kernel: builds the CTA's schedule in shared memory, sums its list lengths and runs the instantiation that
// fits them (a CTA executes only one of the two bodies, so only that one occupies its instruction cache).
__global__ void __launch_bounds__(kAttnThreads, 1)
block_sparse_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmKf,
                         const __grid_constant__ CUtensorMap tmVf, const AttnParams p_in,
                         const int32_t* __restrict__ block_idx, const int32_t* __restrict__ block_cnt,
                         const int32_t* __restrict__ rest_list, const int* __restrict__ pair_header,
                         int pair_min_share, void* __restrict__ out, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  // with a pair kernel in front: the items it left (a list, spread evenly over the CTAs) if it ran, all items if it
  // declined.  In that case this kernel was launched while the pair kernel was running and first waits for it (and
  // so for the classify kernel before it) to end.
  pdl_wait();
  AttnParams p = p_in;
  if (rest_list && pair_path_chosen(pair_header, pair_min_share)) {
    p.item_list = rest_list;
    p.total_items = *reinterpret_cast<const volatile int*>(pair_header + kPairRestCount);
  }
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if ((smem_u32(smem) & 1023u) != 0) {              // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && status) atomicExch(status, static_cast<int>(kDevBadSmemAlign));
    return;
  }
  uint16_t* sch_cnt = reinterpret_cast<uint16_t*>(smem + kAttnSmemTiles + 2 * 2 * 128 * 4 + 512);
  uint16_t* sch_seq0 = sch_cnt + kSchedCap;
  uint16_t* sch_seq1 = sch_seq0 + kSchedCap;
  int* sch_total = reinterpret_cast<int*>(sch_seq1 + kSchedCap);
  const int G = gridDim.x;
  const int n_local = local_item_count(p, G);                       // host guarantees <= kSchedCap
  for (int i = threadIdx.x; i < n_local; i += kAttnThreads) {
    const int c = __ldg(block_cnt + decode_item(p, item_slot(p, i, G)).row);
    sch_cnt[i] = static_cast<uint16_t>(c > 65534 ? 65534 : c);
  }
  __syncthreads();
  if (warp == 0) {
    int running = 0, blocks = 0;
    for (int base = 0; base < n_local; base += 32) {
      const int i = base + lane;
      const int c = i < n_local ? sch_cnt[i] : 0;
      const bool ne = c > 0;
      const unsigned bal = __ballot_sync(0xffffffffu, ne);
      const int k = running + __popc(bal & ((1u << lane) - 1u));
      if (ne) ((k & 1) ? sch_seq1 : sch_seq0)[k >> 1] = static_cast<uint16_t>(i);
      running += __popc(bal);
      blocks += c;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) blocks += __shfl_xor_sync(0xffffffffu, blocks, o);
    if (lane == 0) {
      sch_total[0] = running;
      sch_total[1] = blocks;
    }
  }
  __syncthreads();
  if (2 * sch_total[1] >= kHalfModeMinBlocksX2 * sch_total[0])
    attn_cta<true>(tmQ, tmK, tmV, tmKf, tmVf, p, block_idx, out, status);
  else
    attn_cta<false>(tmQ, tmK, tmV, tmKf, tmVf, p, block_idx, out, status);
}

// ------------------------------------------------------------------------------------------------ item order
// Orders the work items kv head by kv head and, inside a kv head, by list length, longest first; the attention
// kernel then deals that list to its CTAs in rows of gridDim.x, in alternating direction.  Two effects, both for
// masks without an order of their own (non-causal video-diffusion masks: rows list 5 to 891 of 931 blocks, anywhere
// in the sequence):
//  * all CTAs work on one kv head at a time and finish it together (every row of the deal holds items of similar
//    length), so the K/V tiles they gather come from that head's tensors only -- 61 MB at 119K tokens, which stay in
//    L2, where the natural order walks all 24 heads at once (1.46 GB) and re-reads every tile from HBM: measured on
//    random 26-block lists at 119K tokens, 662 TFLOP/s with 24 heads against 914 with two;
//  * no CTA gets the longest item of every row.
// One CTA per (batch, kv head) sorts that head's items with a counting sort (lengths above kOrderBuckets - 1 share
// the first bucket; the order inside a bucket is as the atomics fall, which changes nothing in the result) and
// writes them into the head's segment of the list.
constexpr int kOrderBuckets = 2048;
constexpr int kOrderThreads = 1024;
__global__ void __launch_bounds__(kOrderThreads, 1)
attn_order_kernel(const AttnParams p, const int32_t* __restrict__ block_cnt, int32_t* __restrict__ sorted) {
  __shared__ int hist[kOrderBuckets];
  __shared__ int warp_sum[kOrderThreads / 32];
  pdl_launch_dependents();            // the attention kernel may take its place; it waits for this grid to end
  const int tid = threadIdx.x;
  const int group = p.hq / p.hkv;
  const int b = blockIdx.x / p.hkv, g = blockIdx.x % p.hkv;
  const int n_seg = group * p.q_blocks;                                  // items of this (batch, kv head)
  const size_t row0 = (static_cast<size_t>(b) * p.hq + static_cast<size_t>(g) * group) * p.q_blocks;
  int32_t* seg = sorted + static_cast<size_t>(blockIdx.x) * n_seg;
  for (int i = tid; i < kOrderBuckets; i += kOrderThreads) hist[i] = 0;
  __syncthreads();
  // item j of the segment: query head g * group + j / q_blocks, query block j % q_blocks -- the count array's own
  // order.  The bucket index grows as the list gets shorter.
  auto bucket = [&](int j) {
    const int c = __ldg(block_cnt + row0 + j);
    return kOrderBuckets - 1 - (c < 0 ? 0 : (c > kOrderBuckets - 1 ? kOrderBuckets - 1 : c));
  };
  for (int j = tid; j < n_seg; j += kOrderThreads) atomicAdd(&hist[bucket(j)], 1);
  __syncthreads();
  // exclusive prefix over the buckets, two per thread
  const int h0 = hist[2 * tid], h1 = hist[2 * tid + 1];
  int incl = h0 + h1;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if ((tid & 31) >= o) incl += v;
  }
  if ((tid & 31) == 31) warp_sum[tid >> 5] = incl;
  __syncthreads();
  if (tid < 32) {
    int w = warp_sum[tid];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, w, o);
      if (tid >= o) w += v;
    }
    warp_sum[tid] = w;                 // inclusive over the warps
  }
  __syncthreads();
  const int base = ((tid >> 5) > 0 ? warp_sum[(tid >> 5) - 1] : 0) + incl - h0 - h1;
  __syncthreads();
  hist[2 * tid] = base;                // from here on: the next free position of the bucket
  hist[2 * tid + 1] = base + h0;
  __syncthreads();
  for (int j = tid; j < n_seg; j += kOrderThreads) {
    const int h = g * group + j / p.q_blocks, qb = j % p.q_blocks;
    // the attention kernel's item numbering (decode_item): t = ((q_blocks - 1 - qb) * batch + b) * hq + h
    seg[atomicAdd(&hist[bucket(j)], 1)] = ((p.q_blocks - 1 - qb) * p.batch + b) * p.hq + h;
  }
}

size_t order_workspace_bytes(int batch, int hq, int q_len) {
  return static_cast<size_t>(batch) * hq * ((static_cast<size_t>(q_len) + 127) / 128) * sizeof(int32_t);
}

size_t pair_workspace_bytes(int batch, int hq, int hkv, int q_len);
bool pair_path_applies(int hq, int hkv, int k_len);
int block_sparse_attn_pair_launch(const CUtensorMap& tmQ, const CUtensorMap& tmKf, const CUtensorMap& tmVf,
                                  const AttnParams& p, const int32_t* block_idx, const int32_t* block_cnt, void* out,
                                  void* workspace, size_t workspace_bytes, const int32_t** rest_list,
                                  const int** header, int min_share_pct, int* status, cudaStream_t stream);

// Share (per cent) of a call's listed blocks that must qualify for the pair kernel before the call is split; a
// process-wide setting, read when a call is enqueued.  0: split whenever anything qualifies; > 100: never.
static std::atomic<int> g_pair_min_share{kPairMinSharePct};
int pair_min_share_pct(int set_to) {
  return set_to < 0 ? g_pair_min_share.load() : g_pair_min_share.exchange(set_to);
}

size_t block_sparse_attn_workspace_bytes(int batch, int hq, int hkv, int q_len, int k_len) {
  if (batch < 1 || hq < 1 || hkv < 1 || hq % hkv != 0 || q_len < 1 || k_len < 1) return 0;
  const size_t order = order_workspace_bytes(batch, hq, q_len);
  const size_t pair = pair_path_applies(hq, hkv, k_len) ? pair_workspace_bytes(batch, hq, hkv, q_len) : 0;
  return pair > order ? pair : order;
}

// With a workspace a causal call (with an even number >= 2 of query heads per kv head) runs in two parts: the group
// items whose heads all list the same one or two blocks go to the pair kernel (attention_pair.cu), everything else
// to the general kernel below, which takes its items from the list the pair path leaves.  A non-causal call with a
// workspace has its items ordered kv head by kv head, longest list first inside a head (attn_order_kernel).  Without a workspace the general kernel
// computes everything in the order of the item numbering (rows from the last query block to the first: under a
// causal mask that is longest first already).
int block_sparse_attn_launch(const void* q, const void* k, const void* v, int dtype, int batch, int hq, int hkv,
                             int q_len, int k_len, int head_dim, int64_t qsb, int64_t qsh, int64_t qsl, int64_t ksb,
                             int64_t ksh, int64_t ksl, int64_t vsb, int64_t vsh, int64_t vsl,
                             const int32_t* block_idx, const int32_t* block_cnt, int causal, float scale, void* out,
                             int64_t osb, int64_t osh, int64_t osl, void* workspace, size_t workspace_bytes,
                             int* status, cudaStream_t stream) {
  if (!q || !k || !v || !out || !block_idx || !block_cnt) return XATTN_B200_ERR_ARG;
  if (dtype != XATTN_B200_BF16 && dtype != XATTN_B200_F16) return XATTN_B200_ERR_ARG;
  if (head_dim != 128 || batch < 1 || hq < 1 || hkv < 1 || hq % hkv != 0 || q_len < 1 || k_len < 1)
    return XATTN_B200_ERR_ARG;
  if (causal && k_len < q_len) return XATTN_B200_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (osl % 8) || (osh % 8) || (osb % 8)) return XATTN_B200_ERR_ARG;
  if (!(scale > 0.f)) return XATTN_B200_ERR_ARG;
  int rc;
  if ((rc = check_sm100())) return rc;
  CUtensorMap tmQ, tmK, tmV, tmKf, tmVf;   // K/V as 64-key half tiles and as full 128-key tiles
  if ((rc = make_qkv_map(&tmQ, q, q_len, hq, batch, qsb, qsh, qsl, 128))) return rc;
  if ((rc = make_qkv_map(&tmK, k, k_len, hkv, batch, ksb, ksh, ksl, 64))) return rc;
  if ((rc = make_qkv_map(&tmV, v, k_len, hkv, batch, vsb, vsh, vsl, 64))) return rc;
  if ((rc = make_qkv_map(&tmKf, k, k_len, hkv, batch, ksb, ksh, ksl, 128))) return rc;
  if ((rc = make_qkv_map(&tmVf, v, k_len, hkv, batch, vsb, vsh, vsl, 128))) return rc;
  AttnParams p;
  p.batch = batch; p.hq = hq; p.hkv = hkv; p.q_len = q_len; p.k_len = k_len;
  p.q_blocks = (q_len + 127) / 128; p.list_k_blocks = (k_len + 127) / 128;
  p.causal = causal ? 1 : 0; p.is_bf16 = dtype == XATTN_B200_BF16 ? 1 : 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.osb = osb; p.osh = osh; p.osl = osl;
  p.item_list = nullptr;
  p.snake = 0;
  if (cudaFuncSetAttribute(block_sparse_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem) !=
      cudaSuccess)
    return XATTN_B200_ERR_CUDA;
  const long long items = static_cast<long long>(batch) * hq * p.q_blocks;
  if (items > 0x7fffffffLL) return XATTN_B200_ERR_LIMIT;
  p.total_items = static_cast<int>(items);
  const int sms = sm_count();
  const int grid = items < sms ? static_cast<int>(items) : sms;
  if ((items + grid - 1) / grid > kSchedCap || p.list_k_blocks > 65534) return XATTN_B200_ERR_LIMIT;
  const int32_t* rest = nullptr;
  const int* pair_header = nullptr;
  const int min_share = g_pair_min_share.load();
  if (workspace && !causal) {
    if (workspace_bytes < order_workspace_bytes(batch, hq, q_len)) return XATTN_B200_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0) return XATTN_B200_ERR_ARG;
    int32_t* sorted = static_cast<int32_t*>(workspace);
    attn_order_kernel<<<batch * hkv, kOrderThreads, 0, stream>>>(p, block_cnt, sorted);
    if ((rc = launch_status())) return rc;
    p.item_list = sorted;
    p.snake = 1;
    return launch_dependent(block_sparse_attn_kernel, dim3(grid), dim3(kAttnThreads), kAttnSmem, stream, tmQ, tmK, tmV,
                            tmKf, tmVf, p, block_idx, block_cnt, static_cast<const int32_t*>(nullptr),
                            static_cast<const int*>(nullptr), min_share, out, status);
  }
  if (workspace && pair_path_applies(hq, hkv, k_len)) {
    if ((rc = block_sparse_attn_pair_launch(tmQ, tmKf, tmVf, p, block_idx, block_cnt, out, workspace, workspace_bytes,
                                            &rest, &pair_header, min_share, status, stream)))
      return rc;
  }
  // (a dependent launch in every case: after the pair kernel, or after whatever kernel produced the block lists)
  return launch_dependent(block_sparse_attn_kernel, dim3(grid), dim3(kAttnThreads), kAttnSmem, stream, tmQ, tmK, tmV,
                          tmKf, tmVf, p, block_idx, block_cnt, rest, pair_header, min_share, out, status);
}

}  // namespace xb
