// Definitions shared by the two block-sparse attention kernels (attention.cu: any list length, one work item
// per (head, query block); attention_pair.cu: lists of one or two blocks that the query heads of a kv group share).
#pragma once
#include <math.h>

#include "host_common.cuh"
#include "sm100_primitives.cuh"

namespace xb {

constexpr int kTile16 = 128 * 128 * 2;     // one 128x128 16-bit tile = two 64-column TMA boxes
constexpr int kHalf16 = kTile16 / 2;

struct AttnParams {
  int batch, hq, hkv, q_len, k_len;
  int q_blocks, list_k_blocks;
  int causal, is_bf16;
  int total_items;
  float scale_log2;
  int64_t osb, osh, osl;
  const int32_t* item_list;     // general kernel: its work items (null: all of them, 0 .. total_items - 1)
  int snake;                    // general kernel: deal the items to the CTAs in alternating direction (sorted list)
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
// status word (which must then point to a device buffer of at least 64 + 16*14*XB_TRACE_CAP bytes).  Roles: 0/5
// loader, 1/6 MMA issuer of stream 0/1, 4 epilogue, softmax warp (stream s, quad q): q == 0 ? 2 + s : 7 + 3*s + q - 1.
#ifdef XB_TRACE
#ifndef XB_TRACE_CAP
#define XB_TRACE_CAP 4096          // records per role; 14 roles, first CTA only
#endif
__device__ __forceinline__ void xb_trace(int* status, uint32_t& n, int role, uint32_t tag, uint32_t val) {
  if (blockIdx.x >= 1 || !status || n >= XB_TRACE_CAP) return;
  unsigned long long* buf = reinterpret_cast<unsigned long long*>(status) + 8 +
                            2ull * XB_TRACE_CAP * role;
  buf[2 * n] = (static_cast<unsigned long long>(tag) << 32) | val;
  buf[2 * n + 1] = static_cast<unsigned long long>(clock64());
  ++n;
}
#define XB_TRACE_EV(tag, val) xb_trace(status, trace_n, trace_role, (tag), (val))
#else
#define XB_TRACE_EV(tag, val) ((void)0)
#endif

template <int N, int kLaunchRegs> __device__ __forceinline__ void reg_set_from() {
  if constexpr (N > kLaunchRegs) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
  if constexpr (N < kLaunchRegs) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// [64 columns, rows, 2 column halves, heads, batch]: one box {64, rows, 2, 1, 1} brings `rows` x 128 columns
// with a single TMA instruction, laid out as two 64-column swizzled halves one after the other (Q: 128 rows,
// K/V: 64-key half tiles).
static inline int make_qkv_map(CUtensorMap* m, const void* base, int len, int heads, int batch, int64_t sb, int64_t sh,
                               int64_t sl, uint32_t box_rows, uint32_t box_halves = 2) {
  const uint64_t dims[5] = {64, (uint64_t)len, 2, (uint64_t)heads, (uint64_t)batch};
  // a dimension of extent 1 never moves: give it a harmless valid stride
  const uint64_t s_h = heads > 1 ? (uint64_t)sh * 2 : 256, s_b = batch > 1 ? (uint64_t)sb * 2 : 256;
  const uint64_t str[4] = {(uint64_t)sl * 2, 128, s_h, s_b};
  const uint32_t box[5] = {64, box_rows, box_halves, 1, 1};
  return make_tmap_16bit(m, base, 5, dims, str, box);
}


// ---------------------------------------------------------------- split between the pair and the general kernel
// Workspace header, in 32-bit words: [0] length of the pair list, [1] length of the list of items left to the
// general kernel, [2..3] / [4..5] 64-bit totals of the blocks listed by all items / by the items on the pair list.
constexpr int kPairRestCount = 1, kPairTotalAll = 2, kPairTotalTaken = 4;
constexpr int kPairMinSharePct = 92;

// The split into two kernels costs a second kernel tail, so it pays only when nearly all the work goes to the pair
// kernel: measured on Llama-3.1-8B shapes, 95 % of the blocks on the pair list made the call 8 % faster, 89 % left
// it unchanged and 66 % made it 11 % slower.  Both kernels evaluate this after the classify kernel has finished
// and so agree: below the mark (kPairMinSharePct unless the caller set another, see pair_min_share_pct) the pair
// kernel returns at once and the general kernel computes every item.
__device__ __forceinline__ bool pair_path_chosen(const int* header, int min_share_pct) {
  const unsigned long long all = *reinterpret_cast<const volatile unsigned long long*>(header + kPairTotalAll);
  const unsigned long long taken = *reinterpret_cast<const volatile unsigned long long*>(header + kPairTotalTaken);
  return taken * 100ull >= all * static_cast<unsigned long long>(min_share_pct) && taken > 0;
}

}  // namespace xb
