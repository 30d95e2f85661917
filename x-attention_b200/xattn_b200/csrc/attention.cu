// Phase 3 of the XAttention prefill path: block-sparse FlashAttention forward over 128x128 blocks.
//
// Replaces block_sparse_attn.block_sparse_attn_func (third-party CUDA package; call site
// xattn/src/Xattention.py:377-391).  A work item is one (batch, head, 128-row query block) with its
// ascending list of kept key blocks.  The kernel is persistent (one CTA per SM) and pipelines work items:
// while the softmax / P.V / output store of one item run, the Q tile and the first K/V tiles of the next
// item are already in flight and its first Q.K^T is issued.  Mask rows are short (often 2-10 blocks), so
// hiding the per-item prologue and epilogue matters as much as the inner loop.
//
//   warps 0-3   softmax, one thread per query row: S from TMEM -> registers, token-level causal / tail mask,
//               running max with lazy rescale of O (only when the max grew by more than 2^8), exp2, P packed
//               to 16-bit back into the S columns; the row sum of the item's last block goes to shared memory
//   warps 4-7   epilogue: O / l from TMEM -> global memory, then hands the O buffer back
//   warp 8      (1 thread) TMA: Q tile per item (2 buffers), K and V tiles through one 5-deep ring
//   warp 9      (1 thread) tcgen05: S = Q K^T (operands in shared memory) into one of two TMEM buffers, issued
//               one block ahead of O += P V (P read from TMEM, V from shared memory as an MN-major operand)
//
// TMEM columns: [0,128) S0/P0, [128,256) S1/P1, [256,384) O0, [384,512) O1.
#include <math.h>

#include "host_common.cuh"
#include "sm100_primitives.cuh"

namespace xb {

constexpr int kAttnThreads = 384;
constexpr int kRing = 5;                   // K and V tiles alternate through one ring
constexpr int kTile16 = 128 * 128 * 2;     // one 128x128 16-bit tile = two 64-column TMA boxes
constexpr int kHalf16 = kTile16 / 2;
constexpr int kAttnSmemTiles = kTile16 * (2 + kRing);
constexpr int kAttnSmem = kAttnSmemTiles + 4 * 128 * 4 /*row sums*/ + 256 /*barriers*/;
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

__global__ void __launch_bounds__(kAttnThreads, 1)
block_sparse_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const AttnParams p,
                         const int32_t* __restrict__ block_idx, const int32_t* __restrict__ block_cnt,
                         void* __restrict__ out, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;                               // [2] tiles
  uint8_t* sKV = smem + 2 * kTile16;                // [kRing] tiles
  float* s_l = reinterpret_cast<float*>(smem + kAttnSmemTiles);          // [4][128] final row sums
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kAttnSmemTiles + 4 * 128 * 4);
  const uint32_t q_full0 = smem_u32(bars);                  // [2]
  const uint32_t q_empty0 = smem_u32(bars + 2);             // [2]
  const uint32_t kv_full0 = smem_u32(bars + 4);             // [kRing]
  const uint32_t kv_empty0 = smem_u32(bars + 4 + kRing);    // [kRing]
  const uint32_t s_full0 = smem_u32(bars + 4 + 2 * kRing);  // [2]
  const uint32_t p_ready0 = smem_u32(bars + 6 + 2 * kRing); // [2]
  const uint32_t o_full0 = smem_u32(bars + 8 + 2 * kRing);  // [2]
  const uint32_t o_empty0 = smem_u32(bars + 10 + 2 * kRing);// [2]
  const uint32_t pv_done = smem_u32(bars + 12 + 2 * kRing);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13 + 2 * kRing);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if ((smem_u32(smem) & 1023u) != 0) {              // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && status) atomicExch(status, static_cast<int>(kDevBadSmemAlign));
    return;
  }

  if (threadIdx.x == 0) {
    for (int a = 0; a < 2; ++a) {
      mbar_init(q_full0 + 8 * a, 1);
      mbar_init(q_empty0 + 8 * a, 1);
      mbar_init(s_full0 + 8 * a, 1);
      mbar_init(p_ready0 + 8 * a, 128);
      mbar_init(o_full0 + 8 * a, 1);
      mbar_init(o_empty0 + 8 * a, 128);
    }
    for (int s = 0; s < kRing; ++s) {
      mbar_init(kv_full0 + 8 * s, 1);
      mbar_init(kv_empty0 + 8 * s, 1);
    }
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int group = p.hq / p.hkv;
  const int T = p.total_items;

  if (warp >= 8) {
    reg_dec<56>();
    if (warp == 8 && lane == 0) {
      // ---------------------------------------------------------------- TMA loader
      uint32_t itn = 0, rc = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < T && ok; t += gridDim.x) {
        const Item it = decode_item(p, t);
        const int n = __ldg(block_cnt + it.row);
        if (n == 0) continue;
        const int32_t* list = block_idx + it.row * p.list_k_blocks;
        const int hkv = it.h / group;
        const uint32_t qs = itn & 1;
        if (!mbar_wait(q_empty0 + 8 * qs, ((itn >> 1) & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(q_full0 + 8 * qs, kTile16);
        tma_load_4d(smem_u32(sQ + qs * kTile16), &tmQ, q_full0 + 8 * qs, 0, it.qb * 128, it.h, it.b);
        tma_load_4d(smem_u32(sQ + qs * kTile16) + kHalf16, &tmQ, q_full0 + 8 * qs, 64, it.qb * 128, it.h, it.b);
        for (int j = 0; j < n; ++j) {
          const int k0 = __ldg(list + j) * 128;
#pragma unroll
          for (int kv = 0; kv < 2; ++kv, ++rc) {
            const uint32_t slot = rc % kRing;
            if (!mbar_wait(kv_empty0 + 8 * slot, ((rc / kRing) & 1) ^ 1, abort_flag)) { ok = false; break; }
            mbar_expect_tx(kv_full0 + 8 * slot, kTile16);
            const uint32_t dst = smem_u32(sKV + slot * kTile16);
            const CUtensorMap* tm = kv == 0 ? &tmK : &tmV;
            tma_load_4d(dst, tm, kv_full0 + 8 * slot, 0, k0, hkv, it.b);
            tma_load_4d(dst + kHalf16, tm, kv_full0 + 8 * slot, 64, k0, hkv, it.b);
          }
          if (!ok) break;
        }
        ++itn;
      }
    } else if (warp == 9 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      const uint32_t idesc_qk = make_idesc_f16(128, 128, p.is_bf16 != 0, false, false);
      const uint32_t idesc_pv = make_idesc_f16(128, 128, p.is_bf16 != 0, false, true);
      struct Blk { int t, n, j; uint32_t itn, g; bool valid; };
      auto first_item = [&](int t_start, int& t_out, int& n_out) -> bool {
        for (int t = t_start; t < T; t += gridDim.x) {
          const int n = __ldg(block_cnt + decode_item(p, t).row);
          if (n > 0) { t_out = t; n_out = n; return true; }
        }
        return false;
      };
      auto advance = [&](const Blk& c) -> Blk {
        Blk nx = c;
        nx.g = c.g + 1;
        if (c.j + 1 < c.n) { nx.j = c.j + 1; return nx; }
        nx.valid = first_item(c.t + gridDim.x, nx.t, nx.n);
        nx.j = 0;
        nx.itn = c.itn + 1;
        return nx;
      };
      auto issue_qk = [&](const Blk& c) -> bool {
        const uint32_t qs = c.itn & 1;
        if (c.j == 0 && !mbar_wait(q_full0 + 8 * qs, (c.itn >> 1) & 1, abort_flag)) return false;
        const uint32_t rc = 2 * c.g, slot = rc % kRing;
        if (!mbar_wait(kv_full0 + 8 * slot, (rc / kRing) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t d = tmem_base + (c.g & 1) * 128;
        const uint32_t qa = smem_u32(sQ + qs * kTile16), ka = smem_u32(sKV + slot * kTile16);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t o = (k >> 2) * kHalf16 + (k & 3) * 32;
          mma_ss(d, smem_desc_sw128(qa + o, 16, 1024), smem_desc_sw128(ka + o, 16, 1024), idesc_qk, k > 0 ? 1u : 0u);
        }
        mma_commit(kv_empty0 + 8 * slot);
        mma_commit(s_full0 + 8 * (c.g & 1));
        if (c.j == c.n - 1) mma_commit(q_empty0 + 8 * qs);
        return true;
      };
      auto issue_pv = [&](const Blk& c) -> bool {
        const uint32_t ob = c.itn & 1;
        if (c.j == 0 && !mbar_wait(o_empty0 + 8 * ob, ((c.itn >> 1) & 1) ^ 1, abort_flag)) return false;
        if (!mbar_wait(p_ready0 + 8 * (c.g & 1), (c.g >> 1) & 1, abort_flag)) return false;
        const uint32_t rc = 2 * c.g + 1, slot = rc % kRing;
        if (!mbar_wait(kv_full0 + 8 * slot, (rc / kRing) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t pa = tmem_base + (c.g & 1) * 128;
        const uint32_t od = tmem_base + 256 + ob * 128;
        const uint32_t va = smem_u32(sKV + slot * kTile16);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // 16 keys per step: P columns advance by 8 (two 16-bit values per column), V rows by 16 x 128 B
          mma_ts(od, pa + k * 8, smem_desc_sw128(va + k * 2048, kHalf16, 1024), idesc_pv,
                 (c.j > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(kv_empty0 + 8 * slot);
        mma_commit(pv_done);
        if (c.j == c.n - 1) mma_commit(o_full0 + 8 * ob);
        return true;
      };
      Blk cur;
      cur.j = 0; cur.itn = 0; cur.g = 0;
      cur.valid = first_item(blockIdx.x, cur.t, cur.n);
      bool ok = cur.valid ? issue_qk(cur) : true;
      while (cur.valid && ok) {
        const Blk nx = advance(cur);
        if (nx.valid && !issue_qk(nx)) { ok = false; break; }
        if (!issue_pv(cur)) { ok = false; break; }
        cur = nx;
      }
    }
  } else if (warp < 4) {
    // -------------------------------------------------------------------- softmax
    reg_inc<224>();
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    const int k_off = p.k_len - p.q_len;
    uint32_t itn = 0, g = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < T && ok; t += gridDim.x) {
      const Item it = decode_item(p, t);
      const int n = __ldg(block_cnt + it.row);
      if (n == 0) continue;
      const int32_t* list = block_idx + it.row * p.list_k_blocks;
      const int q_pos = it.qb * 128 + r;
      int row_last = p.k_len - 1;                       // last key position this row may see
      if (p.causal && q_pos + k_off < row_last) row_last = q_pos + k_off;
      const uint32_t tmem_o = tmem_base + 256 + (itn & 1) * 128 + lane_bits;
      float m_used = -INFINITY, l = 0.f;
      for (int j = 0; j < n; ++j, ++g) {
        const int k0 = __ldg(list + j) * 128;
        const int limit = row_last - k0;                // columns c <= limit are visible
        // waits are made warp-uniform: the tensor-memory loads/stores below are warp-collective
        if (!__all_sync(0xffffffffu, mbar_wait(s_full0 + 8 * (g & 1), (g >> 1) & 1, abort_flag))) { ok = false; break; }
        tc_fence_after();
        const uint32_t ts = tmem_base + (g & 1) * 128 + lane_bits;
        float s[128];
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          uint32_t v[32];
          tmem_ld32(ts + c4 * 32, v);
          tc_wait_ld();
#pragma unroll
          for (int k = 0; k < 32; ++k) s[c4 * 32 + k] = __uint_as_float(v[k]);
        }
        float mx = -INFINITY;
        if (limit >= 127) {
#pragma unroll
          for (int c = 0; c < 128; ++c) mx = fmaxf(mx, s[c]);
        } else {
#pragma unroll
          for (int c = 0; c < 128; ++c) {
            s[c] = c <= limit ? s[c] : -INFINITY;
            mx = fmaxf(mx, s[c]);
          }
        }
        const float m_new = fmaxf(m_used, mx * p.scale_log2);
        const bool need = m_new > m_used + kRescaleThreshold || (j == 0) || (m_used == -INFINITY && m_new > -INFINITY);
        if (__any_sync(0xffffffffu, need)) {
          const float alpha = !need ? 1.f : (m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_new));
          if (j > 0) {
            // O is touched only after the previous P.V has completed
            if (!__all_sync(0xffffffffu, mbar_wait(pv_done, (g - 1) & 1, abort_flag))) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              uint32_t v[32];
              tmem_ld32(tmem_o + c4 * 32, v);
              tc_wait_ld();
#pragma unroll
              for (int k = 0; k < 32; ++k) v[k] = __float_as_uint(__uint_as_float(v[k]) * alpha);
              tmem_st32(tmem_o + c4 * 32, v);
            }
            tc_wait_st();
          }
          l *= alpha;
          if (need) m_used = m_new;
        }
        const float m_ref = m_used == -INFINITY ? 0.f : m_used;
        float lsum = 0.f;
#pragma unroll
        for (int c4 = 0; c4 < 2; ++c4) {
          uint32_t v[32];
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const int c = c4 * 64 + 2 * k;
            const float p0 = fast_exp2(fmaf(s[c], p.scale_log2, -m_ref));
            const float p1 = fast_exp2(fmaf(s[c + 1], p.scale_log2, -m_ref));
            lsum += p0 + p1;
            v[k] = pack16(p0, p1, p.is_bf16);
          }
          tmem_st32(ts + c4 * 32, v);
        }
        l += lsum;
        if (j == n - 1) s_l[(itn & 3) * 128 + r] = l;   // read by the epilogue once this item's last P.V is done
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(p_ready0 + 8 * (g & 1));
      }
      ++itn;
    }
  } else {
    // -------------------------------------------------------------------- epilogue (warps 4-7)
    reg_dec<104>();
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t itn = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < T && ok; t += gridDim.x) {
      const Item it = decode_item(p, t);
      const int n = __ldg(block_cnt + it.row);
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
      const uint32_t ob = itn & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(o_full0 + 8 * ob, (itn >> 1) & 1, abort_flag))) { ok = false; break; }
      tc_fence_after();
      const float l = s_l[(itn & 3) * 128 + r];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const uint32_t tmem_o = tmem_base + 256 + ob * 128 + lane_bits;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t v[32];
        tmem_ld32(tmem_o + c4 * 32, v);
        tc_wait_ld();
        if (c4 == 3) {
          // every read of this O buffer is done: the MMA thread may start the item after next in it
          tc_fence_before();
          mbar_arrive(o_empty0 + 8 * ob);
        }
        if (store) {
          uint4* dst = reinterpret_cast<uint4*>(orow + c4 * 64);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w;
            w.x = pack16(__uint_as_float(v[q4 * 8 + 0]) * inv, __uint_as_float(v[q4 * 8 + 1]) * inv, p.is_bf16);
            w.y = pack16(__uint_as_float(v[q4 * 8 + 2]) * inv, __uint_as_float(v[q4 * 8 + 3]) * inv, p.is_bf16);
            w.z = pack16(__uint_as_float(v[q4 * 8 + 4]) * inv, __uint_as_float(v[q4 * 8 + 5]) * inv, p.is_bf16);
            w.w = pack16(__uint_as_float(v[q4 * 8 + 6]) * inv, __uint_as_float(v[q4 * 8 + 7]) * inv, p.is_bf16);
            dst[q4] = w;
          }
        }
      }
      ++itn;
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
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

static int make_qkv_map(CUtensorMap* m, const void* base, int len, int heads, int batch, int64_t sb, int64_t sh,
                        int64_t sl) {
  const uint64_t dims[4] = {128, (uint64_t)len, (uint64_t)heads, (uint64_t)batch};
  // a dimension of extent 1 never moves: give it a harmless valid stride
  const uint64_t s_h = heads > 1 ? (uint64_t)sh * 2 : 256, s_b = batch > 1 ? (uint64_t)sb * 2 : 256;
  const uint64_t str[3] = {(uint64_t)sl * 2, s_h, s_b};
  const uint32_t box[4] = {64, 128, 1, 1};
  return make_tmap_16bit(m, base, 4, dims, str, box);
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
  block_sparse_attn_kernel<<<grid, kAttnThreads, kAttnSmem, stream>>>(tmQ, tmK, tmV, p, block_idx, block_cnt, out,
                                                                      status);
  return launch_status();
}

}  // namespace xb
