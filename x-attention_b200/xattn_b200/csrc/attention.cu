// Phase 3 of the XAttention prefill path: block-sparse FlashAttention forward over 128x128 blocks.
//
// Replaces block_sparse_attn.block_sparse_attn_func (third-party CUDA package; call site
// xattn/src/Xattention.py:377-391).  One CTA owns one (batch, head, 128-row query block) and walks
// that row's ascending list of kept key blocks:
//
//   warp 0   (1 thread)  TMA: Q tile once, then K and V tiles of each listed block through 3-deep rings
//   warp 1   (1 thread)  tcgen05: S = Q K^T into one of two TMEM buffers (so the next block's scores are
//                        computed while the softmax of the current one runs), then O += P V with P read
//                        from TMEM and V from shared memory as an MN-major operand
//   warps 2-5            softmax, one thread per query row: TMEM -> registers, token-level causal / tail
//                        mask, running max with lazy rescale of O (only when the max grew by more than
//                        2^8), exp2, P packed to 16-bit back into the score buffer's columns; at the end
//                        O / l -> global memory
//
// TMEM columns: [0,128) S0/P0, [128,256) S1/P1, [256,384) O.
#include <math.h>

#include "host_common.cuh"
#include "sm100_primitives.cuh"

namespace xb {

constexpr int kAttnThreads = 192;
constexpr int kRing = 3;
constexpr int kTile16 = 128 * 128 * 2;     // one 128x128 16-bit tile = two 64-column TMA boxes
constexpr int kHalf16 = kTile16 / 2;
constexpr int kAttnSmem = kTile16 * (1 + 2 * kRing) + 1024 /*barriers*/ + 1024 /*alignment slack*/;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct AttnParams {
  int batch, hq, hkv, q_len, k_len;
  int q_blocks, list_k_blocks;
  int causal, is_bf16;
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

__global__ void __launch_bounds__(kAttnThreads, 1)
block_sparse_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const AttnParams p,
                         const int32_t* __restrict__ block_idx, const int32_t* __restrict__ block_cnt,
                         void* __restrict__ out, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTile16;
  uint8_t* sV = smem + kTile16 * (1 + kRing);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kTile16 * (1 + 2 * kRing));
  const uint32_t q_full = smem_u32(bars);
  const uint32_t k_full0 = smem_u32(bars + 1);
  const uint32_t k_empty0 = smem_u32(bars + 1 + kRing);
  const uint32_t v_full0 = smem_u32(bars + 1 + 2 * kRing);
  const uint32_t v_empty0 = smem_u32(bars + 1 + 3 * kRing);
  const uint32_t s_full0 = smem_u32(bars + 1 + 4 * kRing);      // [2]
  const uint32_t p_ready0 = smem_u32(bars + 3 + 4 * kRing);     // [2]
  const uint32_t pv_done = smem_u32(bars + 5 + 4 * kRing);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6 + 4 * kRing);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // work item: heaviest query blocks (largest index) first, the heads of a kv group adjacent
  const int item = blockIdx.x;
  const int h = item % p.hq;
  const int rest = item / p.hq;
  const int b = rest % p.batch;
  const int qb = p.q_blocks - 1 - rest / p.batch;
  const int hkv = h / (p.hq / p.hkv);
  const size_t row_id = (static_cast<size_t>(b) * p.hq + h) * p.q_blocks + qb;
  const int n = __ldg(block_cnt + row_id);
  const int32_t* list = block_idx + row_id * p.list_k_blocks;
  const int q0 = qb * 128;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kRing; ++s) {
      mbar_init(k_full0 + 8 * s, 1);
      mbar_init(k_empty0 + 8 * s, 1);
      mbar_init(v_full0 + 8 * s, 1);
      mbar_init(v_empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(s_full0 + 8 * a, 1);
      mbar_init(p_ready0 + 8 * a, 128);
    }
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA loader
    if (lane == 0 && n > 0) {
      mbar_expect_tx(q_full, kTile16);
      tma_load_4d(smem_u32(sQ), &tmQ, q_full, 0, q0, h, b);
      tma_load_4d(smem_u32(sQ) + kHalf16, &tmQ, q_full, 64, q0, h, b);
      for (int j = 0; j < n; ++j) {
        const int st = j % kRing;
        const uint32_t ph = (j / kRing) & 1;
        const int k0 = __ldg(list + j) * 128;
        if (!mbar_wait(k_empty0 + 8 * st, ph ^ 1, abort_flag)) break;
        mbar_expect_tx(k_full0 + 8 * st, kTile16);
        tma_load_4d(smem_u32(sK + st * kTile16), &tmK, k_full0 + 8 * st, 0, k0, hkv, b);
        tma_load_4d(smem_u32(sK + st * kTile16) + kHalf16, &tmK, k_full0 + 8 * st, 64, k0, hkv, b);
        if (!mbar_wait(v_empty0 + 8 * st, ph ^ 1, abort_flag)) break;
        mbar_expect_tx(v_full0 + 8 * st, kTile16);
        tma_load_4d(smem_u32(sV + st * kTile16), &tmV, v_full0 + 8 * st, 0, k0, hkv, b);
        tma_load_4d(smem_u32(sV + st * kTile16) + kHalf16, &tmV, v_full0 + 8 * st, 64, k0, hkv, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n > 0) {
      const uint32_t idesc_qk = make_idesc_f16(128, 128, p.is_bf16 != 0, false, false);
      const uint32_t idesc_pv = make_idesc_f16(128, 128, p.is_bf16 != 0, false, true);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_qk = [&](int j) -> bool {
        const int st = j % kRing;
        if (!mbar_wait(k_full0 + 8 * st, (j / kRing) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t d = tmem_base + (j & 1) * 128;
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + st * kTile16);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t o = (k >> 2) * kHalf16 + (k & 3) * 32;
          mma_ss(d, smem_desc_sw128(qa + o, 16, 1024), smem_desc_sw128(ka + o, 16, 1024), idesc_qk, k > 0 ? 1u : 0u);
        }
        mma_commit(k_empty0 + 8 * st);
        mma_commit(s_full0 + 8 * (j & 1));
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n && ok; ++j) {
        if (j + 1 < n && !issue_qk(j + 1)) { ok = false; break; }
        const int st = j % kRing;
        if (!mbar_wait(p_ready0 + 8 * (j & 1), (j >> 1) & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait(v_full0 + 8 * st, (j / kRing) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t pa = tmem_base + (j & 1) * 128;
        const uint32_t va = smem_u32(sV + st * kTile16);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // 16 keys per step: P columns advance by 8 (two 16-bit values per column), V rows by 16 x 128 B
          mma_ts(tmem_o, pa + k * 8, smem_desc_sw128(va + k * 2048, kHalf16, 1024), idesc_pv,
                 (j > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(v_empty0 + 8 * st);
        mma_commit(pv_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    const int q_pos = q0 + r;
    const int k_off = p.k_len - p.q_len;
    int row_last = p.k_len - 1;                       // last key position this row may see
    if (p.causal && q_pos + k_off < row_last) row_last = q_pos + k_off;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      const int k0 = __ldg(list + j) * 128;
      const int limit = row_last - k0;                // columns c <= limit are visible
      // waits are made warp-uniform: the tensor-memory loads/stores below are warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(s_full0 + 8 * (j & 1), (j >> 1) & 1, abort_flag))) { ok = false; break; }
      tc_fence_after();
      const uint32_t ts = tmem_base + (j & 1) * 128 + lane_bits;
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
          if (!__all_sync(0xffffffffu, mbar_wait(pv_done, (j - 1) & 1, abort_flag))) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t v[32];
            tmem_ld32(tmem_o + lane_bits + c4 * 32, v);
            tc_wait_ld();
#pragma unroll
            for (int k = 0; k < 32; ++k) v[k] = __float_as_uint(__uint_as_float(v[k]) * alpha);
            tmem_st32(tmem_o + lane_bits + c4 * 32, v);
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
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(p_ready0 + 8 * (j & 1));
    }
    // epilogue: O / l
    const bool store = q_pos < p.q_len;
    uint8_t* orow = static_cast<uint8_t*>(out) +
                    2 * (static_cast<int64_t>(b) * p.osb + static_cast<int64_t>(h) * p.osh +
                         static_cast<int64_t>(store ? q_pos : 0) * p.osl);
    if (n > 0 && ok) ok = __all_sync(0xffffffffu, mbar_wait(pv_done, (n - 1) & 1, abort_flag));
    tc_fence_after();
    const float inv = (l > 0.f && ok) ? 1.f / l : 0.f;
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
      uint32_t v[32];
      if (n > 0 && ok) {
        tmem_ld32(tmem_o + lane_bits + c4 * 32, v);
        tc_wait_ld();
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) v[k] = 0u;
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
  if (warp == 1) {
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
  block_sparse_attn_kernel<<<static_cast<int>(items), kAttnThreads, kAttnSmem, stream>>>(tmQ, tmK, tmV, p, block_idx,
                                                                                         block_cnt, out, status);
  return launch_status();
}

}  // namespace xb
