// Phase 1 of the XAttention prefill path: antidiagonal block-importance estimate.
//
//   S'[i,j] = scale * sum_{t<S} Q[S*i + S-1-t, :] . K[S*j + t, :]        (one row/col = S tokens)
//   P = row softmax of S' over the row's visible columns
//   attn_sums[qb,kb] = sum of P over the (block/S) x (block/S) cell
//
// Reference: xattn/src/Xattention.py:71-136,174-252 (torch branch) and xattn/src/kernels.py:5-156,
// 197-235 (Triton kernels).  Here the S' matrix never exists in memory:
//
//   est_setup_kernel     per 128-row tile, the range of 256-column tiles that hold visible columns
//   est_gemm_kernel      persistent, warp-specialised tcgen05 GEMM.  One thread streams the
//                        stride-reshaped operands with TMA (the reshape is a 5-D tensor map: a row of
//                        the A tile for K-step t is token S*i+S-1-t, of the B tile token S*j+t), one
//                        thread issues 128x256x16 MMAs into a double-buffered TMEM accumulator, four
//                        warps run the epilogue: per row, max over the tile's visible columns, exp2,
//                        sums over groups of block/S columns.  Output per (row, key block): an
//                        un-normalised partial sum, plus the max it was taken against per (row, tile).
//   est_rowstat_kernel   per row: combine the tiles' maxima and sums into the row's max and 1/sum
//   est_blocksum_kernel  per (query block, key block): normalise and add the block/S rows (and, when a row
//                        spans at most eight tiles, compute the row statistics itself: no est_rowstat launch).
#include <math.h>

#include "host_common.cuh"
#include "sm100_primitives.cuh"

namespace xb {

constexpr int kTileM = 128;
constexpr int kTileN = 256;                                  // widest column tile; EstGeom::tile_n is 256 or 128
constexpr int kTileK = 64;                                   // elements per TMA box row = 128 bytes
constexpr int kStages = 4;
constexpr int kMaxStages = 6;                                // stages of the kernels whose stage is 32 KiB
constexpr int kABytes = kTileM * kTileK * 2;                 // 16 KiB
constexpr int kBBytes = kTileN * kTileK * 2;                 // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;               // 48 KiB
constexpr int kGemmThreads = 192;                            // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue
constexpr int kGemmSmem = kStages * kStageBytes + 1024 /*barriers*/ + 1024 /*alignment slack*/;

struct EstGeom {
  int batch, hq, hkv;
  int S, d_chunks;             // K loop: S * d_chunks steps of 64 elements
  int rows_total, cols_total;  // padded lengths / S
  int rows_valid, cols_valid;  // rows past rows_valid give zeros; causal: columns past cols_valid are hidden
  int rcs;                     // chunk_size / S
  int row_off;                 // (k_chunks - q_chunks) * rcs: global position of row 0
  int causal, left_blank;      // left_blank: columns left of the row's chunk are hidden (torch branch, un-padded K)
  int rbs, kb_total, qb_total;
  int n_mtiles, n_ntiles;
  int tile_n;                  // columns per tile: 256, or 128 when no row sees more than 128 columns
  int band;                    // attn_sums holds only the chunk's own key blocks (left_blank only): row stride bpc
  int bpc;                     // key blocks per chunk
  // scratch layout: a reshaped row keeps m_pitch (max, sum) pairs and p_pitch partial block sums.  Dense: one per
  // column tile / key block of the whole row.  Compact (left_blank: a row only ever touches the tiles of its own
  // chunk): the column tiles [tile_lo, tile_lo + m_pitch) of its row tile, i.e. key blocks from tile_lo * (tile_n /
  // rbs) on -- 16 floats per row instead of 1024 at 128K tokens.
  int compact, m_pitch, p_pitch;
  // lengths that are no multiple of the stride: the row tile of Q' / column tile of K' that holds the ragged last
  // stride group is read from a zero-padded staging copy of just that tile (-1: none)
  int q_tail_mt, k_tail_nt;
  int head_dim;
  float scale_log2;
  // Tile tables of est_setup_kernel computed on the host and carried in the kernel parameters when they are small
  // (tab_n = n_mtiles <= kTabTiles, e.g. 32 row tiles at 32K tokens, 64 at 128K): every kernel copies them into
  // shared memory and est_setup_kernel is not launched.  Layout: tile_lo[kTabTiles], tile_prefix[kTabTiles + 1],
  // pair_lo[kTabTiles / 2], pair_prefix[kTabTiles / 2 + 1].
  int tab_n;
  int tab[64 + 65 + 32 + 33];
};
constexpr int kTabTiles = 64;
constexpr int kTabInts = kTabTiles + (kTabTiles + 1) + kTabTiles / 2 + (kTabTiles / 2 + 1);
constexpr int kTabPrefix = kTabTiles, kTabPairLo = kTabPrefix + kTabTiles + 1, kTabPairPrefix = kTabPairLo + kTabTiles / 2;
static_assert(kTabInts == 64 + 65 + 32 + 33, "EstGeom::tab");

// Visible columns [lo, hi] of reshaped row i (empty when hi < lo).
// causal, torch branch (Xattention.py:191-225): columns [chunk_start, chunk_start + i_local], minus the
// K padding; when K is not padded the slice `[-0:]` at :201 hides everything left of the chunk too.
// causal, Triton (kernels.py:56): columns <= global position of the row.  non-causal: everything.
__host__ __device__ inline void row_bounds(const EstGeom& g, int i, int& lo, int& hi) {
  if (i >= g.rows_valid) { lo = 1; hi = 0; return; }
  if (!g.causal) { lo = 0; hi = g.cols_total - 1; return; }
  const int chunk_start = (i / g.rcs) * g.rcs + g.row_off;
  lo = g.left_blank ? chunk_start : 0;
  hi = g.row_off + i;
  if (hi > g.cols_valid - 1) hi = g.cols_valid - 1;
}

// first column tile / first key block a row tile's scratch rows are indexed from
__host__ __device__ inline int scratch_tile0(const EstGeom& g, int nlo) { return g.compact ? nlo : 0; }
__host__ __device__ inline int scratch_block0(const EstGeom& g, int nlo) {
  return g.compact ? nlo * (g.tile_n / g.rbs) : 0;
}
// column-tile range of row tile mt: first tile and count (the formula of est_setup_kernel, also used by the host
// to size the compact scratch)
__host__ __device__ inline void row_tile_range(const EstGeom& g, int mt, int& first, int& count) {
  // lo(i) and hi(i) never decrease with i, so the tile's column range is [lo(first row), hi(last valid row)]
  const int i0 = mt * 128;
  int i1 = i0 + 128;
  if (i1 > g.rows_total) i1 = g.rows_total;
  if (i1 > g.rows_valid) i1 = g.rows_valid;
  int lo_min = 0, hi_max = -1;
  if (i1 > i0) {
    int lo, hi;
    row_bounds(g, i0, lo_min, hi);
    row_bounds(g, i1 - 1, lo, hi_max);
  }
  if (hi_max < lo_min) {
    first = 0;
    count = 0;
  } else {
    first = lo_min / g.tile_n;
    count = hi_max / g.tile_n - lo_min / g.tile_n + 1;
  }
}

// tile_lo[mt], tile_prefix[mt] (exclusive prefix of tile counts, n_mtiles+1 entries)
__global__ void est_setup_kernel(EstGeom g, int* __restrict__ tile_lo, int* __restrict__ tile_prefix,
                                 int* __restrict__ pair_lo, int* __restrict__ pair_prefix) {
  extern __shared__ int s_cnt[];                  // [n_mtiles] tile counts, then [n_mtiles] first tiles
  int* s_lo = s_cnt + g.n_mtiles;
  for (int mt = threadIdx.x; mt < g.n_mtiles; mt += blockDim.x) {
    row_tile_range(g, mt, s_lo[mt], s_cnt[mt]);
    tile_lo[mt] = s_lo[mt];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int mt = 0; mt < g.n_mtiles; ++mt) {
      tile_prefix[mt] = acc;
      acc += s_cnt[mt];
    }
    tile_prefix[g.n_mtiles] = acc;
    // pairs of row tiles (2p, 2p+1) for the CTA-pair GEMM: the union of their column-tile ranges
    const int n_pairs = (g.n_mtiles + 1) / 2;
    acc = 0;
    for (int pm = 0; pm < n_pairs; ++pm) {
      int lo = 0x7fffffff, hi = -1;
      for (int mt = 2 * pm; mt < 2 * pm + 2 && mt < g.n_mtiles; ++mt)
        if (s_cnt[mt] > 0) {
          lo = s_lo[mt] < lo ? s_lo[mt] : lo;
          hi = s_lo[mt] + s_cnt[mt] - 1 > hi ? s_lo[mt] + s_cnt[mt] - 1 : hi;
        }
      pair_lo[pm] = hi < 0 ? 0 : lo;
      pair_prefix[pm] = acc;
      acc += hi < 0 ? 0 : hi - lo + 1;
    }
    pair_prefix[n_pairs] = acc;
  }
}

// Tables from the kernel parameters (EstGeom::tab) copied into shared memory by the whole CTA; the caller
// synchronises the CTA before the first use.
__device__ __forceinline__ void load_tables(const EstGeom& g, int* s_tab) {
  for (int i = threadIdx.x; i < kTabInts; i += blockDim.x) s_tab[i] = g.tab[i];
}

// Tile number -> (batch*head, row-tile group, column tile).  With `interleave` > 1 (the query heads per kv head)
// the heads of a kv group take the same (row, column) tile one after the other, so that the K tile they share is
// read from DRAM once and found in L2 by the other heads: it matters when the kernel streams its operands from
// HBM (128-column tiles), where K otherwise came from DRAM about twice.
__device__ __forceinline__ void decode_tile(int n_groups, const int* __restrict__ tile_lo,
                                            const int* __restrict__ tile_prefix, int tiles_per_head, int tile,
                                            int& bh, int& mt, int& nt, int interleave = 1) {
  int rem;
  if (interleave > 1) {
    const int hg = tile % interleave;                  // head inside its kv group
    const int t2 = tile / interleave;
    const int bkv = t2 / tiles_per_head;               // batch * kv heads + kv head
    rem = t2 - bkv * tiles_per_head;
    bh = bkv * interleave + hg;
  } else {
    bh = tile / tiles_per_head;
    rem = tile - bh * tiles_per_head;
  }
  int lo = 0, hi = n_groups;     // find mt with prefix[mt] <= rem < prefix[mt+1]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_prefix[mid] <= rem) lo = mid; else hi = mid;
  }
  mt = lo;
  nt = tile_lo[mt] + rem - tile_prefix[mt];
}

// Epilogue of one accumulator tile for one row (thread): softmax statistics and un-normalised block sums of the
// tile's visible columns [clo, chi].  Two passes over the row in tensor memory (maximum, then exp2 and sums over
// groups of RBS columns), the load of the next 32 columns in flight while the current ones are processed; chunks
// that every lane of the warp sees completely skip the per-element range test.  `release` is called once all
// tensor-memory reads of the tile are done.
template <int RBS, typename Release>
__device__ __forceinline__ void est_epilogue_row(const EstGeom& g, uint32_t taddr, int n_chunks, int clo, int chi,
                                                 bool row_ok, float* __restrict__ prow, int kb0,
                                                 float2* __restrict__ mslot, Release release) {
  auto fully_visible = [&](int c8) { return __all_sync(0xffffffffu, clo <= c8 * 32 && chi >= c8 * 32 + 31); };
  // pass 1: row maximum over the visible columns
  float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  {
    auto max_chunk = [&](const uint32_t (&v)[32], int c8) {
      if (fully_visible(c8)) {
#pragma unroll
        for (int k = 0; k < 32; ++k) mx4[k & 3] = fmaxf(mx4[k & 3], __uint_as_float(v[k]));
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          const int c = c8 * 32 + k;
          if (c >= clo && c <= chi) mx4[k & 3] = fmaxf(mx4[k & 3], __uint_as_float(v[k]));
        }
      }
    };
    uint32_t va[32], vb[32];
    tmem_ld32(taddr, va);
#pragma unroll 1
    for (int c8 = 0; c8 < n_chunks; c8 += 2) {
      tc_wait_ld();
      tmem_ld32(taddr + (c8 + 1) * 32, vb);
      max_chunk(va, c8);
      tc_wait_ld();
      if (c8 + 2 < n_chunks) tmem_ld32(taddr + (c8 + 2) * 32, va);
      max_chunk(vb, c8 + 1);
    }
  }
  const float m_scaled = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * g.scale_log2;     // scale > 0
  // pass 2: exp2 and sums over groups of RBS columns
  float tile_sum = 0.f;
  {
    auto sum_chunk = [&](const uint32_t (&v)[32], int c8) {
      float gs[32 / RBS];
#pragma unroll
      for (int q = 0; q < 32 / RBS; ++q) gs[q] = 0.f;
      if (fully_visible(c8)) {
#pragma unroll
        for (int k = 0; k < 32; ++k) gs[k / RBS] += fast_exp2(fmaf(__uint_as_float(v[k]), g.scale_log2, -m_scaled));
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          const int c = c8 * 32 + k;
          const float x = fmaf(__uint_as_float(v[k]), g.scale_log2, -m_scaled);
          gs[k / RBS] += (c >= clo && c <= chi) ? fast_exp2(x) : 0.f;
        }
      }
#pragma unroll
      for (int q = 0; q < 32 / RBS; ++q) tile_sum += gs[q];
      if (row_ok) {
#pragma unroll
        for (int q = 0; q < 32 / RBS; ++q) {
          const int kb = kb0 + c8 * (32 / RBS) + q;
          if (kb < g.kb_total) prow[kb] = gs[q];
        }
      }
    };
    uint32_t va[32], vb[32];
    tmem_ld32(taddr, va);
#pragma unroll 1
    for (int c8 = 0; c8 < n_chunks; c8 += 2) {
      tc_wait_ld();
      tmem_ld32(taddr + (c8 + 1) * 32, vb);
      sum_chunk(va, c8);
      tc_wait_ld();
      if (c8 + 2 < n_chunks) tmem_ld32(taddr + (c8 + 2) * 32, va);
      else release();                                   // the tile's last load has completed
      sum_chunk(vb, c8 + 1);
    }
  }
  if (row_ok) *mslot = make_float2(m_scaled, tile_sum);
}

// Epilogue for geometries in which a reshaped row sees a single 128-column tile (the torch branch with chunks of
// 128 reshaped rows, e.g. 128K tokens at stride 16): the tile's row maximum and row sum ARE the row's, so the
// normalised block sums are finished here -- exp2 against the row maximum, sums over groups of RBS columns kept in
// registers, division by the row sum, and the sum over the RBS rows of a query block taken across lanes -- and
// written to the chunk-band block sums directly.  Neither the per-row scratch nor the two kernels that would read
// it are needed.  `out` is the 128 / RBS floats of this row's query block (written by its first row's lane).
template <int RBS, typename Release>
__device__ __forceinline__ void est_epilogue_row_direct(const EstGeom& g, uint32_t taddr, int clo, int chi,
                                                        float* __restrict__ out, bool write, Release release) {
  constexpr int kChunks = 4, kPer = 32 / RBS;               // 128 columns; key blocks per 32-column chunk
  auto fully_visible = [&](int c8) { return __all_sync(0xffffffffu, clo <= c8 * 32 && chi >= c8 * 32 + 31); };
  float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  {
    uint32_t va[32], vb[32];
    tmem_ld32(taddr, va);
#pragma unroll
    for (int c8 = 0; c8 < kChunks; c8 += 2) {
      tc_wait_ld();
      tmem_ld32(taddr + (c8 + 1) * 32, vb);
      auto max_chunk = [&](const uint32_t (&v)[32], int c) {
        if (fully_visible(c)) {
#pragma unroll
          for (int k = 0; k < 32; ++k) mx4[k & 3] = fmaxf(mx4[k & 3], __uint_as_float(v[k]));
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const int col = c * 32 + k;
            if (col >= clo && col <= chi) mx4[k & 3] = fmaxf(mx4[k & 3], __uint_as_float(v[k]));
          }
        }
      };
      max_chunk(va, c8);
      tc_wait_ld();
      if (c8 + 2 < kChunks) tmem_ld32(taddr + (c8 + 2) * 32, va);
      max_chunk(vb, c8 + 1);
    }
  }
  const float m_scaled = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * g.scale_log2;     // scale > 0
  float blk[kChunks * kPer];
  float row_sum = 0.f;
  {
    uint32_t va[32], vb[32];
    tmem_ld32(taddr, va);
#pragma unroll
    for (int c8 = 0; c8 < kChunks; c8 += 2) {
      tc_wait_ld();
      tmem_ld32(taddr + (c8 + 1) * 32, vb);
      auto sum_chunk = [&](const uint32_t (&v)[32], int c) {
        float gs[kPer];
#pragma unroll
        for (int q = 0; q < kPer; ++q) gs[q] = 0.f;
        if (fully_visible(c)) {
#pragma unroll
          for (int k = 0; k < 32; ++k) gs[k / RBS] += fast_exp2(fmaf(__uint_as_float(v[k]), g.scale_log2, -m_scaled));
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const int col = c * 32 + k;
            const float x = fmaf(__uint_as_float(v[k]), g.scale_log2, -m_scaled);
            gs[k / RBS] += (col >= clo && col <= chi) ? fast_exp2(x) : 0.f;
          }
        }
#pragma unroll
        for (int q = 0; q < kPer; ++q) {
          row_sum += gs[q];
          blk[c * kPer + q] = gs[q];
        }
      };
      sum_chunk(va, c8);
      tc_wait_ld();
      if (c8 + 2 < kChunks) tmem_ld32(taddr + (c8 + 2) * 32, va);
      else release();                                   // the tile's last load has completed
      sum_chunk(vb, c8 + 1);
    }
  }
  // normalise (a row that sees nothing contributes nothing), then add the RBS rows of the query block: they are RBS
  // consecutive lanes
  const float inv = row_sum > 0.f ? 1.f / row_sum : 0.f;
#pragma unroll
  for (int q = 0; q < kChunks * kPer; ++q) {
    float v = blk[q] * inv;
#pragma unroll
    for (int o = 1; o < RBS; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    blk[q] = v;
  }
  if (write) {
#pragma unroll
    for (int q = 0; q < kChunks * kPer; q += 4)
      *reinterpret_cast<float4*>(out + q) = make_float4(blk[q], blk[q + 1], blk[q + 2], blk[q + 3]);
  }
}

template <int RBS, bool DIRECT>
__global__ void __launch_bounds__(kGemmThreads, 1)
est_gemm_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmQt, const __grid_constant__ CUtensorMap tmKt, const EstGeom g,
                const int* tile_lo, const int* tile_prefix, float* __restrict__ partial,
                float2* __restrict__ mtile, float* __restrict__ sums, const uint32_t idesc, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_tab[kTabInts];
  if (g.tab_n) {                                  // (made visible by the __syncthreads() that ends the prologue)
    load_tables(g, s_tab);
    tile_lo = s_tab;
    tile_prefix = s_tab + kTabPrefix;
  }
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // 128-column tiles (every operand tile is used once: the kernel streams Q and K from HBM) take six 32 KiB
  // stages, 256-column tiles four 48 KiB ones: 192 KiB in flight either way
  const int n_stages = g.tile_n == 128 ? kMaxStages : kStages;
  const int stage_bytes = kABytes + g.tile_n * kTileK * 2;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  const uint32_t full0 = smem_u32(bars);                       // [kMaxStages]
  const uint32_t empty0 = smem_u32(bars + kMaxStages);         // [kMaxStages]
  const uint32_t tfull0 = smem_u32(bars + 2 * kMaxStages);     // [2]
  const uint32_t tempty0 = smem_u32(bars + 2 * kMaxStages + 2);// [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_per_head = tile_prefix[g.n_mtiles];
  const int total_tiles = tiles_per_head * g.batch * g.hq;
  const int k_steps = g.S * g.d_chunks;
  const int group = g.hq / g.hkv;
  const int interleave = g.tile_n == 128 ? group : 1;      // streaming case only: see decode_tile

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one thread)
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
        int bh, mt, nt;
        decode_tile(g.n_mtiles, tile_lo, tile_prefix, tiles_per_head, tile, bh, mt, nt, interleave);
        const int b = bh / g.hq, h = bh - b * g.hq;
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % n_stages;
          const uint32_t ph = (it / n_stages) & 1;
          if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag)) break;
          const int t = ks / g.d_chunks;
          const int dc = ks - t * g.d_chunks;
          const uint32_t dstA = smem_u32(smem + s * stage_bytes);
          mbar_expect_tx(full0 + 8 * s, stage_bytes);
          // (the tile that holds a ragged last stride group comes from its zero-padded staging copy)
          const bool qt = mt == g.q_tail_mt, kt = nt == g.k_tail_nt;
          tma_load_5d(dstA, qt ? &tmQt : &tmQ, full0 + 8 * s, dc * kTileK, g.S - 1 - t, qt ? 0 : mt * kTileM, h, b);
          tma_load_5d(dstA + kABytes, kt ? &tmKt : &tmK, full0 + 8 * s, dc * kTileK, t, kt ? 0 : nt * g.tile_n,
                      h / group, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      uint32_t it = 0, local_tile = 0;
      const uint64_t a_desc0 = smem_desc_sw128(smem_u32(smem), 16, 1024);
      const uint64_t b_desc0 = smem_desc_sw128(smem_u32(smem) + kABytes, 16, 1024);
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++local_tile) {
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait(tempty0 + 8 * acc, acc_ph ^ 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kTileN;
        bool ok = true;
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % n_stages;
          const uint32_t ph = (it / n_stages) & 1;
          if (!mbar_wait(full0 + 8 * s, ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          // descriptors differ from the stage-0 ones only in the start-address field (units of 16 bytes)
          const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(s * (stage_bytes >> 4));
          const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(s * (stage_bytes >> 4));
#pragma unroll
          for (int k4 = 0; k4 < kTileK / 16; ++k4)
            mma_ss(d_tmem, a_desc + k4 * 2, b_desc + k4 * 2, idesc, (ks > 0 || k4 > 0) ? 1u : 0u);
          mma_commit(empty0 + 8 * s);          // stage reusable once these MMAs have read it
        }
        if (!ok) break;
        mma_commit(tfull0 + 8 * acc);          // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps, thread = tile row)
    const int quad = warp & 3;                  // TMEM lane quarter this warp may access
    const int r = quad * 32 + lane;
    const int kGroups = g.tile_n / RBS;         // key blocks per tile
    const int n_chunks = g.tile_n / 32;
    uint32_t local_tile = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local_tile) {
      int bh, mt, nt;
      decode_tile(g.n_mtiles, tile_lo, tile_prefix, tiles_per_head, tile, bh, mt, nt, interleave);
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      const int i = mt * kTileM + r;
      int lo, hi;
      row_bounds(g, i, lo, hi);
      const int n0 = nt * g.tile_n;
      const int clo = lo - n0 > 0 ? lo - n0 : 0;
      const int chi = hi - n0 < g.tile_n - 1 ? hi - n0 : g.tile_n - 1;
      // warp-uniform: the tensor-memory loads below are warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * acc, acc_ph, abort_flag))) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * kTileN + (static_cast<uint32_t>(quad * 32) << 16);
      const bool row_ok = i < g.rows_total;
      const size_t rrow = static_cast<size_t>(bh) * g.rows_total + (row_ok ? i : 0);
      const int nlo = tile_lo[mt];
      auto release = [&]() {
        // all TMEM reads of this accumulator are done: hand it back to the MMA thread
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
      };
      if constexpr (DIRECT) {
        // the query block of this row, and its first row's lane as the writer (RBS divides 32)
        const int qb = i / RBS;
        est_epilogue_row_direct<RBS>(g, taddr, clo, chi,
                                     sums + (static_cast<size_t>(bh) * g.qb_total + (qb < g.qb_total ? qb : 0)) * g.bpc,
                                     (lane % RBS) == 0 && qb < g.qb_total, release);
      } else {
        est_epilogue_row<RBS>(g, taddr, n_chunks, clo, chi, row_ok,
                              partial + rrow * g.p_pitch - scratch_block0(g, nlo), nt * kGroups,
                              mtile + rrow * g.m_pitch + nt - scratch_tile0(g, nlo), release);
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give copies and MMAs still in flight time to land before shared/tensor memory is released
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

// The same GEMM on CTA PAIRS (thread-block clusters of 2, tcgen05 cta_group::2): a pair computes a 256x256 tile.
// Each CTA loads its own 128 rows of A and HALF of the tile's 256 columns of B (32 KiB per K step instead of 48),
// the even CTA issues 256x256x16 MMAs that read both CTAs' shared memory, and each CTA finds the accumulator of
// its own 128 rows in its own tensor memory, where its four epilogue warps work exactly as in the single-CTA
// kernel.  The single-CTA kernel is bound by operand bytes in flight per SM (L2 latency x shared-memory
// capacity); the pair moves a third fewer bytes per FLOP and has six 32 KiB stages in flight.
//   full[s]   (even CTA)  1 arrival (its producer's expect_tx of both CTAs' bytes) + the bytes of four TMA loads
//   empty[s]  (each CTA)  1 arrival: the commit of the MMAs that read stage s, delivered to both CTAs
//   tfull[a]  (each CTA)  1 arrival: the commit of a tile's last MMA, delivered to both CTAs
//   tempty[a] (even CTA)  8 arrivals: four epilogue warps of each CTA
constexpr int kPairStages = 6;
constexpr int kPairBBytes = 128 * kTileK * 2;                // this CTA's half of the B tile: 16 KiB
constexpr int kPairStageBytes = kABytes + kPairBBytes;       // 32 KiB
constexpr int kPairSmem = kPairStages * kPairStageBytes + 1024 /*barriers*/ + 1024 /*alignment slack*/;

template <int RBS>
__global__ void __launch_bounds__(kGemmThreads, 1)
est_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKh,
                     const __grid_constant__ CUtensorMap tmQt, const __grid_constant__ CUtensorMap tmKt,
                     const EstGeom g, const int* pair_lo, const int* pair_prefix,
                     float* __restrict__ partial, float2* __restrict__ mtile, const uint32_t idesc, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_tab[kTabInts];
  if (g.tab_n) {                                  // (made visible by the __syncthreads() that ends the prologue)
    load_tables(g, s_tab);
    pair_lo = s_tab + kTabPairLo;
    pair_prefix = s_tab + kTabPairPrefix;
  }
  // the same offset in both CTAs of the pair (the dynamic shared memory of a kernel starts at the same address
  // in every CTA), which the MMA descriptors rely on
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);
  const uint32_t full0 = smem_u32(bars);                            // [kPairStages]
  const uint32_t empty0 = smem_u32(bars + kPairStages);             // [kPairStages]
  const uint32_t tfull0 = smem_u32(bars + 2 * kPairStages);         // [2]
  const uint32_t tempty0 = smem_u32(bars + 2 * kPairStages + 2);    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kPairStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                  // 0: issues the MMAs
  const int pair = blockIdx.x >> 1, n_pairs_grid = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmKh);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();               // barriers of both CTAs are initialised before any remote arrival or copy
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_groups = (g.n_mtiles + 1) / 2;
  const int tiles_per_head = pair_prefix[n_groups];
  const int total_tiles = tiles_per_head * g.batch * g.hq;
  const int k_steps = g.S * g.d_chunks;
  const int group = g.hq / g.hkv;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one thread per CTA)
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = pair; tile < total_tiles && !*abort_flag; tile += n_pairs_grid) {
        int bh, pm, nt;
        decode_tile(n_groups, pair_lo, pair_prefix, tiles_per_head, tile, bh, pm, nt);
        const int b = bh / g.hq, h = bh - b * g.hq;
        const int mt = 2 * pm + static_cast<int>(rank);
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % kPairStages;
          const uint32_t ph = (it / kPairStages) & 1;
          if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag)) break;
          const int t = ks / g.d_chunks;
          const int dc = ks - t * g.d_chunks;
          const uint32_t dstA = smem_u32(smem + s * kPairStageBytes);
          // all four loads of a stage are counted on the even CTA's barrier
          const uint32_t full_even = mapa_shared(full0 + 8 * s, 0);
          if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * kPairStageBytes);
          const bool qt = mt == g.q_tail_mt, kt = nt == g.k_tail_nt;
          tma_load_5d_pair(dstA, qt ? &tmQt : &tmQ, full_even, dc * kTileK, g.S - 1 - t, qt ? 0 : mt * kTileM, h, b);
          tma_load_5d_pair(dstA + kABytes, kt ? &tmKt : &tmKh, full_even, dc * kTileK, t,
                           (kt ? 0 : nt * kTileN) + static_cast<int>(rank) * 128, h / group, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (one thread of the even CTA)
    if (lane == 0 && rank == 0) {
      uint32_t it = 0, local_tile = 0;
      const uint64_t a_desc0 = smem_desc_sw128(smem_u32(smem), 16, 1024);
      const uint64_t b_desc0 = smem_desc_sw128(smem_u32(smem) + kABytes, 16, 1024);
      for (int tile = pair; tile < total_tiles && !*abort_flag; tile += n_pairs_grid, ++local_tile) {
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait(tempty0 + 8 * acc, acc_ph ^ 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kTileN;
        bool ok = true;
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % kPairStages;
          const uint32_t ph = (it / kPairStages) & 1;
          if (!mbar_wait(full0 + 8 * s, ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(s * (kPairStageBytes >> 4));
          const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(s * (kPairStageBytes >> 4));
#pragma unroll
          for (int k4 = 0; k4 < kTileK / 16; ++k4)
            mma_ss_pair(d_tmem, a_desc + k4 * 2, b_desc + k4 * 2, idesc, (ks > 0 || k4 > 0) ? 1u : 0u);
          mma_commit_pair(empty0 + 8 * s, 3);  // stage reusable in both CTAs once these MMAs have read it
        }
        if (!ok) break;
        mma_commit_pair(tfull0 + 8 * acc, 3);  // accumulator complete in both CTAs
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps, thread = tile row)
    const int quad = warp & 3;                  // TMEM lane quarter this warp may access
    const int r = quad * 32 + lane;
    constexpr int kGroups = kTileN / RBS;       // key blocks per tile
    constexpr int n_chunks = kTileN / 32;
    uint32_t local_tile = 0;
    for (int tile = pair; tile < total_tiles; tile += n_pairs_grid, ++local_tile) {
      int bh, pm, nt;
      decode_tile(n_groups, pair_lo, pair_prefix, tiles_per_head, tile, bh, pm, nt);
      const int mt = 2 * pm + static_cast<int>(rank);
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      const int i = mt * kTileM + r;
      int lo, hi;
      row_bounds(g, i < g.rows_total ? i : g.rows_total, lo, hi);   // rows past the end see nothing
      const int n0 = nt * kTileN;
      const int clo = lo - n0 > 0 ? lo - n0 : 0;
      const int chi = hi - n0 < kTileN - 1 ? hi - n0 : kTileN - 1;
      // warp-uniform: the tensor-memory loads below are warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * acc, acc_ph, abort_flag))) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * kTileN + (static_cast<uint32_t>(quad * 32) << 16);
      const bool row_ok = i < g.rows_total;
      const size_t rrow = static_cast<size_t>(bh) * g.rows_total + (row_ok ? i : 0);
      // (compact scratch: both row tiles of a pair lie in one chunk and start at the pair's first column tile)
      const int nlo = pair_lo[pm];
      est_epilogue_row<RBS>(g, taddr, n_chunks, clo, chi, row_ok,
                            partial + rrow * g.p_pitch - scratch_block0(g, nlo), nt * kGroups,
                            mtile + rrow * g.m_pitch + nt - scratch_tile0(g, nlo), [&]() {
                              // all TMEM reads of this accumulator are done: hand it back to the MMA thread of
                              // the even CTA
                              tc_fence_before();
                              __syncwarp();
                              if (lane == 0) mbar_arrive_cluster(mapa_shared(tempty0 + 8 * acc, 0));
                            });
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give copies and MMAs still in flight time to land before shared/tensor memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) { __nanosleep(1000); }
    if (threadIdx.x == 0 && status) atomicExch(status, static_cast<int>(kDevWaitTimeout));
  }
  // neither CTA may release tensor memory, or leave while the other can still signal its barriers
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// Normalisation of the partial sums, as two streaming kernels.
//   est_rowstat_kernel  one thread per reshaped row i:  m_i = max_t m_{i,t},
//                       1/l_i with l_i = sum_t s_{i,t} 2^(m_{i,t} - m_i)      (m, s = per-tile max and sum)
//   est_blocksum_kernel one thread per (query block, key block):
//                       out[qb][kb] = sum_{i in qb} partial[i][kb] * 2^(m_{i,t(kb)} - m_i) / l_i
__global__ void __launch_bounds__(256)
est_rowstat_kernel(const EstGeom g, const int* tile_lo, const int* tile_prefix,
                   const float2* __restrict__ mtile, float2* __restrict__ rowstat, int total_rows) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_rows) return;
  const int i = idx % g.rows_total;
  const int mt = i / kTileM;
  // (the three table entries a row needs come straight from the kernel parameters when the tables are there)
  const int nlo = g.tab_n ? g.tab[mt] : tile_lo[mt];
  const int ncnt = g.tab_n ? g.tab[kTabPrefix + mt + 1] - g.tab[kTabPrefix + mt] : tile_prefix[mt + 1] - tile_prefix[mt];
  const float2* mrow = mtile + static_cast<size_t>(idx) * g.m_pitch + nlo - scratch_tile0(g, nlo);
  float m = -INFINITY, l = 0.f;
  if (i < g.rows_valid) {
    for (int t = 0; t < ncnt; ++t) m = fmaxf(m, mrow[t].x);
    if (m > -INFINITY)
      for (int t = 0; t < ncnt; ++t) {
        const float2 ms = mrow[t];
        if (ms.x > -INFINITY) l += ms.y * exp2f(ms.x - m);
      }
  }
  rowstat[idx] = make_float2(m, l > 0.f ? 1.f / l : 0.f);
}

// VEC consecutive key blocks per thread (4 when kb_total is a multiple of 4: one 16-byte store; they share a tile)
// FUSED: the query block's row statistics are computed here (eight threads per row, one (max, sum) pair each, so
// a row costs one memory round trip) instead of being read from est_rowstat_kernel's output; for geometries whose
// rows span at most eight column tiles.
template <int VEC, bool FUSED>
__global__ void __launch_bounds__(256)
est_blocksum_kernel(const EstGeom g, const int* tile_lo, const int* tile_prefix,
                    const float* __restrict__ partial, const float2* __restrict__ mtile,
                    const float2* __restrict__ rowstat, float* __restrict__ sums) {
  __shared__ float2 s_stat[32];                            // FUSED: (m_i, 1/l_i) of the query block's rows (rbs <= 32)
  const int qb = blockIdx.y, bh = blockIdx.z;
  const int i0 = qb * g.rbs;
  if (FUSED) {
    const int mt_ = i0 / kTileM;
    const int nlo_ = g.tab_n ? g.tab[mt_] : tile_lo[mt_];
    const int ncnt_ = g.tab_n ? g.tab[kTabPrefix + mt_ + 1] - g.tab[kTabPrefix + mt_]
                              : tile_prefix[mt_ + 1] - tile_prefix[mt_];
    int rows_ = g.rows_valid - i0;
    rows_ = rows_ > g.rbs ? g.rbs : rows_;
    const int row = threadIdx.x >> 3, slot = threadIdx.x & 7;
    if (row < g.rbs) {                                     // whole 8-lane groups take the branch together
      float2 ms = make_float2(-INFINITY, 0.f);
      if (row < rows_ && slot < ncnt_)
        ms = mtile[(static_cast<size_t>(bh) * g.rows_total + i0 + row) * g.m_pitch + nlo_ - scratch_tile0(g, nlo_) + slot];
      const unsigned grp = 0xffu << (threadIdx.x & 24);    // the eight lanes of this row
      float m = ms.x;
      m = fmaxf(m, __shfl_xor_sync(grp, m, 1));
      m = fmaxf(m, __shfl_xor_sync(grp, m, 2));
      m = fmaxf(m, __shfl_xor_sync(grp, m, 4));
      const float term = (m > -INFINITY && ms.x > -INFINITY) ? ms.y * exp2f(ms.x - m) : 0.f;
      float l = 0.f;                                       // summed in tile order, as est_rowstat_kernel does
#pragma unroll
      for (int k = 0; k < 8; ++k) l += __shfl_sync(grp, term, (threadIdx.x & 24) + k);
      if (slot == 0) s_stat[row] = make_float2(m, l > 0.f ? 1.f / l : 0.f);
    }
    __syncthreads();
  }
  // band layout: only the key blocks of the query block's own chunk, [cur, cur + bpc)
  const int cur = g.band ? (g.row_off + (i0 / g.rcs) * g.rcs) / g.rbs : 0;
  const int kb_local = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (kb_local >= (g.band ? g.bpc : g.kb_total)) return;
  const int kb = cur + kb_local;
  const int mt = i0 / kTileM;
  const int nlo = g.tab_n ? g.tab[mt] : tile_lo[mt];
  const int ncnt = g.tab_n ? g.tab[kTabPrefix + mt + 1] - g.tab[kTabPrefix + mt] : tile_prefix[mt + 1] - tile_prefix[mt];
  const int gpt = g.tile_n / g.rbs;                       // key blocks per tile (a multiple of 4)
  const int t = kb / gpt;
  float acc[VEC];
#pragma unroll
  for (int q = 0; q < VEC; ++q) acc[q] = 0.f;
  if (t >= nlo && t < nlo + ncnt) {
    const size_t r0 = static_cast<size_t>(bh) * g.rows_total + i0;
    int rows = g.rows_valid - i0;                         // rows past rows_valid contribute nothing
    rows = rows > g.rbs ? g.rbs : rows;
#pragma unroll 2
    for (int row = 0; row < rows; ++row) {
      const float2 st = FUSED ? s_stat[row] : rowstat[r0 + row];
      const float mx = mtile[(r0 + row) * g.m_pitch + t - scratch_tile0(g, nlo)].x;
      const float f = (st.y > 0.f && mx > -INFINITY) ? exp2f(mx - st.x) * st.y : 0.f;
      const float* pp = partial + (r0 + row) * g.p_pitch + kb - scratch_block0(g, nlo);
      if (VEC == 4) {
        const float4 pv = *reinterpret_cast<const float4*>(pp);
        if (f != 0.f) { acc[0] += pv.x * f; acc[1 % VEC] += pv.y * f; acc[2 % VEC] += pv.z * f; acc[3 % VEC] += pv.w * f; }
      } else {
        if (f != 0.f) acc[0] += pp[0] * f;
      }
    }
  }
  float* out = sums + (static_cast<size_t>(bh) * g.qb_total + qb) * (g.band ? g.bpc : g.kb_total) + kb_local;
  if (VEC == 4) *reinterpret_cast<float4*>(out) = make_float4(acc[0], acc[1 % VEC], acc[2 % VEC], acc[3 % VEC]);
  else out[0] = acc[0];
}

// x = hi + mid + lo in bf16; rows widened to 6*D (see the header).
// Rows l >= len_valid are written as zeros (a length rounded up to the stride).
__global__ void split_f32_kernel(const float* __restrict__ x, int heads, int len, int len_valid, int D, int64_t sb,
                                 int64_t sh, int64_t sl, int role, __nv_bfloat16* __restrict__ out, size_t total) {
  for (size_t e = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; e < total;
       e += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int d = static_cast<int>(e % D);
    size_t rest = e / D;
    const int l = static_cast<int>(rest % len);
    rest /= len;
    const int h = static_cast<int>(rest % heads);
    const int b = static_cast<int>(rest / heads);
    const float v = l < len_valid ? x[b * sb + h * sh + l * sl + d] : 0.f;
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
    __nv_bfloat16* o = out + (e / D) * (6 * static_cast<size_t>(D)) + d;
    if (role == 0) {
      o[0] = hi; o[D] = hi; o[2 * D] = mid; o[3 * D] = hi; o[4 * D] = lo; o[5 * D] = mid;
    } else {
      o[0] = hi; o[D] = mid; o[2 * D] = hi; o[3 * D] = lo; o[4 * D] = hi; o[5 * D] = mid;
    }
  }
}

// Zero-padded copy of `n_tokens` tokens starting at `first_token` of every head ([batch, heads, n_tokens, D] 16-bit,
// contiguous): the tile that holds the ragged last stride group, so that the tokens past the end read as the zeros
// the reference pads with (xattn/src/Xattention.py:42-51) instead of the next head's data.  16 bytes per thread.
__global__ void est_tail_kernel(const uint4* __restrict__ src, int64_t sb, int64_t sh, int64_t sl, int heads, int len,
                                int D, int first_token, int n_tokens, uint4* __restrict__ dst, size_t total_vec) {
  const int vec_per_row = D / 8;
  for (size_t e = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; e < total_vec;
       e += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(e % vec_per_row);
    size_t rest = e / vec_per_row;
    const int tok = static_cast<int>(rest % n_tokens);
    rest /= n_tokens;
    const int h = static_cast<int>(rest % heads);
    const int b = static_cast<int>(rest / heads);
    const int t = first_token + tok;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (t < len) v = src[(b * sb + h * sh + static_cast<int64_t>(t) * sl) / 8 + c];
    dst[e] = v;
  }
}

// ------------------------------------------------------------------------------------ host side
struct EstWorkspace {
  size_t off_tile_lo, off_tile_prefix, off_pair_lo, off_pair_prefix, off_rowstat, off_mtile, off_partial;
  size_t off_qtail, off_ktail, total;
};

static int fill_geometry(int batch, int hq, int hkv, int q_len, int k_len, int head_dim, int stride, int block_size,
                         int chunk_size, float scale, int causal, int semantics, EstGeom& g) {
  if (batch < 1 || hq < 1 || hkv < 1 || hq % hkv != 0 || q_len < 1 || k_len < 1) return XATTN_B200_ERR_ARG;
  if (stride != 4 && stride != 8 && stride != 16 && stride != 32) return XATTN_B200_ERR_ARG;
  if (block_size != 128 || chunk_size < block_size || chunk_size % block_size != 0) return XATTN_B200_ERR_ARG;
  if (head_dim < kTileK || head_dim % kTileK != 0) return XATTN_B200_ERR_ARG;
  const int k_pad = (chunk_size - k_len % chunk_size) % chunk_size;
  const int q_pad = (chunk_size - q_len % chunk_size) % chunk_size;
  const int lq = q_len + q_pad, lk = k_len + k_pad;
  if (lk / chunk_size < lq / chunk_size) return XATTN_B200_ERR_ARG;   // Xattention.py:39
  g.batch = batch; g.hq = hq; g.hkv = hkv;
  g.S = stride; g.d_chunks = head_dim / kTileK;
  g.rows_total = lq / stride; g.cols_total = lk / stride;
  g.rows_valid = g.rows_total - q_pad / stride;
  g.cols_valid = g.cols_total - k_pad / stride;
  g.rcs = chunk_size / stride;
  g.row_off = (lk / chunk_size - lq / chunk_size) * g.rcs;
  g.causal = causal ? 1 : 0;
  g.left_blank = (causal && semantics != XATTN_B200_SEMANTICS_TRITON && k_pad / stride == 0) ? 1 : 0;
  g.band = semantics == XATTN_B200_SEMANTICS_TORCH_BAND ? 1 : 0;
  g.bpc = chunk_size / block_size;
  if (g.band && !g.left_blank) return XATTN_B200_ERR_ARG;
  g.rbs = block_size / stride;
  g.kb_total = lk / block_size; g.qb_total = lq / block_size;
  g.n_mtiles = (g.rows_total + kTileM - 1) / kTileM;
  // narrow tiles when every row sees at most one 128-column span (torch branch with chunk_size <= 128*stride):
  // a 256-wide tile would spend half of its MMA work on hidden columns
  g.tile_n = (g.left_blank && g.rcs <= 128) ? 128 : kTileN;
  g.n_ntiles = (g.cols_total + g.tile_n - 1) / g.tile_n;
  g.scale_log2 = scale * 1.4426950408889634f;
  g.head_dim = head_dim;
  g.tab_n = 0;
  g.q_tail_mt = q_len % stride ? (q_len / stride) / kTileM : -1;
  g.k_tail_nt = k_len % stride ? (k_len / stride) / g.tile_n : -1;
  g.compact = g.left_blank;
  g.m_pitch = g.n_ntiles;
  g.p_pitch = g.kb_total;
  if (g.compact) {
    int max_cnt = 1;
    for (int mt = 0; mt < g.n_mtiles; ++mt) {
      int first, cnt;
      row_tile_range(g, mt, first, cnt);
      max_cnt = cnt > max_cnt ? cnt : max_cnt;
    }
    g.m_pitch = max_cnt;
    g.p_pitch = max_cnt * (g.tile_n / g.rbs);
  }
  return XATTN_B200_OK;
}

static EstWorkspace workspace_layout(const EstGeom& g) {
  EstWorkspace w;
  auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
  size_t o = 0;
  w.off_tile_lo = o; o = up(o + sizeof(int) * g.n_mtiles);
  w.off_tile_prefix = o; o = up(o + sizeof(int) * (g.n_mtiles + 1));
  w.off_pair_lo = o; o = up(o + sizeof(int) * ((g.n_mtiles + 1) / 2));
  w.off_pair_prefix = o; o = up(o + sizeof(int) * ((g.n_mtiles + 1) / 2 + 1));
  const size_t rows = static_cast<size_t>(g.batch) * g.hq * g.rows_total;
  w.off_rowstat = o; o = up(o + sizeof(float2) * rows);
  w.off_mtile = o; o = up(o + sizeof(float2) * rows * g.m_pitch);
  w.off_partial = o; o = up(o + sizeof(float) * rows * g.p_pitch);
  // staging tiles [batch, heads, tile * S tokens, head_dim], 16 bit
  w.off_qtail = o;
  if (g.q_tail_mt >= 0) o = up(o + static_cast<size_t>(g.batch) * g.hq * kTileM * g.S * g.head_dim * 2);
  w.off_ktail = o;
  if (g.k_tail_nt >= 0) o = up(o + static_cast<size_t>(g.batch) * g.hkv * g.tile_n * g.S * g.head_dim * 2);
  w.total = o;
  return w;
}

// Scratch of one estimate call: exact for the given mask and semantics, or (causal < 0) enough for any.
size_t estimate_workspace_bytes(int batch, int hq, int q_len, int k_len, int stride, int block_size, int chunk_size,
                                int causal, int semantics) {
  EstGeom g;
  const int ql = q_len, kl = k_len;      // (head_dim 128 and hkv = hq assumed for the staging tiles of ragged lengths)
  if (causal >= 0) {
    if (fill_geometry(batch, hq, hq, ql, kl, 128, stride, block_size, chunk_size, 1.f, causal, semantics, g) !=
        XATTN_B200_OK)
      return 0;
    return workspace_layout(g).total;
  }
  size_t need = 0;
  for (int c = 0; c < 2; ++c) {
    if (fill_geometry(batch, hq, hq, ql, kl, 128, stride, block_size, chunk_size, 1.f, c, c ? XATTN_B200_SEMANTICS_TRITON : 0, g) !=
        XATTN_B200_OK)
      return 0;
    const size_t t = workspace_layout(g).total;
    need = t > need ? t : need;
  }
  return need;
}

int estimate_launch(const void* q, const void* k, int dtype, int batch, int hq, int hkv, int q_len, int k_len,
                    int head_dim, int64_t qsb, int64_t qsh, int64_t qsl, int64_t ksb, int64_t ksh, int64_t ksl,
                    int stride, int block_size, int chunk_size, float scale, int causal, int semantics,
                    float* attn_sums, void* workspace, size_t workspace_bytes, int* status, cudaStream_t stream) {
  if (!q || !k || !attn_sums) return XATTN_B200_ERR_ARG;
  if (dtype != XATTN_B200_BF16 && dtype != XATTN_B200_F16) return XATTN_B200_ERR_ARG;
  if (semantics != XATTN_B200_SEMANTICS_TORCH && semantics != XATTN_B200_SEMANTICS_TRITON &&
      semantics != XATTN_B200_SEMANTICS_TORCH_BAND)
    return XATTN_B200_ERR_ARG;
  if (!(scale > 0.f)) return XATTN_B200_ERR_ARG;
  EstGeom g;
  int rc = fill_geometry(batch, hq, hkv, q_len, k_len, head_dim, stride, block_size, chunk_size, scale, causal,
                         semantics, g);
  if (rc) return rc;
  const EstWorkspace w = workspace_layout(g);
  if (!workspace || workspace_bytes < w.total) return XATTN_B200_ERR_WORKSPACE;
  if ((rc = check_sm100())) return rc;
  // every stated maximum is checked before the first launch, so that a refusal leaves no work in flight
  const long long total_rows = static_cast<long long>(batch) * hq * g.rows_total;
  if (g.n_mtiles > 8192 || total_rows > 0x7fffffffLL || static_cast<long long>(batch) * hq > 65535 ||
      g.qb_total > 65535)
    return XATTN_B200_ERR_LIMIT;

  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int* tile_lo = reinterpret_cast<int*>(ws + w.off_tile_lo);
  int* tile_prefix = reinterpret_cast<int*>(ws + w.off_tile_prefix);
  int* pair_lo = reinterpret_cast<int*>(ws + w.off_pair_lo);
  int* pair_prefix = reinterpret_cast<int*>(ws + w.off_pair_prefix);
  float2* mtile = reinterpret_cast<float2*>(ws + w.off_mtile);
  float2* rowstat = reinterpret_cast<float2*>(ws + w.off_rowstat);
  float* partial = reinterpret_cast<float*>(ws + w.off_partial);

  // 5-D views [head_dim, S, len/S, heads, batch] whose second coordinate picks the token inside a stride group
  CUtensorMap tmQ, tmK;
  {
    const uint64_t dims[5] = {(uint64_t)head_dim, (uint64_t)stride, (uint64_t)(q_len / stride), (uint64_t)hq,
                              (uint64_t)batch};
    const uint64_t str[4] = {(uint64_t)qsl * 2, (uint64_t)qsl * 2 * stride, (uint64_t)qsh * 2, (uint64_t)qsb * 2};
    const uint32_t box[5] = {kTileK, 1, kTileM, 1, 1};
    if ((rc = make_tmap_16bit(&tmQ, q, 5, dims, str, box))) return rc;
  }
  {
    const uint64_t dims[5] = {(uint64_t)head_dim, (uint64_t)stride, (uint64_t)(k_len / stride), (uint64_t)hkv,
                              (uint64_t)batch};
    const uint64_t str[4] = {(uint64_t)ksl * 2, (uint64_t)ksl * 2 * stride, (uint64_t)ksh * 2, (uint64_t)ksb * 2};
    const uint32_t box[5] = {kTileK, 1, (uint32_t)g.tile_n, 1, 1};
    if ((rc = make_tmap_16bit(&tmK, k, 5, dims, str, box))) return rc;
  }

  // up to 64 KiB of dynamic shared memory (8192 row tiles): above the 48 KiB a kernel gets without asking
  if (cudaFuncSetAttribute(est_setup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * sizeof(int) * 8192) !=
      cudaSuccess)
    return XATTN_B200_ERR_CUDA;
  // CTA pairs (256x256 tiles) when tiles are 256 columns wide and the two row tiles of a pair see about the
  // same columns (always, except when a 128-row chunk of the torch branch blanks everything left of it)
  bool use_pairs = g.tile_n == kTileN && g.n_mtiles >= 2 && (!g.left_blank || g.rcs % (2 * kTileM) == 0);
#ifdef XB_EST_NO_PAIRS
  use_pairs = false;
#endif
  // Chunks of exactly one 128-row, 128-column tile under the torch branch (128K tokens at stride 16): a row's only
  // tile holds exactly the key blocks of its chunk-band output, so the GEMM's epilogue finishes the block sums
  // itself and neither the scratch arrays nor est_rowstat_kernel / est_blocksum_kernel are needed.
  bool direct = !use_pairs && g.band && g.left_blank && g.compact && g.m_pitch == 1 && g.tile_n == 128 &&
                g.rcs == kTileM && g.row_off % 128 == 0 && g.rbs <= 32 && 32 % g.rbs == 0 &&
                g.bpc == 128 / g.rbs && g.bpc % 4 == 0 && (reinterpret_cast<uintptr_t>(attn_sums) & 15) == 0;
  for (int mt = 0; direct && mt < g.n_mtiles; ++mt) {
    int first, count;
    row_tile_range(g, mt, first, count);
    direct = count == 1 && first * 128 == (mt * kTileM / g.rcs) * g.rcs + g.row_off;
  }
#ifdef XB_EST_NO_DIRECT
  direct = false;
#endif
  // ragged lengths: stage the tile with the last (partial) stride group and map it like the tensor itself
  CUtensorMap tmQt = tmQ, tmKt = tmK;
  auto stage_tail = [&](const void* src, int64_t sb, int64_t sh, int64_t sl, int heads, int len, int tile_rows,
                        int tail_tile, size_t off, uint32_t box_rows, CUtensorMap* map) -> int {
    if ((sb % 8) || (sh % 8) || (sl % 8) || (head_dim % 8)) return XATTN_B200_ERR_ARG;
    const int n_tokens = tile_rows * stride;
    const size_t total_vec = static_cast<size_t>(batch) * heads * n_tokens * (head_dim / 8);
    size_t blocks = (total_vec + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    est_tail_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
        static_cast<const uint4*>(src), sb, sh, sl, heads, len, head_dim, tail_tile * n_tokens, n_tokens,
        reinterpret_cast<uint4*>(ws + off), total_vec);
    int r = launch_status();
    if (r) return r;
    const uint64_t dims[5] = {(uint64_t)head_dim, (uint64_t)stride, (uint64_t)tile_rows, (uint64_t)heads,
                              (uint64_t)batch};
    const uint64_t tok = (uint64_t)head_dim * 2;
    const uint64_t s_h = heads > 1 ? tok * n_tokens : 256, s_b = batch > 1 ? tok * n_tokens * heads : 256;
    const uint64_t str[4] = {tok, tok * stride, s_h, s_b};
    const uint32_t box[5] = {kTileK, 1, box_rows, 1, 1};
    return make_tmap_16bit(map, ws + off, 5, dims, str, box);
  };
  if (g.q_tail_mt >= 0 &&
      (rc = stage_tail(q, qsb, qsh, qsl, hq, q_len, kTileM, g.q_tail_mt, w.off_qtail, kTileM, &tmQt)))
    return rc;
  if (g.k_tail_nt >= 0 && (rc = stage_tail(k, ksb, ksh, ksl, hkv, k_len, g.tile_n, g.k_tail_nt, w.off_ktail,
                                           use_pairs ? 128 : static_cast<uint32_t>(g.tile_n), &tmKt)))
    return rc;

  if (g.n_mtiles <= kTabTiles) {
    // few row tiles: the tables travel in the kernel parameters (the arithmetic of est_setup_kernel, on the host)
    int* t_lo = g.tab, *t_prefix = g.tab + kTabPrefix, *p_lo = g.tab + kTabPairLo, *p_prefix = g.tab + kTabPairPrefix;
    int cnt[kTabTiles];
    int acc = 0;
    for (int mt = 0; mt < g.n_mtiles; ++mt) {
      row_tile_range(g, mt, t_lo[mt], cnt[mt]);
      t_prefix[mt] = acc;
      acc += cnt[mt];
    }
    t_prefix[g.n_mtiles] = acc;
    const int n_pairs = (g.n_mtiles + 1) / 2;
    acc = 0;
    for (int pm = 0; pm < n_pairs; ++pm) {
      int lo = 0x7fffffff, hi = -1;
      for (int mt = 2 * pm; mt < 2 * pm + 2 && mt < g.n_mtiles; ++mt)
        if (cnt[mt] > 0) {
          lo = t_lo[mt] < lo ? t_lo[mt] : lo;
          hi = t_lo[mt] + cnt[mt] - 1 > hi ? t_lo[mt] + cnt[mt] - 1 : hi;
        }
      p_lo[pm] = hi < 0 ? 0 : lo;
      p_prefix[pm] = acc;
      acc += hi < 0 ? 0 : hi - lo + 1;
    }
    p_prefix[n_pairs] = acc;
    g.tab_n = g.n_mtiles;
  } else {
    est_setup_kernel<<<1, 256, 2 * sizeof(int) * g.n_mtiles, stream>>>(g, tile_lo, tile_prefix, pair_lo, pair_prefix);
    if ((rc = launch_status())) return rc;
  }

  const int sms = sm_count();
  if (use_pairs) {
    CUtensorMap tmKh;                     // K with a box of 128 rows: one CTA's half of a 256-column tile
    {
      const uint64_t dims[5] = {(uint64_t)head_dim, (uint64_t)stride, (uint64_t)(k_len / stride), (uint64_t)hkv,
                                (uint64_t)batch};
      const uint64_t str[4] = {(uint64_t)ksl * 2, (uint64_t)ksl * 2 * stride, (uint64_t)ksh * 2, (uint64_t)ksb * 2};
      const uint32_t box[5] = {kTileK, 1, 128, 1, 1};
      if ((rc = make_tmap_16bit(&tmKh, k, 5, dims, str, box))) return rc;
    }
    const uint32_t idesc2 = make_idesc_f16(2 * kTileM, kTileN, dtype == XATTN_B200_BF16, false, false);
    auto launch_pair = [&](auto kern) -> int {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem) != cudaSuccess)
        return XATTN_B200_ERR_CUDA;
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(static_cast<unsigned>(sms & ~1), 1, 1);
      cfg.blockDim = dim3(kGemmThreads, 1, 1);
      cfg.dynamicSmemBytes = kPairSmem;
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      // every pair must be resident at once (persistent kernel): shrink the grid to what the device can hold
      int max_clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess || max_clusters < 1)
        return XATTN_B200_ERR_CUDA;
      if (static_cast<unsigned>(2 * max_clusters) < cfg.gridDim.x) cfg.gridDim.x = 2 * max_clusters;
      if (cudaLaunchKernelEx(&cfg, kern, tmQ, tmKh, tmQt, tmKt, g, (const int*)pair_lo, (const int*)pair_prefix,
                             partial, mtile, idesc2, status) != cudaSuccess)
        return XATTN_B200_ERR_CUDA;
      return launch_status();
    };
    switch (g.rbs) {
      case 4: rc = launch_pair(est_gemm_pair_kernel<4>); break;
      case 8: rc = launch_pair(est_gemm_pair_kernel<8>); break;
      case 16: rc = launch_pair(est_gemm_pair_kernel<16>); break;
      case 32: rc = launch_pair(est_gemm_pair_kernel<32>); break;
      default: rc = XATTN_B200_ERR_ARG;
    }
    if (rc) return rc;
  } else {
  const uint32_t idesc = make_idesc_f16(kTileM, g.tile_n, dtype == XATTN_B200_BF16, false, false);
  const int grid = sms;
  auto launch = [&](auto kern) -> int {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem) != cudaSuccess)
      return XATTN_B200_ERR_CUDA;
    kern<<<grid, kGemmThreads, kGemmSmem, stream>>>(tmQ, tmK, tmQt, tmKt, g, tile_lo, tile_prefix, partial, mtile,
                                                    attn_sums, idesc, status);
    return launch_status();
  };
  if (direct) {
    switch (g.rbs) {
      case 4: rc = launch(est_gemm_kernel<4, true>); break;
      case 8: rc = launch(est_gemm_kernel<8, true>); break;
      case 16: rc = launch(est_gemm_kernel<16, true>); break;
      case 32: rc = launch(est_gemm_kernel<32, true>); break;
      default: rc = XATTN_B200_ERR_ARG;
    }
    return rc;                                         // the block sums are complete
  }
  switch (g.rbs) {
    case 4: rc = launch(est_gemm_kernel<4, false>); break;
    case 8: rc = launch(est_gemm_kernel<8, false>); break;
    case 16: rc = launch(est_gemm_kernel<16, false>); break;
    case 32: rc = launch(est_gemm_kernel<32, false>); break;
    default: rc = XATTN_B200_ERR_ARG;
  }
  if (rc) return rc;
  }

  // rows that span at most eight column tiles: their statistics are computed inside est_blocksum_kernel
  const int max_tiles_per_row = g.m_pitch;             // (dense scratch: every column tile of the row)
  const int out_cols = g.band ? g.bpc : g.kb_total;
  const bool vec4 = g.kb_total % 4 == 0 && out_cols % 4 == 0 && (reinterpret_cast<uintptr_t>(attn_sums) & 15) == 0;
  const int per_row = vec4 ? out_cols / 4 : out_cols;
  // (and a query block with enough key blocks to amortise the extra round trip: measured -11 us at 32K, where a
  // CTA sums 128 key blocks, and +10 us at 128K, where it sums 16)
#ifndef XB_FUSE_MIN
#define XB_FUSE_MIN 32
#endif
  const bool fused = max_tiles_per_row <= 8 && per_row >= XB_FUSE_MIN;
  if (!fused) {
    est_rowstat_kernel<<<static_cast<int>((total_rows + 255) / 256), 256, 0, stream>>>(
        g, tile_lo, tile_prefix, mtile, rowstat, static_cast<int>(total_rows));
    if ((rc = launch_status())) return rc;
  }
  int bt = per_row >= 256 ? 256 : ((per_row + 31) / 32) * 32;
  if (fused && bt < 8 * g.rbs) bt = 8 * g.rbs;           // eight threads per row for the statistics (rbs <= 32)
  const dim3 fgrid((per_row + bt - 1) / bt, g.qb_total, batch * hq);
  if (vec4) {
    if (fused) est_blocksum_kernel<4, true><<<fgrid, bt, 0, stream>>>(g, tile_lo, tile_prefix, partial, mtile, rowstat, attn_sums);
    else est_blocksum_kernel<4, false><<<fgrid, bt, 0, stream>>>(g, tile_lo, tile_prefix, partial, mtile, rowstat, attn_sums);
  } else {
    if (fused) est_blocksum_kernel<1, true><<<fgrid, bt, 0, stream>>>(g, tile_lo, tile_prefix, partial, mtile, rowstat, attn_sums);
    else est_blocksum_kernel<1, false><<<fgrid, bt, 0, stream>>>(g, tile_lo, tile_prefix, partial, mtile, rowstat, attn_sums);
  }
  return launch_status();
}

int split_f32_launch(const float* x, int batch, int heads, int len, int len_valid, int head_dim, int64_t sb, int64_t sh,
                     int64_t sl, int role, void* out, cudaStream_t stream) {
  if (!x || !out || batch < 1 || heads < 1 || len < 1 || len_valid < 1 || len_valid > len || head_dim < 1 ||
      (role != 0 && role != 1))
    return XATTN_B200_ERR_ARG;
  const size_t total = static_cast<size_t>(batch) * heads * len * head_dim;
  const int block = 256;
  size_t blocks = (total + block - 1) / block;
  if (blocks > 148 * 32) blocks = 148 * 32;
  split_f32_kernel<<<static_cast<int>(blocks), block, 0, stream>>>(x, heads, len, len_valid, head_dim, sb, sh, sl, role,
                                                                    static_cast<__nv_bfloat16*>(out), total);
  return launch_status();
}

}  // namespace xb
