// Block-scaled FP8 GEMM (dense and expert-grouped) for sm_100a.
//
//   C[m,n] = out_t( sum_kb a_s[m,kb] * b_s[n/128,kb] * sum_{k in kb} A[m,k] * B[n,k] )
//
// One persistent CTA per SM walks 128 x BN output tiles.  BN = 192 with two TMEM accumulator buffers where there
// are waves of full tiles (fewest bytes per FLOP from L2, fewest tiles; its 32-column pieces never straddle a
// 128-wide scale block), BN = 128 with four buffers for small and medium row counts and for the expert-grouped
// form (more tiles to spread, a deeper hand-off between the MMAs and the promotion).  Per 128-wide K slab:
//   * warp 0 (one elected lane) issues two TMA tile loads (A 128 rows x 128 B, B BN rows x 128 B,
//     128-byte swizzle) into a shared-memory ring, signalled through `full` mbarriers;
//   * warp 1 (one elected lane) issues four tcgen05.mma kind::f8f6f4 (128 x BN x 32) that write the
//     slab's partial sums into one of the TMEM buffers, then commits the slab to the
//     `empty` barrier of the ring slot and to the `tmem_full` barrier of the buffer;
//   * warps 4-11 (two per TMEM lane quadrant, BN/2 columns each) pull the partial sums out of TMEM with
//     32-column tcgen05.ld issued back to back, release the buffer, and promote them into float32 register
//     accumulators with the slab's scale a_s[m,kb]*b_s[nb,kb] (DeepSeek-style 128-block float scales cannot be
//     folded into the hardware's power-of-two MX scaling, so promotion runs on the CUDA cores, overlapped with
//     the next slabs' MMAs through the TMEM buffers), two columns per instruction (packed float32 FMA).  A
//     thread's activation scales are prefetched into registers four slabs at a time; the slab loop has no
//     barrier between warps;
//   * warp 3 (the scout) runs one unit ahead of the promotion warps and leaves, in one of two descriptor slots in
//     shared memory, the next unit's tile coordinates, K range, weight-block scales and the activation scales of its
//     first four slabs, so that a promotion warp starts a unit with shared-memory reads instead of integer divisions
//     and exposed global loads (per tile that start cost as much as a slab and a half of MMAs);
//   * warp 2 (one elected lane) hands finished tiles to the TMA engine: the promotion threads park their rounded
//     part of a tile in shared memory and arrive on an mbarrier, never waiting for each other or for a store.
// The kernel runs latency-, power- and issue-limited rather than tensor-limited (the tensor pipe is busy 40-50 %
// of the cycles): every instruction a promotion warp executes or a waiting warp spends polling costs time,
// so the per-slab loops are kept short, waits suspend in hardware (mbarrier.try_wait with a time hint) and
// each promotion warp owns as many columns as the register file allows (fewer warps = less per-slab overhead).
// The epilogue rounds to bf16/fp16, parks the tile in swizzled shared memory, from where TMA stores drain it
// during the next tile; in grouped "scatter" mode it multiplies by the routing
// weight and writes 16 bytes at a time to the token-major row named by sorted_token_ids.
// Scheduling: with fewer than two waves of tiles and a long K the tiles x slabs space is cut into one equal run
// of slabs per SM (stream-K; a run covers the end of one tile, possibly a whole tile, and the start of the next);
// otherwise the tiles of a short last wave are split along K.  Split work writes float32 partial sums that a
// second kernel adds in ascending K order.  In push mode (row-parallel layers under tensor parallelism) a tile is
// stored through the tensor map of the staging buffer of the GPU that owns its rows, which folds the
// reduce-scatter of the all-reduce into the epilogue.
//
// Every mbarrier wait is bounded; on expiry the role raises a flag in shared memory and leaves its loops, the other
// roles sit out their own limits, the CTA sets a status word, drains, frees its TMEM and returns
// (sglb200_gemm_status() reports it).
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace sglb200 {

constexpr int BM = 128, BK = 128;
constexpr int kScaleBlockN = 128;         // weight scales cover 128 output rows
constexpr int kTmemCols = 512;
constexpr int kEpiWarp0 = 4;              // warp 0 TMA, warp 1 MMA + TMEM owner, warps 4.. promotion + epilogue
constexpr int kEpiWarps = 8;
constexpr int kGemmThreads = 128 + kEpiWarps * 32;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kColGroups = kEpiWarps / 4;  // promotion warps per TMEM lane quadrant
constexpr uint32_t kTileBytesA = BM * BK;  // fp8
// A pipeline wait: a bounded run of suspending probes (seconds at most).  `p.wait_probes == kProbesNone` (a
// diagnostic setting) makes every wait give up at once, which exercises the give-up path on a healthy GPU.
// (Measured: also polling the CTA's abort flag between runs of probes, so that one role's expiry ends the others'
// waits early, cost 5 % of the large-M rate; each role sits out its own limit instead.)
// Measurement builds (-DSGLB_TRACE): clock stamps of one promotion warp per column group of CTA 0, per unit.
#ifdef SGLB_TRACE
constexpr int kTraceUnits = 64, kTraceStamps = 8;
__device__ long long g_trace[3][kTraceUnits][kTraceStamps];  // [2] = the scout warp
#define SGLB_SCOUT_STAMP(i)                                                                             \
  do {                                                                                                  \
    if (blockIdx.x == 0 && lane == 0 && scout_unit < kTraceUnits) g_trace[2][scout_unit][i] = clock64(); \
  } while (0)
#define SGLB_STAMP(i)                                                                                  \
  do {                                                                                                 \
    if (blockIdx.x == 0 && q == 0 && lane == 0 && trace_unit < kTraceUnits) g_trace[cgrp][trace_unit][i] = clock64(); \
  } while (0)
#else
#define SGLB_STAMP(i)
#define SGLB_SCOUT_STAMP(i)
#endif

#define SGLB_WAIT(bar, parity) (p.wait_probes != ptx::kProbesNone && ptx::mbar_wait_quiet(bar, parity))
#ifndef SGLB_FMA2
#define SGLB_FMA2 1                        // promotion with packed float32 FMAs (two columns per instruction)
#endif

// Tile width BN: 192 columns with two TMEM accumulator buffers (the fewest bytes per FLOP from L2 and the fewest
// tiles: best where there are waves of full tiles), or 128 columns with four buffers (more tiles for the same
// problem and a deeper hand-off between the MMAs and the promotion: best where tiles are few or short).
template <int BN_>
struct TileCfg {
  static constexpr int BN = BN_;
  static constexpr int kStages = BN_ >= 192 ? 4 : 5;
  static constexpr int kAccBufs = kTmemCols / BN_;   // TMEM accumulator buffers in flight
  static constexpr int kAccStride = BN_;             // TMEM columns between buffers
  static constexpr int kEpiCols = BN_ / kColGroups;  // columns of a buffer owned by one promotion warp
  static constexpr uint32_t kTileBytesB = BN_ * BK;
  static constexpr uint32_t kStageBytes = kTileBytesA + kTileBytesB;
  // output staging for the TMA store: per 64 columns a [128 rows][64 columns] 2-byte tile in the 128-byte swizzle
  static constexpr int kOutGroups = BN_ / 64;
  static constexpr uint32_t kOutGroupBytes = BM * 64 * 2;
  static constexpr uint32_t kOutBytes = kOutGroups * kOutGroupBytes;
  static_assert(kEpiWarps % 4 == 0 && BN_ % kColGroups == 0 && kEpiCols % 32 == 0 && BN_ % 64 == 0 &&
                    kAccBufs * kAccStride <= kTmemCols && BN_ <= 256 && kStageBytes % 1024 == 0,
                "accumulator layout");
};

__device__ int g_gemm_status = 0;  // 0 ok, 1 = a pipeline wait expired

struct GemmParams {
  const float* a_s;
  const float* b_s;
  void* C;
  const void* bias;
  const int32_t* sorted_ids;   // grouped
  const int32_t* expert_ids;   // grouped
  const int32_t* num_rows_dev; // grouped: rows in use (multiple of 128)
  const float* row_weights;    // grouped scatter, optional
  int64_t M;                   // dense: rows of A; grouped: max rows
  int64_t N, K;
  int64_t as_stride_m, as_stride_k;
  int64_t numel;               // grouped scatter: valid ids are < numel
  int kb_total;                // ceil(K/128)
  int full_units;              // dense: the first `full_units` tiles are one unit each ...
  int splits;                  // ... and every later tile is cut into `splits` units along K (1 = none)
  int kb_per_split;            // K slabs per unit of a split tile
  float* partial;              // float32 partial sums of the split tiles: [slot][BM x BN block]
  int partial_rowmajor;        // layout of a block: 1 = [row][BN] (few rows), 0 = [column / 4][row][4] (full tiles)
  int nb_total;                // ceil(N/128): weight scale blocks along N
  int tiles_n;                 // ceil(N/BN)
  int scatter;
  int out_fp16;
  int tma_out;                 // rows of C are written with TMA tile stores (map_c is valid)
  int group_m;                 // m-tiles per rasterization group
  // push mode (row-parallel layers): the output rows are owned in equal blocks by `world` GPUs and each tile
  // is stored into its owner's staging buffer [source rank][rows per owner][N] through that buffer's tensor map
  const CUtensorMap* push_maps;  // [world] in global memory, nullptr = ordinary output through map_c
  int push_rows_per_owner;       // a multiple of BM
  int push_rank;                 // this GPU's slot in the owners' staging buffers
  // stream-K mode (fewer than two waves of tiles): the tiles x slabs space is cut into `sk_ctas` equal runs of
  // `sk_share` slabs, one per CTA; a run covers at most `sk_pieces` tiles (the end of one, the start of the next,
  // with a whole tile between them when sk_share exceeds kb_total)
  int sk_share;                  // 0 = off; otherwise <= (sk_pieces - 1) * kb_total
  int sk_ctas;
  int sk_pieces;                 // 2 or 3
  int sk_total;                  // tiles * kb_total
  uint32_t wait_probes;          // probes after which a pipeline wait gives up
};

constexpr int kDescSlabs = 512;  // K slabs of one unit whose weight-block scales a unit descriptor holds (K <= 65536)

// What the scout warp prepares for the promotion warps while they work on the previous unit: where the unit lies and
// the scales its first slabs need, so that a promotion warp starts a unit with a few shared-memory reads instead of
// integer divisions and global loads whose latency nothing hides.
struct UnitDesc {
  float a4[BM][4];          // activation scales of the unit's first four slabs, per tile row
  float b[2][kDescSlabs];   // weight-block scales of the unit's slabs for the (at most two) 128-column blocks of the tile
  int m_tile, n_tile, expert, kb_begin;
  int kb_stop, split, slot, pad;
};

template <class Cfg>
struct SharedCtl {
  UnitDesc desc[2];
  uint64_t desc_full[2];   // the descriptor is written (every scout lane arrives)
  uint64_t desc_empty[2];  // every promotion thread has read what it needs from it
  uint64_t full[Cfg::kStages];
  uint64_t empty[Cfg::kStages];
  uint64_t tmem_full[Cfg::kAccBufs];
  uint64_t tmem_empty[Cfg::kAccBufs];
  uint64_t out_full;  // the output staging holds a rounded tile (every promotion thread arrives)
  uint64_t out_free;  // the TMA stores of the previous tile have read the staging (the storing thread arrives)
  uint32_t tmem_base;
  int abort_flag;
};

struct TileCoord {
  int m_tile, n_tile, expert;
};

// tile index -> (m_tile, n_tile): groups of `group_m` m-tiles sweep over n together, m fastest inside a group.
// The activation rows of a group stay in L2 while the weight matrix streams past them once per group.
__device__ __forceinline__ void tile_coord(int t, int tiles_m, int tiles_n, int group_m, int& m_tile, int& n_tile) {
  const int per_group = group_m * tiles_n;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int gsz = min(tiles_m - first_m, group_m);
  const int r = t - g * per_group;
  m_tile = first_m + r % gsz;
  n_tile = r / gsz;
}

// A unit of work = one output tile x one K range.  Dense problems number their units: the tiles
// [0, full_units) whole, then `splits` consecutive units per remaining tile.
struct Unit {
  int tile, kb_begin, kb_stop;
  int slot;  // split units: which [BM][BN] float32 block of the partial-sum scratch
  bool split;
};
template <bool kGrouped>
__device__ __forceinline__ Unit decode_unit(const GemmParams& p, int u) {
  Unit x;
  x.slot = 0;
  if (!kGrouped && p.sk_share > 0) {
    // unit u = piece u / sk_ctas of the run of CTA u % sk_ctas
    const int piece = u / p.sk_ctas, c = u - piece * p.sk_ctas;
    const int lo = c * p.sk_share, hi = min(lo + p.sk_share, p.sk_total);
    const int t0 = lo / p.kb_total;
    x.tile = t0 + piece, x.slot = u, x.split = true;
    // the run restricted to the slabs of tile t0 + piece (empty ranges are skipped by every role)
    const int tb = x.tile * p.kb_total;
    x.kb_begin = max(lo, tb) - tb;
    x.kb_stop = max(min(hi, tb + p.kb_total) - tb, x.kb_begin);
    return x;
  }
  if (kGrouped || u < p.full_units) {
    x.tile = u, x.kb_begin = 0, x.kb_stop = p.kb_total, x.split = false;
  } else {
    const int v = u - p.full_units;
    x.tile = p.full_units + v / p.splits;
    const int sp = v - (x.tile - p.full_units) * p.splits;
    x.kb_begin = sp * p.kb_per_split;
    x.kb_stop = min(p.kb_total, x.kb_begin + p.kb_per_split);
    x.slot = v;
    x.split = true;
  }
  return x;
}

template <typename OutT, int kCols>
__device__ __forceinline__ void store_row_chunk(OutT* dst, const float* v, const void* bias_v, int n0, int N) {
  // up to kCols consecutive columns starting at n0 and ending before N, 8 per 16-byte store
#pragma unroll
  for (int j = 0; j < kCols / 8; ++j) {
    const int n = n0 + j * 8;
    if (n + 8 <= N) {
      float x[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = v[j * 8 + i];
      if (bias_v != nullptr) {
        const uint4 braw = __ldg(reinterpret_cast<const uint4*>(static_cast<const OutT*>(bias_v) + n));
        const OutT* b = reinterpret_cast<const OutT*>(&braw);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] += ElemTraits<OutT>::to_f32(b[i]);
      }
      uint4 raw;
      OutT* o = reinterpret_cast<OutT*>(&raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = ElemTraits<OutT>::from_f32(x[i]);
      *reinterpret_cast<uint4*>(dst + j * 8) = raw;
    } else {
      for (int i = 0; i < 8 && n + i < N; ++i) {
        float x = v[j * 8 + i];
        if (bias_v != nullptr) x += ElemTraits<OutT>::to_f32(static_cast<const OutT*>(bias_v)[n + i]);
        dst[j * 8 + i] = ElemTraits<OutT>::from_f32(x);
      }
    }
  }
}

template <bool kGrouped, int BN_>
__global__ void __launch_bounds__(kGemmThreads, 1)
    fp8_blockscale_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                               const __grid_constant__ CUtensorMap map_c, const GemmParams p) {
  using Cfg = TileCfg<BN_>;
  constexpr int BN = Cfg::BN, kStages = Cfg::kStages, kAccBufs = Cfg::kAccBufs, kAccStride = Cfg::kAccStride,
                kEpiCols = Cfg::kEpiCols, kOutGroups = Cfg::kOutGroups;
  constexpr uint32_t kStageBytes = Cfg::kStageBytes, kOutGroupBytes = Cfg::kOutGroupBytes, kOutBytes = Cfg::kOutBytes;
  extern __shared__ uint8_t smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* out_stage = tiles + kStages * kStageBytes;
  SharedCtl<Cfg>* ctl = reinterpret_cast<SharedCtl<Cfg>*>(out_stage + kOutBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &ctl->abort_flag;

  int64_t rows = p.M;
  if (kGrouped) {
    const int64_t lim = *p.num_rows_dev;
    rows = lim < rows ? lim : rows;
  }
  const int tiles_m = (int)((rows + BM - 1) / BM);
  const int tiles_n = p.tiles_n;
  const int num_tiles = tiles_m * tiles_n;
  const int kb_total = p.kb_total;
  const int num_units = kGrouped         ? num_tiles
                        : p.sk_share > 0 ? p.sk_pieces * p.sk_ctas
                                         : p.full_units + (num_tiles - p.full_units) * p.splits;

  // (the reduction kernel that follows a split launch is launched programmatically: letting it be scheduled now
  // hides its launch latency; it waits for this grid to complete before it reads a partial sum)
  ptx::launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->empty[s]), 1);
    }
    for (int b = 0; b < kAccBufs; ++b) {
      ptx::mbar_init(ptx::smem_u32(&ctl->tmem_full[b]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->tmem_empty[b]), kEpiWarps);
    }
    for (int d = 0; d < 2; ++d) {
      ptx::mbar_init(ptx::smem_u32(&ctl->desc_full[d]), 32);
      ptx::mbar_init(ptx::smem_u32(&ctl->desc_empty[d]), kEpiThreads);
    }
    ptx::mbar_init(ptx::smem_u32(&ctl->out_full), kEpiThreads);
    ptx::mbar_init(ptx::smem_u32(&ctl->out_free), 1);
    ctl->abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&map_a);
    ptx::tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&ctl->tmem_base), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const bool vec_scales = p.as_stride_k == 1 && (p.as_stride_m & 3) == 0 &&
                          (reinterpret_cast<uintptr_t>(p.a_s) & 15u) == 0;
  // activation scales of slabs kb .. kb+3 of the row `a_row` points at (zero past the last slab)
  auto load_a4_row = [&](const float* a_row, int kb) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (vec_scales && kb + 3 < kb_total && (kb & 3) == 0) {
      v = __ldg(reinterpret_cast<const float4*>(a_row + kb));
    } else {
      if (kb + 0 < kb_total) v.x = __ldg(a_row + (int64_t)(kb + 0) * p.as_stride_k);
      if (kb + 1 < kb_total) v.y = __ldg(a_row + (int64_t)(kb + 1) * p.as_stride_k);
      if (kb + 2 < kb_total) v.z = __ldg(a_row + (int64_t)(kb + 2) * p.as_stride_k);
      if (kb + 3 < kb_total) v.w = __ldg(a_row + (int64_t)(kb + 3) * p.as_stride_k);
    }
    return v;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (ptx::elect_one()) {
      const uint32_t bar_empty0 = ptx::smem_u32(&ctl->empty[0]), bar_full0 = ptx::smem_u32(&ctl->full[0]);
      const uint32_t tiles0 = ptx::smem_u32(tiles);
      uint32_t s = 0, ph = 0;
      bool alive = true;
      for (int u = blockIdx.x; u < num_units && alive; u += gridDim.x) {
        const Unit un = decode_unit<kGrouped>(p, u);
        const int t = un.tile, kb_begin = un.kb_begin, kb_stop = un.kb_stop;
        if (kb_begin >= kb_stop) continue;  // (an empty piece of a stream-K run)
        int m_tile, n_tile;
        tile_coord(t, tiles_m, tiles_n, p.group_m, m_tile, n_tile);
        int e = 0;
        if (kGrouped) {
          e = p.expert_ids[m_tile];
          if (e < 0) continue;
        }
        // this thread shares its scheduler with promotion warps that always have work: every instruction it
        // spends per slab delays the loads, so the loop keeps only 32-bit counters that step
        const int row_a = m_tile * BM, row_b = n_tile * BN;
        for (int k0 = kb_begin * BK; k0 < kb_stop * BK; k0 += BK) {
          if (!SGLB_WAIT(bar_empty0 + s * 8, ph ^ 1u)) { *abort_flag = 1; alive = false; break; }
          const uint32_t bar = bar_full0 + s * 8;
          ptx::mbar_arrive_expect_tx(bar, kStageBytes);
          const uint32_t dst_a = tiles0 + s * kStageBytes;
          ptx::tma_load_2d(dst_a, &map_a, bar, k0, row_a);
          ptx::tma_load_3d(dst_a + kTileBytesA, &map_b, bar, k0, row_b, e);
          if (++s == (uint32_t)kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::make_idesc_e4m3_f32(BM, BN);
      // Operand descriptor (K-major, 128-byte swizzle): low word = address/16 | LBO(1) << 16, high word =
      // SBO(1024/16) | version 1 (bit 46) | layout SWIZZLE_128B (2 at bit 61).  Only the low word changes.
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t desc_lo0 = ((ptx::smem_u32(tiles) & 0x3ffffu) >> 4) | (1u << 16);
      const uint32_t bar_full0 = ptx::smem_u32(&ctl->full[0]), bar_empty0 = ptx::smem_u32(&ctl->empty[0]);
      const uint32_t bar_tfull0 = ptx::smem_u32(&ctl->tmem_full[0]), bar_tempty0 = ptx::smem_u32(&ctl->tmem_empty[0]);
      uint32_t s = 0, ph = 0, buf = 0, aph = 0;
      bool alive = true;
      for (int u = blockIdx.x; u < num_units && alive; u += gridDim.x) {
        const Unit un = decode_unit<kGrouped>(p, u);
        const int t = un.tile, kb_begin = un.kb_begin, kb_stop = un.kb_stop;
        if (kb_begin >= kb_stop) continue;
        if (kGrouped) {
          int m_tile, n_tile;
          tile_coord(t, tiles_m, tiles_n, p.group_m, m_tile, n_tile);
          if (p.expert_ids[m_tile] < 0) continue;
        }
        for (int kb = kb_begin; kb < kb_stop; ++kb) {
          if (!SGLB_WAIT(bar_tempty0 + buf * 8, aph ^ 1u)) { *abort_flag = 1; alive = false; break; }
          if (!SGLB_WAIT(bar_full0 + s * 8, ph)) { *abort_flag = 1; alive = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_lo = desc_lo0 + s * (kStageBytes >> 4);
          const uint32_t b_lo = a_lo + (kTileBytesA >> 4);
          const uint32_t d_tmem = tmem_base + buf * kAccStride;
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            // advancing 32 bytes along K inside the 128-byte swizzled row = +2 in the descriptor's 16-byte units
            ptx::mma_f8f6f4(d_tmem, ptx::pack_f32x2(a_lo + 2 * k, kDescHi), ptx::pack_f32x2(b_lo + 2 * k, kDescHi), idesc,
                            k > 0 ? 1u : 0u);
          }
          ptx::mma_commit(bar_empty0 + s * 8);
          ptx::mma_commit(bar_tfull0 + buf * 8);
          if (++s == (uint32_t)kStages) {
            s = 0;
            ph ^= 1u;
          }
          if (++buf == (uint32_t)kAccBufs) {
            buf = 0;
            aph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------ output stores ------------------------------
    // One thread hands every finished tile to the TMA engine: it waits until all promotion threads have parked their
    // part of the tile in the staging area, issues the stores, waits until they have read the staging and gives it
    // back.  The promotion warps never wait for each other or for a store to be issued: each goes on to its next
    // unit as soon as its own part is parked.
    if (p.tma_out && ptx::elect_one()) {
      const uint32_t bar_out_full = ptx::smem_u32(&ctl->out_full), bar_out_free = ptx::smem_u32(&ctl->out_free);
      uint32_t oph = 0;
      for (int u = blockIdx.x; u < num_units; u += gridDim.x) {
        const Unit un = decode_unit<kGrouped>(p, u);
        if (un.kb_begin >= un.kb_stop || un.split) continue;
        if (!SGLB_WAIT(bar_out_full, oph)) {
          *abort_flag = 1;
          break;
        }
        oph ^= 1u;
        if (*abort_flag == 0) {  // (after a give-up the tile is incomplete: nothing is stored)
          int m_tile, n_tile;
          tile_coord(un.tile, tiles_m, tiles_n, p.group_m, m_tile, n_tile);
          const int n_end = (int)min((int64_t)n_tile * BN + BN, p.N);
          const CUtensorMap* cmap = &map_c;
          int out_row0 = m_tile * BM;
          if (p.push_maps != nullptr) {
            const int owner = out_row0 / p.push_rows_per_owner;
            cmap = p.push_maps + owner;
            out_row0 += (p.push_rank - owner) * p.push_rows_per_owner;
          }
#pragma unroll
          for (int g = 0; g < kOutGroups; ++g) {
            if (n_tile * BN + g * 64 < n_end)
              ptx::tma_store_2d(cmap, ptx::smem_u32(out_stage) + g * kOutGroupBytes, n_tile * BN + g * 64, out_row0);
          }
          ptx::tma_store_commit();
        }
        ptx::tma_store_wait_read();
        ptx::mbar_arrive(bar_out_free);
      }
      // tiles pushed to other GPUs have landed before the kernel counts as finished
      if (p.push_maps != nullptr) ptx::tma_store_wait_all();
    }
  } else if (warp == 3) {
    // ------------------------------ unit scout ------------------------------
    // Walks the CTA's units one ahead of the promotion warps and leaves a descriptor of each in one of two slots:
    // tile coordinates and K range (every unit, empty stream-K pieces included, so that the two sides count alike),
    // and for units with work the activation scales of the first four slabs of all 128 rows and the unit's
    // weight-block scales.  All 32 lanes probe the same barrier word, so the outcome of a wait is uniform.
    const uint32_t bar_dfull0 = ptx::smem_u32(&ctl->desc_full[0]), bar_dempty0 = ptx::smem_u32(&ctl->desc_empty[0]);
    uint32_t ds = 0, dph = 0;
#ifdef SGLB_TRACE
    int scout_unit = -1;
#endif
    for (int u = blockIdx.x; u < num_units; u += gridDim.x) {
#ifdef SGLB_TRACE
      ++scout_unit;
#endif
      SGLB_SCOUT_STAMP(0);
      if (!SGLB_WAIT(bar_dempty0 + ds * 8, dph ^ 1u)) {
        *abort_flag = 1;
        break;
      }
      SGLB_SCOUT_STAMP(1);
      const Unit un = decode_unit<kGrouped>(p, u);
      UnitDesc* d = &ctl->desc[ds];
      int m_tile = 0, n_tile = 0, e = 0;
      const bool work = un.kb_begin < un.kb_stop;
      if (work) {
        tile_coord(un.tile, tiles_m, tiles_n, p.group_m, m_tile, n_tile);
        if (kGrouped) e = p.expert_ids[m_tile];
      }
      if (lane == 0) {
        d->m_tile = m_tile, d->n_tile = n_tile, d->expert = e, d->kb_begin = un.kb_begin;
        d->kb_stop = un.kb_stop, d->split = un.split ? 1 : 0, d->slot = un.slot, d->pad = 0;
      }
      SGLB_SCOUT_STAMP(2);
      if (work && e >= 0) {
        // every load of the descriptor is requested before the first value is stored: one round trip to L2, not one
        // per row
        const int nb_tile = min(n_tile * BN / kScaleBlockN, p.nb_total - 1);
        const float* b_row0 = p.b_s + ((int64_t)e * p.nb_total + nb_tile) * kb_total + un.kb_begin;
        const float* b_row1 = p.b_s + ((int64_t)e * p.nb_total + min(nb_tile + 1, p.nb_total - 1)) * kb_total + un.kb_begin;
        const int n = min(un.kb_stop - un.kb_begin, kDescSlabs);
        float4 av[BM / 32];
        float bv0[4], bv1[4];
#pragma unroll
        for (int k = 0; k < BM / 32; ++k) {
          const int64_t row = (int64_t)m_tile * BM + lane + 32 * k;  // rows past M read a valid row; never stored
          av[k] = load_a4_row(p.a_s + min(row, rows - 1) * p.as_stride_m, un.kb_begin);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int i = lane + 32 * k;
          bv0[k] = i < n ? __ldg(b_row0 + i) : 0.f;
          bv1[k] = i < n ? __ldg(b_row1 + i) : 0.f;
        }
        const uint32_t d_addr = ptx::smem_u32(d);
#pragma unroll
        for (int k = 0; k < BM / 32; ++k)
          ptx::sts_128(d_addr + (uint32_t)offsetof(UnitDesc, a4) + (uint32_t)(lane + 32 * k) * 16u,
                       make_uint4(__float_as_uint(av[k].x), __float_as_uint(av[k].y), __float_as_uint(av[k].z),
                                  __float_as_uint(av[k].w)));
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int i = lane + 32 * k;
          if (i < n) {
            d->b[0][i] = bv0[k];
            d->b[1][i] = bv1[k];
          }
        }
        for (int i = lane + 128; i < n; i += 32) {  // (K beyond 16384)
          d->b[0][i] = __ldg(b_row0 + i);
          d->b[1][i] = __ldg(b_row1 + i);
        }
      }
      ptx::mbar_arrive(bar_dfull0 + ds * 8);  // every lane: its own writes are released with its arrival
      SGLB_SCOUT_STAMP(3);
      if (++ds == 2u) {
        ds = 0;
        dph ^= 1u;
      }
    }
  } else if (warp >= kEpiWarp0) {
    // ------------------------------ promotion + epilogue ------------------------------
    // A thread that sees the abort flag keeps walking the same loops (without waiting or touching TMEM) so
    // that the storing thread always collects all kEpiThreads arrivals per tile.
    const int q = warp & 3;                     // TMEM lane quadrant this warp may read
    const int cgrp = (warp - kEpiWarp0) >> 2;   // column group: columns cgrp*kEpiCols .. of the tile
    constexpr int kPiecesMax = kEpiCols / 32;
    const int row_in_tile = q * 32 + lane;
    const uint32_t bar_tfull0 = ptx::smem_u32(&ctl->tmem_full[0]), bar_tempty0 = ptx::smem_u32(&ctl->tmem_empty[0]);
    const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + cgrp * kEpiCols;
    const uint32_t bar_out_full = ptx::smem_u32(&ctl->out_full), bar_out_free = ptx::smem_u32(&ctl->out_free);
    const uint32_t bar_dfull0 = ptx::smem_u32(&ctl->desc_full[0]), bar_dempty0 = ptx::smem_u32(&ctl->desc_empty[0]);
    const uint32_t desc_addr0 = ptx::smem_u32(&ctl->desc[0]);
    uint32_t buf = 0, aph = 0, oph = 0, ds = 0, dph = 0;
    bool alive = true;
#ifdef SGLB_TRACE
    int trace_unit = -1;
#endif
    for (int u = blockIdx.x; u < num_units; u += gridDim.x) {
#ifdef SGLB_TRACE
      ++trace_unit;
#endif
      SGLB_STAMP(0);
      // the unit as the scout warp described it (without a descriptor there is nothing to walk: leave)
      if (!SGLB_WAIT(bar_dfull0 + ds * 8, dph)) {
        *abort_flag = 1;
        break;
      }
      const uint32_t desc_addr = desc_addr0 + ds * (uint32_t)sizeof(UnitDesc);
      // the descriptor is handed back (by every thread) once nothing more is read from it
      auto release_desc = [&]() {
        ptx::mbar_arrive(bar_dempty0 + ds * 8);
        if (++ds == 2u) {
          ds = 0;
          dph ^= 1u;
        }
      };
      const float4 h0 = ptx::lds_f32x4(desc_addr + (uint32_t)offsetof(UnitDesc, m_tile));
      const int m_tile = __float_as_int(h0.x), n_tile = __float_as_int(h0.y), kb_begin = __float_as_int(h0.w);
      const int kb_stop = __float_as_int(ptx::lds_f32(desc_addr + (uint32_t)offsetof(UnitDesc, kb_stop)));
      if (kb_begin >= kb_stop) {  // (an empty piece of a stream-K run; uniform over the CTA)
        release_desc();
        continue;
      }
      const int64_t row = (int64_t)m_tile * BM + row_in_tile;
      const int n0 = n_tile * BN + cgrp * kEpiCols;            // first of this warp's columns
      const int n_end = (int)min((int64_t)n_tile * BN + BN, p.N);  // one past the tile's last valid column
      const int e = kGrouped ? __float_as_int(h0.z) : 0;
      float acc[kEpiCols];
#pragma unroll
      for (int j = 0; j < kEpiCols; ++j) acc[j] = 0.f;
      if (e >= 0) {
        // Activation scales live in registers: the four scales of a thread's row for the unit's first four slabs come
        // from the descriptor; per later group of four slabs the thread loads them itself, the load for the next
        // group issued before the current group is promoted, a few thousand cycles ahead of its use.  The
        // weight-block scales (uniform across a warp: at most two 128-wide blocks per tile, one value per slab each)
        // are read from the descriptor slab by slab.  No barrier between the promotion warps.
        // A 32-column piece never straddles a weight block; a piece wholly past N is clamped to the last block.
        const int nb_tile = min(n_tile * BN / kScaleBlockN, p.nb_total - 1);
        bool piece_in_blk1[kPiecesMax];
#pragma unroll
        for (int i = 0; i < kPiecesMax; ++i)
          piece_in_blk1[i] = min((n0 + 32 * i) / kScaleBlockN, p.nb_total - 1) != nb_tile;
        const float* a_row = p.a_s + min(row, rows - 1) * p.as_stride_m;  // rows past M read a valid row; never stored
        auto load_a4 = [&](int kb) { return load_a4_row(a_row, kb); };
        float4 a_cur = ptx::lds_f32x4(desc_addr + (uint32_t)offsetof(UnitDesc, a4) + (uint32_t)row_in_tile * 16u);
        float4 a_nxt = a_cur;
        const int n_slabs = kb_stop - kb_begin;
        uint32_t b_addr = desc_addr + (uint32_t)offsetof(UnitDesc, b);
        SGLB_STAMP(1);
        for (int g = 0; g < n_slabs; ++g) {
          const int j = g & 3;
          if (j == 0) {
            if (g > 0) a_cur = a_nxt;
            if (g + 4 < n_slabs) a_nxt = load_a4(kb_begin + g + 4);
          }
          const float a_sc = j == 0 ? a_cur.x : j == 1 ? a_cur.y : j == 2 ? a_cur.z : a_cur.w;
          const float sc0 = a_sc * ptx::lds_f32(b_addr), sc1 = a_sc * ptx::lds_f32(b_addr + kDescSlabs * 4);
          b_addr += 4;
          // (the 32 lanes probe the same word in the same instruction, so the outcome is uniform across the
          // warp, as the warp-wide tcgen05.ld below requires)
          if (alive && !SGLB_WAIT(bar_tfull0 + buf * 8, aph)) {
            *abort_flag = 1;
            alive = false;
          }
          if (alive) {
            ptx::tc_fence_after();
            const uint32_t taddr = taddr0 + buf * kAccStride;
            // All 32-column pieces of the slab are requested before the one wait (tcgen05.wait::ld waits for
            // every outstanding load of the thread): one TMEM round trip per slab sits on the hand-off chain
            // MMA -> commit -> promotion -> release.  The buffer goes back to the MMA thread as soon as the
            // pieces are in registers.
            uint32_t r[kPiecesMax][32];
#pragma unroll
            for (int i = 0; i < kPiecesMax; ++i) ptx::tmem_ld_32x32(taddr + 32 * i, r[i]);
            ptx::tmem_ld_wait();
            ptx::tc_fence_before();
            ptx::mbar_arrive_if(bar_tempty0 + buf * 8, lane == 0);
#pragma unroll
            for (int i = 0; i < kPiecesMax; ++i) {
              const float sc = piece_in_blk1[i] ? sc1 : sc0;
#if SGLB_FMA2
              // two columns per instruction (packed float32 FMA: the same two IEEE operations): half the issue slots
#pragma unroll
              for (int jj = 0; jj < 32; jj += 2) ptx::fma2(acc[32 * i + jj], acc[32 * i + jj + 1], r[i][jj], r[i][jj + 1], sc);
#else
#pragma unroll
              for (int jj = 0; jj < 32; ++jj) acc[32 * i + jj] = fmaf(__uint_as_float(r[i][jj]), sc, acc[32 * i + jj]);
#endif
            }
          }
          if (++buf == (uint32_t)kAccBufs) {
            buf = 0;
            aph ^= 1u;
          }
        }
      }
      // (whether the unit is a piece of a split tile, and its slot among the partial sums, are read only now: two
      // registers fewer across the slab loop)
      Unit un;
      {
        const float4 h1 = ptx::lds_f32x4(desc_addr + (uint32_t)offsetof(UnitDesc, kb_stop));
        un.tile = 0, un.kb_begin = kb_begin, un.kb_stop = kb_stop;
        un.split = __float_as_int(h1.y) != 0, un.slot = __float_as_int(h1.z);
      }
      release_desc();
      // ---- store ----
      SGLB_STAMP(2);
      if (un.split) {
        // this unit's float32 partial sums, tile-local layout; a second kernel adds the units of a tile in a
        // fixed order, adds the bias and rounds once
        if (alive && row < rows) {  // (rows past M are never read back)
          // Layout of a block: with full tiles [column / 4][row][4], so that the 32 lanes of a warp (32 consecutive
          // rows) write 512 contiguous bytes per store; with a handful of rows (weight streaming) [row][BN], where
          // a row's columns stay together.  The reduction kernel reads it the same way.
          if (p.partial_rowmajor) {
            float* dst = p.partial + (int64_t)un.slot * (BM * BN) + row_in_tile * BN + cgrp * kEpiCols;
#pragma unroll
            for (int j = 0; j < kEpiCols / 4; ++j)
              *reinterpret_cast<float4*>(dst + j * 4) = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
          } else {
            float* dst = p.partial + (int64_t)un.slot * (BM * BN) + ((int64_t)(cgrp * kEpiCols / 4) * BM + row_in_tile) * 4;
#pragma unroll
            for (int j = 0; j < kEpiCols / 4; ++j)
              *reinterpret_cast<float4*>(dst + (int64_t)j * BM * 4) =
                  make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
          }
        }
        continue;
      }
      if (p.tma_out) {
        // Rows of C are contiguous: round to the output type, park the warp's 32 x 64 block in shared memory
        // (128-byte rows, 16-byte chunks XOR-swizzled by the row so that the 32 lanes of a store spread over
        // all banks); the storing thread (warp 2) hands the 128 x 64 blocks to the TMA engine, which clips them to
        // the tensor.  The store drains while the next tile is being promoted.
        // The staging area is free once the stores of the previous tile have read it (a thread whose wait expired
        // skips the data movement and still arrives, so that the storing thread is released).
        if (alive && !SGLB_WAIT(bar_out_free, oph ^ 1u)) {
          *abort_flag = 1;
          alive = false;
        }
        oph ^= 1u;
        SGLB_STAMP(3);
        if (alive && n0 < n_end) {
          if (p.bias != nullptr) {
            // (tile columns past N are clipped by the store; their bias reads are clamped to stay in bounds)
            const uint16_t* bsrc = static_cast<const uint16_t*>(p.bias);
#pragma unroll
            for (int j = 0; j < kEpiCols; ++j) {
              const uint16_t raw16 = __ldg(bsrc + min(n0 + j, (int)p.N - 1));
              acc[j] += p.out_fp16 ? __half2float(__ushort_as_half(raw16)) : __bfloat162float(__ushort_as_bfloat16(raw16));
            }
          }
          // round pairs of adjacent columns with one packed conversion each, then 16-byte shared-memory stores
          uint32_t packed[kEpiCols / 2];
          if (p.out_fp16) {
#pragma unroll
            for (int j = 0; j < kEpiCols / 2; ++j) {
              const __half2 h = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
              packed[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
          } else {
#pragma unroll
            for (int j = 0; j < kEpiCols / 2; ++j) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
              packed[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
          }
          const uint32_t stage0 = ptx::smem_u32(out_stage) + row_in_tile * 128;
          const uint32_t swz = (uint32_t)(row_in_tile & 7);
#pragma unroll
          for (int j = 0; j < kEpiCols / 8; ++j) {
            const int col = cgrp * kEpiCols + j * 8;  // within the tile: 64-column group col / 64, 16-byte chunk (col % 64) / 8
            ptx::sts_128(stage0 + (col >> 6) * kOutGroupBytes + ((((col & 63) >> 3) ^ swz) << 4),
                         make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]));
          }
          ptx::fence_async_smem();  // this thread's part is visible to the TMA engine before it arrives
        }
        SGLB_STAMP(4);
        ptx::mbar_arrive(bar_out_full);
        SGLB_STAMP(5);
        SGLB_STAMP(6);
        continue;
      }
      if (!alive) continue;
      int64_t out_row = row;
      bool store_ok = row < rows;
      if (kGrouped && p.scatter) {
        const int32_t id = store_ok ? p.sorted_ids[row] : -1;
        store_ok = id >= 0 && id < p.numel;
        out_row = id;
        if (store_ok && p.row_weights != nullptr) {
          const float w = __ldg(p.row_weights + id);
#pragma unroll
          for (int j = 0; j < kEpiCols; ++j) acc[j] *= w;
        }
      }
      if (store_ok && n0 < n_end) {
        if (p.out_fp16) {
          store_row_chunk<__half, kEpiCols>(static_cast<__half*>(p.C) + out_row * p.N + n0, acc, p.bias, n0, n_end);
        } else {
          store_row_chunk<__nv_bfloat16, kEpiCols>(static_cast<__nv_bfloat16*>(p.C) + out_row * p.N + n0, acc, p.bias, n0,
                                                   n_end);
        }
      }
    }
  }

  // ------------------------------ teardown ------------------------------
  // (the storing thread has waited for its last stores to read their source, in push mode to land, before it
  // reaches the barrier below)
  ptx::tc_fence_before();
  __syncthreads();
  if (ctl->abort_flag != 0 && threadIdx.x == 0) {
    atomicExch(&g_gemm_status, 1);
    // give TMA copies that may still be in flight time to land before the CTA's shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
  }
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Offset of element (row r of the tile, column c, a multiple of 4) inside a unit's partial sums: 128-row blocks one
// after the other, each laid out [column / 4][row][4] or, with `rowmajor`, [row][BN]; `step` = distance between
// the two float4 halves of an 8-column group.
__device__ __forceinline__ int64_t partial_offset(int r, int c, int BN, int rowmajor) {
  const int64_t blk = (int64_t)(r / BM) * (BM * BN);
  return rowmajor ? blk + (int64_t)(r % BM) * BN + c : blk + ((int64_t)(c >> 2) * BM + (r % BM)) * 4;
}
// Thread i of a tile's reduction -> (row, first of 8 columns): columns fastest for the row-major layout, rows
// fastest for the other, so that neighbouring threads read neighbouring words either way.
__device__ __forceinline__ void reduce_coord(int i, int tile_rows, int BN, int rowmajor, int& r, int& c8) {
  if (rowmajor) {
    r = i / (BN / 8);
    c8 = (i - r * (BN / 8)) * 8;
  } else {
    c8 = (i / tile_rows) * 8;
    r = i - (i / tile_rows) * tile_rows;
  }
}

// Sums the partial tiles of every split output tile in ascending split order (deterministic), adds the bias,
// rounds once and writes the part of the tile that lies inside C.  One thread per 8 consecutive columns of a row;
// grid = (split tiles, BM * BN / 8 / 256).
template <typename OutT>
__global__ void __launch_bounds__(256)
    split_reduce_kernel(const float* __restrict__ partial, OutT* __restrict__ C, const OutT* __restrict__ bias,
                        int64_t M, int64_t N, int BN, int tile_rows, int tiles_m, int tiles_n, int group_m,
                        int full_units, int splits, int rowmajor) {
  ptx::grid_dependency_wait();  // the GEMM's partial sums are complete and visible
  const int tile = full_units + blockIdx.x;
  int m_tile, n_tile;
  tile_coord(tile, tiles_m, tiles_n, group_m, m_tile, n_tile);
  // one thread per (row, 8-column group)
  int r, c8;
  reduce_coord(blockIdx.y * 256 + threadIdx.x, tile_rows, BN, rowmajor, r, c8);
  const int half = rowmajor ? 4 : BM * 4;
  const int64_t row = (int64_t)m_tile * tile_rows + r;
  const int64_t col = (int64_t)n_tile * BN + c8;
  if (c8 >= BN || r >= tile_rows || row >= M || col >= N) return;  // N is a multiple of 8: a group is inside or outside as a whole
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int64_t tile_elems = (int64_t)tile_rows * BN;  // (a pair's unit = two 128-row blocks one after the other)
  const float* src = partial + (int64_t)blockIdx.x * splits * tile_elems + partial_offset(r, c8, BN, rowmajor);
  for (int s = 0; s < splits; ++s, src += tile_elems) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(src)), b = __ldg(reinterpret_cast<const float4*>(src + half));
    acc[0] += a.x, acc[1] += a.y, acc[2] += a.z, acc[3] += a.w;
    acc[4] += b.x, acc[5] += b.y, acc[6] += b.z, acc[7] += b.w;
  }
  if (bias != nullptr) {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += ElemTraits<OutT>::to_f32(bias[col + j]);
  }
  uint4 raw;
  OutT* o = reinterpret_cast<OutT*>(&raw);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = ElemTraits<OutT>::from_f32(acc[j]);
  *reinterpret_cast<uint4*>(C + row * N + col) = raw;
}

// The same for stream-K runs: output tile `blockIdx.x` is the sum, in ascending K order, of the pieces of the runs
// that cover its slabs; run c covers slabs [c * share, (c + 1) * share) of the tiles x slabs space and its piece
// for this tile sits in slot c + ctas * (tile - first tile of the run).
template <typename OutT>
__global__ void __launch_bounds__(256)
    streamk_reduce_kernel(const float* __restrict__ partial, OutT* __restrict__ C, const OutT* __restrict__ bias,
                          int64_t M, int64_t N, int BN, int tile_rows, int tiles_m, int tiles_n, int group_m,
                          int kb_total, int share, int ctas, int rowmajor) {
  ptx::grid_dependency_wait();  // the GEMM's partial sums are complete and visible
  const int tile = blockIdx.x;
  int m_tile, n_tile;
  tile_coord(tile, tiles_m, tiles_n, group_m, m_tile, n_tile);
  int r, c8;
  reduce_coord(blockIdx.y * 256 + threadIdx.x, tile_rows, BN, rowmajor, r, c8);
  const int half = rowmajor ? 4 : BM * 4;
  const int64_t row = (int64_t)m_tile * tile_rows + r;
  const int64_t col = (int64_t)n_tile * BN + c8;
  if (c8 >= BN || r >= tile_rows || row >= M || col >= N) return;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int c_first = tile * kb_total / share, c_last = ((tile + 1) * kb_total - 1) / share;
  for (int c = c_first; c <= c_last; ++c) {
    const int slot = c + ctas * (tile - c * share / kb_total);
    const float* src = partial + (int64_t)slot * tile_rows * BN + partial_offset(r, c8, BN, rowmajor);
    const float4 a = __ldg(reinterpret_cast<const float4*>(src)), b = __ldg(reinterpret_cast<const float4*>(src + half));
    acc[0] += a.x, acc[1] += a.y, acc[2] += a.z, acc[3] += a.w;
    acc[4] += b.x, acc[5] += b.y, acc[6] += b.z, acc[7] += b.w;
  }
  if (bias != nullptr) {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += ElemTraits<OutT>::to_f32(bias[col + j]);
  }
  uint4 raw;
  OutT* o = reinterpret_cast<OutT*>(&raw);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = ElemTraits<OutT>::from_f32(acc[j]);
  *reinterpret_cast<uint4*>(C + row * N + col) = raw;
}

// How a dense problem is cut into units.
//  * Few tiles, long K, M <= 128 (weight streaming): stream-K over all SMs while the partial sums cost less than a
//    quarter of the weight bytes.
//  * Fewer than two waves of tiles with a long K otherwise (M = 256 or so): stream-K when its run of slabs plus
//    the cost of the partial sums is shorter than the whole waves it replaces.
//  * More tiles than SMs with a last wave that fills at most half of them: the tiles of that wave are split so
//    that the tail takes 1/splits of a tile time instead of a whole one (the other tiles are untouched).
#ifndef SGLB_TAIL_SPLIT
#define SGLB_TAIL_SPLIT 1
#endif
constexpr bool kTailSplit = SGLB_TAIL_SPLIT != 0;
#ifndef SGLB_STREAM_K
#define SGLB_STREAM_K 1
#endif
constexpr bool kStreamK = SGLB_STREAM_K != 0;
struct UnitPlan {
  int full_units, splits, kb_per_split;
  int64_t split_tiles;
  int sk_share, sk_ctas, sk_pieces;  // stream-K (sk_share > 0): supersedes the fields above
  int64_t scratch_blocks() const { return sk_share > 0 ? (int64_t)sk_pieces * sk_ctas : split_tiles * splits; }
};
// `tile_rows` x BN tiles shared among `sms` workers (SMs, or pairs of SMs for 256-row tiles).
static UnitPlan plan_units(int64_t M, int64_t N, int64_t K, int BN, int tile_rows, int sms) {
  const int kb_total = (int)((K + BK - 1) / BK);
  const int64_t tiles = ((M + tile_rows - 1) / tile_rows) * ((N + BN - 1) / BN);
  UnitPlan pl{(int)tiles, 1, kb_total, 0, 0, 0, 2};
  int64_t s = 1, split_tiles = 0;
  if (kStreamK && tiles < 2 * sms && kb_total >= 8 && kb_total % 4 == 0) {
    // Equal runs of slabs over ALL SMs (splitting every tile the same number of ways leaves sms mod tiles of
    // them idle).
    const int64_t total = tiles * kb_total;
    int64_t share = (total + sms - 1) / sms;
    share = (share + 3) / 4 * 4;  // runs start on multiples of four slabs: aligned 128-bit loads of the activation scales
    const int64_t ctas = (total + share - 1) / share;
    const int64_t rows = M < tile_rows ? M : tile_rows;
    const int pieces = share <= kb_total ? 2 : 3;
    bool take = false;
    if (tiles * 2 <= sms && pieces == 2) {
      // weight streaming: the partial sums (two pieces per CTA, M rows each, written and read back) stay below a
      // quarter of the weight bytes
      take = 2 * ctas * rows * BN * 4 * 2 * 4 <= N * K;
    } else if (share <= 2 * (int64_t)kb_total) {
      // Compared in slab times (about 0.45 us each): the run plus the partial sums (one piece per run and per
      // tile boundary, written and read back at about 4 TB/s, plus the second launch) against the whole waves.
      const int64_t waves = (tiles + sms - 1) / sms;
      const double partial_bytes = (double)(ctas + tiles) * tile_rows * BN * 4 * 2;
      const double cost = (double)share + partial_bytes / 1.8e6 + 6.0;
      take = cost < 0.9 * (double)(waves * kb_total);
    }
    if (take) {
      pl.sk_share = (int)share, pl.sk_ctas = (int)ctas, pl.sk_pieces = pieces;
      return pl;
    }
  }
  if (tiles * 2 <= sms && kb_total >= 8) {
    // (measured: splitting further, to several units per SM, costs more in partial-sum traffic and per-unit
    // start-up than it gains in balance)
    s = sms / tiles;
    const int64_t by_traffic = K / (32 * M);
    if (s > by_traffic) s = by_traffic;
    if (s > kb_total / 4) s = kb_total / 4;
    if (s > 16) s = 16;
    split_tiles = tiles;
  } else if (kTailSplit && tiles > sms && kb_total >= 32) {
    const int64_t tail = tiles % sms;
    if (tail > 0 && tail * 2 <= sms) {
      s = sms / tail;
      if (s > kb_total / 8) s = kb_total / 8;
      if (s > 8) s = 8;
      split_tiles = tail;
    }
  }
  if (s > 1) {
    int per = (int)((kb_total + s - 1) / s);
    per = (per + 3) / 4 * 4;  // keeps the 128-bit loads of the activation scales aligned
    pl.splits = (kb_total + per - 1) / per;
    pl.kb_per_split = per;
    if (pl.splits > 1) {
      pl.split_tiles = split_tiles;
      pl.full_units = (int)(tiles - split_tiles);
    } else {
      pl.kb_per_split = kb_total;
    }
  }
  return pl;
}

// ---------------------------------------------------------------------------------------------
// Host side: tensor maps (encoded through the driver entry point, cached per argument tuple)
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  uint64_t d0, d1, d2;
  uint32_t box_rows, rank;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && box_rows == o.box_rows && rank == o.rank;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ k.d0;
    h = h * 1000003u ^ k.d1;
    h = h * 1000003u ^ k.d2;
    return (h * 1000003u ^ k.box_rows) * 31u + k.rank;
  }
};

// uint8 tensor [d2][d1][d0] (d0 contiguous) described with `rank` (2 or 3) dimensions,
// box = 128 x box_rows (x 1), 128-byte swizzle, out-of-range elements read as zero.
static int get_tensor_map(const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t box_rows, uint32_t rank,
                          CUtensorMap* out) {
  static thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr, d0, d1, d2, box_rows, rank};
  auto itc = cache.find(key);
  if (itc != cache.end()) {
    *out = itc->second;
    return SGLB200_OK;
  }
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return fail(SGLB200_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {d0, d0 * d1};  // bytes (1-byte elements)
  cuuint32_t box[3] = {(cuuint32_t)BK, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SGLB200_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return SGLB200_OK;
}

// Output tensor [rows][N] of 2-byte elements, box = 64 columns x 128 rows, 128-byte swizzle (matches the
// staging layout written by the epilogue).
static int get_out_map(const void* ptr, uint64_t N, uint64_t rows, int out_fp16, CUtensorMap* out) {
  static thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr, N, rows, (uint64_t)out_fp16, 0, 0};
  auto itc = cache.find(key);
  if (itc != cache.end()) {
    *out = itc->second;
    return SGLB200_OK;
  }
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return fail(SGLB200_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {N, rows};
  cuuint64_t strides[1] = {N * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)BM};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, out_fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SGLB200_E_CUDA, "cuTensorMapEncodeTiled (output) failed with CUresult %d", (int)r);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return SGLB200_OK;
}

// m-tiles per rasterization group: as many as keep the group's activation rows (128*K bytes per m-tile) within
// a quarter of the L2 (measured: with half of it the streaming weight tiles start evicting the rows), in groups
// of equal size, so that the weights are read from DRAM once per group and the activations once in all.
static int choose_group_m(int64_t rows, int64_t K, int tile_rows = BM) {
  const int64_t budget = 32ll << 20;
  int64_t gmax = budget / (tile_rows * K);
  if (gmax < 2) gmax = 2;
  if (gmax < 4 && tile_rows == BM) gmax = 4;
  const int64_t tiles_m = (rows + tile_rows - 1) / tile_rows;
  const int64_t groups = (tiles_m + gmax - 1) / gmax;
  return (int)((tiles_m + groups - 1) / groups);
}

// Tile width of a dense problem (TileCfg).  Where the 192-wide tiling streams weights (stream-K, split tiles) or
// makes several waves, it wins: fewer tiles, fewer bytes per FLOP, and at large M the 128-wide tile runs at about
// 0.85 of its rate.  Where one wave of 192-wide tiles leaves SMs idle and K is not split, the 128-wide tile's
// extra tiles fill them.  Compared as waves x tile width, the 128-wide tile charged 150 instead of 128.
#ifndef SGLB_FORCE_BN
#define SGLB_FORCE_BN 0  // 128 or 192: one tile width for everything (measurements)
#endif
static int choose_bn(int64_t M, int64_t N, int64_t K) {
  if (SGLB_FORCE_BN) return SGLB_FORCE_BN;
  const int sms = sm_count();
  const UnitPlan p192 = plan_units(M, N, K, 192, BM, sms);
  if (p192.scratch_blocks() > 0) return 192;
  const int64_t tiles_m = (M + BM - 1) / BM;
  const int64_t waves192 = (tiles_m * ((N + 191) / 192) + sms - 1) / sms;
  const int64_t waves128 = (tiles_m * ((N + 127) / 128) + sms - 1) / sms;
  return waves128 * 150 < waves192 * 192 ? 128 : 192;
}
// The expert-grouped form: rows per expert are not known on the host; with a handful of routed rows (decode) the
// 128-wide tile spreads the few row blocks over more SMs, otherwise the 192-wide tile is ahead by 5-10 %.
static int choose_bn_grouped(int64_t numel) {
  if (SGLB_FORCE_BN) return SGLB_FORCE_BN;
  return numel <= 64 ? 128 : 192;
}

// How a dense problem runs: tile width and the cut into units.
struct DensePlan {
  int bn;
  UnitPlan units;
  int64_t scratch_bytes() const { return units.scratch_blocks() * (int64_t)BM * bn * (int64_t)sizeof(float); }
};
static DensePlan plan_dense(int64_t M, int64_t N, int64_t K) {
  DensePlan d;
  d.bn = choose_bn(M, N, K);
  d.units = plan_units(M, N, K, d.bn, BM, sm_count());
  return d;
}

static uint32_t g_wait_probes = ptx::kProbeLimit;  // sglb200_gemm_set_wait_probes

template <class Cfg>
static size_t gemm_smem_bytes() {
  return (size_t)Cfg::kStages * Cfg::kStageBytes + Cfg::kOutBytes + sizeof(SharedCtl<Cfg>) + 1024;
}

template <bool kGrouped, int BN>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const GemmParams& p,
                       int64_t max_units, cudaStream_t st, int sm_margin = 0) {
  const size_t smem = gemm_smem_bytes<TileCfg<BN>>();
  static thread_local bool attr_set[64] = {false};  // the opt-in is per function and per device
  int dev = 0;
  SGLB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    SGLB_CUDA(cudaFuncSetAttribute(fp8_blockscale_gemm_kernel<kGrouped, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)smem));
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  int sms = sm_count() - sm_margin;  // SMs left free run a concurrent kernel (the reduce-and-gather of an earlier chunk)
  if (sms < 1) sms = 1;
  const unsigned grid = (unsigned)(max_units < sms ? max_units : sms);
  fp8_blockscale_gemm_kernel<kGrouped, BN><<<grid, kGemmThreads, smem, st>>>(ma, mb, mc, p);
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}

template <int BN>
static int dense_mm(const DensePlan& dp, const void* A, const void* B, const float* a_s, const float* b_s, void* C,
                    const void* bias, int64_t M, int64_t N, int64_t K, int64_t as_stride_m, int64_t as_stride_k,
                    int out_dtype, void* workspace, int64_t workspace_bytes, cudaStream_t st) {
  constexpr int kTileRows = BM;
  CUtensorMap ma, mb;
  int rc = get_tensor_map(A, (uint64_t)K, (uint64_t)M, 1, BM, 2, &ma);
  if (rc) return rc;
  // B is addressed as [1][N][K] so that dense and grouped kernels share the 3-D load
  rc = get_tensor_map(B, (uint64_t)K, (uint64_t)N, 1, BN, 3, &mb);
  if (rc) return rc;
  GemmParams p{};
  p.a_s = a_s, p.b_s = b_s, p.C = C, p.bias = bias;
  p.M = M, p.N = N, p.K = K;
  p.as_stride_m = as_stride_m, p.as_stride_k = as_stride_k;
  p.kb_total = (int)((K + BK - 1) / BK), p.nb_total = (int)((N + kScaleBlockN - 1) / kScaleBlockN);
  p.tiles_n = (int)((N + BN - 1) / BN);
  p.group_m = choose_group_m(M, K, kTileRows);
  p.out_fp16 = out_dtype;
  p.wait_probes = g_wait_probes;
  UnitPlan pl = dp.units;
  const int64_t tiles = ((M + kTileRows - 1) / kTileRows) * p.tiles_n;
  if (pl.scratch_blocks() > 0 &&
      (workspace == nullptr || !aligned16(workspace) || workspace_bytes < dp.scratch_bytes()))
    pl = UnitPlan{(int)tiles, 1, p.kb_total, 0, 0, 0, 2};  // no scratch offered: one unit per tile
  p.full_units = pl.full_units, p.splits = pl.splits, p.kb_per_split = pl.kb_per_split;
  p.sk_share = pl.sk_share, p.sk_ctas = pl.sk_ctas, p.sk_pieces = pl.sk_pieces, p.sk_total = (int)(tiles * p.kb_total);
  p.partial = static_cast<float*>(workspace);
  p.partial_rowmajor = M <= 32 ? 1 : 0;
  CUtensorMap mc{};
  p.tma_out = pl.sk_share == 0 && pl.full_units > 0;
  if (p.tma_out) {
    rc = get_out_map(C, (uint64_t)N, (uint64_t)M, out_dtype, &mc);
    if (rc) return rc;
  }
  rc = launch_gemm<false, BN>(ma, mb, mc, p, pl.sk_share > 0 ? pl.sk_ctas : pl.full_units + pl.split_tiles * pl.splits, st);
  if (rc != SGLB200_OK || pl.scratch_blocks() == 0) return rc;
  const int tiles_m = (int)((M + kTileRows - 1) / kTileRows);
  const unsigned ygrid = (unsigned)((kTileRows * BN / 8 + 255) / 256);
  // The reduction is launched programmatically (it may be scheduled while the GEMM's last CTAs drain).
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(256, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int rowmajor = p.partial_rowmajor, bn = BN, tile_rows = kTileRows;
  if (pl.sk_share > 0) {
    cfg.gridDim = dim3((unsigned)tiles, ygrid, 1);
    if (out_dtype == 0)
      SGLB_CUDA(cudaLaunchKernelEx(&cfg, streamk_reduce_kernel<__nv_bfloat16>, (const float*)p.partial,
                                   static_cast<__nv_bfloat16*>(C), static_cast<const __nv_bfloat16*>(bias), M, N, bn,
                                   tile_rows, tiles_m, p.tiles_n, p.group_m, p.kb_total, pl.sk_share, pl.sk_ctas, rowmajor));
    else
      SGLB_CUDA(cudaLaunchKernelEx(&cfg, streamk_reduce_kernel<__half>, (const float*)p.partial, static_cast<__half*>(C),
                                   static_cast<const __half*>(bias), M, N, bn, tile_rows, tiles_m, p.tiles_n, p.group_m,
                                   p.kb_total, pl.sk_share, pl.sk_ctas, rowmajor));
    return SGLB200_OK;
  }
  cfg.gridDim = dim3((unsigned)pl.split_tiles, ygrid, 1);
  if (out_dtype == 0)
    SGLB_CUDA(cudaLaunchKernelEx(&cfg, split_reduce_kernel<__nv_bfloat16>, (const float*)p.partial,
                                 static_cast<__nv_bfloat16*>(C), static_cast<const __nv_bfloat16*>(bias), M, N, bn, tile_rows,
                                 tiles_m, p.tiles_n, p.group_m, pl.full_units, pl.splits, rowmajor));
  else
    SGLB_CUDA(cudaLaunchKernelEx(&cfg, split_reduce_kernel<__half>, (const float*)p.partial, static_cast<__half*>(C),
                                 static_cast<const __half*>(bias), M, N, bn, tile_rows, tiles_m, p.tiles_n, p.group_m,
                                 pl.full_units, pl.splits, rowmajor));
  return SGLB200_OK;
}

template <int BN>
static int grouped_mm(const void* A, const float* a_s, const void* B, const float* b_s, void* C,
                      const int32_t* sorted_token_ids, const int32_t* expert_ids, const int32_t* num_rows_dev,
                      const float* row_weights, int64_t max_rows, int64_t numel, int num_experts, int64_t N, int64_t K,
                      int scatter, int out_dtype, cudaStream_t st) {
  CUtensorMap ma, mb;
  int rc = get_tensor_map(A, (uint64_t)K, (uint64_t)max_rows, 1, BM, 2, &ma);
  if (rc) return rc;
  rc = get_tensor_map(B, (uint64_t)K, (uint64_t)N, (uint64_t)num_experts, BN, 3, &mb);
  if (rc) return rc;
  GemmParams p{};
  p.a_s = a_s, p.b_s = b_s, p.C = C, p.bias = nullptr;
  p.sorted_ids = sorted_token_ids, p.expert_ids = expert_ids, p.num_rows_dev = num_rows_dev;
  p.row_weights = row_weights;
  p.M = max_rows, p.N = N, p.K = K;
  p.kb_total = (int)((K + BK - 1) / BK), p.nb_total = (int)((N + kScaleBlockN - 1) / kScaleBlockN);
  p.tiles_n = (int)((N + BN - 1) / BN);
  p.group_m = choose_group_m(max_rows, K);
  p.as_stride_m = p.kb_total, p.as_stride_k = 1;
  p.numel = numel, p.scatter = scatter, p.out_fp16 = out_dtype;
  p.wait_probes = g_wait_probes;
  p.full_units = 0, p.splits = 1, p.kb_per_split = p.kb_total, p.partial = nullptr;  // grouped: one unit per tile
  p.sk_pieces = 2;
  CUtensorMap mc{};
  p.tma_out = !scatter;  // sorted-row output is contiguous; the scatter form writes token-major rows one by one
  if (p.tma_out) {
    rc = get_out_map(C, (uint64_t)N, (uint64_t)max_rows, out_dtype, &mc);
    if (rc) return rc;
  }
  const int64_t tiles = ((max_rows + BM - 1) / BM) * p.tiles_n;
  return launch_gemm<true, BN>(ma, mb, mc, p, tiles, st);
}

}  // namespace sglb200

using namespace sglb200;

extern "C" int sglb200_gemm_status_clear(void) {
  const int zero = 0;
  SGLB_CUDA(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int)));
  return SGLB200_OK;
}

extern "C" int sglb200_gemm_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

extern "C" void sglb200_gemm_set_wait_probes(uint32_t probes) { g_wait_probes = probes == 0 ? ptx::kProbeLimit : probes; }

extern "C" int64_t sglb200_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return plan_dense(M, N, K).scratch_bytes();
}

extern "C" int sglb200_fp8_blockwise_scaled_mm(const void* A, const void* B, const float* a_s, const float* b_s,
                                               void* C, const void* bias, int64_t M, int64_t N, int64_t K,
                                               int64_t as_stride_m, int64_t as_stride_k, int out_dtype,
                                               void* workspace, int64_t workspace_bytes, void* stream) {
  SGLB_REQUIRE(M >= 0 && N > 0 && K > 0, "fp8_blockwise_scaled_mm: bad shape M=%lld N=%lld K=%lld", (long long)M,
               (long long)N, (long long)K);
  SGLB_REQUIRE(K % 16 == 0, "fp8_blockwise_scaled_mm: K=%lld must be a multiple of 16", (long long)K);
  SGLB_REQUIRE(K <= (int64_t)kDescSlabs * BK, "fp8_blockwise_scaled_mm: K=%lld exceeds %d", (long long)K, kDescSlabs * BK);
  SGLB_REQUIRE(N % 8 == 0, "fp8_blockwise_scaled_mm: N=%lld must be a multiple of 8", (long long)N);
  SGLB_REQUIRE(out_dtype == 0 || out_dtype == 1, "fp8_blockwise_scaled_mm: out_dtype %d (0 bf16, 1 fp16)", out_dtype);
  if (M == 0) return SGLB200_OK;
  SGLB_REQUIRE(A && B && a_s && b_s && C, "fp8_blockwise_scaled_mm: null pointer");
  SGLB_REQUIRE(aligned16(A) && aligned16(B) && aligned16(C) && (bias == nullptr || aligned16(bias)),
               "fp8_blockwise_scaled_mm: A, B, C and bias must be 16-byte aligned");
  SGLB_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "fp8_blockwise_scaled_mm: dimension too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const DensePlan dp = plan_dense(M, N, K);
  if (dp.bn == 128)
    return dense_mm<128>(dp, A, B, a_s, b_s, C, bias, M, N, K, as_stride_m, as_stride_k, out_dtype, workspace,
                         workspace_bytes, st);
  return dense_mm<192>(dp, A, B, a_s, b_s, C, bias, M, N, K, as_stride_m, as_stride_k, out_dtype, workspace,
                       workspace_bytes, st);
}

extern "C" int sglb200_fp8_blockwise_grouped_mm(const void* A, const float* a_s, const void* B, const float* b_s,
                                                void* C, const int32_t* sorted_token_ids, const int32_t* expert_ids,
                                                const int32_t* num_rows_dev, const float* row_weights,
                                                int64_t max_rows, int64_t numel, int num_experts, int64_t N, int64_t K,
                                                int scatter, int out_dtype, void* stream) {
  SGLB_REQUIRE(max_rows >= 0 && N > 0 && K > 0 && num_experts >= 1, "grouped_mm: bad shape rows=%lld N=%lld K=%lld E=%d",
               (long long)max_rows, (long long)N, (long long)K, num_experts);
  SGLB_REQUIRE(K % 16 == 0 && N % 8 == 0, "grouped_mm: K must be a multiple of 16 and N of 8");
  SGLB_REQUIRE(K <= (int64_t)kDescSlabs * BK, "grouped_mm: K=%lld exceeds %d", (long long)K, kDescSlabs * BK);
  SGLB_REQUIRE(out_dtype == 0 || out_dtype == 1, "grouped_mm: out_dtype %d (0 bf16, 1 fp16)", out_dtype);
  if (max_rows == 0) return SGLB200_OK;
  SGLB_REQUIRE(A && a_s && B && b_s && C && expert_ids && num_rows_dev, "grouped_mm: null pointer");
  SGLB_REQUIRE(!scatter || sorted_token_ids, "grouped_mm: scatter mode needs sorted_token_ids");
  SGLB_REQUIRE(aligned16(A) && aligned16(B) && aligned16(C), "grouped_mm: A, B and C must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (choose_bn_grouped(numel) == 128)
    return grouped_mm<128>(A, a_s, B, b_s, C, sorted_token_ids, expert_ids, num_rows_dev, row_weights, max_rows, numel,
                           num_experts, N, K, scatter, out_dtype, st);
  return grouped_mm<192>(A, a_s, B, b_s, C, sorted_token_ids, expert_ids, num_rows_dev, row_weights, max_rows, numel,
                         num_experts, N, K, scatter, out_dtype, st);
}


// ---------------------------------------------------------------------------------------------
// Push mode: the GEMM of a row-parallel layer with the reduce-scatter folded into its epilogue.
// ---------------------------------------------------------------------------------------------
namespace sglb200 {

// Device copy of the per-owner output tensor maps, built once per (staging buffers, shape) and kept.
struct PushKey {
  const void* ptrs[8];
  uint64_t N, rows;
  int world, out_fp16;
  bool operator==(const PushKey& o) const {
    for (int i = 0; i < 8; ++i)
      if (ptrs[i] != o.ptrs[i]) return false;
    return N == o.N && rows == o.rows && world == o.world && out_fp16 == o.out_fp16;
  }
};
struct PushKeyHash {
  size_t operator()(const PushKey& k) const {
    size_t h = k.N * 1000003u ^ k.rows;
    for (int i = 0; i < 8; ++i) h = h * 1000003u ^ reinterpret_cast<size_t>(k.ptrs[i]);
    return h * 31u + (size_t)k.world * 2 + (size_t)k.out_fp16;
  }
};

static int get_push_maps(void* const* stage_ptrs, int world, uint64_t N, uint64_t rows, int out_fp16,
                         const CUtensorMap** out) {
  static thread_local std::unordered_map<PushKey, CUtensorMap*, PushKeyHash> cache;
  PushKey key{};
  for (int i = 0; i < world; ++i) key.ptrs[i] = stage_ptrs[i];
  key.N = N, key.rows = rows, key.world = world, key.out_fp16 = out_fp16;
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return SGLB200_OK;
  }
  CUtensorMap host[8];
  for (int i = 0; i < world; ++i) {
    const int rc = get_out_map(stage_ptrs[i], N, rows, out_fp16, &host[i]);
    if (rc) return rc;
  }
  CUtensorMap* dev = nullptr;
  SGLB_CUDA(cudaMalloc(&dev, sizeof(CUtensorMap) * 8));
  SGLB_CUDA(cudaMemcpy(dev, host, sizeof(CUtensorMap) * world, cudaMemcpyHostToDevice));
  cache.emplace(key, dev);
  *out = dev;
  return SGLB200_OK;
}

template <int BN>
static int push_mm(const void* A, const void* B, const float* a_s, const float* b_s, void* const* stage_ptrs, int world,
                   int rank, int64_t M, int64_t N, int64_t K, int64_t as_stride_m, int64_t as_stride_k, int out_dtype,
                   int sm_margin, cudaStream_t st) {
  constexpr int kTileRows = BM;
  CUtensorMap ma, mb;
  int rc = get_tensor_map(A, (uint64_t)K, (uint64_t)M, 1, BM, 2, &ma);
  if (rc) return rc;
  rc = get_tensor_map(B, (uint64_t)K, (uint64_t)N, 1, BN, 3, &mb);
  if (rc) return rc;
  GemmParams p{};
  p.a_s = a_s, p.b_s = b_s, p.C = nullptr, p.bias = nullptr;
  p.M = M, p.N = N, p.K = K;
  p.as_stride_m = as_stride_m, p.as_stride_k = as_stride_k;
  p.kb_total = (int)((K + BK - 1) / BK), p.nb_total = (int)((N + kScaleBlockN - 1) / kScaleBlockN);
  p.tiles_n = (int)((N + BN - 1) / BN);
  p.group_m = choose_group_m(M, K, kTileRows);
  p.out_fp16 = out_dtype;
  p.wait_probes = g_wait_probes;
  const int64_t tiles = ((M + kTileRows - 1) / kTileRows) * p.tiles_n;
  p.full_units = (int)tiles, p.splits = 1, p.kb_per_split = p.kb_total, p.partial = nullptr;  // one unit per tile
  p.sk_pieces = 2;
  p.tma_out = 1;
  // rows are owned in blocks of rpo = ceil(M / world) rounded up to whole tiles (the last owners may hold fewer
  // rows, or none); every owner's staging buffer is [world][rpo][N]
  const int64_t rpo = sglb200_push_rows_per_owner(M, world);
  rc = get_push_maps(stage_ptrs, world, (uint64_t)N, (uint64_t)(rpo * world), out_dtype, &p.push_maps);
  if (rc) return rc;
  p.push_rows_per_owner = (int)rpo, p.push_rank = rank;
  CUtensorMap mc = {};
  rc = get_out_map(stage_ptrs[rank], (uint64_t)N, (uint64_t)(rpo * world), out_dtype, &mc);  // unused by the stores; keeps map_c valid
  if (rc) return rc;
  return launch_gemm<false, BN>(ma, mb, mc, p, tiles, st, sm_margin);
}

}  // namespace sglb200

extern "C" int64_t sglb200_push_rows_per_owner(int64_t M, int world) {
  if (M <= 0 || world <= 0) return 0;
  const int64_t per = (M + world - 1) / world;
  return (per + BM - 1) / BM * BM;
}

extern "C" int sglb200_push_prepare(void* const* stage_ptrs, int world, int64_t M, int64_t N, int out_dtype) {
  SGLB_REQUIRE(world >= 2 && world <= 8 && stage_ptrs != nullptr, "push_prepare: world %d", world);
  SGLB_REQUIRE(M > 0 && N > 0 && N % 8 == 0 && (out_dtype == 0 || out_dtype == 1), "push_prepare: bad shape or dtype");
  for (int i = 0; i < world; ++i)
    SGLB_REQUIRE(stage_ptrs[i] != nullptr && aligned16(stage_ptrs[i]), "push_prepare: staging buffer %d missing or unaligned", i);
  const int64_t rpo = sglb200_push_rows_per_owner(M, world);
  const CUtensorMap* maps = nullptr;
  return get_push_maps(stage_ptrs, world, (uint64_t)N, (uint64_t)(rpo * world), out_dtype, &maps);
}

extern "C" int sglb200_fp8_blockwise_scaled_mm_push(const void* A, const void* B, const float* a_s, const float* b_s,
                                                    void* const* stage_ptrs, int world, int rank, int64_t M, int64_t N,
                                                    int64_t K, int64_t as_stride_m, int64_t as_stride_k, int out_dtype,
                                                    int sm_margin, void* stream) {
  SGLB_REQUIRE(world >= 2 && world <= 8 && rank >= 0 && rank < world, "mm_push: world %d, rank %d", world, rank);
  SGLB_REQUIRE(sm_margin >= 0 && sm_margin < sm_count(), "mm_push: sm_margin %d", sm_margin);
  SGLB_REQUIRE(M > 0 && N > 0 && K > 0, "mm_push: bad shape M=%lld N=%lld K=%lld", (long long)M, (long long)N,
               (long long)K);
  SGLB_REQUIRE(K % 16 == 0 && N % 8 == 0, "mm_push: K=%lld must be a multiple of 16 and N=%lld of 8", (long long)K,
               (long long)N);
  SGLB_REQUIRE(K <= (int64_t)kDescSlabs * BK, "mm_push: K=%lld exceeds %d", (long long)K, kDescSlabs * BK);
  SGLB_REQUIRE(out_dtype == 0 || out_dtype == 1, "mm_push: out_dtype %d (0 bf16, 1 fp16)", out_dtype);
  SGLB_REQUIRE(A && B && a_s && b_s && stage_ptrs, "mm_push: null pointer");
  for (int i = 0; i < world; ++i)
    SGLB_REQUIRE(stage_ptrs[i] != nullptr && aligned16(stage_ptrs[i]), "mm_push: staging buffer %d missing or unaligned", i);
  SGLB_REQUIRE(aligned16(A) && aligned16(B), "mm_push: A and B must be 16-byte aligned");
  SGLB_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "mm_push: dimension too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (choose_bn(M, N, K) == 128)
    return push_mm<128>(A, B, a_s, b_s, stage_ptrs, world, rank, M, N, K, as_stride_m, as_stride_k, out_dtype, sm_margin, st);
  return push_mm<192>(A, B, a_s, b_s, stage_ptrs, world, rank, M, N, K, as_stride_m, as_stride_k, out_dtype, sm_margin, st);
}

#ifdef SGLB_TRACE
extern "C" int sglb200_debug_trace(void* host_buf, int64_t bytes) {
  if (bytes != (int64_t)sizeof(long long) * 3 * kTraceUnits * kTraceStamps) return -1;
  return cudaMemcpyFromSymbol(host_buf, g_trace, (size_t)bytes) == cudaSuccess ? 0 : -2;
}
#endif
