// Block-scaled FP8 GEMM (dense and expert-grouped) for sm_100a.
//
//   C[m,n] = out_t( sum_kb a_s[m,kb] * b_s[n/128,kb] * sum_{k in kb} A[m,k] * B[n,k] )
//
// One persistent CTA per SM walks 128 x BN output tiles.  BN = 192 for long K (a 128x128 tile needs 128 B/clk
// per SM from L2 at full tensor rate, more than the fabric delivers; 128x192 needs 107, and its 32-column
// pieces never straddle a 128-wide scale block); BN = 128 with four accumulator buffers for short K, where a
// whole tile's partial sums fit in tensor memory and the MMAs of the next tile run under the epilogue of the
// current one.  Per 128-wide K slab:
//   * warp 0 (one elected lane) issues two TMA tile loads (A 128 rows x 128 B, B BN rows x 128 B,
//     128-byte swizzle) into a shared-memory ring, signalled through `full` mbarriers;
//   * warp 1 (one elected lane) issues four tcgen05.mma kind::f8f6f4 (128 x BN x 32) that write the
//     slab's partial sums into one of the TMEM buffers, then commits the slab to the `empty` barrier of
//     the ring slot and to the `tmem_full` barrier of the buffer;
//   * warps 4-11 (two per TMEM lane quadrant, BN/2 columns each) pull the partial sums out of TMEM with
//     32-column tcgen05.ld issued back to back, release the buffer, and promote them into float32 register
//     accumulators with the slab's scale a_s[m,kb]*b_s[nb,kb] (DeepSeek-style 128-block float scales cannot be
//     folded into the hardware's power-of-two MX scaling, so promotion runs on the CUDA cores, overlapped with
//     the next slab's MMAs through the TMEM buffers).  The slab loop is unrolled four ways: every unit starts
//     at buffer 0, so buffer, barrier and TMEM addresses are compile-time constants and the four activation
//     scales of a group are the components of one 128-bit load issued a group ahead.  The weight-block scales
//     of the tile are staged by each warp for itself in its own strip of shared memory (64 slabs at a time,
//     double-buffered), so the slab loop has no barrier between warps.
// The kernel runs power- and issue-limited rather than tensor-limited: every instruction a promotion warp
// executes or a waiting warp spends polling costs time, so the per-slab code is kept short and waits suspend
// in hardware (mbarrier.try_wait with a time hint).
// Epilogue: each promotion warp rounds its 32 rows x BN/2 columns to bf16/fp16, parks them in its own part of
// shared memory (32 x 32 pieces, 64-byte swizzle) and its lane 0 hands the pieces to the TMA engine; the
// stores drain during the next tile, and no barrier spans the warps.  The scales of the NEXT unit are requested
// before the epilogue so that they arrive under it.  In grouped "scatter" mode the epilogue multiplies by the
// routing weight and writes 16 bytes at a time to the token-major row named by sorted_token_ids.
// Scheduling: with fewer than two waves of tiles and a long K the tiles x slabs space is cut into one equal
// run of slabs per SM (stream-K; a run covers the end of one tile, possibly a whole tile, and the start of the
// next); otherwise the tiles of a short last wave are split along K.  Split work writes float32 partial sums
// that a second kernel adds in ascending K order.  In push mode (row-parallel layers under tensor parallelism)
// a tile is stored through the tensor map of the staging buffer of the GPU that owns its rows, which folds the
// reduce-scatter of the all-reduce into the epilogue.
//
// Every mbarrier wait is bounded; on expiry the role raises a flag in shared memory that the other waiters
// poll, the CTA sets a status word, drains, frees its TMEM and returns (sglb200_gemm_status() reports it).
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
#ifndef SGLB_EPI_WARPS_128
#define SGLB_EPI_WARPS_128 8              // promotion warps of the 128-wide tile (8 or 16); the 192-wide tile has 8
#endif
constexpr uint32_t kTileBytesA = BM * BK;  // fp8
constexpr int kBChunk = 64;                // slabs of weight-block scales a promotion warp stages at a time
#ifndef SGLB_LOOKAHEAD_ALL
#define SGLB_LOOKAHEAD_ALL 0
#endif
#ifndef SGLB_FMA2
#define SGLB_FMA2 1                        // promotion with packed float32 FMAs (two columns per instruction)
#endif
#ifndef SGLB_SHORT_K
#define SGLB_SHORT_K 1000000               // problems with at most this many K slabs use the 128-wide tile (all of
                                           // them: measured equal to the 192-wide tile at M >= 1024 and 10-30 % ahead
                                           // of it below, dense and grouped; the 192-wide tile stays selectable)
#endif

// kPair: two CTAs (a cluster of two SMs) share 256 x BN tiles through tcgen05.mma.cta_group::2; each stages its own
// 128 rows of A and HALF of the BN rows of B, so a slab costs 28 KB of shared-memory writes and 28 KB of operand
// reads per SM instead of 40 + 40 (shared memory moves 128 B/clk: a single CTA is capped at about 60 % of the
// tensor rate by it).
template <int BN_, bool kPair_ = false>
struct TileCfg {
  static constexpr int BN = BN_;
  static constexpr bool kPair = kPair_;
  static constexpr int kBRows = kPair_ ? BN_ / 2 : BN_;  // rows of B this CTA stages per slab
  static constexpr int kStages = kPair_ ? (BN_ >= 192 ? 6 : 7) : (BN_ >= 192 ? 4 : 5);
  static constexpr int kAccBufs = kTmemCols / BN_;   // TMEM accumulator buffers in flight
  static constexpr int kAccStride = BN_;             // TMEM columns between buffers
  static constexpr int kEpiWarps = BN_ == 128 ? SGLB_EPI_WARPS_128 : 8;  // promotion + epilogue warps
  static constexpr int kColGroups = kEpiWarps / 4;   // promotion warps per TMEM lane quadrant
  static constexpr int kThreads = kEpiWarp0 * 32 + kEpiWarps * 32;
  static constexpr int kEpiCols = BN_ / kColGroups;  // columns of a buffer owned by one promotion warp
  static constexpr int kPieces = kEpiCols / 32;      // 32-column pieces per warp
  static constexpr uint32_t kTileBytesB = kBRows * BK;
  static constexpr uint32_t kStageBytes = kTileBytesA + kTileBytesB;
  // output staging for the TMA store: per TMEM lane quadrant and 64 columns a [32 rows][64 columns] 2-byte block in
  // the 128-byte swizzle
  static constexpr int kOutGroups = BN_ / 64;
  static constexpr uint32_t kGroupBytes = 32 * 64 * 2;
  static constexpr uint32_t kOutBytes = 4 * kOutGroups * kGroupBytes;
  static_assert(kEpiWarps % 4 == 0 && kEpiCols % 32 == 0 && BN_ % 64 == 0 && (4 % kAccBufs) == 0 && kAccBufs * kAccStride <= kTmemCols && BN_ <= 256 &&
                    kStageBytes % 1024 == 0,
                "accumulator layout");
};

__device__ int g_gemm_status = 0;  // 0 ok, 1 = a pipeline wait expired

#ifdef SGLB_TRACE
// Development builds only: per-slab clock stamps of the roles of CTAs 0 and 1 (sglb200_debug_trace copies them out).
constexpr int kTraceSlabs = 256, kTraceEvents = 4, kTraceRoles = 3;
__device__ long long g_trace[2][kTraceRoles][kTraceSlabs][kTraceEvents];
#define SGLB_STAMP(role, n, ev)                                                                  \
  do {                                                                                           \
    if (blockIdx.x < 2 && (n) < kTraceSlabs) g_trace[blockIdx.x][role][n][ev] = clock64();       \
  } while (0)
#else
#define SGLB_STAMP(role, n, ev) \
  do {                          \
  } while (0)
#endif

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

template <class Cfg>
struct SharedCtl {
  float b_strip[Cfg::kEpiWarps][2][2][kBChunk];  // per promotion warp: [buffer][weight block within the tile][slab]
  uint64_t full[Cfg::kStages];
  uint64_t empty[Cfg::kStages];
  uint64_t tmem_full[Cfg::kAccBufs];
  uint64_t tmem_empty[Cfg::kAccBufs];
  uint32_t tmem_base;
  int abort_flag;
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

// One K slab of one promotion warp: wait for the slab's partial sums in TMEM buffer B, pull this warp's columns
// into registers, hand the buffer back, and add them, scaled, to the accumulators.  `bsc[i]` is the weight-block
// scale of the warp's i-th 32-column piece for this slab.  Returns false when the wait expired.
template <class Cfg>
__device__ __forceinline__ void release_buffer(uint32_t bar, uint32_t lane0) {
  if (Cfg::kPair)
    ptx::mbar_arrive_cluster_if(bar, lane0);
  else
    ptx::mbar_arrive_if(bar, lane0);
}
template <class Cfg, int B>
__device__ __forceinline__ bool promote_slab(uint32_t bar_tfull0, uint32_t bar_tempty0, uint32_t taddr0,
                                             uint32_t (&par)[Cfg::kAccBufs], uint32_t lane0, bool active, float a_sc,
                                             const float (&bsc)[Cfg::kPieces], float (&acc)[Cfg::kEpiCols],
                                             volatile int* abort_flag, uint32_t probes, int tn = -1) {
  (void)tn;  // (slab counter of the development trace: stamps only where tn >= 0)
  // (the 32 lanes probe the same word in the same instruction, so the outcome is uniform across the warp, as
  // the warp-wide tcgen05.ld below requires)
  if (tn >= 0) SGLB_STAMP(2, tn, 0);
  if (!ptx::mbar_wait_bounded(bar_tfull0 + B * 8, par[B], abort_flag, probes)) return false;
  if (tn >= 0) SGLB_STAMP(2, tn, 1);
  par[B] ^= 1u;
  ptx::tc_fence_after();
#ifdef SGLB_DBG_NOLDTM
  active = false;  // (development: promotion only hands the buffer back)
#endif
  if (active) {
    // All pieces of the slab are requested before the one wait (tcgen05.wait::ld waits for every outstanding
    // load of the thread): one TMEM round trip per slab sits on the hand-off chain MMA -> commit -> promotion
    // -> release.  The buffer goes back to the MMA thread as soon as the pieces are in registers.
    uint32_t r[Cfg::kPieces][32];
#pragma unroll
    for (int i = 0; i < Cfg::kPieces; ++i) ptx::tmem_ld_32x32(taddr0 + B * Cfg::kAccStride + 32 * i, r[i]);
    ptx::tmem_ld_wait();
    ptx::tc_fence_before();
    release_buffer<Cfg>(bar_tempty0 + B * 8, lane0);
    if (tn >= 0) SGLB_STAMP(2, tn, 2);
#ifdef SGLB_DBG_NOFMA
    // (development: one add per piece keeps the loads alive)
#pragma unroll
    for (int i = 0; i < Cfg::kPieces; ++i) acc[32 * i] += __uint_as_float(r[i][0] ^ r[i][31]) * a_sc * bsc[i];
#elif SGLB_FMA2
    // two columns per instruction (packed float32 FMA): half the issue slots of the promotion
#pragma unroll
    for (int i = 0; i < Cfg::kPieces; ++i) {
      const float sc = a_sc * bsc[i];
#pragma unroll
      for (int jj = 0; jj < 32; jj += 2)
        ptx::fma2(acc[32 * i + jj], acc[32 * i + jj + 1], r[i][jj], r[i][jj + 1], sc);
    }
#else
#pragma unroll
    for (int i = 0; i < Cfg::kPieces; ++i) {
      const float sc = a_sc * bsc[i];
#pragma unroll
      for (int jj = 0; jj < 32; ++jj) acc[32 * i + jj] = fmaf(__uint_as_float(r[i][jj]), sc, acc[32 * i + jj]);
    }
#endif
    if (tn >= 0) SGLB_STAMP(2, tn, 3);
  } else {
    // a warp whose 32 rows all lie past M has nothing to add: it only keeps the buffer hand-off in step
    ptx::tc_fence_before();
    release_buffer<Cfg>(bar_tempty0 + B * 8, lane0);
  }
  return true;
}

template <bool kGrouped, int BN_, bool kPair>
__global__ void __launch_bounds__((TileCfg<BN_, kPair>::kThreads), 1)
    fp8_blockscale_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                               const __grid_constant__ CUtensorMap map_c, const GemmParams p) {
  static_assert(!(kGrouped && kPair), "the rows of a pair tile share one weight matrix");
  using Cfg = TileCfg<BN_, kPair>;
  constexpr int kTileRows = kPair ? 2 * BM : BM;  // rows of a scheduling tile
  constexpr int kEpiWarps = Cfg::kEpiWarps;
  constexpr int BN = Cfg::BN, kStages = Cfg::kStages, kAccBufs = Cfg::kAccBufs, kEpiCols = Cfg::kEpiCols,
                kPieces = Cfg::kPieces;
  constexpr uint32_t kStageBytes = Cfg::kStageBytes, kGroupBytes = Cfg::kGroupBytes;
  extern __shared__ uint8_t smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* out_stage = tiles + kStages * kStageBytes;
  SharedCtl<Cfg>* ctl = reinterpret_cast<SharedCtl<Cfg>*>(out_stage + Cfg::kOutBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &ctl->abort_flag;
  const uint32_t probes = p.wait_probes;

  int64_t rows = p.M;
  if (kGrouped) {
    const int64_t lim = *p.num_rows_dev;
    rows = lim < rows ? lim : rows;
  }
  const int tiles_m = (int)((rows + kTileRows - 1) / kTileRows);
  const int tiles_n = p.tiles_n;
  const int num_tiles = tiles_m * tiles_n;
  // a pair walks its units together: both CTAs see the same sequence
  const uint32_t crank = kPair ? ptx::cluster_ctarank() : 0u;
  const int unit0 = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int unit_step = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int kb_total = p.kb_total;
  const int num_units = kGrouped         ? num_tiles
                        : p.sk_share > 0 ? p.sk_pieces * p.sk_ctas
                                         : p.full_units + (num_tiles - p.full_units) * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->empty[s]), 1);
    }
    for (int b = 0; b < kAccBufs; ++b) {
      ptx::mbar_init(ptx::smem_u32(&ctl->tmem_full[b]), 1);
      // (a pair: the leader's barrier collects the promotion warps of both CTAs)
      ptx::mbar_init(ptx::smem_u32(&ctl->tmem_empty[b]), kPair ? 2 * kEpiWarps : kEpiWarps);
    }
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
  if (kPair) ptx::cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  ptx::tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  auto raise_abort = [&]() {
    *abort_flag = 1;
    if (kPair) ptx::st_cluster_u32(ptx::mapa(ptx::smem_u32(&ctl->abort_flag), crank ^ 1u), 1u);  // the peer leaves too
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (ptx::elect_one()) {
      const uint32_t bar_empty0 = ptx::smem_u32(&ctl->empty[0]), bar_full0 = ptx::smem_u32(&ctl->full[0]);
      // (a pair: the bytes of both CTAs are counted on the leader's barrier, which the leader arms for both)
      const uint32_t bar_full_lead0 = kPair ? ptx::mapa(bar_full0, 0) : bar_full0;
      const uint32_t tiles0 = ptx::smem_u32(tiles);
      uint32_t s = 0, ph = 0;
      bool alive = true;
      int tn = 0;
      (void)tn;
      for (int u = unit0; u < num_units && alive; u += unit_step) {
        const Unit un = decode_unit<kGrouped>(p, u);
        const int kb_begin = un.kb_begin, kb_stop = un.kb_stop;
        if (kb_begin >= kb_stop) continue;
        int m_tile, n_tile;
        tile_coord(un.tile, tiles_m, tiles_n, p.group_m, m_tile, n_tile);
        if (kPair) m_tile = 2 * m_tile + (int)crank;
        int e = 0;
        if (kGrouped) {
          e = p.expert_ids[m_tile];
          if (e < 0) continue;
        }
        // this thread shares its scheduler with promotion warps that always have work: every instruction it
        // spends per slab delays the loads, so the loop keeps only 32-bit counters that step
        const int row_a = m_tile * BM, row_b = n_tile * BN + (int)crank * Cfg::kBRows;
        for (int k0 = kb_begin * BK; k0 < kb_stop * BK; k0 += BK) {
          SGLB_STAMP(0, tn, 0);
          if (!ptx::mbar_wait_bounded(bar_empty0 + s * 8, ph ^ 1u, abort_flag, probes)) {
            raise_abort();
            alive = false;
            break;
          }
          SGLB_STAMP(0, tn, 1);
          ++tn;
          const uint32_t dst_a = tiles0 + s * kStageBytes;
          if (kPair) {
            if (crank == 0) ptx::mbar_arrive_expect_tx(bar_full0 + s * 8, 2 * kStageBytes);
            const uint32_t bar = bar_full_lead0 + s * 8;
            ptx::tma_load_2d_pair(dst_a, &map_a, bar, k0, row_a);
            ptx::tma_load_3d_pair(dst_a + kTileBytesA, &map_b, bar, k0, row_b, e);
          } else {
            const uint32_t bar = bar_full0 + s * 8;
            ptx::mbar_arrive_expect_tx(bar, kStageBytes);
            ptx::tma_load_2d(dst_a, &map_a, bar, k0, row_a);
            ptx::tma_load_3d(dst_a + kTileBytesA, &map_b, bar, k0, row_b, e);
          }
          if (++s == (uint32_t)kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (ptx::elect_one() && crank == 0) {  // (of a pair, the leader issues the MMAs for both CTAs)
      constexpr uint32_t idesc = ptx::make_idesc_e4m3_f32(kTileRows, BN);
      // Operand descriptor (K-major, 128-byte swizzle): low word = address/16 | LBO(1) << 16, high word =
      // SBO(1024/16) | version 1 (bit 46) | layout SWIZZLE_128B (2 at bit 61).  Only the low word changes.
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t desc_lo0 = ((ptx::smem_u32(tiles) & 0x3ffffu) >> 4) | (1u << 16);
      const uint32_t bar_full0 = ptx::smem_u32(&ctl->full[0]), bar_empty0 = ptx::smem_u32(&ctl->empty[0]);
      const uint32_t bar_tfull0 = ptx::smem_u32(&ctl->tmem_full[0]), bar_tempty0 = ptx::smem_u32(&ctl->tmem_empty[0]);
      uint32_t s = 0, ph = 0;
      uint32_t tpar = 0;  // bit b: parity of the last completed release of TMEM buffer b
      bool alive = true;
      for (int u = unit0; u < num_units && alive; u += unit_step) {
        const Unit un = decode_unit<kGrouped>(p, u);
        const int kb_begin = un.kb_begin, kb_stop = un.kb_stop;
        if (kb_begin >= kb_stop) continue;
        if (kGrouped) {
          int m_tile, n_tile;
          tile_coord(un.tile, tiles_m, tiles_n, p.group_m, m_tile, n_tile);
          if (p.expert_ids[m_tile] < 0) continue;
        }
        uint32_t buf = 0;  // every unit starts at buffer 0 (the promotion warps count on it)
        bool ok = true;
        for (int kb = kb_begin; kb < kb_stop; ++kb) {
          // (Measured: doing the next slab's waits between this slab's MMAs instead gains nothing with four TMEM
          // buffers and loses a quarter with two, where the next buffer is still being read.)
          ok = ptx::mbar_wait_bounded(bar_tempty0 + buf * 8, ((tpar >> buf) & 1u) ^ 1u, abort_flag, probes) &&
               ptx::mbar_wait_bounded(bar_full0 + s * 8, ph, abort_flag, probes);
          if (!ok) break;
          ptx::tc_fence_after();
          const uint32_t a_lo = desc_lo0 + s * (kStageBytes >> 4);
          const uint32_t b_lo = a_lo + (kTileBytesA >> 4);
          const uint32_t d_tmem = tmem_base + buf * Cfg::kAccStride;
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            // advancing 32 bytes along K inside the 128-byte swizzled row = +2 in the descriptor's 16-byte units
            if (kPair)
              ptx::mma_f8f6f4_pair(d_tmem, ptx::pack_f32x2(a_lo + 2 * k, kDescHi), ptx::pack_f32x2(b_lo + 2 * k, kDescHi),
                                   idesc, k > 0 ? 1u : 0u);
            else
              ptx::mma_f8f6f4(d_tmem, ptx::pack_f32x2(a_lo + 2 * k, kDescHi), ptx::pack_f32x2(b_lo + 2 * k, kDescHi), idesc,
                              k > 0 ? 1u : 0u);
          }
          if (kPair) {  // (both CTAs' ring slots are free, both CTAs' promotion warps may read)
            ptx::mma_commit_pair(bar_empty0 + s * 8);
            ptx::mma_commit_pair(bar_tfull0 + buf * 8);
          } else {
            ptx::mma_commit(bar_empty0 + s * 8);
            ptx::mma_commit(bar_tfull0 + buf * 8);
          }
          if (++s == (uint32_t)kStages) {
            s = 0;
            ph ^= 1u;
          }
          tpar ^= 1u << buf;
          if (++buf == (uint32_t)kAccBufs) buf = 0;
        }
        if (!ok) {
          raise_abort();
          alive = false;
        }
      }
    }
  } else if (warp >= kEpiWarp0) {
    // ------------------------------ promotion + epilogue ------------------------------
    const int pw = warp - kEpiWarp0;
    const int q = warp & 3;      // TMEM lane quadrant this warp may read
    const int cgrp = pw >> 2;    // column group: columns cgrp*kEpiCols .. of the tile
    const int row_in_tile = q * 32 + lane;
    const uint32_t lane0 = lane == 0 ? 1u : 0u;
    const bool vec_scales = p.as_stride_k == 1 && (p.as_stride_m & 3) == 0 &&
                            (reinterpret_cast<uintptr_t>(p.a_s) & 15u) == 0;
    // (a pair: buffers are handed back on the leader's barrier, through the cluster's shared-memory window)
    const uint32_t bar_tfull0 = ptx::smem_u32(&ctl->tmem_full[0]);
    const uint32_t bar_tempty0 = kPair ? ptx::mapa(ptx::smem_u32(&ctl->tmem_empty[0]), 0) : ptx::smem_u32(&ctl->tmem_empty[0]);
    const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + cgrp * kEpiCols;
    const uint32_t strip0 = ptx::smem_u32(&ctl->b_strip[pw][0][0][0]);
    constexpr uint32_t kStripBytes = 2 * kBChunk * 4;  // one buffer of the strip: two weight blocks x kBChunk slabs
    const uint32_t stage_q = ptx::smem_u32(out_stage) + q * Cfg::kOutGroups * kGroupBytes;  // this quadrant's staging
    uint32_t par[kAccBufs];
#pragma unroll
    for (int b = 0; b < kAccBufs; ++b) par[b] = 0;
    bool alive = true;
#ifdef SGLB_TRACE
    int tslab = 0;  // slabs this warp has promoted (development trace, first promotion warp's lane 0 only)
#define SGLB_TN ((pw == 0 && lane == 0) ? tslab++ : -1)
#else
#define SGLB_TN (-1)
#endif

    // what a promotion warp needs to know about a unit
    struct Hdr {
      int m_tile, n_tile, e, kb_begin, kb_stop, slot;
      bool split, work;
    };
    auto header = [&](int u) {
      Hdr h;
      const Unit un = decode_unit<kGrouped>(p, u);
      tile_coord(un.tile, tiles_m, tiles_n, p.group_m, h.m_tile, h.n_tile);
      if (kPair) h.m_tile = 2 * h.m_tile + (int)crank;
      h.kb_begin = un.kb_begin, h.kb_stop = un.kb_stop, h.slot = un.slot, h.split = un.split;
      h.work = un.kb_begin < un.kb_stop;  // (an empty piece of a stream-K run: skipped by every role)
      h.e = 0;
      if (kGrouped) h.e = p.expert_ids[h.m_tile];
      return h;
    };
    // activation scales of slabs kb .. kb+3 of one row (zero past the last slab)
    auto load_a4 = [&](const float* a_row, int kb) {
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
    auto a_row_of = [&](const Hdr& h) {  // rows past M read a valid row; never stored
      const int64_t row = (int64_t)h.m_tile * BM + row_in_tile;
      return p.a_s + (row < rows ? row : rows - 1) * p.as_stride_m;
    };
    // weight-block scales (uniform across a warp: at most two 128-wide blocks per tile, one value per slab each)
    auto b_rows_of = [&](const Hdr& h, const float*& r0, const float*& r1) {
      const int nb_tile = min(h.n_tile * BN / kScaleBlockN, p.nb_total - 1);
      r0 = p.b_s + ((int64_t)h.e * p.nb_total + nb_tile) * kb_total;
      r1 = p.b_s + ((int64_t)h.e * p.nb_total + min(nb_tile + 1, p.nb_total - 1)) * kb_total;
    };
    // lane l fetches slabs kb0 + l and kb0 + 32 + l of both blocks (clamped: values past the last slab are unused)
    auto fetch_b = [&](const float* r0, const float* r1, int kb0, float (&v)[4]) {
      const int k0 = min(kb0 + lane, kb_total - 1), k1 = min(kb0 + 32 + lane, kb_total - 1);
      v[0] = __ldg(r0 + k0), v[1] = __ldg(r0 + k1), v[2] = __ldg(r1 + k0), v[3] = __ldg(r1 + k1);
    };
    auto store_b = [&](uint32_t strip, const float (&v)[4]) {
      __syncwarp();  // every lane is done reading what the buffer held
      ptx::sts_f32(strip + lane * 4, v[0]);
      ptx::sts_f32(strip + (32 + lane) * 4, v[1]);
      ptx::sts_f32(strip + (kBChunk + lane) * 4, v[2]);
      ptx::sts_f32(strip + (kBChunk + 32 + lane) * 4, v[3]);
      __syncwarp();
    };

    // The scales a unit starts with (its first four activation scales, its first chunk of weight-block scales)
    // are requested one unit ahead, before the previous unit's epilogue, and so arrive under it.
    float4 a_first = make_float4(0.f, 0.f, 0.f, 0.f);
    float bv[4] = {0.f, 0.f, 0.f, 0.f};
    auto prefetch = [&](const Hdr& h) {
      if (!h.work || h.e < 0) return;
      const float *r0, *r1;
      b_rows_of(h, r0, r1);
      fetch_b(r0, r1, h.kb_begin, bv);
      a_first = load_a4(a_row_of(h), h.kb_begin);
    };

    // (with the 192-wide tile the registers do not stretch to carrying them across the epilogue: its units fetch
    // their first scales when they start, which their many slabs amortise)
    constexpr bool kLookahead = SGLB_LOOKAHEAD_ALL || BN < 192;
    int u = unit0;
    bool have = u < num_units;
    Hdr h{};
    if (have) {
      h = header(u);
      if (kLookahead) prefetch(h);
    }
    uint32_t cb = 0;  // which half of the strip the next chunk of weight-block scales goes to
    while (have) {
      const int64_t row = (int64_t)h.m_tile * BM + row_in_tile;
      const int n0 = h.n_tile * BN + cgrp * kEpiCols;                  // first of this warp's columns
      const int n_end = (int)min((int64_t)h.n_tile * BN + BN, p.N);    // one past the tile's last valid column
      float acc[kEpiCols];
#pragma unroll
      for (int j = 0; j < kEpiCols; ++j) acc[j] = 0.f;
      if (h.work && h.e >= 0 && alive) {
        if (!kLookahead) prefetch(h);
        const float* a_row = a_row_of(h);
        // A 32-column piece never straddle a weight block; a piece wholly past N is clamped to the last block.
        const int nb_tile = min(h.n_tile * BN / kScaleBlockN, p.nb_total - 1);
        uint32_t poff[kPieces];
#pragma unroll
        for (int i = 0; i < kPieces; ++i)
          poff[i] = (BN != kScaleBlockN && min((n0 + 32 * i) / kScaleBlockN, p.nb_total - 1) != nb_tile) ? kBChunk * 4 : 0;
        uint32_t b_base = strip0 + cb * kStripBytes;
        store_b(b_base, bv);
        float4 a_cur = a_first;
        const int n_slabs = h.kb_stop - h.kb_begin;
        const bool active = kGrouped || (int64_t)h.m_tile * BM + q * 32 < rows;
        int g = 0;
        while (g < n_slabs && alive) {
          const int chunk_end = min(n_slabs, g + kBChunk);  // (g is a multiple of kBChunk here)
          const bool more = chunk_end < n_slabs;
          if (more) {  // (K beyond 8192: the next 64 slabs' weight-block scales, fetched a chunk ahead)
            const float *b_row0, *b_row1;
            b_rows_of(h, b_row0, b_row1);
            fetch_b(b_row0, b_row1, h.kb_begin + chunk_end, bv);
          }
          uint32_t b_addr = b_base;
          for (; g + 4 <= chunk_end; g += 4, b_addr += 16) {
            const float4 a_nxt = load_a4(a_row, h.kb_begin + g + 4);
            // (the weight-block scales are read slab by slab: holding a group's worth in registers spills)
            float bsc[kPieces];
#define SGLB_SLAB(J, A_SC)                                                                                          \
  {                                                                                                                 \
    _Pragma("unroll") for (int i = 0; i < kPieces; ++i) bsc[i] = ptx::lds_f32(b_addr + poff[i] + 4 * (J));          \
    alive = promote_slab<Cfg, (J) % kAccBufs>(bar_tfull0, bar_tempty0, taddr0, par, lane0, active, A_SC, bsc, acc,  \
                                              abort_flag, probes, SGLB_TN);                                         \
  }
            SGLB_SLAB(0, a_cur.x)
            if (alive) SGLB_SLAB(1, a_cur.y)
            if (alive) SGLB_SLAB(2, a_cur.z)
            if (alive) SGLB_SLAB(3, a_cur.w)
            if (!alive) break;
            a_cur = a_nxt;
          }
          if (alive && g < chunk_end) {
            // one to three trailing slabs (only a unit's last group can be short)
            const int rem = chunk_end - g;
            float bsc[kPieces];
            SGLB_SLAB(0, a_cur.x)
            if (alive && rem > 1) SGLB_SLAB(1, a_cur.y)
            if (alive && rem > 2) SGLB_SLAB(2, a_cur.z)
#undef SGLB_SLAB
            g = chunk_end;
          }
          if (more && alive) {
            cb ^= 1u;
            b_base = strip0 + cb * kStripBytes;
            store_b(b_base, bv);
          }
        }
        if (!alive) raise_abort();
        cb ^= 1u;
      }
      // the next unit's header and first scales, requested before this unit's epilogue
      const Hdr cur = h;
      u += unit_step;
      have = u < num_units;
      if (have) {
        h = header(u);
        if (alive && kLookahead) prefetch(h);
      }
      if (!cur.work) continue;
      // ---- store ----
      if (cur.split) {
        // this unit's float32 partial sums, tile-local layout; a second kernel adds the units of a tile in a
        // fixed order, adds the bias and rounds once
        if (alive && row < rows) {  // (rows past M are never read back)
          // (a pair: the two CTAs' 128-row blocks of a unit follow each other)
          // Layout of a block: with full tiles [column / 4][row][4], so that the 32 lanes of a warp (32 consecutive
          // rows) write 512 contiguous bytes per store; with a handful of rows (weight streaming) [row][BN], where
          // a row's columns stay together.  The reduction kernel reads it the same way.
          const int64_t blk = kPair ? (int64_t)cur.slot * 2 + crank : (int64_t)cur.slot;
          if (p.partial_rowmajor) {
            float* dst = p.partial + blk * (BM * BN) + row_in_tile * BN + cgrp * kEpiCols;
#pragma unroll
            for (int j = 0; j < kEpiCols / 4; ++j)
              *reinterpret_cast<float4*>(dst + j * 4) = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
          } else {
            float* dst = p.partial + blk * (BM * BN) + ((int64_t)(cgrp * kEpiCols / 4) * BM + row_in_tile) * 4;
#pragma unroll
            for (int j = 0; j < kEpiCols / 4; ++j)
              *reinterpret_cast<float4*>(dst + (int64_t)j * BM * 4) =
                  make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
          }
        }
        continue;
      }
      if (p.tma_out) {
        // Rows of C are contiguous: round to the output type and park the 32 rows x BN columns of this TMEM lane
        // quadrant in shared memory (per 64 columns a block of 128-byte rows, 16-byte chunks XOR-swizzled by the
        // row so that the lanes of a store spread over all banks); the quadrant's two warps each write their half
        // of the columns, meet at a barrier of their own (64 threads, same scheduler), and one lane hands the
        // blocks to the TMA engine, which clips them to the tensor.  The stores drain while the next tile is being
        // promoted; their source is reclaimed at the next epilogue.  No barrier spans the quadrants.
        // (A warp whose wait expired still joins both barriers; only the data movement is skipped.)
        const bool issuer = cgrp == 0 && lane == 0;
        if (issuer) ptx::tma_store_wait_read();
        ptx::bar_sync(2 + q, 32 * Cfg::kColGroups);
        const bool rows_in = (int64_t)cur.m_tile * BM + q * 32 < rows;
        if (alive && n0 < n_end && rows_in) {
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
              const __half2 hh = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
              packed[j] = *reinterpret_cast<const uint32_t*>(&hh);
            }
          } else {
#pragma unroll
            for (int j = 0; j < kEpiCols / 2; ++j) {
              const __nv_bfloat162 hh = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
              packed[j] = *reinterpret_cast<const uint32_t*>(&hh);
            }
          }
          const uint32_t dst0 = stage_q + lane * 128;
          const uint32_t swz = (uint32_t)(lane & 7);
#pragma unroll
          for (int j = 0; j < kEpiCols / 8; ++j) {
            const int col = cgrp * kEpiCols + j * 8;  // within the tile: 64-column group col / 64, 16-byte chunk (col % 64) / 8
            ptx::sts_128(dst0 + (col >> 6) * kGroupBytes + ((((uint32_t)(col & 63) >> 3) ^ swz) << 4),
                         make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]));
          }
          ptx::fence_async_smem();
        }
        ptx::bar_sync(2 + q, 32 * Cfg::kColGroups);
        if (issuer && alive && rows_in) {
          const CUtensorMap* cmap = &map_c;
          int out_row0 = cur.m_tile * BM;
          if (p.push_maps != nullptr) {
            const int owner = out_row0 / p.push_rows_per_owner;
            cmap = p.push_maps + owner;
            out_row0 += (p.push_rank - owner) * p.push_rows_per_owner;
          }
#pragma unroll
          for (int g = 0; g < Cfg::kOutGroups; ++g) {
            if (cur.n_tile * BN + g * 64 < n_end)
              ptx::tma_store_2d(cmap, stage_q + g * kGroupBytes, cur.n_tile * BN + g * 64, out_row0 + q * 32);
          }
          ptx::tma_store_commit();
        }
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
    // this warp's tile stores: sources stay valid until read; tiles pushed to other GPUs have landed before the
    // kernel counts as finished
    if (cgrp == 0 && lane == 0) {
      if (p.push_maps != nullptr)
        ptx::tma_store_wait_all();
      else
        ptx::tma_store_wait_read();
    }
  }

  // ------------------------------ teardown ------------------------------
  ptx::tc_fence_before();
  __syncthreads();
  // (a pair: neither CTA releases shared or tensor memory that its peer's instructions may still touch)
  if (kPair) ptx::cluster_sync_all();
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

// Tile width of a problem: the 128-wide tile (four accumulator buffers) where K is short.
static int choose_bn(int64_t K) { return (K + BK - 1) / BK <= SGLB_SHORT_K ? 128 : 192; }

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

// Output tensor [rows][N] of 2-byte elements, box = 64 columns x 32 rows, 128-byte swizzle (matches the
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
  cuuint32_t box[2] = {64u, 32u};
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

// How a dense problem runs: tile width, single CTAs or CTA pairs, and the cut into units.
#ifndef SGLB_PAIR_MIN_M
#define SGLB_PAIR_MIN_M 0    // from this many rows on, pairs of CTAs share 256-row tiles (0 = never)
#endif
#ifndef SGLB_PAIR_BN
#define SGLB_PAIR_BN 128     // tile width of a pair whatever K is (0 = as a single CTA would choose)
#endif
struct DensePlan {
  int bn;
  bool pair;
  int tile_rows, workers;
  UnitPlan units;
  int64_t scratch_bytes() const { return units.scratch_blocks() * (int64_t)tile_rows * bn * (int64_t)sizeof(float); }
};
static DensePlan plan_dense(int64_t M, int64_t N, int64_t K) {
  DensePlan d;
  d.pair = SGLB_PAIR_MIN_M > 0 && M >= SGLB_PAIR_MIN_M;
  d.bn = d.pair && SGLB_PAIR_BN > 0 ? SGLB_PAIR_BN : choose_bn(K);
  d.tile_rows = d.pair ? 2 * BM : BM;
  d.workers = d.pair ? sm_count() / 2 : sm_count();
  d.units = plan_units(M, N, K, d.bn, d.tile_rows, d.workers);
  return d;
}

static uint32_t g_wait_probes = ptx::kProbeLimit;  // sglb200_gemm_set_wait_probes

template <class Cfg>
static size_t gemm_smem_bytes() {
  return (size_t)Cfg::kStages * Cfg::kStageBytes + Cfg::kOutBytes + sizeof(SharedCtl<Cfg>) + 1024;
}

template <bool kGrouped, int BN, bool kPair = false>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const GemmParams& p,
                       int64_t max_units, cudaStream_t st, int sm_margin = 0) {
  const size_t smem = gemm_smem_bytes<TileCfg<BN, kPair>>();
  static thread_local bool attr_set[64] = {false};  // the opt-in is per function and per device
  int dev = 0;
  SGLB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    SGLB_CUDA(cudaFuncSetAttribute(fp8_blockscale_gemm_kernel<kGrouped, BN, kPair>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  int sms = sm_count() - sm_margin;  // SMs left free run a concurrent kernel (the reduce-and-gather of an earlier chunk)
  if (sms < 1) sms = 1;
  if (!kPair) {
    const unsigned grid = (unsigned)(max_units < sms ? max_units : sms);
    fp8_blockscale_gemm_kernel<kGrouped, BN, kPair><<<grid, TileCfg<BN, kPair>::kThreads, smem, st>>>(ma, mb, mc, p);
    SGLB_CUDA(cudaGetLastError());
    return SGLB200_OK;
  }
  // pairs: a cluster of two CTAs per unit in flight (one cluster per two SMs)
  int64_t clusters = sms / 2;
  if (clusters < 1) clusters = 1;
  if (max_units < clusters) clusters = max_units;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
  cfg.blockDim = dim3(TileCfg<BN, kPair>::kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  SGLB_CUDA(cudaLaunchKernelEx(&cfg, fp8_blockscale_gemm_kernel<kGrouped, BN, kPair>, ma, mb, mc, p));
  return SGLB200_OK;
}

template <int BN, bool kPair>
static int dense_mm(const DensePlan& dp, const void* A, const void* B, const float* a_s, const float* b_s, void* C,
                    const void* bias, int64_t M, int64_t N, int64_t K, int64_t as_stride_m, int64_t as_stride_k,
                    int out_dtype, void* workspace, int64_t workspace_bytes, cudaStream_t st) {
  constexpr int kTileRows = kPair ? 2 * BM : BM;
  CUtensorMap ma, mb;
  int rc = get_tensor_map(A, (uint64_t)K, (uint64_t)M, 1, BM, 2, &ma);
  if (rc) return rc;
  // B is addressed as [1][N][K] so that dense and grouped kernels share the 3-D load
  rc = get_tensor_map(B, (uint64_t)K, (uint64_t)N, 1, TileCfg<BN, kPair>::kBRows, 3, &mb);
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
  rc = launch_gemm<false, BN, kPair>(ma, mb, mc, p,
                                     pl.sk_share > 0 ? pl.sk_ctas : pl.full_units + pl.split_tiles * pl.splits, st);
  if (rc != SGLB200_OK || pl.scratch_blocks() == 0) return rc;
  const int tiles_m = (int)((M + kTileRows - 1) / kTileRows);
  const unsigned ygrid = (unsigned)((kTileRows * BN / 8 + 255) / 256);
  if (pl.sk_share > 0) {
    const dim3 sgrid((unsigned)tiles, ygrid);
    if (out_dtype == 0)
      streamk_reduce_kernel<__nv_bfloat16><<<sgrid, 256, 0, st>>>(
          p.partial, static_cast<__nv_bfloat16*>(C), static_cast<const __nv_bfloat16*>(bias), M, N, BN, kTileRows, tiles_m,
          p.tiles_n, p.group_m, p.kb_total, pl.sk_share, pl.sk_ctas, p.partial_rowmajor);
    else
      streamk_reduce_kernel<__half><<<sgrid, 256, 0, st>>>(p.partial, static_cast<__half*>(C),
                                                           static_cast<const __half*>(bias), M, N, BN, kTileRows,
                                                           tiles_m, p.tiles_n, p.group_m, p.kb_total, pl.sk_share,
                                                           pl.sk_ctas, p.partial_rowmajor);
    SGLB_CUDA(cudaGetLastError());
    return SGLB200_OK;
  }
  const dim3 grid((unsigned)pl.split_tiles, ygrid);
  if (out_dtype == 0)
    split_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p.partial, static_cast<__nv_bfloat16*>(C),
                                                             static_cast<const __nv_bfloat16*>(bias), M, N, BN, kTileRows,
                                                             tiles_m, p.tiles_n, p.group_m, pl.full_units, pl.splits,
                                                             p.partial_rowmajor);
  else
    split_reduce_kernel<__half><<<grid, 256, 0, st>>>(p.partial, static_cast<__half*>(C),
                                                      static_cast<const __half*>(bias), M, N, BN, kTileRows, tiles_m,
                                                      p.tiles_n, p.group_m, pl.full_units, pl.splits, p.partial_rowmajor);
  SGLB_CUDA(cudaGetLastError());
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
  return launch_gemm<true, BN, false>(ma, mb, mc, p, tiles, st);
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

#ifdef SGLB_TRACE
extern "C" int sglb200_debug_trace(void* out, int64_t bytes) {
  if (bytes > (int64_t)sizeof(long long) * 2 * kTraceRoles * kTraceSlabs * kTraceEvents)
    bytes = (int64_t)sizeof(long long) * 2 * kTraceRoles * kTraceSlabs * kTraceEvents;
  SGLB_CUDA(cudaMemcpyFromSymbol(out, g_trace, (size_t)bytes));
  return SGLB200_OK;
}
#endif

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
  SGLB_REQUIRE(N % 8 == 0, "fp8_blockwise_scaled_mm: N=%lld must be a multiple of 8", (long long)N);
  SGLB_REQUIRE(out_dtype == 0 || out_dtype == 1, "fp8_blockwise_scaled_mm: out_dtype %d (0 bf16, 1 fp16)", out_dtype);
  if (M == 0) return SGLB200_OK;
  SGLB_REQUIRE(A && B && a_s && b_s && C, "fp8_blockwise_scaled_mm: null pointer");
  SGLB_REQUIRE(aligned16(A) && aligned16(B) && aligned16(C) && (bias == nullptr || aligned16(bias)),
               "fp8_blockwise_scaled_mm: A, B, C and bias must be 16-byte aligned");
  SGLB_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "fp8_blockwise_scaled_mm: dimension too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const DensePlan dp = plan_dense(M, N, K);
  if (dp.bn == 128 && dp.pair)
    return dense_mm<128, true>(dp, A, B, a_s, b_s, C, bias, M, N, K, as_stride_m, as_stride_k, out_dtype, workspace,
                               workspace_bytes, st);
  if (dp.bn == 128)
    return dense_mm<128, false>(dp, A, B, a_s, b_s, C, bias, M, N, K, as_stride_m, as_stride_k, out_dtype, workspace,
                                workspace_bytes, st);
  if (dp.pair)
    return dense_mm<192, true>(dp, A, B, a_s, b_s, C, bias, M, N, K, as_stride_m, as_stride_k, out_dtype, workspace,
                               workspace_bytes, st);
  return dense_mm<192, false>(dp, A, B, a_s, b_s, C, bias, M, N, K, as_stride_m, as_stride_k, out_dtype, workspace,
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
  SGLB_REQUIRE(out_dtype == 0 || out_dtype == 1, "grouped_mm: out_dtype %d (0 bf16, 1 fp16)", out_dtype);
  if (max_rows == 0) return SGLB200_OK;
  SGLB_REQUIRE(A && a_s && B && b_s && C && expert_ids && num_rows_dev, "grouped_mm: null pointer");
  SGLB_REQUIRE(!scatter || sorted_token_ids, "grouped_mm: scatter mode needs sorted_token_ids");
  SGLB_REQUIRE(aligned16(A) && aligned16(B) && aligned16(C), "grouped_mm: A, B and C must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (choose_bn(K) == 128)
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

template <int BN, bool kPair>
static int push_mm(const void* A, const void* B, const float* a_s, const float* b_s, void* const* stage_ptrs, int world,
                   int rank, int64_t M, int64_t N, int64_t K, int64_t as_stride_m, int64_t as_stride_k, int out_dtype,
                   int sm_margin, cudaStream_t st) {
  constexpr int kTileRows = kPair ? 2 * BM : BM;
  CUtensorMap ma, mb;
  int rc = get_tensor_map(A, (uint64_t)K, (uint64_t)M, 1, BM, 2, &ma);
  if (rc) return rc;
  rc = get_tensor_map(B, (uint64_t)K, (uint64_t)N, 1, TileCfg<BN, kPair>::kBRows, 3, &mb);
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
  return launch_gemm<false, BN, kPair>(ma, mb, mc, p, tiles, st, sm_margin);
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
  SGLB_REQUIRE(out_dtype == 0 || out_dtype == 1, "mm_push: out_dtype %d (0 bf16, 1 fp16)", out_dtype);
  SGLB_REQUIRE(A && B && a_s && b_s && stage_ptrs, "mm_push: null pointer");
  for (int i = 0; i < world; ++i)
    SGLB_REQUIRE(stage_ptrs[i] != nullptr && aligned16(stage_ptrs[i]), "mm_push: staging buffer %d missing or unaligned", i);
  SGLB_REQUIRE(aligned16(A) && aligned16(B), "mm_push: A and B must be 16-byte aligned");
  SGLB_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "mm_push: dimension too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const DensePlan dp = plan_dense(M, N, K);  // (tile shape only: a pushed tile is never split along K)
#define SGLB_PUSH(BN_, PAIR_)                                                                                        \
  return push_mm<BN_, PAIR_>(A, B, a_s, b_s, stage_ptrs, world, rank, M, N, K, as_stride_m, as_stride_k, out_dtype, \
                             sm_margin, st)
  if (dp.bn == 128 && dp.pair) SGLB_PUSH(128, true);
  if (dp.bn == 128) SGLB_PUSH(128, false);
  if (dp.pair) SGLB_PUSH(192, true);
  SGLB_PUSH(192, false);
#undef SGLB_PUSH
}
