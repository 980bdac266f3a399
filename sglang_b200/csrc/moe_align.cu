// moe_align_block_size for sm_100a: a deterministic (stable) counting sort of the flat
// top-k expert ids into expert segments padded to a multiple of block_size.
//
// Bucket b = id + 1 (id -1, "expert not on this rank", is bucket 0 and is reported as
// expert -1).  Within a bucket entries keep ascending flat index, so the output is a pure
// function of the input (the reference kernel's atomicAdd scatter yields an arbitrary
// permutation inside each expert segment; this order is one of its valid outputs and is the
// order of the reference's CPU implementation and test oracle).
//
// The ids are cut into chunks of consecutive entries, one CTA per chunk (1024 ids, or longer chunks
// when the input would otherwise need more than 128 CTAs: ranking costs about seven warp instructions per
// id, so a chunk is bound by instruction issue on its SM and short chunks on many SMs finish first); inside
// a CTA each of the 32 warps
// owns one contiguous span of the chunk and walks it 32 ids at a time.  Rank of an
// entry = (padded start of its bucket) + (entries of that bucket in earlier chunks) + (in
// earlier warps of the chunk) + (in earlier steps of the warp) + (in lower lanes of the step,
// from one ballot per id bit).  Up to kSingleMax ids run as ONE CTA; up to kLargeMin ids as one cooperative
// kernel (histogram, grid barrier, scatter) or, where a cooperative launch is not possible, as histogram ->
// scan -> scatter launches over a small global workspace; above that the tile-sorted path.  No global atomics.
#include <cooperative_groups.h>

#include <mutex>

#include "common.cuh"

namespace sglb200 {

constexpr int kAlignThreads = 1024;
constexpr int kAlignWarps = kAlignThreads / 32;
constexpr int kChunk = kAlignWarps * 256;          // 8192 ids per CTA: the longest chunk of the multi-CTA path (at 2^20 ids)
constexpr int64_t kSingleMax = 2048;               // up to here one CTA sorts everything in one launch
constexpr int kMidMaxChunks = 128;                 // CTAs of the multi-CTA path: at most one per SM, all resident
#ifndef SGLB_ALIGN_COOP
#define SGLB_ALIGN_COOP 1
#endif
constexpr bool kAlignCoop = SGLB_ALIGN_COOP != 0;  // one cooperative launch instead of three for 8192 < ids <= 1 M
constexpr int kMaxChunks = 296;                    // about two CTAs per SM; longer inputs get longer chunks

__device__ __forceinline__ int warp_incl_scan(int v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, v, off);
    if (lane >= off) v += n;
  }
  return v;
}

// Lanes of the warp holding the same key, from one ballot per key bit (match.any iterates over the distinct
// values of the warp, about 30 of them here, and is several times slower).
__device__ __forceinline__ unsigned peers_of(int key, int nbits) {
  unsigned peers = 0xffffffffu;
  for (int k = 0; k < nbits; ++k) {
    const unsigned set = __ballot_sync(0xffffffffu, (key >> k) & 1);
    peers &= ((key >> k) & 1) ? set : ~set;
  }
  return peers;
}

// The same with the bit count known at compile time (fully unrolled, no loop bookkeeping).
template <int NBITS>
__device__ __forceinline__ unsigned peers_of_fixed(int key) {
  unsigned peers = 0xffffffffu;
#pragma unroll
  for (int k = 0; k < NBITS; ++k) {
    const bool bit = (key >> k) & 1;
    const unsigned set = __ballot_sync(0xffffffffu, bit);
    peers &= set ^ (bit ? 0u : 0xffffffffu);
  }
  return peers;
}

constexpr int kBatch = 8;  // steps whose id loads are issued together: hides the load latency of a long span

// Per-warp bucket counts of the chunk [chunk_begin, chunk_end) into wc[warp][B] (smem, zeroed by caller).
__device__ __forceinline__ void count_chunk(const int32_t* __restrict__ ids, int64_t chunk_begin, int64_t chunk_end,
                                            int span, int B, int* wc) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t seg = chunk_begin + (int64_t)warp * span;
  const int64_t seg_end = seg + span < chunk_end ? seg + span : chunk_end;
  for (int64_t s0 = seg; s0 < seg_end; s0 += 32 * kBatch) {
    int v[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int64_t i = s0 + j * 32 + lane;
      v[j] = i < seg_end ? ids[i] + 1 : -1;
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j)
      if (v[j] >= 0 && v[j] < B) atomicAdd(&wc[warp * B + v[j]], 1);  // shared-memory atomic, contended only inside the warp
  }
}

// Turns wc[warp][b] into exclusive prefixes over warps; returns this CTA's total per bucket in tot[b].
__device__ __forceinline__ void scan_over_warps(int B, int* wc, int* tot) {
  for (int b = threadIdx.x; b < B; b += kAlignThreads) {
    int run = 0;
#pragma unroll 8
    for (int w = 0; w < kAlignWarps; ++w) {
      const int c = wc[w * B + b];
      wc[w * B + b] = run;
      run += c;
    }
    tot[b] = run;
  }
}

// prefix[0..B] = exclusive scan of ceil(tot[b]/block)*block.  `scratch` holds 33 ints.  NT = threads of the CTA.
template <int NT = kAlignThreads>
__device__ __forceinline__ void padded_prefix(int B, int block_size, const int* tot, int* prefix, int* scratch) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int carry = 0;
  for (int base = 0; base < B; base += NT) {
    const int b = base + threadIdx.x;
    const int v = b < B ? (tot[b] + block_size - 1) / block_size * block_size : 0;
    const int incl = warp_incl_scan(v);
    if (lane == 31) scratch[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const int w = lane < NT / 32 ? scratch[lane] : 0;
      const int wi = warp_incl_scan(w);
      scratch[lane] = wi - w;
      if (lane == 31) scratch[32] = wi;
    }
    __syncthreads();
    if (b < B) prefix[b] = carry + scratch[warp] + incl - v;
    carry += scratch[32];
    __syncthreads();
  }
  if (threadIdx.x == 0) prefix[B] = carry;
  __syncthreads();
}

// Writes sorted_token_ids for the chunk.  base[b] = padded start of bucket b + entries in earlier chunks.
template <int NBITS = 0>  // > 0: the number of key bits is known at compile time (unrolled ballots)
__device__ __forceinline__ void scatter_chunk(const int32_t* __restrict__ ids, int64_t chunk_begin, int64_t chunk_end,
                                              int span, int B, int* wc, const int* base, int32_t* __restrict__ sorted) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t seg = chunk_begin + (int64_t)warp * span;
  const int64_t seg_end = seg + span < chunk_end ? seg + span : chunk_end;
  const int nbits = 32 - __clz(B + 31);  // keys run up to B + 31
  for (int64_t s0 = seg; s0 < seg_end; s0 += 32 * kBatch) {  // uniform over the warp
    int v[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int64_t i = s0 + j * 32 + lane;
      int b = i < seg_end ? ids[i] + 1 : -1;
      if (b >= B) b = -1;
      v[j] = b;
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (s0 + j * 32 >= seg_end) break;  // uniform
      const int b = v[j];
      const int key = b >= 0 ? b : B + lane;  // invalid lanes match nobody
      const unsigned peers = NBITS > 0 ? peers_of_fixed<(NBITS > 0 ? NBITS : 1)>(key) : peers_of(key, nbits);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      int start = 0;
      if (b >= 0) start = wc[warp * B + b];
      __syncwarp();
      if (b >= 0) {
        sorted[(int64_t)base[b] + start + rank] = (int32_t)(s0 + j * 32 + lane);
        if (lane == 31 - __clz(peers)) wc[warp * B + b] = start + __popc(peers);
      }
      __syncwarp();
    }
  }
}

// expert_ids for blocks [first, first+stride, ...) and the padding tails of buckets b = first_b, first_b+stride_b, ...
template <int NT = kAlignThreads>
__device__ __forceinline__ void fill_meta(int B, int block_size, int64_t numel, const int* prefix, const int* tot_all,
                                          int32_t* __restrict__ expert_ids, int32_t* __restrict__ sorted,
                                          bool pad_sorted, int part, int parts) {
  const int num_blocks = prefix[B] / block_size;
  for (int i = part * NT + threadIdx.x; i < num_blocks; i += parts * NT) {
    const int pos = i * block_size;
    int lo = 0, hi = B;  // first bucket whose end is > pos
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (prefix[mid + 1] <= pos) lo = mid + 1; else hi = mid;
    }
    expert_ids[i] = lo - 1;
  }
  if (pad_sorted) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int b = part * (NT / 32) + warp; b < B; b += parts * (NT / 32)) {
      const int begin = prefix[b] + tot_all[b], end = prefix[b + 1];
      for (int p = begin + lane; p < end; p += 32) sorted[p] = (int32_t)numel;
    }
  }
}

// ---- numel <= kChunk: everything in one CTA -------------------------------------------------
__global__ void __launch_bounds__(kAlignThreads)
    moe_align_single_kernel(const int32_t* __restrict__ ids, int64_t numel, int span, int B, int block_size,
                            int32_t* __restrict__ sorted, int32_t* __restrict__ expert_ids,
                            int32_t* __restrict__ post_pad, int32_t* __restrict__ cumsum, bool pad_sorted) {
  extern __shared__ int smem[];
  int* wc = smem;                       // [32][B]
  int* tot = wc + kAlignWarps * B;      // [B]
  int* prefix = tot + B;                // [B+1]
  int* scratch = prefix + B + 1;        // [33]
  for (int i = threadIdx.x; i < kAlignWarps * B; i += kAlignThreads) wc[i] = 0;
  __syncthreads();
  count_chunk(ids, 0, numel, span, B, wc);
  __syncthreads();
  scan_over_warps(B, wc, tot);
  __syncthreads();
  padded_prefix(B, block_size, tot, prefix, scratch);
  for (int b = threadIdx.x; b <= B; b += kAlignThreads) cumsum[b] = prefix[b];
  if (threadIdx.x == 0) *post_pad = prefix[B];
  fill_meta(B, block_size, numel, prefix, tot, expert_ids, sorted, pad_sorted, 0, 1);
  scatter_chunk(ids, 0, numel, span, B, wc, prefix, sorted);
}

// ---- numel > kChunk: histogram per chunk -> scan over chunks -> scatter ----------------------
__global__ void __launch_bounds__(kAlignThreads)
    moe_align_hist_kernel(const int32_t* __restrict__ ids, int64_t numel, int span, int B,
                          int* __restrict__ chunk_hist) {
  extern __shared__ int smem[];
  int* wc = smem;
  int* tot = wc + kAlignWarps * B;
  for (int i = threadIdx.x; i < kAlignWarps * B; i += kAlignThreads) wc[i] = 0;
  __syncthreads();
  const int64_t chunk_len = (int64_t)span * kAlignWarps;
  const int64_t begin = (int64_t)blockIdx.x * chunk_len;
  const int64_t end = begin + chunk_len < numel ? begin + chunk_len : numel;
  count_chunk(ids, begin, end, span, B, wc);
  __syncthreads();
  scan_over_warps(B, wc, tot);
  __syncthreads();
  for (int b = threadIdx.x; b < B; b += kAlignThreads) chunk_hist[(int64_t)blockIdx.x * B + b] = tot[b];
}

// One warp per bucket: chunk_hist[:, b] becomes its exclusive scan over chunks; totals[b] = sum.
__global__ void __launch_bounds__(kAlignThreads)
    moe_align_scan_kernel(int* __restrict__ chunk_hist, int* __restrict__ totals, int num_chunks, int B) {
  const int b = blockIdx.x * kAlignWarps + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= B) return;
  int run = 0;
  for (int c0 = 0; c0 < num_chunks; c0 += 32) {
    const int c = c0 + lane;
    const int v = c < num_chunks ? chunk_hist[(int64_t)c * B + b] : 0;
    const int incl = warp_incl_scan(v);
    if (c < num_chunks) chunk_hist[(int64_t)c * B + b] = run + incl - v;
    run += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) totals[b] = run;
}

__global__ void __launch_bounds__(kAlignThreads)
    moe_align_scatter_kernel(const int32_t* __restrict__ ids, int64_t numel, int span, int B, int block_size,
                             const int* __restrict__ chunk_hist, const int* __restrict__ totals,
                             int32_t* __restrict__ sorted, int32_t* __restrict__ expert_ids,
                             int32_t* __restrict__ post_pad, int32_t* __restrict__ cumsum, bool pad_sorted) {
  extern __shared__ int smem[];
  int* wc = smem;                       // [32][B]
  int* tot = wc + kAlignWarps * B;      // [B]   this chunk's totals (unused after scan) / all-chunk totals
  int* prefix = tot + B;                // [B+1]
  int* base = prefix + B + 1;           // [B]
  int* scratch = base + B;              // [33]
  for (int i = threadIdx.x; i < kAlignWarps * B; i += kAlignThreads) wc[i] = 0;
  for (int b = threadIdx.x; b < B; b += kAlignThreads) tot[b] = totals[b];
  __syncthreads();
  padded_prefix(B, block_size, tot, prefix, scratch);
  for (int b = threadIdx.x; b < B; b += kAlignThreads) base[b] = prefix[b] + chunk_hist[(int64_t)blockIdx.x * B + b];
  if (blockIdx.x == 0) {
    for (int b = threadIdx.x; b <= B; b += kAlignThreads) cumsum[b] = prefix[b];
    if (threadIdx.x == 0) *post_pad = prefix[B];
  }
  fill_meta(B, block_size, numel, prefix, tot, expert_ids, sorted, pad_sorted, blockIdx.x, gridDim.x);
  __syncthreads();  // fill_meta is done with tot[] before it is reused below
  const int64_t chunk_len = (int64_t)span * kAlignWarps;
  const int64_t begin = (int64_t)blockIdx.x * chunk_len;
  const int64_t end = begin + chunk_len < numel ? begin + chunk_len : numel;
  count_chunk(ids, begin, end, span, B, wc);
  __syncthreads();
  scan_over_warps(B, wc, tot);
  __syncthreads();
  scatter_chunk(ids, begin, end, span, B, wc, base, sorted);
}

// ---- kSingleMax < numel <= kLargeMin, one launch ------------------------------------------------
// The same three steps in ONE cooperative kernel: every CTA counts its chunk, publishes the chunk's histogram,
// all CTAs meet at a grid barrier, then every CTA sums the histograms of the chunks before it (and of all chunks)
// for itself and scatters, reusing the per-warp counts it already holds in shared memory.  Saves two launches
// and the second count; the grid barrier is legal because the launch is cooperative (all CTAs are resident).
template <int NBITS>
__global__ void __launch_bounds__(kAlignThreads)
    moe_align_coop_kernel(const int32_t* __restrict__ ids, int64_t numel, int span, int B, int block_size,
                          int* __restrict__ chunk_hist, int32_t* __restrict__ sorted, int32_t* __restrict__ expert_ids,
                          int32_t* __restrict__ post_pad, int32_t* __restrict__ cumsum, bool pad_sorted) {
  extern __shared__ int smem[];
  int* wc = smem;                       // [32][B]
  int* tot = wc + kAlignWarps * B;      // [B]   this chunk's totals, then the totals over all chunks
  int* prefix = tot + B;                // [B+1]
  int* base = prefix + B + 1;           // [B]
  int* scratch = base + B;              // [33]
  for (int i = threadIdx.x; i < kAlignWarps * B; i += kAlignThreads) wc[i] = 0;
  __syncthreads();
  const int64_t chunk_len = (int64_t)span * kAlignWarps;
  const int64_t begin = (int64_t)blockIdx.x * chunk_len;
  const int64_t end = begin + chunk_len < numel ? begin + chunk_len : numel;
  count_chunk(ids, begin, end, span, B, wc);
  __syncthreads();
  scan_over_warps(B, wc, tot);  // wc becomes the exclusive prefix over the warps of this chunk
  __syncthreads();
  for (int b = threadIdx.x; b < B; b += kAlignThreads) chunk_hist[(int64_t)blockIdx.x * B + b] = tot[b];
  __threadfence();
  cooperative_groups::this_grid().sync();
  // totals over all chunks and entries in earlier chunks, per bucket: all threads walk the [chunks][B] table once
  // (coalesced, independent loads) and add into shared memory
  for (int b = threadIdx.x; b < B; b += kAlignThreads) tot[b] = 0, base[b] = 0;
  __syncthreads();
  {
    const int n = (int)gridDim.x * B, mine_end = (int)blockIdx.x * B;
    constexpr int kU = 4;
    for (int i0 = threadIdx.x; i0 < n; i0 += kAlignThreads * kU) {
      int v[kU];
#pragma unroll
      for (int k = 0; k < kU; ++k) {
        const int i = i0 + k * kAlignThreads;
        v[k] = i < n ? __ldcg(chunk_hist + i) : 0;  // written by other CTAs: read through L2
      }
#pragma unroll
      for (int k = 0; k < kU; ++k) {
        const int i = i0 + k * kAlignThreads;
        if (i < n && v[k] != 0) {
          const int b = i % B;
          atomicAdd(&tot[b], v[k]);
          if (i < mine_end) atomicAdd(&base[b], v[k]);
        }
      }
    }
  }
  __syncthreads();
  padded_prefix(B, block_size, tot, prefix, scratch);
  for (int b = threadIdx.x; b < B; b += kAlignThreads) base[b] += prefix[b];
  if (blockIdx.x == 0) {
    for (int b = threadIdx.x; b <= B; b += kAlignThreads) cumsum[b] = prefix[b];
    if (threadIdx.x == 0) *post_pad = prefix[B];
  }
  fill_meta(B, block_size, numel, prefix, tot, expert_ids, sorted, pad_sorted, blockIdx.x, gridDim.x);
  __syncthreads();
  scatter_chunk<NBITS>(ids, begin, end, span, B, wc, base, sorted);
}

static bool g_align_coop_enabled = true;  // sglb200_moe_align_set_cooperative

using CoopKernel = void (*)(const int32_t*, int64_t, int, int, int, int*, int32_t*, int32_t*, int32_t*, int32_t*, bool);
static CoopKernel coop_kernel_for(int B) {
  switch (32 - __builtin_clz((unsigned)(B + 31))) {  // keys run up to B + 31
    case 6: return moe_align_coop_kernel<6>;
    case 7: return moe_align_coop_kernel<7>;
    case 8: return moe_align_coop_kernel<8>;
    case 9: return moe_align_coop_kernel<9>;
    case 10: return moe_align_coop_kernel<10>;
    default: return moe_align_coop_kernel<0>;
  }
}

// Whether `chunks` CTAs of the cooperative kernel can be resident at once on the current device (cached per device
// and shared-memory size class).
static bool coop_fits(CoopKernel kern, int64_t chunks, size_t smem) {
  static thread_local int last_dev = -1;
  static thread_local size_t last_smem = 0;
  static thread_local int64_t last_cap = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  if (dev != last_dev || smem != last_smem) {
    int coop = 0, per_sm = 0;
    int64_t cap = 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) == cudaSuccess && coop &&
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kAlignThreads, smem) ==
            cudaSuccess)
      cap = (int64_t)per_sm * sm_count();
    last_dev = dev, last_smem = smem, last_cap = cap;
  }
  return chunks <= last_cap;
}

// ---- numel > kLargeMin: tile-sorted scatter ---------------------------------------------------
// With the per-warp scatter above every (CTA, warp, bucket) is an output stream of its own that grows four
// bytes at a time; at tens of millions of ids those streams (millions of half-written 32-byte sectors) no
// longer fit the L2 and the sort is bound by partial-sector traffic.  Here a CTA sorts a tile of kTsTile ids
// in shared memory first (ranks from the same ballots, then a scan over the warps and over the buckets of the
// tile) and writes each bucket's run of the tile with consecutive threads, so a CTA has one stream per bucket
// and writes it in runs.
constexpr int kTsThreads = 512;
constexpr int kTsWarps = kTsThreads / 32;
constexpr int kTsItems = 8;
constexpr int kTsTile = kTsThreads * kTsItems;  // 4096 ids
constexpr int64_t kLargeMin = 1 << 20;          // inputs above this take the tile-sorted path

template <int NBITS>
__global__ void __launch_bounds__(kTsThreads, 2)
    moe_align_tile_scatter_kernel(const int32_t* __restrict__ ids, int64_t numel, int64_t chunk_len, int B,
                                  int block_size, const int* __restrict__ chunk_hist, const int* __restrict__ totals,
                                  int32_t* __restrict__ sorted, int32_t* __restrict__ expert_ids,
                                  int32_t* __restrict__ post_pad, int32_t* __restrict__ cumsum, bool pad_sorted) {
  extern __shared__ int smem[];
  int* wc = smem;                        // [16][B]  per-warp counts of the tile, then exclusive over warps
  int* tot_all = wc + kTsWarps * B;      // [B]      totals over all chunks
  int* prefix = tot_all + B;             // [B+1]    padded starts of the buckets in the output
  int* base = prefix + B + 1;            // [B]      where this CTA's next entry of a bucket goes
  int* ttot = base + B;                  // [B]      totals of the tile
  int* tstart = ttot + B;                // [B+1]    starts of the buckets inside the sorted tile
  int* scratch = tstart + B + 1;         // [40]
  int* val = scratch + 40;               // [kTsTile] the tile in sorted order: bucket << 12 | index inside the tile
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  for (int b = tid; b < B; b += kTsThreads) tot_all[b] = totals[b];
  __syncthreads();
  padded_prefix<kTsThreads>(B, block_size, tot_all, prefix, scratch);
  for (int b = tid; b < B; b += kTsThreads) base[b] = prefix[b] + chunk_hist[(int64_t)blockIdx.x * B + b];
  if (blockIdx.x == 0) {
    for (int b = tid; b <= B; b += kTsThreads) cumsum[b] = prefix[b];
    if (tid == 0) *post_pad = prefix[B];
  }
  fill_meta<kTsThreads>(B, block_size, numel, prefix, tot_all, expert_ids, sorted, pad_sorted, blockIdx.x, gridDim.x);

  const int64_t begin = (int64_t)blockIdx.x * chunk_len;
  const int64_t end = begin + chunk_len < numel ? begin + chunk_len : numel;
  const unsigned below = (1u << lane) - 1u;
  for (int64_t t0 = begin; t0 < end; t0 += kTsTile) {
    for (int b = lane; b < B; b += 32) wc[warp * B + b] = 0;
    const int64_t w0 = t0 + warp * (32 * kTsItems);
    int key[kTsItems], loc[kTsItems];
#pragma unroll
    for (int j = 0; j < kTsItems; ++j) {
      const int64_t i = w0 + j * 32 + lane;
      int b = i < end ? ids[i] + 1 : -1;
      if (b >= B) b = -1;
      key[j] = b;
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < kTsItems; ++j) {
      const int b = key[j];
      const unsigned peers = peers_of_fixed<NBITS>(b >= 0 ? b : B + lane);  // invalid lanes match nobody
      int start = 0;
      if (b >= 0) start = wc[warp * B + b];
      __syncwarp();
      if (b >= 0 && lane == 31 - __clz(peers)) wc[warp * B + b] = start + __popc(peers);
      __syncwarp();
      loc[j] = start + __popc(peers & below);
    }
    __syncthreads();
    for (int b = tid; b < B; b += kTsThreads) {
      int run = 0;
#pragma unroll
      for (int w = 0; w < kTsWarps; ++w) {
        const int c = wc[w * B + b];
        wc[w * B + b] = run;
        run += c;
      }
      ttot[b] = run;
    }
    __syncthreads();
    padded_prefix<kTsThreads>(B, 1, ttot, tstart, scratch);
#pragma unroll
    for (int j = 0; j < kTsItems; ++j) {
      const int b = key[j];
      if (b >= 0) {
        const int pos = tstart[b] + wc[warp * B + b] + loc[j];
        val[pos] = (b << 12) | (warp * (32 * kTsItems) + j * 32 + lane);
      }
    }
    // ttot[b] becomes the offset from a position in the sorted tile to its place in the output
    for (int b = tid; b < B; b += kTsThreads) {
      const int c = ttot[b];
      ttot[b] = base[b] - tstart[b];
      base[b] += c;
    }
    __syncthreads();
    const int n = tstart[B];
    const int t_lo = (int)t0;  // numel < 2^31
    for (int p = tid; p < n; p += kTsThreads) {
      const int e = val[p];
      sorted[ttot[e >> 12] + p] = t_lo + (e & (kTsTile - 1));
    }
    __syncthreads();
  }
}

static size_t tile_scatter_smem_bytes(int B) {
  return sizeof(int) * ((size_t)kTsWarps * B + 5 * (size_t)B + 2 + 40 + kTsTile);
}

// Chunks of the tile-sorted path: two CTAs per SM, chunk lengths a multiple of the tile (and of the histogram
// kernel's 32 warps x 32 ids).
static void align_plan_large(int64_t numel, int64_t* chunks, int64_t* chunk_len) {
  int64_t len = (numel + kMaxChunks - 1) / kMaxChunks;
  len = (len + kTsTile - 1) / kTsTile * kTsTile;
  *chunk_len = len;
  *chunks = (numel + len - 1) / len;
}

// How the ids are cut: number of chunks (CTAs) and ids per warp (a multiple of 32).
static void align_plan(int64_t numel, int64_t* chunks, int* span) {
  if (numel <= kSingleMax) {
    *chunks = 1;
    const int64_t per_warp = (numel + kAlignWarps - 1) / kAlignWarps;
    *span = (int)((per_warp + 31) / 32 * 32);
    if (*span == 0) *span = 32;
    return;
  }
  int64_t c = (numel + 1023) / 1024;
  if (c > kMidMaxChunks) c = kMidMaxChunks;
  int64_t chunk_len = (numel + c - 1) / c;
  chunk_len = (chunk_len + 1023) / 1024 * 1024;  // 32 warps x a multiple of 32 ids
  *span = (int)(chunk_len / kAlignWarps);
  *chunks = (numel + chunk_len - 1) / chunk_len;
}

static size_t align_smem_bytes(int B) { return sizeof(int) * ((size_t)kAlignWarps * B + 3 * (size_t)B + 1 + 33 + 8); }

}  // namespace sglb200

using namespace sglb200;

extern "C" void sglb200_moe_align_set_cooperative(int on) { g_align_coop_enabled = on != 0; }

extern "C" int64_t sglb200_moe_align_workspace_bytes(int64_t numel, int num_experts) {
  if (numel <= kSingleMax) return 0;
  int64_t chunks = 0;
  if (numel > kLargeMin) {
    int64_t chunk_len = 0;
    align_plan_large(numel, &chunks, &chunk_len);
  } else {
    int span = 0;
    align_plan(numel, &chunks, &span);
  }
  return (chunks + 1) * (int64_t)num_experts * (int64_t)sizeof(int);
}

extern "C" int sglb200_moe_align_block_size(const int32_t* topk_ids, int64_t numel, int num_experts, int block_size,
                                            int32_t* sorted_token_ids, int32_t* expert_ids,
                                            int32_t* num_tokens_post_pad, int32_t* cumsum_buffer,
                                            int pad_sorted_token_ids, void* workspace, int64_t workspace_bytes,
                                            void* stream) {
  SGLB_REQUIRE(numel >= 0 && numel < (1ll << 31) - (int64_t)num_experts * block_size, "moe_align: numel %lld too large",
               (long long)numel);
  SGLB_REQUIRE(num_experts >= 1 && block_size >= 1, "moe_align: num_experts %d, block_size %d", num_experts, block_size);
  SGLB_REQUIRE(sorted_token_ids && expert_ids && num_tokens_post_pad && cumsum_buffer && (topk_ids || numel == 0),
               "moe_align: null pointer");
  const int B = num_experts;
  const size_t smem = align_smem_bytes(B);
  SGLB_REQUIRE(smem <= 200 * 1024, "moe_align: %d buckets need %zu bytes of shared memory (limit 200 KiB)", B, smem);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (smem > 48 * 1024) {
    // opt in to more than 48 KiB of dynamic shared memory (a per-function, per-device attribute; cheap to repeat)
    SGLB_CUDA(cudaFuncSetAttribute(moe_align_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    SGLB_CUDA(cudaFuncSetAttribute(moe_align_hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    SGLB_CUDA(cudaFuncSetAttribute(moe_align_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  }
  if (numel > kLargeMin) {
    SGLB_REQUIRE(B <= 8160, "moe_align: %d buckets exceed the bucket field of the large-input path", B);
    const size_t ts_smem = tile_scatter_smem_bytes(B);
    SGLB_REQUIRE(ts_smem <= 200 * 1024, "moe_align: %d buckets need %zu bytes of shared memory (limit 200 KiB)", B,
                 ts_smem);
    const int nbits = 32 - __builtin_clz((unsigned)(B + 31));  // keys run up to B + 31
    int64_t lchunks = 0, chunk_len = 0;
    align_plan_large(numel, &lchunks, &chunk_len);
    const int64_t lneed = (lchunks + 1) * (int64_t)B * (int64_t)sizeof(int);
    if (workspace == nullptr || workspace_bytes < lneed)
      return fail(SGLB200_E_WORKSPACE, "moe_align: workspace of %lld bytes required, got %lld", (long long)lneed,
                  (long long)workspace_bytes);
    int* hist = static_cast<int*>(workspace);
    int* tot = hist + lchunks * B;
    moe_align_hist_kernel<<<(unsigned)lchunks, kAlignThreads, smem, st>>>(topk_ids, numel, (int)(chunk_len / kAlignWarps),
                                                                          B, hist);
    moe_align_scan_kernel<<<(unsigned)((B + kAlignWarps - 1) / kAlignWarps), kAlignThreads, 0, st>>>(hist, tot,
                                                                                                     (int)lchunks, B);
#define SGLB_TILE_SCATTER(NB)                                                                                       \
  case NB:                                                                                                          \
    if (ts_smem > 48 * 1024)                                                                                        \
      SGLB_CUDA(cudaFuncSetAttribute(moe_align_tile_scatter_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                     200 * 1024));                                                                  \
    moe_align_tile_scatter_kernel<NB><<<(unsigned)lchunks, kTsThreads, ts_smem, st>>>(                              \
        topk_ids, numel, chunk_len, B, block_size, hist, tot, sorted_token_ids, expert_ids, num_tokens_post_pad,    \
        cumsum_buffer, pad_sorted_token_ids != 0);                                                                  \
    break
    switch (nbits) {
      SGLB_TILE_SCATTER(6);
      SGLB_TILE_SCATTER(7);
      SGLB_TILE_SCATTER(8);
      SGLB_TILE_SCATTER(9);
      SGLB_TILE_SCATTER(10);
      SGLB_TILE_SCATTER(11);
      SGLB_TILE_SCATTER(12);
      default: SGLB_TILE_SCATTER(13);
    }
#undef SGLB_TILE_SCATTER
    SGLB_CUDA(cudaGetLastError());
    return SGLB200_OK;
  }
  int64_t chunks = 0;
  int span = 0;
  align_plan(numel, &chunks, &span);
  if (chunks == 1) {
    moe_align_single_kernel<<<1, kAlignThreads, smem, st>>>(topk_ids, numel, span, B, block_size, sorted_token_ids, expert_ids,
                                                            num_tokens_post_pad, cumsum_buffer,
                                                            pad_sorted_token_ids != 0);
    SGLB_CUDA(cudaGetLastError());
    return SGLB200_OK;
  }
  const int64_t need = sglb200_moe_align_workspace_bytes(numel, num_experts);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(SGLB200_E_WORKSPACE, "moe_align: workspace of %lld bytes required, got %lld", (long long)need,
                (long long)workspace_bytes);
  int* chunk_hist = static_cast<int*>(workspace);
  int* totals = chunk_hist + chunks * B;
  if (kAlignCoop && g_align_coop_enabled) {
    const CoopKernel kern = coop_kernel_for(B);
    if (smem > 48 * 1024)
      SGLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    if (coop_fits(kern, chunks, smem)) {
      bool pad = pad_sorted_token_ids != 0;
      void* args[] = {&topk_ids, &numel, &span, (void*)&B, &block_size, &chunk_hist, &sorted_token_ids, &expert_ids,
                      &num_tokens_post_pad, &cumsum_buffer, &pad};
      SGLB_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kern),
                                            dim3((unsigned)chunks), dim3(kAlignThreads), args, smem, st));
      return SGLB200_OK;
    }
  }
  moe_align_hist_kernel<<<(unsigned)chunks, kAlignThreads, smem, st>>>(topk_ids, numel, span, B, chunk_hist);
  moe_align_scan_kernel<<<(unsigned)((B + kAlignWarps - 1) / kAlignWarps), kAlignThreads, 0, st>>>(chunk_hist, totals,
                                                                                                   (int)chunks, B);
  moe_align_scatter_kernel<<<(unsigned)chunks, kAlignThreads, smem, st>>>(topk_ids, numel, span, B, block_size, chunk_hist,
                                                                          totals, sorted_token_ids, expert_ids,
                                                                          num_tokens_post_pad, cumsum_buffer,
                                                                          pad_sorted_token_ids != 0);
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant.
//
// Some callers of this library cannot obtain device memory at the moment they need the sort: code
// running while a stream is being captured into a CUDA graph with the allocator frozen, a serving
// process whose memory pool has been handed over entirely to the KV cache, or a host program that is
// not built on torch and has no allocator of its own to ask.  For them the scratch the sort needs (the
// padded prefix and the per-chunk histograms) lives in a fixed array inside the library image instead
// of in caller-provided buffers.  Every GPU that loads the library holds this array until exit.
// ---------------------------------------------------------------------------------------------
namespace sglb200 {

constexpr int kNoAllocMaxBuckets = 1024;                               // experts + 1
constexpr int64_t kNoAllocMaxNumel = 1 << 20;                          // flat top-k ids
constexpr int64_t kNoAllocMaxChunks = kNoAllocMaxNumel / kChunk;       // 128 (align_plan never uses more for 2^20 ids)
constexpr int64_t kNoAllocScratchInts =
    (kNoAllocMaxBuckets + 1) + (kNoAllocMaxChunks + 1) * kNoAllocMaxBuckets;  // prefix + histograms + totals

static __device__ __align__(256) int g_noalloc_scratch[kNoAllocScratchInts];

// Device address of g_noalloc_scratch for the CURRENT device, resolved once per device.  In host code
// the array's name is only a handle for the runtime, never a pointer a kernel may dereference.
static int noalloc_scratch_ptr(int** out) {
  static std::mutex mu;
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  SGLB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(SGLB200_E_INVALID, "moe_align (no-alloc): device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    SGLB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    ptrs[dev] = static_cast<int*>(p);
  }
  *out = ptrs[dev];
  return SGLB200_OK;
}

}  // namespace sglb200

extern "C" int sglb200_moe_align_block_size_noalloc(const int32_t* topk_ids, int64_t numel, int num_experts,
                                                    int block_size, int32_t* sorted_token_ids, int32_t* expert_ids,
                                                    int32_t* num_tokens_post_pad, int pad_sorted_token_ids,
                                                    void* stream) {
  if (num_experts > kNoAllocMaxBuckets)
    return fail(SGLB200_E_INVALID,
                "moe_align (no-alloc): %d buckets exceed the built-in scratch (at most %d, i.e. %d experts + 1); use "
                "sglb200_moe_align_block_size with caller-provided buffers",
                num_experts, kNoAllocMaxBuckets, kNoAllocMaxBuckets - 1);
  if (numel > kNoAllocMaxNumel)
    return fail(SGLB200_E_INVALID,
                "moe_align (no-alloc): %lld ids exceed the built-in scratch (at most %lld); use "
                "sglb200_moe_align_block_size with caller-provided buffers",
                (long long)numel, (long long)kNoAllocMaxNumel);
  int* scratch = nullptr;
  const int rc = noalloc_scratch_ptr(&scratch);
  if (rc != SGLB200_OK) return rc;
  // layout: [0, B+1) padded prefix; then the chunk histograms and totals.  The kernels overwrite every
  // word they later read, so nothing has to be cleared between calls.
  int32_t* cumsum = scratch;
  void* workspace = scratch + (kNoAllocMaxBuckets + 1);
  const int64_t workspace_bytes = (kNoAllocMaxChunks + 1) * (int64_t)kNoAllocMaxBuckets * (int64_t)sizeof(int);
  return sglb200_moe_align_block_size(topk_ids, numel, num_experts, block_size, sorted_token_ids, expert_ids,
                                      num_tokens_post_pad, cumsum, pad_sorted_token_ids, workspace, workspace_bytes,
                                      stream);
}
