// 1 x G activation quantizer (float8_e4m3fn codes + float32 scales) and the fused
// silu_and_mul + quantizer, for sm_100a.
//
// Both are streaming kernels on one skeleton: persistent CTAs walk tiles of 8192 elements that one thread
// stages with bulk copies (cp.async.bulk) into a ring of shared-memory buffers completing on mbarriers, so
// the bytes in flight per SM do not depend on registers or occupancy; every input byte is read from HBM
// once; a thread owns 32 elements of one group per tile, the group maximum takes two shuffle rounds, and
// every quad of lanes writes one full 32-byte sector of codes.
//
// Arithmetic contract (bit-exact with the reference CUDA kernel built without fast-math):
//   amax  = max(|x|, eps)            scale = amax / fp8_max      (div.rn.f32)
//   code  = cvt.rn.satfinite.e4m3( min(max(x / scale, fp8_min), fp8_max) )   (div.rn.f32)
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace sglb200 {

// ---- streaming skeleton shared by the quantizer and the fused activation + quantizer ----------------
//
// A CTA walks tiles of kTileElems consecutive elements (tile t, t + gridDim.x, ...).  One thread stages
// each tile with a 1-D bulk copy (cp.async.bulk) into a ring of kStreamStages shared-memory buffers that
// complete on mbarriers, so the bytes in flight per SM are set by the ring and not by registers or
// occupancy.  A thread owns kThreadElems = 32 elements of ONE group per tile (a 128-group is shared by four
// lanes: two shuffle rounds per 32 elements), read as 16-byte chunks interleaved over the lanes of the
// group so that shared-memory reads are conflict-free and every quad of lanes writes one full 32-byte
// sector of codes.
constexpr int kStreamThreads = 256;
constexpr int kThreadElems = 32;
constexpr int kTileElems = kStreamThreads * kThreadElems;  // 8192
template <typename T>
constexpr int kStagesOf = sizeof(T) == 4 ? 3 : 4;  // 64 KB (16-bit types) or 96 KB (float32) of ring per CTA

__device__ int g_stream_status = 0;  // 0 ok, 1 = a wait for a staged tile expired
static uint32_t g_stream_wait_probes = ptx::kProbeLimit;  // sglb200_stream_set_wait_probes

// A CTA that gave up a wait: it records the failure and then holds its shared memory for about a millisecond, so
// that bulk copies it has already issued into other ring slots land before the SM hands the memory to another CTA.
__device__ __forceinline__ void stream_give_up(int tid) {
  if (tid == 0) {
    atomicExch(&g_stream_status, 1);
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) {
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ uint4 lds_128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// max(m, |a|, |b|) that returns NaN if any input is NaN: one group-wide test then tells whether the group
// holds a NaN or an infinity and must take the careful path.
__device__ __forceinline__ float max3_abs_nan(float m, float a, float b) {
  float r;
  asm("{\n\t.reg .f32 ta, tb;\n\t"
      "abs.f32 ta, %2;\n\tabs.f32 tb, %3;\n\t"
      "max.NaN.f32 %0, %1, ta, tb;\n\t}"
      : "=f"(r)
      : "f"(m), "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

template <typename T>
struct Chunk {  // a 16-byte chunk of T
  static constexpr int kElems = 16 / (int)sizeof(T);
  static constexpr int kPerThread = kThreadElems / kElems;  // chunks a thread owns per tile
};

template <typename T>
__device__ __forceinline__ void unpack_chunk(const uint4& raw, float* v);
template <>
__device__ __forceinline__ void unpack_chunk<__nv_bfloat16>(const uint4& raw, float* v) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void unpack_chunk<__half>(const uint4& raw, float* v) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void unpack_chunk<float>(const uint4& raw, float* v) {
  v[0] = __uint_as_float(raw.x), v[1] = __uint_as_float(raw.y);
  v[2] = __uint_as_float(raw.z), v[3] = __uint_as_float(raw.w);
}

// Sign bits of the chunk's elements, one per byte (bit 7), in element order.
template <typename T>
__device__ __forceinline__ void chunk_signs(const uint4& raw, uint32_t* s) {
  if constexpr (sizeof(T) == 2) {
    s[0] = __byte_perm(raw.x, raw.y, 0x7531) & 0x80808080u;
    s[1] = __byte_perm(raw.z, raw.w, 0x7531) & 0x80808080u;
  } else {
    s[0] = __byte_perm(__byte_perm(raw.x, raw.y, 0x0073), __byte_perm(raw.z, raw.w, 0x0073), 0x5410) & 0x80808080u;
  }
}

// Codes of one chunk when every element of the group is finite and the scale is in the range where the
// division-free quotient is exact (see quant_chunk_careful).  With the standard range no clamp is needed: a quotient can
// exceed 448 only by rounding and the conversion saturates; the sign of a zero quotient is taken from the
// input bits (it is the only case in which the computed sign can differ from the numerator's).
template <typename T, bool kStdRange>
__device__ __forceinline__ void quant_chunk_fast(const uint4& raw, const float* v, float scale, float r, float qmin,
                                                 float qmax, uint32_t* codes) {
  constexpr int CE = Chunk<T>::kElems;
  float q[CE];
#pragma unroll
  for (int i = 0; i < CE; ++i) {
    const float q0 = __fmul_rn(v[i], r);
    const float e = __fmaf_rn(-q0, scale, v[i]);
    q[i] = __fmaf_rn(e, r, q0);
    if (!kStdRange) q[i] = fminf(fmaxf(copysignf(q[i], v[i]), qmin), qmax);
  }
#pragma unroll
  for (int i = 0; i < CE / 4; ++i) codes[i] = pack_e4m3x4(q[4 * i], q[4 * i + 1], q[4 * i + 2], q[4 * i + 3]);
  if (kStdRange) {
    uint32_t s[CE / 4];
    chunk_signs<T>(raw, s);
#pragma unroll
    for (int i = 0; i < CE / 4; ++i) codes[i] |= s[i];
  }
}

// Codes of one chunk by the full contract (any input, any scale).
//
// The contract is code = e4m3(min(max(RN(x / scale), qmin), qmax)) with an IEEE float32 division.  A
// div.rn.f32 costs about ten instructions per element, which makes the kernel issue-bound, so the quotient
// is formed without dividing: with r = RN(1/scale) computed once per group,
//     q0 = RN(x*r);  e = fma(-q0, scale, x) (exact residual);  q = fma(e, r, q0);  q = copysign(q, x)
// equals RN(x / scale) bit for bit whenever |q| >= 2^-20 (checked exhaustively for every bf16 / fp16 input
// pair and on ~1e8 random float32 pairs by tests/exact_div_check.c); smaller quotients may differ in float32
// but encode as the same signed zero.  copysign restores the sign of a zero numerator.  Scales outside
// [1e-30, 1e36] (an infinite group maximum, or a caller-chosen eps near zero) take the IEEE division.
// Both clamps are applied: the lower one is also what turns a NaN quotient into -448, as in the reference.
template <typename T>
__device__ __forceinline__ void quant_chunk_careful(const float* v, float scale, float qmin, float qmax,
                                                    uint32_t* codes) {
  constexpr int CE = Chunk<T>::kElems;
  float q[CE];
  if (scale >= 1e-30f && scale <= 1e36f) {
    const float r = __frcp_rn(scale);
#pragma unroll
    for (int i = 0; i < CE; ++i) {
      const float q0 = __fmul_rn(v[i], r);
      const float e = __fmaf_rn(-q0, scale, v[i]);
      q[i] = copysignf(__fmaf_rn(e, r, q0), v[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < CE; ++i) q[i] = __fdiv_rn(v[i], scale);
  }
#pragma unroll
  for (int i = 0; i < CE; ++i) q[i] = fminf(fmaxf(q[i], qmin), qmax);
#pragma unroll
  for (int i = 0; i < CE / 4; ++i) codes[i] = pack_e4m3x4(q[4 * i], q[4 * i + 1], q[4 * i + 2], q[4 * i + 3]);
}

// Interleaving of a group's 16-byte chunks over its LPG lanes: lane l reads chunk (LPG * j + l + rot) mod GC at
// step j, where rot depends on the group's position so that the eight threads of a quarter warp always touch
// eight different 16-byte bank groups.
template <typename T, int LPG>
__device__ __forceinline__ int chunk_rotation(int g) {
  constexpr int GC = LPG * Chunk<T>::kPerThread;  // chunks per group
  if (LPG >= 8) return 0;
  if (LPG == 1) return GC >= 8 ? (g & 7) : ((g >> 1) & (GC - 1));
  return LPG * (g & (8 / LPG - 1));
}

// Scale and codes of the group this thread shares with LPG - 1 neighbouring lanes.  v holds the thread's 32
// values (chunk-major), raw the bits they came from.  Every lane of the warp calls this together.
template <typename T, int LPG, bool kStdRange>
__device__ __forceinline__ float quant_group(const uint4* raw, const float* v, float eps, float qmin, float qmax,
                                             uint32_t (*codes)[Chunk<T>::kElems / 4]) {
  constexpr int CE = Chunk<T>::kElems, NCH = Chunk<T>::kPerThread;
  float m = eps;
#pragma unroll
  for (int i = 0; i < NCH * CE; i += 2) m = max3_abs_nan(m, v[i], v[i + 1]);
#pragma unroll
  for (int off = LPG / 2; off >= 1; off >>= 1) m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, off));
  float scale = __fdiv_rn(m, qmax);
  if (m < __int_as_float(0x7f800000) && scale >= 1e-30f && scale <= 1e36f) {
    const float r = __frcp_rn(scale);
#pragma unroll
    for (int j = 0; j < NCH; ++j) quant_chunk_fast<T, kStdRange>(raw[j], v + j * CE, scale, r, qmin, qmax, codes[j]);
  } else {
    // a NaN or an infinity in the group, or an extreme scale: the reference's maximum ignores NaNs
    const unsigned lane = threadIdx.x & 31u;
    const unsigned gmask = (LPG == 32 ? 0xffffffffu : ((1u << LPG) - 1u)) << (lane & ~(unsigned)(LPG - 1));
    float a = eps;
#pragma unroll
    for (int i = 0; i < NCH * CE; ++i) a = fmaxf(a, fabsf(v[i]));
#pragma unroll
    for (int off = LPG / 2; off >= 1; off >>= 1) a = fmaxf(a, __shfl_xor_sync(gmask, a, off));
    scale = __fdiv_rn(a, qmax);
#pragma unroll
    for (int j = 0; j < NCH; ++j) quant_chunk_careful<T>(v + j * CE, scale, qmin, qmax, codes[j]);
  }
  return scale;
}

// The quantizer.  `issue(i)` (thread 0) arms the slot's mbarrier with the byte count of this CTA's i-th tile and
// starts its copy.

template <typename T, int LPG, bool kStdRange>
__global__ void __launch_bounds__(kStreamThreads, 3)
    quant_stream_kernel(const T* __restrict__ x, uint8_t* __restrict__ out_q, float* __restrict__ out_s,
                        int64_t total_elems, int groups_per_row, int64_t s_stride_token, int64_t s_stride_group,
                        bool s_contiguous, float eps, float qmin, float qmax, uint32_t probes) {
  constexpr int CE = Chunk<T>::kElems, NCH = Chunk<T>::kPerThread, GC = LPG * NCH;
  constexpr int G = LPG * kThreadElems;
  constexpr int kStreamStages = kStagesOf<T>;
  constexpr uint32_t kTileBytes = kTileElems * sizeof(T);
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[kStreamStages];
  __shared__ int s_abort;
  const uint32_t smem_base = ptx::smem_u32(smem_raw);
  const int tid = threadIdx.x;
  const int64_t tiles = (total_elems + kTileElems - 1) / kTileElems;
  const int64_t my_tiles = (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;  // > 0: the grid never exceeds tiles

  auto issue = [&](int64_t i) {  // thread 0 only
    const int slot = (int)(i % kStreamStages);
    const int64_t e0 = (blockIdx.x + i * gridDim.x) * (int64_t)kTileElems;
    const int64_t left = total_elems - e0;
    const uint32_t bytes = left >= kTileElems ? kTileBytes : (uint32_t)(left * sizeof(T));
    const uint32_t bar = ptx::smem_u32(&bars[slot]);
    ptx::mbar_arrive_expect_tx(bar, bytes);
    bulk_load_1d(smem_base + slot * kTileBytes, x + e0, bytes, bar);
  };

  if (tid == 0) {
    s_abort = 0;
#pragma unroll
    for (int s = 0; s < kStreamStages; ++s) ptx::mbar_init(ptx::smem_u32(&bars[s]), 1);
    ptx::mbar_fence_init();
    for (int64_t i = 0; i < kStreamStages && i < my_tiles; ++i) issue(i);
  }
  __syncthreads();

  const int g_local = tid / LPG, l = tid % LPG;
  const int rot = chunk_rotation<T, LPG>(g_local);
  int cj[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) cj[j] = (LPG * j + l + rot) % GC;

  for (int64_t i = 0; i < my_tiles; ++i) {
    const int slot = (int)(i % kStreamStages);
    const uint32_t parity = (uint32_t)((i / kStreamStages) & 1);
    if (!ptx::mbar_probe(ptx::smem_u32(&bars[slot]), parity, probes)) s_abort = 1;
    uint4 raw[NCH];
    const uint32_t src = smem_base + slot * kTileBytes + (uint32_t)(g_local * GC) * 16u;
#pragma unroll
    for (int j = 0; j < NCH; ++j) raw[j] = lds_128(src + (uint32_t)cj[j] * 16u);
    __syncthreads();  // every thread holds its part of the slot in registers: the slot can be refilled
    if (s_abort) {  // (uniform: read after the barrier)
      stream_give_up(tid);
      return;
    }
    if (tid == 0 && i + kStreamStages < my_tiles) issue(i + kStreamStages);

    float v[NCH * CE];
#pragma unroll
    for (int j = 0; j < NCH; ++j) unpack_chunk<T>(raw[j], v + j * CE);
    uint32_t codes[NCH][CE / 4];
    const float scale = quant_group<T, LPG, kStdRange>(raw, v, eps, qmin, qmax, codes);

    const int64_t e0 = (blockIdx.x + i * gridDim.x) * (int64_t)kTileElems;
    const int64_t ge = e0 + (int64_t)g_local * G;  // first element of this thread's group
    if (ge < total_elems) {
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        uint8_t* dst = out_q + ge + cj[j] * CE;
        if constexpr (CE == 8) {
          *reinterpret_cast<uint2*>(dst) = make_uint2(codes[j][0], codes[j][1]);
        } else {
          *reinterpret_cast<uint32_t*>(dst) = codes[j][0];
        }
      }
      if (l == 0) {
        const int64_t g = ge / G;
        if (s_contiguous) {
          out_s[g] = scale;
        } else {
          const int64_t t = g / groups_per_row;
          out_s[t * s_stride_token + (g - t * groups_per_row) * s_stride_group] = scale;
        }
      }
    }
  }
}

// Fused silu_and_mul + quantizer on the same skeleton.  x is [rows, 2d] (gate | up); a tile is kTileElems
// consecutive OUTPUT elements of the flat [rows, d] result, staged as one or more (gate, up) pairs of row
// segments.  h = T(T(silu(gate)) * up): silu in float32 rounded to T, then one packed multiply (the product of
// two 16-bit floats is exact in float32, so its single rounding equals rounding the float32 product), then
// the quantizer arithmetic on h in registers.
template <typename T>
struct Packed2;
template <>
struct Packed2<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t round_mul(float a, float b, uint32_t up) {
    const __nv_bfloat162 act = __floats2bfloat162_rn(a, b);
    const __nv_bfloat162 h = __hmul2(act, *reinterpret_cast<const __nv_bfloat162*>(&up));
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};
template <>
struct Packed2<__half> {
  static __device__ __forceinline__ uint32_t round_mul(float a, float b, uint32_t up) {
    const __half2 act = __floats2half2_rn(a, b);
    const __half2 h = __hmul2(act, *reinterpret_cast<const __half2*>(&up));
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};

constexpr int kSiluStages = 2;  // 2 x (16 KB gate + 16 KB up) per CTA, three CTAs per SM (80 registers)

constexpr int kMaskedMaxExperts = 1024;  // experts of one masked call (four per thread in the tile count scan)

// kMasked: the input is [experts, rows_per_expert, 2d] and only the first masked_m[e] rows of expert e are valid
// (the layout of python/sglang/srt/layers/moe/ep_moe/kernels.py:287-361).  The valid rows of every expert are cut
// into tiles of their own, numbered one expert after the other; rows beyond masked_m[e] are neither read nor written.
template <typename T, int LPG, bool kMasked>
__global__ void __launch_bounds__(kStreamThreads, 3)
    silu_mul_quant_stream_kernel(const T* __restrict__ x, uint8_t* __restrict__ out_q, float* __restrict__ out_s,
                                 int64_t rows, int d, const int32_t* __restrict__ num_rows_dev, float eps, float qmin,
                                 float qmax, uint32_t probes, const int32_t* __restrict__ masked_m, int num_experts,
                                 int64_t rows_per_expert) {
  static_assert(sizeof(T) == 2, "16-bit inputs only");
  constexpr int CE = 8, NCH = 4, GC = LPG * NCH, G = LPG * kThreadElems;
  constexpr uint32_t kHalfBytes = kTileElems * 2;  // gate part of a stage; the up part follows it
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[kSiluStages];
  __shared__ int s_abort;
  __shared__ int s_tiles_before[kMasked ? kMaskedMaxExperts + 1 : 1];  // tiles of the experts before e
  __shared__ int s_warp_sum[kStreamThreads / 32];
  if (num_rows_dev != nullptr) {
    const int64_t lim = *num_rows_dev;
    rows = lim < rows ? lim : rows;
  }
  const uint32_t smem_base = ptx::smem_u32(smem_raw);
  const int tid = threadIdx.x;
  int64_t total_elems = rows * d;
  int64_t tiles = (total_elems + kTileElems - 1) / kTileElems;
  auto valid_rows = [&](int e) -> int64_t {
    const int64_t m = masked_m[e];
    return m < 0 ? 0 : (m > rows_per_expert ? rows_per_expert : m);
  };
  if constexpr (kMasked) {
    // exclusive scan of the experts' tile counts: four experts per thread, then the warps' sums
    int cnt[4], mine = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int e = tid * 4 + k;
      cnt[k] = e < num_experts ? (int)((valid_rows(e) * d + kTileElems - 1) / kTileElems) : 0;
      mine += cnt[k];
    }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if ((tid & 31) >= o) incl += up;
    }
    if ((tid & 31) == 31) s_warp_sum[tid >> 5] = incl;
    __syncthreads();
    int before = incl - mine;
    for (int w = 0; w < (tid >> 5); ++w) before += s_warp_sum[w];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int e = tid * 4 + k;
      if (e < num_experts) s_tiles_before[e] = before;
      before += cnt[k];
    }
    if (tid == kStreamThreads - 1) s_tiles_before[num_experts] = before;  // (experts beyond num_experts count 0)
    __syncthreads();
    tiles = s_tiles_before[num_experts];
  }
  if ((int64_t)blockIdx.x >= tiles) return;  // the grid is sized from the host-side bound on rows
  const int64_t my_tiles = (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;

  // tile i of this CTA: first element within its expert (or within the whole input), that range's element count, and
  // the range's first row
  auto locate = [&](int64_t i, int64_t& e0, int64_t& lim, int64_t& row_base) {
    const int64_t gt = blockIdx.x + i * gridDim.x;
    if constexpr (kMasked) {
      int lo = 0, hi = num_experts;  // the expert with s_tiles_before[e] <= gt < s_tiles_before[e + 1]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((int64_t)s_tiles_before[mid] <= gt) lo = mid; else hi = mid;
      }
      e0 = (gt - s_tiles_before[lo]) * (int64_t)kTileElems;
      lim = valid_rows(lo) * d;
      row_base = (int64_t)lo * rows_per_expert;
    } else {
      e0 = gt * (int64_t)kTileElems;
      lim = total_elems;
      row_base = 0;
    }
  };

  auto issue = [&](int64_t i) {  // thread 0 only
    const int slot = (int)(i % kSiluStages);
    int64_t e0, lim, row_base;
    locate(i, e0, lim, row_base);
    const int64_t left = lim - e0;
    const int n = left >= kTileElems ? kTileElems : (int)left;
    const uint32_t bar = ptx::smem_u32(&bars[slot]);
    const uint32_t dst = smem_base + slot * (2 * kHalfBytes);
    ptx::mbar_arrive_expect_tx(bar, (uint32_t)n * 4u);
    int64_t r = e0 / d;
    int c = (int)(e0 - r * d);
    r += row_base;
    for (int off = 0; off < n;) {
      const int seg = (d - c) < (n - off) ? (d - c) : (n - off);
      const T* row = x + r * 2 * (int64_t)d + c;
      bulk_load_1d(dst + off * 2, row, (uint32_t)seg * 2u, bar);
      bulk_load_1d(dst + kHalfBytes + off * 2, row + d, (uint32_t)seg * 2u, bar);
      off += seg;
      c = 0;
      ++r;
    }
  };

  if (tid == 0) {
    s_abort = 0;
#pragma unroll
    for (int s = 0; s < kSiluStages; ++s) ptx::mbar_init(ptx::smem_u32(&bars[s]), 1);
    ptx::mbar_fence_init();
    for (int64_t i = 0; i < kSiluStages && i < my_tiles; ++i) issue(i);
  }
  __syncthreads();

  const int g_local = tid / LPG, l = tid % LPG;
  const int rot = chunk_rotation<T, LPG>(g_local);
  int cj[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) cj[j] = (LPG * j + l + rot) % GC;

  for (int64_t i = 0; i < my_tiles; ++i) {
    const int slot = (int)(i % kSiluStages);
    const uint32_t parity = (uint32_t)((i / kSiluStages) & 1);
    if (!ptx::mbar_probe(ptx::smem_u32(&bars[slot]), parity, probes)) s_abort = 1;
    uint4 graw[NCH], uraw[NCH];
    const uint32_t src = smem_base + slot * (2 * kHalfBytes) + (uint32_t)(g_local * GC) * 16u;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      graw[j] = lds_128(src + (uint32_t)cj[j] * 16u);
      uraw[j] = lds_128(src + kHalfBytes + (uint32_t)cj[j] * 16u);
    }
    __syncthreads();  // the slot is in registers and can be refilled
    if (s_abort) {  // (uniform: read after the barrier)
      stream_give_up(tid);
      return;
    }
    if (tid == 0 && i + kSiluStages < my_tiles) issue(i + kSiluStages);

    uint4 hraw[NCH];
    float v[NCH * CE];
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      float g[CE];
      unpack_chunk<T>(graw[j], g);
      const uint32_t up[4] = {uraw[j].x, uraw[j].y, uraw[j].z, uraw[j].w};
      uint32_t h[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) h[k] = Packed2<T>::round_mul(silu_f32(g[2 * k]), silu_f32(g[2 * k + 1]), up[k]);
      hraw[j] = make_uint4(h[0], h[1], h[2], h[3]);
      unpack_chunk<T>(hraw[j], v + j * CE);
    }
    uint32_t codes[NCH][CE / 4];
    const float scale = quant_group<T, LPG, true>(hraw, v, eps, qmin, qmax, codes);

    int64_t e0, lim, row_base;
    locate(i, e0, lim, row_base);
    const int64_t ge_in = e0 + (int64_t)g_local * G;
    if (ge_in < lim) {
      const int64_t ge = row_base * d + ge_in;
#pragma unroll
      for (int j = 0; j < NCH; ++j)
        *reinterpret_cast<uint2*>(out_q + ge + cj[j] * CE) = make_uint2(codes[j][0], codes[j][1]);
      if (l == 0) out_s[ge / G] = scale;
    }
  }
}

template <typename T, int LPG, bool kStd>
static int launch_quant_inst(const void* input, void* output_q, float* output_s, int64_t total_elems,
                             int groups_per_row, int64_t s_stride_token, int64_t s_stride_group, bool contiguous,
                             float eps, float qmin, float qmax, cudaStream_t stream) {
  constexpr size_t smem = (size_t)kStagesOf<T> * kTileElems * sizeof(T);
  auto kern = quant_stream_kernel<T, LPG, kStd>;
  // opt in to the ring's dynamic shared memory (a per-function, per-device attribute; cheap to repeat)
  SGLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int64_t tiles = (total_elems + kTileElems - 1) / kTileElems;
  const int64_t resident = (int64_t)sm_count() * (sizeof(T) == 4 ? 2 : 3);
  const unsigned grid = (unsigned)(tiles < resident ? tiles : resident);
  kern<<<grid, kStreamThreads, smem, stream>>>(static_cast<const T*>(input), static_cast<uint8_t*>(output_q), output_s,
                                               total_elems, groups_per_row, s_stride_token, s_stride_group, contiguous,
                                               eps, qmin, qmax, g_stream_wait_probes);
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}

template <typename T>
static int launch_quant(const void* input, void* output_q, float* output_s, int64_t num_tokens, int64_t hidden,
                        int group_size, float eps, float qmin, float qmax, int64_t s_stride_token,
                        int64_t s_stride_group, cudaStream_t stream) {
  const int64_t total = num_tokens * hidden;
  const int groups_per_row = (int)(hidden / group_size);
  const bool contiguous = (s_stride_group == 1 && s_stride_token == groups_per_row);
  if (total == 0) return SGLB200_OK;
  const bool std_range = (qmin == -448.0f && qmax == 448.0f);
#define SGLB_LAUNCH_Q(LPG)                                                                                          \
  return std_range ? launch_quant_inst<T, LPG, true>(input, output_q, output_s, total, groups_per_row,              \
                                                     s_stride_token, s_stride_group, contiguous, eps, qmin, qmax,   \
                                                     stream)                                                        \
                   : launch_quant_inst<T, LPG, false>(input, output_q, output_s, total, groups_per_row,             \
                                                      s_stride_token, s_stride_group, contiguous, eps, qmin, qmax,  \
                                                      stream)
  switch (group_size) {
    case 32: SGLB_LAUNCH_Q(1);
    case 64: SGLB_LAUNCH_Q(2);
    case 128: SGLB_LAUNCH_Q(4);
    case 256: SGLB_LAUNCH_Q(8);
    default: return fail(SGLB200_E_INVALID, "quantizer: group_size %d not in {32,64,128,256}", group_size);
  }
#undef SGLB_LAUNCH_Q
}

template <typename T, int LPG, bool kMasked>
static int launch_silu_mul_quant_kernel(const void* input, void* output_q, float* output_s, int64_t rows, int64_t d,
                                        float eps, const int32_t* num_rows_dev, const int32_t* masked_m,
                                        int num_experts, int64_t rows_per_expert, cudaStream_t stream) {
  constexpr size_t smem = (size_t)kSiluStages * 2 * kTileElems * sizeof(T);
  auto kern = silu_mul_quant_stream_kernel<T, LPG, kMasked>;
  SGLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  // (masked: every expert's last tile may be partial, so the bound counts the experts' tiles one by one)
  const int64_t tiles = kMasked ? (int64_t)num_experts * ((rows_per_expert * d + kTileElems - 1) / kTileElems)
                                : (rows * d + kTileElems - 1) / kTileElems;
  const int64_t resident = (int64_t)sm_count() * 3;
  const unsigned grid = (unsigned)(tiles < resident ? tiles : resident);
  kern<<<grid, kStreamThreads, smem, stream>>>(static_cast<const T*>(input), static_cast<uint8_t*>(output_q), output_s,
                                               rows, (int)d, num_rows_dev, eps, -448.0f, 448.0f, g_stream_wait_probes,
                                               masked_m, num_experts, rows_per_expert);
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}

template <typename T, int LPG>
static int launch_silu_mul_quant_inst(const void* input, void* output_q, float* output_s, int64_t rows, int64_t d,
                                      float eps, const int32_t* num_rows_dev, cudaStream_t stream,
                                      const int32_t* masked_m = nullptr, int num_experts = 0,
                                      int64_t rows_per_expert = 0) {
  if (masked_m != nullptr)
    return launch_silu_mul_quant_kernel<T, LPG, true>(input, output_q, output_s, rows, d, eps, nullptr, masked_m,
                                                      num_experts, rows_per_expert, stream);
  return launch_silu_mul_quant_kernel<T, LPG, false>(input, output_q, output_s, rows, d, eps, num_rows_dev, nullptr, 0, 0,
                                                     stream);
}

template <typename T>
static int launch_silu_mul_quant(const void* input, void* output_q, float* output_s, int64_t rows, int64_t d,
                                 int group_size, float eps, const int32_t* num_rows_dev, cudaStream_t stream) {
  if (rows * d == 0) return SGLB200_OK;
  SGLB_REQUIRE(d < (1ll << 30), "silu_mul_quant: d %lld too large", (long long)d);
  switch (group_size) {
    case 32: return launch_silu_mul_quant_inst<T, 1>(input, output_q, output_s, rows, d, eps, num_rows_dev, stream);
    case 64: return launch_silu_mul_quant_inst<T, 2>(input, output_q, output_s, rows, d, eps, num_rows_dev, stream);
    case 128: return launch_silu_mul_quant_inst<T, 4>(input, output_q, output_s, rows, d, eps, num_rows_dev, stream);
    case 256: return launch_silu_mul_quant_inst<T, 8>(input, output_q, output_s, rows, d, eps, num_rows_dev, stream);
    default: return fail(SGLB200_E_INVALID, "silu_mul_quant: group_size %d not in {32,64,128,256}", group_size);
  }
}

template <typename T>
static int launch_silu_mul_quant_masked(const void* input, void* output_q, float* output_s, int num_experts,
                                        int64_t rows_per_expert, int64_t d, int group_size, float eps,
                                        const int32_t* masked_m, cudaStream_t stream) {
  const int64_t rows = (int64_t)num_experts * rows_per_expert;
#define SGLB_MASKED(LPG)                                                                                         \
  return launch_silu_mul_quant_inst<T, LPG>(input, output_q, output_s, rows, d, eps, nullptr, stream, masked_m, \
                                            num_experts, rows_per_expert)
  switch (group_size) {
    case 32: SGLB_MASKED(1);
    case 64: SGLB_MASKED(2);
    case 128: SGLB_MASKED(4);
    case 256: SGLB_MASKED(8);
    default: return fail(SGLB200_E_INVALID, "silu_mul_quant: group_size %d not in {32,64,128,256}", group_size);
  }
#undef SGLB_MASKED
}

}  // namespace sglb200

using namespace sglb200;

extern "C" int sglb200_silu_and_mul_masked_quant_fp8(const void* input, int dtype, void* output_q, float* output_s,
                                                     int num_experts, int64_t rows_per_expert, int64_t d,
                                                     int group_size, float eps, const int32_t* masked_m,
                                                     void* stream) {
  SGLB_REQUIRE(num_experts >= 0 && num_experts <= kMaskedMaxExperts && rows_per_expert >= 0 && d > 0 &&
                   group_size > 0 && d % group_size == 0 && d < (1ll << 30),
               "silu_mul_masked_quant: bad shape experts=%d (at most %d) rows_per_expert=%lld d=%lld group=%d",
               num_experts, kMaskedMaxExperts, (long long)rows_per_expert, (long long)d, group_size);
  if (num_experts == 0 || rows_per_expert == 0) return SGLB200_OK;
  SGLB_REQUIRE(rows_per_expert * d < (1ll << 40), "silu_mul_masked_quant: expert of %lld x %lld elements too large",
               (long long)rows_per_expert, (long long)d);
  SGLB_REQUIRE(input && output_q && output_s && masked_m, "silu_mul_masked_quant: null pointer");
  SGLB_REQUIRE(aligned16(input) && (reinterpret_cast<uintptr_t>(output_q) & 7u) == 0,
               "silu_mul_masked_quant: input must be 16-byte and output_q 8-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case 0:
      return launch_silu_mul_quant_masked<__nv_bfloat16>(input, output_q, output_s, num_experts, rows_per_expert, d,
                                                         group_size, eps, masked_m, st);
    case 1:
      return launch_silu_mul_quant_masked<__half>(input, output_q, output_s, num_experts, rows_per_expert, d,
                                                  group_size, eps, masked_m, st);
    default:
      return fail(SGLB200_E_UNSUPPORTED, "silu_mul_masked_quant: dtype code %d (0 bf16, 1 fp16)", dtype);
  }
}

extern "C" int sglb200_per_token_group_quant_fp8(const void* input, int in_dtype, void* output_q, float* output_s,
                                                 int64_t num_tokens, int64_t hidden, int group_size, float eps,
                                                 float fp8_min, float fp8_max, int64_t s_stride_token,
                                                 int64_t s_stride_group, void* stream) {
  SGLB_REQUIRE(num_tokens >= 0 && hidden > 0, "quantizer: bad shape [%lld, %lld]", (long long)num_tokens,
               (long long)hidden);
  SGLB_REQUIRE(group_size > 0 && hidden % group_size == 0, "quantizer: hidden %lld not divisible by group_size %d",
               (long long)hidden, group_size);
  if (num_tokens == 0) return SGLB200_OK;
  SGLB_REQUIRE(input && output_q && output_s, "quantizer: null pointer");
  SGLB_REQUIRE(aligned16(input) && (reinterpret_cast<uintptr_t>(output_q) & 7u) == 0,
               "quantizer: input must be 16-byte and output_q 8-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (in_dtype) {
    case 0:
      return launch_quant<__nv_bfloat16>(input, output_q, output_s, num_tokens, hidden, group_size, eps, fp8_min,
                                         fp8_max, s_stride_token, s_stride_group, st);
    case 1:
      return launch_quant<__half>(input, output_q, output_s, num_tokens, hidden, group_size, eps, fp8_min, fp8_max,
                                  s_stride_token, s_stride_group, st);
    case 2:
      return launch_quant<float>(input, output_q, output_s, num_tokens, hidden, group_size, eps, fp8_min, fp8_max,
                                 s_stride_token, s_stride_group, st);
    default:
      return fail(SGLB200_E_UNSUPPORTED, "quantizer: dtype code %d (0 bf16, 1 fp16, 2 fp32)", in_dtype);
  }
}

extern "C" int sglb200_silu_and_mul_quant_fp8(const void* input, int dtype, void* output_q, float* output_s,
                                              int64_t rows, int64_t d, int group_size, float eps,
                                              const int32_t* num_rows_dev, void* stream) {
  SGLB_REQUIRE(rows >= 0 && d > 0 && group_size > 0 && d % group_size == 0,
               "silu_mul_quant: bad shape rows=%lld d=%lld group=%d", (long long)rows, (long long)d, group_size);
  if (rows == 0) return SGLB200_OK;
  SGLB_REQUIRE(input && output_q && output_s, "silu_mul_quant: null pointer");
  SGLB_REQUIRE(aligned16(input) && (reinterpret_cast<uintptr_t>(output_q) & 7u) == 0,
               "silu_mul_quant: input must be 16-byte and output_q 8-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case 0:
      return launch_silu_mul_quant<__nv_bfloat16>(input, output_q, output_s, rows, d, group_size, eps, num_rows_dev,
                                                  st);
    case 1:
      return launch_silu_mul_quant<__half>(input, output_q, output_s, rows, d, group_size, eps, num_rows_dev, st);
    default:
      return fail(SGLB200_E_UNSUPPORTED, "silu_mul_quant: dtype code %d (0 bf16, 1 fp16)", dtype);
  }
}

extern "C" void sglb200_stream_set_wait_probes(uint32_t probes) {
  g_stream_wait_probes = probes == 0 ? ptx::kProbeLimit : probes;
}

extern "C" int sglb200_stream_status_clear(void) {
  const int zero = 0;
  SGLB_CUDA(cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int)));
  return SGLB200_OK;
}

extern "C" int sglb200_stream_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_stream_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}
