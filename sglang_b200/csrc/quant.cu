// 1 x G activation quantizer (float8_e4m3fn codes + float32 scales) and the fused
// silu_and_mul + quantizer, for sm_100a.
//
// Both kernels are pure streaming kernels: every input byte is read once with a 128-bit
// load, the group maximum is reduced with warp shuffles, and codes leave as 64-bit stores.
// Each thread keeps UNROLL independent 16-byte loads in flight so that a full SM holds
// enough bytes in flight to cover HBM latency.
//
// Arithmetic contract (bit-exact with the reference CUDA kernel built without fast-math):
//   amax  = max(|x|, eps)            scale = amax / fp8_max      (div.rn.f32)
//   code  = cvt.rn.satfinite.e4m3( min(max(x / scale, fp8_min), fp8_max) )   (div.rn.f32)
#include "common.cuh"

namespace sglb200 {

constexpr int kQuantThreads = 256;
constexpr int kQuantUnroll = 4;

template <int TPG>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
  for (int off = TPG / 2; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);

template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 raw = ld_nc_16(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[8]) {
  uint4 raw = ld_nc_16(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  uint4 a = ld_nc_16(p), b = ld_nc_16(p + 4);
  v[0] = __uint_as_float(a.x), v[1] = __uint_as_float(a.y), v[2] = __uint_as_float(a.z), v[3] = __uint_as_float(a.w);
  v[4] = __uint_as_float(b.x), v[5] = __uint_as_float(b.y), v[6] = __uint_as_float(b.z), v[7] = __uint_as_float(b.w);
}

// Quantise 8 values held by this thread given the group scale; returns 8 packed codes.
//
// The contract is code = e4m3(min(max(RN(x / scale), qmin), qmax)) with an IEEE float32 division.  A
// div.rn.f32 costs about ten instructions per element, which makes the kernel issue-bound, so the quotient
// is formed without dividing: with r = RN(1/scale) computed once per group,
//     q0 = RN(x*r);  e = fma(-q0, scale, x) (exact residual);  q = fma(e, r, q0);  q = copysign(q, x)
// equals RN(x / scale) bit for bit whenever |q| >= 2^-20 (checked exhaustively for every bf16 / fp16 input
// pair and on ~1e8 random float32 pairs by tests/exact_div_check.c); smaller quotients may differ in float32
// but encode as the same signed zero.  copysign restores the sign of a zero numerator.  Scales outside
// [1e-30, 1e36] (an infinite group maximum, or a caller-chosen eps near zero) take the IEEE division.
// With the standard range +-448 the upper clamp is what the saturating conversion does anyway and is
// dropped; the lower clamp stays because it is also what turns a NaN quotient into -448, as in the reference.
template <bool kStdRange>
__device__ __forceinline__ uint2 quant8(const float (&v)[8], float scale, float qmin, float qmax) {
  float q[8];
  if (scale >= 1e-30f && scale <= 1e36f) {
    const float r = __frcp_rn(scale);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float q0 = __fmul_rn(v[i], r);
      const float e = __fmaf_rn(-q0, scale, v[i]);
      q[i] = copysignf(__fmaf_rn(e, r, q0), v[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = __fdiv_rn(v[i], scale);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    q[i] = fmaxf(q[i], qmin);
    if (!kStdRange) q[i] = fminf(q[i], qmax);
  }
  uint2 out;
  out.x = pack_e4m3x4(q[0], q[1], q[2], q[3]);
  out.y = pack_e4m3x4(q[4], q[5], q[6], q[7]);
  return out;
}

// One thread owns 8 consecutive elements (a "chunk"); TPG consecutive lanes own one group.
template <typename T, int TPG, bool kStdRange>
__global__ void __launch_bounds__(kQuantThreads)
    per_token_group_quant_kernel(const T* __restrict__ x, uint2* __restrict__ out_q, float* __restrict__ out_s,
                                 int64_t total_chunks, int groups_per_row, int64_t s_stride_token,
                                 int64_t s_stride_group, bool s_contiguous, float eps, float qmin, float qmax) {
  const int64_t base = (int64_t)blockIdx.x * (kQuantThreads * kQuantUnroll) + threadIdx.x;
  float v[kQuantUnroll][8];
  bool ok[kQuantUnroll];
#pragma unroll
  for (int u = 0; u < kQuantUnroll; ++u) {
    const int64_t c = base + (int64_t)u * kQuantThreads;
    ok[u] = c < total_chunks;
    if (ok[u]) {
      load8<T>(x + c * 8, v[u]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[u][i] = 0.f;
    }
  }
#pragma unroll
  for (int u = 0; u < kQuantUnroll; ++u) {
    const int64_t c = base + (int64_t)u * kQuantThreads;
    float amax = eps;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[u][i]));
    amax = group_max<TPG>(amax);
    const float scale = __fdiv_rn(amax, qmax);
    if (ok[u]) {
      out_q[c] = quant8<kStdRange>(v[u], scale, qmin, qmax);
      if ((threadIdx.x & (TPG - 1)) == 0) {
        const int64_t g = c / TPG;
        if (s_contiguous) {
          out_s[g] = scale;
        } else {
          const int64_t t = g / groups_per_row;
          const int64_t gi = g - t * groups_per_row;
          out_s[t * s_stride_token + gi * s_stride_group] = scale;
        }
      }
    }
  }
}

// Fused silu_and_mul + quantizer.  x is [rows, 2d]; chunk c of row r covers outputs [8c, 8c+8).
template <typename T, int TPG>
__global__ void __launch_bounds__(kQuantThreads)
    silu_mul_quant_kernel(const T* __restrict__ x, uint2* __restrict__ out_q, float* __restrict__ out_s, int64_t rows,
                          int chunks_per_row, const int32_t* __restrict__ num_rows_dev, float eps, float qmin,
                          float qmax) {
  if (num_rows_dev != nullptr) {
    const int64_t lim = *num_rows_dev;
    rows = lim < rows ? lim : rows;
  }
  const int64_t total_chunks = rows * chunks_per_row;
  const int64_t base = (int64_t)blockIdx.x * (kQuantThreads * 2) + threadIdx.x;
  if ((int64_t)blockIdx.x * (kQuantThreads * 2) >= total_chunks) return;  // whole block past the end
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int64_t c = base + (int64_t)u * kQuantThreads;
    const bool ok = c < total_chunks;
    float g[8], up[8], h[8];
    if (ok) {
      const int64_t r = c / chunks_per_row;
      const int64_t cc = c - r * chunks_per_row;
      const T* row = x + r * (int64_t)chunks_per_row * 16;
      load8<T>(row + cc * 8, g);
      load8<T>(row + (int64_t)chunks_per_row * 8 + cc * 8, up);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) g[i] = 0.f, up[i] = 0.f;
    }
    float amax = eps;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // silu in float32, rounded to T, times `up` rounded to T: the reference's two rounding points
      const float act = ElemTraits<T>::to_f32(ElemTraits<T>::from_f32(silu_f32(g[i])));
      h[i] = ElemTraits<T>::to_f32(ElemTraits<T>::from_f32(act * up[i]));
      amax = fmaxf(amax, fabsf(h[i]));
    }
    amax = group_max<TPG>(amax);
    const float scale = __fdiv_rn(amax, qmax);
    if (ok) {
      out_q[c] = quant8<true>(h, scale, qmin, qmax);
      if ((threadIdx.x & (TPG - 1)) == 0) out_s[c / TPG] = scale;
    }
  }
}

template <typename T>
static int launch_quant(const void* input, void* output_q, float* output_s, int64_t num_tokens, int64_t hidden,
                        int group_size, float eps, float qmin, float qmax, int64_t s_stride_token,
                        int64_t s_stride_group, cudaStream_t stream) {
  const int64_t total_chunks = num_tokens * hidden / 8;
  const int groups_per_row = (int)(hidden / group_size);
  const bool contiguous = (s_stride_group == 1 && s_stride_token == groups_per_row);
  const int64_t per_block = (int64_t)kQuantThreads * kQuantUnroll;
  const int64_t blocks = (total_chunks + per_block - 1) / per_block;
  if (blocks == 0) return SGLB200_OK;
  SGLB_REQUIRE(blocks < (1ll << 31), "quantizer: input too large (%lld chunks)", (long long)total_chunks);
  const bool std_range = (qmin == -448.0f && qmax == 448.0f);
#define SGLB_LAUNCH_Q2(TPG, STD)                                                                                 \
  per_token_group_quant_kernel<T, TPG, STD><<<(unsigned)blocks, kQuantThreads, 0, stream>>>(                     \
      static_cast<const T*>(input), static_cast<uint2*>(output_q), output_s, total_chunks, groups_per_row,       \
      s_stride_token, s_stride_group, contiguous, eps, qmin, qmax)
#define SGLB_LAUNCH_Q(TPG)         \
  do {                             \
    if (std_range)                 \
      SGLB_LAUNCH_Q2(TPG, true);   \
    else                           \
      SGLB_LAUNCH_Q2(TPG, false);  \
  } while (0)
  switch (group_size) {
    case 32: SGLB_LAUNCH_Q(4); break;
    case 64: SGLB_LAUNCH_Q(8); break;
    case 128: SGLB_LAUNCH_Q(16); break;
    case 256: SGLB_LAUNCH_Q(32); break;
    default: return fail(SGLB200_E_INVALID, "quantizer: group_size %d not in {32,64,128,256}", group_size);
  }
#undef SGLB_LAUNCH_Q
#undef SGLB_LAUNCH_Q2
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}

template <typename T>
static int launch_silu_mul_quant(const void* input, void* output_q, float* output_s, int64_t rows, int64_t d,
                                 int group_size, float eps, const int32_t* num_rows_dev, cudaStream_t stream) {
  const int chunks_per_row = (int)(d / 8);
  const int64_t total_chunks = rows * chunks_per_row;
  const int64_t per_block = (int64_t)kQuantThreads * 2;
  const int64_t blocks = (total_chunks + per_block - 1) / per_block;
  if (blocks == 0) return SGLB200_OK;
  SGLB_REQUIRE(blocks < (1ll << 31), "silu_mul_quant: input too large");
#define SGLB_LAUNCH_SQ(TPG)                                                                           \
  silu_mul_quant_kernel<T, TPG><<<(unsigned)blocks, kQuantThreads, 0, stream>>>(                      \
      static_cast<const T*>(input), static_cast<uint2*>(output_q), output_s, rows, chunks_per_row,    \
      num_rows_dev, eps, -448.0f, 448.0f)
  switch (group_size) {
    case 32: SGLB_LAUNCH_SQ(4); break;
    case 64: SGLB_LAUNCH_SQ(8); break;
    case 128: SGLB_LAUNCH_SQ(16); break;
    case 256: SGLB_LAUNCH_SQ(32); break;
    default: return fail(SGLB200_E_INVALID, "silu_mul_quant: group_size %d not in {32,64,128,256}", group_size);
  }
#undef SGLB_LAUNCH_SQ
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}

}  // namespace sglb200

using namespace sglb200;

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
