// Memory-bound helpers of the MoE path for sm_100a: silu_and_mul, the top-k sum, and the row
// gather into expert-sorted order.  All use 128-bit accesses and one pass over the data.
#include "common.cuh"

namespace sglb200 {

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const T* p = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = ElemTraits<T>::to_f32(p[i]);
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 raw;
  T* p = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) p[i] = ElemTraits<T>::from_f32(v[i]);
  return raw;
}

// out[r, 8c..8c+8) = T(T(silu(x[r, 8c..])) * x[r, d + 8c..]); one thread per 8 outputs.
template <typename T>
__global__ void __launch_bounds__(256)
    silu_and_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t total_chunks, int chunks_per_row) {
  const int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (c >= total_chunks) return;
  const int64_t r = c / chunks_per_row;
  const int64_t cc = c - r * chunks_per_row;
  const T* row = x + r * (int64_t)chunks_per_row * 16;
  float g[8], u[8], h[8];
  unpack8<T>(ld_nc_16(row + cc * 8), g);
  unpack8<T>(ld_nc_16(row + (int64_t)chunks_per_row * 8 + cc * 8), u);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float act = ElemTraits<T>::to_f32(ElemTraits<T>::from_f32(silu_f32(g[i])));
    h[i] = act * u[i];
  }
  reinterpret_cast<uint4*>(out)[c] = pack8<T>(h);
}

// out[t, 8c..] = T(scale * sum_k x[t, k, 8c..]); one thread per 8 outputs, k ascending.
template <typename T>
__global__ void __launch_bounds__(256)
    moe_sum_reduce_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t total_chunks, int chunks_per_row,
                          int topk, float scale) {
  const int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (c >= total_chunks) return;
  const int64_t t = c / chunks_per_row;
  const int64_t cc = c - t * chunks_per_row;
  const T* src = x + (t * topk) * (int64_t)chunks_per_row * 8 + cc * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  int k = 0;
  for (; k + 4 <= topk; k += 4) {  // four independent loads in flight
    uint4 raw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) raw[j] = ld_nc_16(src + (int64_t)(k + j) * chunks_per_row * 8);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v[8];
      unpack8<T>(raw[j], v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i];
    }
  }
  for (; k < topk; ++k) {
    float v[8];
    unpack8<T>(ld_nc_16(src + (int64_t)k * chunks_per_row * 8), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += v[i];
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] *= scale;
  reinterpret_cast<uint4*>(out)[c] = pack8<T>(acc);
}

// The same sum over the slots whose expert id is not negative: under expert parallelism a token's slots for experts
// of other ranks are never written by the grouped GEMM and must not be read.
template <typename T>
__global__ void __launch_bounds__(256)
    moe_sum_reduce_masked_kernel(const T* __restrict__ x, const int32_t* __restrict__ ids, T* __restrict__ out,
                                 int64_t total_chunks, int chunks_per_row, int topk, float scale) {
  const int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (c >= total_chunks) return;
  const int64_t t = c / chunks_per_row;
  const int64_t cc = c - t * chunks_per_row;
  const T* src = x + (t * topk) * (int64_t)chunks_per_row * 8 + cc * 8;
  const int32_t* id = ids + t * topk;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < topk; k0 += 4) {  // up to four independent loads in flight
    uint4 raw[4];
    bool on[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      on[j] = k0 + j < topk && __ldg(id + k0 + j) >= 0;
      if (on[j]) raw[j] = ld_nc_16(src + (int64_t)(k0 + j) * chunks_per_row * 8);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (on[j]) {
        float v[8];
        unpack8<T>(raw[j], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += v[i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] *= scale;
  reinterpret_cast<uint4*>(out)[c] = pack8<T>(acc);
}

// Sorted order without its leading segment of filtered ids (bucket 0 = expert -1): everything after it moves to the
// front, so that the kernels bounded by num_tokens_post_pad never touch rows of experts that are not on this rank.
__global__ void __launch_bounds__(256)
    drop_filtered_kernel(const int32_t* __restrict__ sorted_in, const int32_t* __restrict__ eids_in,
                         const int32_t* __restrict__ cumsum, const int32_t* __restrict__ post_in,
                         int32_t* __restrict__ sorted_out, int32_t* __restrict__ eids_out, int32_t* __restrict__ post_out,
                         int block) {
  const int begin = cumsum[1];  // padded length of bucket 0, a multiple of `block`
  const int n = *post_in - begin;
  const int stride = gridDim.x * 256;
  for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += stride) sorted_out[i] = sorted_in[begin + i];
  const int nb = n / block, b0 = begin / block;
  for (int j = blockIdx.x * 256 + threadIdx.x; j < nb; j += stride) eids_out[j] = eids_in[b0 + j];
  if (blockIdx.x == 0 && threadIdx.x == 0) *post_out = n;
}

// out[t, 8c..] = T(scale * sum_j src[slot[t, j], 8c..]) over the j with 0 <= slot[t, j] < src_rows, ascending j,
// float32 accumulation; one thread per 8 outputs.
template <typename T>
__global__ void __launch_bounds__(256)
    gather_sum_rows_kernel(const T* __restrict__ src, const int64_t* __restrict__ slot, T* __restrict__ out,
                           int64_t total_chunks, int chunks_per_row, int per_token, int64_t src_rows, float scale) {
  const int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (c >= total_chunks) return;
  const int64_t t = c / chunks_per_row;
  const int64_t cc = c - t * chunks_per_row;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < per_token; ++j) {
    const int64_t r = slot[t * per_token + j];
    if (r < 0 || r >= src_rows) continue;
    float v[8];
    unpack8<T>(ld_nc_16(src + (r * chunks_per_row + cc) * 8), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += v[i];
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] *= scale;
  reinterpret_cast<uint4*>(out)[c] = pack8<T>(acc);
}

// out[t, 8c..] = T( sum_j f[t, j] * in[perm[t * topk + j], 8c..] ), float32 accumulation in ascending j; factors in
// the output type (or absent = 1).  One thread per 8 outputs.
template <typename T>
__global__ void __launch_bounds__(256)
    shuffle_mul_sum_kernel(const T* __restrict__ in, T* __restrict__ out, const int32_t* __restrict__ perm,
                           const T* __restrict__ factors, int64_t total_chunks, int chunks_per_row, int topk) {
  const int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (c >= total_chunks) return;
  const int64_t t = c / chunks_per_row;
  const int64_t cc = c - t * chunks_per_row;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < topk; ++j) {
    const int64_t r = perm[t * topk + j];
    const float f = factors != nullptr ? ElemTraits<T>::to_f32(factors[t * topk + j]) : 1.0f;
    float v[8];
    unpack8<T>(ld_nc_16(in + (r * chunks_per_row + cc) * 8), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += f * v[i];
  }
  reinterpret_cast<uint4*>(out)[c] = pack8<T>(acc);
}

// One CTA per destination row r: copies hidden bytes (16 B per thread per step) and `groups` scales.
__global__ void __launch_bounds__(256)
    gather_rows_kernel(const uint4* __restrict__ src_q, const float* __restrict__ src_s, uint4* __restrict__ dst_q,
                       float* __restrict__ dst_s, const int32_t* __restrict__ sorted_ids,
                       const int32_t* __restrict__ num_rows_dev, int64_t numel, int topk, int vecs_per_row,
                       int groups) {
  const int64_t rows = *num_rows_dev;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const int32_t id = sorted_ids[r];
    uint4* dq = dst_q + r * vecs_per_row;
    float* ds = dst_s + r * groups;
    if (id >= 0 && id < numel) {
      const int64_t t = id / topk;
      const uint4* sq = src_q + t * vecs_per_row;
      for (int i = threadIdx.x; i < vecs_per_row; i += 256) dq[i] = __ldg(sq + i);
      for (int i = threadIdx.x; i < groups; i += 256) ds[i] = __ldg(src_s + t * groups + i);
    } else {
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int i = threadIdx.x; i < vecs_per_row; i += 256) dq[i] = z;
      for (int i = threadIdx.x; i < groups; i += 256) ds[i] = 0.f;
    }
  }
}

}  // namespace sglb200

using namespace sglb200;

extern "C" int sglb200_silu_and_mul(void* out, const void* input, int dtype, int64_t rows, int64_t d, void* stream) {
  SGLB_REQUIRE(rows >= 0 && d > 0 && d % 8 == 0, "silu_and_mul: rows=%lld d=%lld (d must be a multiple of 8)",
               (long long)rows, (long long)d);
  if (rows == 0) return SGLB200_OK;
  SGLB_REQUIRE(out && input && aligned16(out) && aligned16(input), "silu_and_mul: pointers must be 16-byte aligned");
  const int64_t total = rows * (d / 8);
  const int64_t blocks = (total + 255) / 256;
  SGLB_REQUIRE(blocks < (1ll << 31), "silu_and_mul: input too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    silu_and_mul_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(input),
                                                                         static_cast<__nv_bfloat16*>(out), total,
                                                                         (int)(d / 8));
  else if (dtype == 1)
    silu_and_mul_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __half*>(input),
                                                                  static_cast<__half*>(out), total, (int)(d / 8));
  else
    return fail(SGLB200_E_UNSUPPORTED, "silu_and_mul: dtype code %d (0 bf16, 1 fp16)", dtype);
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}

extern "C" int sglb200_moe_sum_reduce(const void* x, void* out, int dtype, int64_t tokens, int64_t topk,
                                      int64_t hidden, float scale, void* stream) {
  SGLB_REQUIRE(tokens >= 0 && topk >= 1 && hidden > 0 && hidden % 8 == 0,
               "moe_sum_reduce: tokens=%lld topk=%lld hidden=%lld (hidden must be a multiple of 8)", (long long)tokens,
               (long long)topk, (long long)hidden);
  if (tokens == 0) return SGLB200_OK;
  SGLB_REQUIRE(x && out && aligned16(x) && aligned16(out), "moe_sum_reduce: pointers must be 16-byte aligned");
  const int64_t total = tokens * (hidden / 8);
  const int64_t blocks = (total + 255) / 256;
  SGLB_REQUIRE(blocks < (1ll << 31), "moe_sum_reduce: input too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    moe_sum_reduce_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), total, (int)(hidden / 8), (int)topk,
        scale);
  else if (dtype == 1)
    moe_sum_reduce_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __half*>(x),
                                                                    static_cast<__half*>(out), total,
                                                                    (int)(hidden / 8), (int)topk, scale);
  else
    return fail(SGLB200_E_UNSUPPORTED, "moe_sum_reduce: dtype code %d (0 bf16, 1 fp16)", dtype);
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}

extern "C" int sglb200_gather_sum_rows(const void* src, const int64_t* slot, void* out, int dtype, int64_t tokens,
                                       int per_token, int64_t src_rows, int64_t hidden, float scale, void* stream) {
  SGLB_REQUIRE(tokens >= 0 && per_token >= 1 && src_rows >= 0 && hidden > 0 && hidden % 8 == 0,
               "gather_sum_rows: tokens=%lld per_token=%d hidden=%lld (hidden must be a multiple of 8)",
               (long long)tokens, per_token, (long long)hidden);
  if (tokens == 0) return SGLB200_OK;
  SGLB_REQUIRE(slot && out && (src || src_rows == 0) && aligned16(src) && aligned16(out),
               "gather_sum_rows: null or misaligned pointer");
  const int64_t total = tokens * (hidden / 8);
  const int64_t blocks = (total + 255) / 256;
  SGLB_REQUIRE(blocks < (1ll << 31), "gather_sum_rows: input too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    gather_sum_rows_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(src), slot, static_cast<__nv_bfloat16*>(out), total, (int)(hidden / 8),
        per_token, src_rows, scale);
  else if (dtype == 1)
    gather_sum_rows_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __half*>(src), slot,
                                                                     static_cast<__half*>(out), total, (int)(hidden / 8),
                                                                     per_token, src_rows, scale);
  else
    return fail(SGLB200_E_UNSUPPORTED, "gather_sum_rows: dtype code %d (0 bf16, 1 fp16)", dtype);
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}

extern "C" int sglb200_shuffle_mul_sum(const void* input, void* output, const int32_t* permutation, const void* factors,
                                       int dtype, int64_t tokens, int topk, int64_t hidden, void* stream) {
  SGLB_REQUIRE(tokens >= 0 && topk >= 1 && hidden > 0 && hidden % 8 == 0,
               "shuffle_mul_sum: tokens=%lld topk=%d hidden=%lld (hidden must be a multiple of 8)", (long long)tokens,
               topk, (long long)hidden);
  if (tokens == 0) return SGLB200_OK;
  SGLB_REQUIRE(input && output && permutation && aligned16(input) && aligned16(output),
               "shuffle_mul_sum: null or misaligned pointer");
  const int64_t total = tokens * (hidden / 8);
  const int64_t blocks = (total + 255) / 256;
  SGLB_REQUIRE(blocks < (1ll << 31), "shuffle_mul_sum: input too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    shuffle_mul_sum_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(input), static_cast<__nv_bfloat16*>(output), permutation,
        static_cast<const __nv_bfloat16*>(factors), total, (int)(hidden / 8), topk);
  else if (dtype == 1)
    shuffle_mul_sum_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __half*>(input),
                                                                     static_cast<__half*>(output), permutation,
                                                                     static_cast<const __half*>(factors), total,
                                                                     (int)(hidden / 8), topk);
  else
    return fail(SGLB200_E_UNSUPPORTED, "shuffle_mul_sum: dtype code %d (0 bf16, 1 fp16)", dtype);
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}

extern "C" int sglb200_gather_rows_fp8(const void* src_q, const float* src_s, void* dst_q, float* dst_s,
                                       const int32_t* sorted_token_ids, const int32_t* num_rows_dev, int64_t max_rows,
                                       int64_t numel, int topk, int64_t hidden, int64_t groups, void* stream) {
  SGLB_REQUIRE(hidden > 0 && hidden % 16 == 0 && topk >= 1 && groups >= 0, "gather_rows: hidden=%lld topk=%d",
               (long long)hidden, topk);
  if (max_rows == 0) return SGLB200_OK;
  SGLB_REQUIRE(src_q && dst_q && sorted_token_ids && num_rows_dev && aligned16(src_q) && aligned16(dst_q),
               "gather_rows: null or misaligned pointer");
  SGLB_REQUIRE(groups == 0 || (src_s && dst_s), "gather_rows: scale pointers missing");
  const int64_t blocks = max_rows < 148 * 16 ? max_rows : 148 * 16;
  gather_rows_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src_q), src_s, static_cast<uint4*>(dst_q), dst_s, sorted_token_ids, num_rows_dev, numel,
      topk, (int)(hidden / 16), (int)groups);
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}

extern "C" int sglb200_moe_sum_reduce_masked(const void* x, const int32_t* topk_ids, void* out, int dtype, int64_t tokens,
                                             int64_t topk, int64_t hidden, float scale, void* stream) {
  SGLB_REQUIRE(tokens >= 0 && topk >= 1 && hidden > 0 && hidden % 8 == 0,
               "moe_sum_reduce_masked: tokens=%lld topk=%lld hidden=%lld (hidden must be a multiple of 8)",
               (long long)tokens, (long long)topk, (long long)hidden);
  if (tokens == 0) return SGLB200_OK;
  SGLB_REQUIRE(x && topk_ids && out && aligned16(x) && aligned16(out), "moe_sum_reduce_masked: null or misaligned pointer");
  const int64_t total = tokens * (hidden / 8);
  const int64_t blocks = (total + 255) / 256;
  SGLB_REQUIRE(blocks < (1ll << 31), "moe_sum_reduce_masked: input too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    moe_sum_reduce_masked_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), topk_ids, static_cast<__nv_bfloat16*>(out), total, (int)(hidden / 8),
        (int)topk, scale);
  else if (dtype == 1)
    moe_sum_reduce_masked_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const __half*>(x), topk_ids, static_cast<__half*>(out), total, (int)(hidden / 8), (int)topk, scale);
  else
    return fail(SGLB200_E_UNSUPPORTED, "moe_sum_reduce_masked: dtype code %d (0 bf16, 1 fp16)", dtype);
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}

extern "C" int sglb200_moe_align_drop_filtered(const int32_t* sorted_in, const int32_t* expert_ids_in,
                                               const int32_t* cumsum, const int32_t* post_in, int32_t* sorted_out,
                                               int32_t* expert_ids_out, int32_t* post_out, int64_t max_rows,
                                               int block_size, void* stream) {
  SGLB_REQUIRE(sorted_in && expert_ids_in && cumsum && post_in && sorted_out && expert_ids_out && post_out,
               "moe_align_drop_filtered: null pointer");
  SGLB_REQUIRE(sorted_in != sorted_out && expert_ids_in != expert_ids_out, "moe_align_drop_filtered: outputs must not alias inputs");
  SGLB_REQUIRE(max_rows >= 0 && max_rows < (1ll << 31) && block_size >= 1, "moe_align_drop_filtered: bad sizes");
  int64_t blocks = (max_rows + 255) / 256;
  if (blocks < 1) blocks = 1;
  const int64_t cap = (int64_t)sm_count() * 4;
  if (blocks > cap) blocks = cap;
  drop_filtered_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      sorted_in, expert_ids_in, cumsum, post_in, sorted_out, expert_ids_out, post_out, block_size);
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}
