// Routing kernels that feed moe_align: softmax / sigmoid top-k and the grouped, biased "fused gate" of
// DeepSeek-V3.  One warp per token row; expert e lives in lane e % 32, register e / 32 (coalesced loads,
// up to 1024 experts).  Each of the k picks is a warp arg-max (value descending, index ascending on ties),
// after which the winner's register is retired.  The whole row stays in registers; nothing is written but
// the k weights and ids.
#include <cfloat>

#include "common.cuh"

namespace sglb200 {

constexpr int kGateWarps = 8;          // rows per CTA
constexpr int kGateMaxPerLane = 32;    // experts <= 1024
constexpr float kNegInf = -INFINITY;

// (value, index) arg-max over the warp: larger value wins, lower index on equal values.
__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, m);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, m);
    if (ov > v || (ov == v && oi < idx)) {
      v = ov;
      idx = oi;
    }
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}

// Picks the k best of sel[] (one value per expert, kPerLane registers per lane); reports the matching
// entries of wgt[] in pick order through lane 0.  `out_w` / `out_i` are this row's k output slots.
template <int kPerLane>
__device__ __forceinline__ float pick_topk(float (&sel)[kPerLane], const float (&wgt)[kPerLane], int lane, int k,
                                           float* out_w, int32_t* out_i) {
  float sum = 0.f;
  for (int pick = 0; pick < k; ++pick) {
    float best = kNegInf;
    int best_e = INT_MAX;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      if (sel[j] > best) {  // ascending j = ascending expert index within the lane: first hit keeps the lower index
        best = sel[j];
        best_e = j * 32 + lane;
      }
    }
    warp_argmax(best, best_e);
    if (best_e == INT_MAX) best_e = 0;  // fewer candidates than k: every remaining value is -inf
    const int owner = best_e & 31, slot = best_e >> 5;
    float w = 0.f;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      if (j == slot && lane == owner) {
        w = wgt[j];
        sel[j] = kNegInf;
      }
    }
    w = __shfl_sync(0xffffffffu, w, owner);
    if (lane == 0) {
      out_w[pick] = w;
      out_i[pick] = best_e;
    }
    sum += w;  // same order and values in every lane
  }
  return sum;
}

// mode 0: softmax(x [tanh-capped] [+ bias]) ; weight = probability
// mode 1: sigmoid(x) [+ bias] for the selection; weight = (sigmoid + bias) - bias, as the reference reports it
template <typename T, int kPerLane, int kMode>
__global__ void __launch_bounds__(kGateWarps * 32)
    topk_gate_kernel(const T* __restrict__ gating, const float* __restrict__ bias, int64_t rows, int E, int k,
                     int renormalize, float softcap, float* __restrict__ out_w, int32_t* __restrict__ out_i) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kGateWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* x = gating + row * E;
  float sel[kPerLane], wgt[kPerLane];
#pragma unroll
  for (int j = 0; j < kPerLane; ++j) {
    const int e = j * 32 + lane;
    float v = kNegInf;
    if (e < E) {
      v = ElemTraits<T>::to_f32(x[e]);
      if (kMode == 0) {
        if (softcap != 0.f) v = tanhf(v / softcap) * softcap;
        if (bias != nullptr) v += bias[e];
      } else {
        v = 1.0f / (1.0f + expf(-v));
        if (bias != nullptr) v += bias[e];
      }
    }
    sel[j] = v;
  }
  if (kMode == 0) {
    float mx = kNegInf;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) mx = fmaxf(mx, sel[j]);
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      sel[j] = (j * 32 + lane < E) ? expf(sel[j] - mx) : 0.f;
      s += sel[j];
    }
    const float inv = 1.f / warp_sum(s);
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      wgt[j] = sel[j] * inv;
      sel[j] = (j * 32 + lane < E) ? wgt[j] : kNegInf;
    }
  } else {
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      const int e = j * 32 + lane;
      wgt[j] = (bias != nullptr && e < E) ? sel[j] - bias[e] : sel[j];
    }
  }
  float* ow = out_w + row * k;
  int32_t* oi = out_i + row * k;
  const float sum = pick_topk<kPerLane>(sel, wgt, lane, k, ow, oi);
  if (renormalize) {
    __syncwarp();
    const float inv = 1.f / sum;
    for (int p = lane; p < k; p += 32) ow[p] = ow[p] * inv;
  }
}

// DeepSeek-V3 gate.  All arithmetic on the scores happens in the input type T, as in the reference:
//   s = T(sigmoid_f32(x)); b = s + bias (T); group score = sum of the group's two largest b (T);
//   keep the topk_group groups with the largest score (lower group index on ties); pick the top-k b among the
//   kept groups (lower expert index on ties); weights = s, divided by their sum, optionally times the scaling
//   factor.  Fused shared experts take ids E, E+1, .. and weight sum / factor before the normalisation.
template <typename T, int kPerLane>
__global__ void __launch_bounds__(kGateWarps * 32)
    fused_gate_kernel(const T* __restrict__ input, const T* __restrict__ bias, int64_t rows, int E, int G, int topk_group,
                      int topk, int n_shared, float factor, int scale_output, float* __restrict__ out_w,
                      int32_t* __restrict__ out_i) {
  extern __shared__ float gate_smem[];  // per warp: E biased scores
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = (int64_t)blockIdx.x * kGateWarps + warp;
  if (row >= rows) return;
  float* b_sh = gate_smem + warp * E;
  const T* x = input + row * E;
  float sel[kPerLane], wgt[kPerLane];
#pragma unroll
  for (int j = 0; j < kPerLane; ++j) {
    const int e = j * 32 + lane;
    sel[j] = kNegInf;
    wgt[j] = 0.f;
    if (e < E) {
      const float xv = ElemTraits<T>::to_f32(x[e]);
      const T s = ElemTraits<T>::from_f32(1.0f / (1.0f + expf(-xv)));
      const T b = ElemTraits<T>::from_f32(ElemTraits<T>::to_f32(s) + ElemTraits<T>::to_f32(bias[e]));
      wgt[j] = ElemTraits<T>::to_f32(s);
      sel[j] = ElemTraits<T>::to_f32(b);
      b_sh[e] = sel[j];
    }
  }
  __syncwarp();
  // group scores: lane g < G scans its group
  const int gs = E / G;
  float gscore = kNegInf;
  if (lane < G) {
    float m1 = -FLT_MAX, m2 = -FLT_MAX;
    for (int i = 0; i < gs; ++i) {
      const float v = b_sh[lane * gs + i];
      if (v > m1) {
        m2 = m1;
        m1 = v;
      } else if (v > m2) {
        m2 = v;
      }
    }
    gscore = ElemTraits<T>::to_f32(ElemTraits<T>::from_f32(m1 + m2));
  }
  // a group is kept when fewer than topk_group groups beat it (larger score, or equal score and lower index)
  int beaten_by = 0;
  for (int g = 0; g < G; ++g) {
    const float og = __shfl_sync(0xffffffffu, gscore, g);
    if (og > gscore || (og == gscore && g < lane)) ++beaten_by;
  }
  const uint32_t keep_mask = __ballot_sync(0xffffffffu, lane < G && beaten_by < topk_group);
#pragma unroll
  for (int j = 0; j < kPerLane; ++j) {
    const int e = j * 32 + lane;
    if (e < E && !((keep_mask >> (e / gs)) & 1u)) sel[j] = kNegInf;
  }
  const int k_routed = topk - n_shared;
  float* ow = out_w + row * topk;
  int32_t* oi = out_i + row * topk;
  const float sum = pick_topk<kPerLane>(sel, wgt, lane, k_routed, ow, oi);
  __syncwarp();
  if (lane == 0) {
    for (int i = 0; i < n_shared; ++i) {
      oi[k_routed + i] = E + i;
      ow[k_routed + i] = sum / factor;
    }
    for (int p = 0; p < topk; ++p) {
      float w = ow[p] / sum;
      if (scale_output) w *= factor;
      ow[p] = w;
    }
  }
}

template <typename T, int kMode>
static int launch_topk(const void* gating, const float* bias, int64_t rows, int E, int k, int renorm, float softcap,
                       float* out_w, int32_t* out_i, cudaStream_t st) {
  const unsigned grid = (unsigned)((rows + kGateWarps - 1) / kGateWarps);
  const T* g = static_cast<const T*>(gating);
#define SGLB_GATE_CASE(P)                                                                                        \
  if (E <= 32 * P) {                                                                                             \
    topk_gate_kernel<T, P, kMode><<<grid, kGateWarps * 32, 0, st>>>(g, bias, rows, E, k, renorm, softcap, out_w, out_i); \
    SGLB_CUDA(cudaGetLastError());                                                                               \
    return SGLB200_OK;                                                                                           \
  }
  SGLB_GATE_CASE(1) SGLB_GATE_CASE(2) SGLB_GATE_CASE(4) SGLB_GATE_CASE(8) SGLB_GATE_CASE(16) SGLB_GATE_CASE(32)
#undef SGLB_GATE_CASE
  return fail(SGLB200_E_UNSUPPORTED, "top-k gate: %d experts (at most %d)", E, 32 * kGateMaxPerLane);
}

template <typename T>
static int launch_fused_gate(const void* input, const void* bias, int64_t rows, int E, int G, int topk_group, int topk,
                             int n_shared, float factor, int scale_output, float* out_w, int32_t* out_i,
                             cudaStream_t st) {
  const unsigned grid = (unsigned)((rows + kGateWarps - 1) / kGateWarps);
  const size_t smem = (size_t)kGateWarps * E * sizeof(float);
  const T* x = static_cast<const T*>(input);
  const T* b = static_cast<const T*>(bias);
#define SGLB_GATE_CASE(P)                                                                                      \
  if (E <= 32 * P) {                                                                                           \
    fused_gate_kernel<T, P><<<grid, kGateWarps * 32, smem, st>>>(x, b, rows, E, G, topk_group, topk, n_shared, \
                                                                 factor, scale_output, out_w, out_i);         \
    SGLB_CUDA(cudaGetLastError());                                                                             \
    return SGLB200_OK;                                                                                         \
  }
  SGLB_GATE_CASE(1) SGLB_GATE_CASE(2) SGLB_GATE_CASE(4) SGLB_GATE_CASE(8) SGLB_GATE_CASE(16) SGLB_GATE_CASE(32)
#undef SGLB_GATE_CASE
  return fail(SGLB200_E_UNSUPPORTED, "fused gate: %d experts (at most %d)", E, 32 * kGateMaxPerLane);
}

}  // namespace sglb200

using namespace sglb200;

static int check_gate_args(const char* what, const void* gating, int dtype, int64_t rows, int E, int topk,
                           const float* out_w, const int32_t* out_i) {
  SGLB_REQUIRE(rows >= 0 && E >= 1 && topk >= 1 && topk <= E, "%s: rows=%lld experts=%d topk=%d", what, (long long)rows,
               E, topk);
  SGLB_REQUIRE(dtype >= 0 && dtype <= 2, "%s: dtype %d (0 bf16, 1 fp16, 2 fp32)", what, dtype);
  SGLB_REQUIRE(rows == 0 || (gating && out_w && out_i), "%s: null pointer", what);
  return SGLB200_OK;
}

extern "C" int sglb200_topk_softmax(const void* gating, int dtype, int64_t rows, int num_experts, int topk,
                                    int renormalize, float moe_softcapping, const float* correction_bias,
                                    float* topk_weights, int32_t* topk_ids, void* stream) {
  int rc = check_gate_args("topk_softmax", gating, dtype, rows, num_experts, topk, topk_weights, topk_ids);
  if (rc || rows == 0) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    return launch_topk<__nv_bfloat16, 0>(gating, correction_bias, rows, num_experts, topk, renormalize, moe_softcapping,
                                         topk_weights, topk_ids, st);
  if (dtype == 1)
    return launch_topk<__half, 0>(gating, correction_bias, rows, num_experts, topk, renormalize, moe_softcapping,
                                  topk_weights, topk_ids, st);
  return launch_topk<float, 0>(gating, correction_bias, rows, num_experts, topk, renormalize, moe_softcapping,
                               topk_weights, topk_ids, st);
}

extern "C" int sglb200_topk_sigmoid(const void* gating, int dtype, int64_t rows, int num_experts, int topk,
                                    int renormalize, const float* correction_bias, float* topk_weights,
                                    int32_t* topk_ids, void* stream) {
  int rc = check_gate_args("topk_sigmoid", gating, dtype, rows, num_experts, topk, topk_weights, topk_ids);
  if (rc || rows == 0) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    return launch_topk<__nv_bfloat16, 1>(gating, correction_bias, rows, num_experts, topk, renormalize, 0.f, topk_weights,
                                         topk_ids, st);
  if (dtype == 1)
    return launch_topk<__half, 1>(gating, correction_bias, rows, num_experts, topk, renormalize, 0.f, topk_weights,
                                  topk_ids, st);
  return launch_topk<float, 1>(gating, correction_bias, rows, num_experts, topk, renormalize, 0.f, topk_weights, topk_ids,
                               st);
}

extern "C" int sglb200_moe_fused_gate(const void* input, const void* bias, int dtype, int64_t rows, int num_experts,
                                      int num_expert_group, int topk_group, int topk, int num_fused_shared_experts,
                                      float routed_scaling_factor, int apply_routed_scaling_factor_on_output,
                                      float* topk_weights, int32_t* topk_ids, void* stream) {
  int rc = check_gate_args("moe_fused_gate", input, dtype, rows, num_experts, topk, topk_weights, topk_ids);
  if (rc) return rc;
  SGLB_REQUIRE(num_expert_group >= 1 && num_expert_group <= 32 && num_experts % num_expert_group == 0,
               "moe_fused_gate: %d groups for %d experts (1..32 groups of equal size)", num_expert_group, num_experts);
  SGLB_REQUIRE(topk_group >= 1 && topk_group <= num_expert_group, "moe_fused_gate: topk_group %d of %d groups",
               topk_group, num_expert_group);
  SGLB_REQUIRE(num_fused_shared_experts >= 0 && num_fused_shared_experts < topk,
               "moe_fused_gate: %d fused shared experts with topk %d", num_fused_shared_experts, topk);
  SGLB_REQUIRE(topk - num_fused_shared_experts <= topk_group * (num_experts / num_expert_group),
               "moe_fused_gate: topk %d exceeds the experts of %d kept groups", topk, topk_group);
  SGLB_REQUIRE(num_fused_shared_experts == 0 || routed_scaling_factor != 0.f,
               "moe_fused_gate: fused shared experts need a non-zero routed_scaling_factor");
  if (rows == 0) return SGLB200_OK;
  SGLB_REQUIRE(bias != nullptr, "moe_fused_gate: null bias");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    return launch_fused_gate<__nv_bfloat16>(input, bias, rows, num_experts, num_expert_group, topk_group, topk,
                                            num_fused_shared_experts, routed_scaling_factor,
                                            apply_routed_scaling_factor_on_output, topk_weights, topk_ids, st);
  if (dtype == 1)
    return launch_fused_gate<__half>(input, bias, rows, num_experts, num_expert_group, topk_group, topk,
                                     num_fused_shared_experts, routed_scaling_factor,
                                     apply_routed_scaling_factor_on_output, topk_weights, topk_ids, st);
  return launch_fused_gate<float>(input, bias, rows, num_experts, num_expert_group, topk_group, topk,
                                  num_fused_shared_experts, routed_scaling_factor, apply_routed_scaling_factor_on_output,
                                  topk_weights, topk_ids, st);
}
