// Shared host/device helpers for the sm_100a block-FP8 kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/sglang_b200.h"

namespace sglb200 {

// Records the message returned by sglb200_last_error() and yields `code`.
int fail(int code, const char* fmt, ...);

#define SGLB_REQUIRE(cond, ...)                                   \
  do {                                                            \
    if (!(cond)) return ::sglb200::fail(SGLB200_E_INVALID, __VA_ARGS__); \
  } while (0)

#define SGLB_CUDA(expr)                                                                              \
  do {                                                                                               \
    cudaError_t _e = (expr);                                                                         \
    if (_e != cudaSuccess)                                                                           \
      return ::sglb200::fail(SGLB200_E_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                             __FILE__, __LINE__);                                                    \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per device).
int sm_count();

template <typename T>
struct ElemTraits;
template <>
struct ElemTraits<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct ElemTraits<__half> {
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <>
struct ElemTraits<float> {
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};

// 16-byte streaming load that does not allocate in L1 (data is touched once).
__device__ __forceinline__ uint4 ld_nc_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Two float32 -> two e4m3 codes (lo in bits 0-7, hi in bits 8-15), RNE, saturate-to-finite.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// silu(x) = x / (1 + e^-x) in float32 with the hardware exponential and reciprocal.  The result is rounded to
// bf16/fp16 by every caller, so the few-ulp float32 error of the approximations shows only at rounding ties
// (the unfused and fused activation kernels share this function and stay bit-identical to each other).
__device__ __forceinline__ float silu_f32(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// Four float32 -> four e4m3 codes packed little-endian (a in bits 0-7 ... d in bits 24-31).
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint32_t r;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}"
      : "=r"(r)
      : "f"(a), "f"(b), "f"(c), "f"(d));
  return r;
}

}  // namespace sglb200
