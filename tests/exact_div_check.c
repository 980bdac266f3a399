/* Checks, on the CPU, the division-free quotient the quantizer kernel uses:
 *     r = RN(1/s);  q0 = RN(x*r);  e = fma(-q0, s, x);  q = fma(e, r, q0);  q = copysign(q, x)
 * against the IEEE quotient RN(x/s) it must reproduce, for s = RN(amax/448):
 *   mode 0: every bf16 amax > 0 and every bf16 x with |x| <= amax   (exhaustive)
 *   mode 1: every fp16 amax > 0 and every fp16 x with |x| <= amax   (exhaustive)
 *   mode 2: random float32 pairs
 * Prints the number of pairs whose float32 quotients differ with magnitude >= 2^-20 or whose signs differ
 * (expected 0; below 2^-20 every value encodes as a signed zero).  Build: gcc -O2 -mfma -fopenmp
 * -ffp-contract=off.  fmaf() is a single fused operation with -mfma. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float f16_to_f32(uint16_t h) {
  uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 0x1f, m = h & 0x3ff;
  if (e == 0) { float f = (float)m * 5.9604644775390625e-08f; return s ? -f : f; }
  return bits_f32(s | ((e + 112) << 23) | (m << 13));
}

static inline int differs(float x, float s) {
  const float ref = x / s;
  const float r = 1.0f / s;
  const float q0 = x * r;
  const float e = fmaf(-q0, s, x);
  float q = fmaf(e, r, q0);
  q = copysignf(q, x);
  if (f32_bits(q) == f32_bits(ref)) return 0;
  /* Quotients far below half of the smallest e4m3 subnormal (2^-10) all encode as +-0: there the two may
   * differ in float32 (the residual underflows) without any effect on the code, as long as the sign agrees. */
  if (fabsf(ref) < 0x1p-20f && fabsf(q) < 0x1p-20f && signbit(q) == signbit(ref)) return 0;
  return 1;
}

int main(int argc, char** argv) {
  int mode = argc > 1 ? atoi(argv[1]) : 0;
  long long bad = 0, total = 0;
  if (mode == 0 || mode == 1) {
    int n_amax = mode == 0 ? 0x7f80 : 0x7c00; /* positive finite patterns */
#pragma omp parallel for schedule(dynamic, 64) reduction(+ : bad, total)
    for (int a = 1; a < n_amax; ++a) {
      float amax = mode == 0 ? bits_f32((uint32_t)a << 16) : f16_to_f32((uint16_t)a);
      if (amax < 1e-10f) amax = 1e-10f;
      float s = amax / 448.0f;
      if (!(s >= 1e-30f && s <= 1e36f)) continue; /* the kernel takes its IEEE-division path here */
      for (int b = 0; b <= a; ++b) {
        float x = mode == 0 ? bits_f32((uint32_t)b << 16) : f16_to_f32((uint16_t)b);
        bad += differs(x, s) + differs(-x, s);
        total += 2;
      }
    }
  } else {
    uint64_t st = 88172645463325252ull;
    for (long long i = 0; i < 150000000ll; ++i) {
      st ^= st << 13; st ^= st >> 7; st ^= st << 17;
      float amax = bits_f32((uint32_t)(st >> 33) & 0x7fffffffu);
      if (!(amax < INFINITY) || amax < 1e-10f) continue;
      float s = amax / 448.0f;
      if (!(s >= 1e-30f && s <= 1e36f)) continue;
      uint32_t xb = (uint32_t)st;
      float x = bits_f32(xb);
      if (!(fabsf(x) <= amax)) { x = bits_f32((xb & 0x807fffffu) | (f32_bits(amax) & 0x7f800000u)); if (!(fabsf(x) <= amax)) x *= 0.5f; }
      bad += differs(x, s);
      total += 1;
    }
  }
  printf("%lld %lld\n", bad, total);
  return 0;
}
