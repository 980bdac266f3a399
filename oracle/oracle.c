/* Plain-C restatement of the integer / byte-exact parts of the block-FP8 path
 * (TEST INFRASTRUCTURE ONLY: linked by the tests, the smoke check and the CPU
 * baseline leg of the benchmark; never by the product library).
 *
 * It mirrors oracle/block_fp8_oracle.py function by function so that large
 * parity cases finish in seconds; tests/test_oracle_c.py checks the two against
 * each other.  Reference citations (paths relative to the reference root):
 *   quantizer      sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:44-113
 *   moe_align      sgl-kernel/csrc/moe/moe_align_kernel.cu:28-41,56-228 with the
 *                  stable order of sgl-kernel/csrc/cpu/moe.cpp:134-189
 *   block GEMM     python/sglang/test/test_block_fp8.py:273-325
 * Compile with -ffp-contract=off: every float operation below is a single
 * IEEE-754 binary32 operation, as in the CUDA kernel built without fast-math.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static inline float f16_to_f32(uint16_t h) {
  uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 0x1f, m = h & 0x3ff, u;
  if (e == 0) {
    if (m == 0) {
      u = s;
    } else {
      float f = (float)m * 5.9604644775390625e-08f; /* m * 2^-24, exact */
      memcpy(&u, &f, 4);
      u |= s;
    }
  } else if (e == 31) {
    u = s | 0x7f800000u | (m << 13);
  } else {
    u = s | ((e + 112) << 23) | (m << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* float32 -> float8_e4m3fn, round-to-nearest-even, saturate-to-finite
 * (the conversion `__nv_fp8_e4m3(float)` performs). */
static inline uint8_t f32_to_e4m3(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint8_t sign = (uint8_t)((u >> 24) & 0x80);
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return 0x7f;            /* NaN */
  if (a >= 0x43e00000u) return sign | 0x7e;    /* |x| >= 448 -> 448 */
  if (a < 0x3c800000u) {                       /* |x| < 2^-6: subnormal codes, step 2^-9 */
    float af;
    memcpy(&af, &a, 4);
    float r = nearbyintf(af * 512.0f);         /* exact scaling; ties-to-even in default mode */
    return sign | (uint8_t)r;                  /* r in 0..8; 8 == 0x08 == 2^-6 */
  }
  /* normal: keep 3 mantissa bits, RNE on the 20 dropped bits */
  uint32_t r = a + 0x7ffffu + ((a >> 20) & 1u);
  uint32_t e = (r >> 23) - 120;                /* rebias 127 -> 7 */
  uint32_t m = (r >> 20) & 7u;
  uint32_t code = (e << 3) | m;
  if (code > 0x7e) code = 0x7e;
  return sign | (uint8_t)code;
}

static const float E4M3_MAX = 448.0f;

static float e4m3_table[256];
static int e4m3_table_ready = 0;
static void build_table(void) {
  for (int c = 0; c < 256; ++c) {
    int e = (c >> 3) & 0xf, m = c & 7;
    float v = e == 0 ? ldexpf((float)m / 8.0f, -6) : ldexpf(1.0f + (float)m / 8.0f, e - 7);
    if ((c & 0x7f) == 0x7f) v = NAN;
    e4m3_table[c] = (c & 0x80) ? -v : v;
  }
  e4m3_table_ready = 1;
}

void oracle_e4m3_encode(const float* x, int64_t n, uint8_t* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = f32_to_e4m3(x[i]);
}

/* dtype: 0 = bf16 bits, 1 = fp16 bits, 2 = float32 */
void oracle_quant(const void* x, int dtype, int64_t num_groups, int group_size, float eps, uint8_t* q, float* s) {
#pragma omp parallel for schedule(static)
  for (int64_t g = 0; g < num_groups; ++g) {
    float amax = eps;
    float buf[1024];
    for (int i = 0; i < group_size; ++i) {
      int64_t idx = g * group_size + i;
      float v = dtype == 0 ? bf16_to_f32(((const uint16_t*)x)[idx])
                : dtype == 1 ? f16_to_f32(((const uint16_t*)x)[idx])
                             : ((const float*)x)[idx];
      buf[i] = v;
      amax = fmaxf(amax, fabsf(v));
    }
    float ys = amax / E4M3_MAX;
    s[g] = ys;
    for (int i = 0; i < group_size; ++i) {
      float qv = fminf(fmaxf(buf[i] / ys, -E4M3_MAX), E4M3_MAX);
      q[g * group_size + i] = f32_to_e4m3(qv);
    }
  }
}

/* topk_ids in [-1, num_experts); outputs sized as in the reference wrapper.
 * Entries beyond *post_pad are left untouched. */
void oracle_moe_align(const int32_t* ids, int64_t numel, int num_experts, int block, int32_t* sorted_ids,
                      int32_t* expert_ids, int32_t* post_pad) {
  int buckets = num_experts + 1;
  int64_t* cnt = (int64_t*)calloc((size_t)buckets + 1, sizeof(int64_t));
  int64_t* cum = (int64_t*)calloc((size_t)buckets + 1, sizeof(int64_t));
  for (int64_t i = 0; i < numel; ++i) cnt[ids[i] + 1]++;
  for (int e = 0; e < buckets; ++e) {
    cum[e + 1] = cum[e] + (cnt[e] + block - 1) / block * block;
    for (int64_t k = cum[e]; k < cum[e + 1]; k += block) expert_ids[k / block] = e - 1;
  }
  int64_t total = cum[buckets];
  for (int64_t i = 0; i < total; ++i) sorted_ids[i] = (int32_t)numel;
  memset(cnt, 0, sizeof(int64_t) * (size_t)buckets);
  for (int64_t i = 0; i < numel; ++i) {
    int b = ids[i] + 1;
    sorted_ids[cum[b] + cnt[b]++] = (int32_t)i;
  }
  *post_pad = (int32_t)total;
  free(cnt);
  free(cum);
}

/* C[m,n] = bf16( sum_kb (a_s[m,kb]*b_s[n/bn,kb]) * sum_{k in kb} A[m,k]*B[n,k] ), float32 throughout. */
void oracle_block_gemm(const uint8_t* a, const float* a_s, const uint8_t* b, const float* b_s, int64_t M, int64_t N,
                       int64_t K, int bn, int bk, uint16_t* c_bf16, float* c_f32) {
  if (!e4m3_table_ready) build_table();
  int64_t kt = (K + bk - 1) / bk;
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t n = 0; n < N; ++n) {
      float acc = 0.f;
      for (int64_t t = 0; t < kt; ++t) {
        int64_t k1 = (t + 1) * bk < K ? (t + 1) * bk : K;
        float part = 0.f;
        for (int64_t k = t * bk; k < k1; ++k) part += e4m3_table[a[m * K + k]] * e4m3_table[b[n * K + k]];
        acc += part * (a_s[m * kt + t] * b_s[(n / bn) * kt + t]);
      }
      if (c_bf16) c_bf16[m * N + n] = f32_to_bf16(acc);
      if (c_f32) c_f32[m * N + n] = acc;
    }
  }
}

/* h = bf16( bf16(silu(gate)) * up ); x is [rows, 2d] bf16 bits (activation.cu:55-60). */
void oracle_silu_and_mul(const uint16_t* x, int64_t rows, int64_t d, uint16_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t i = 0; i < d; ++i) {
      float g = bf16_to_f32(x[r * 2 * d + i]);
      float u = bf16_to_f32(x[r * 2 * d + d + i]);
      float act = bf16_to_f32(f32_to_bf16(g / (1.0f + expf(-g))));
      out[r * d + i] = f32_to_bf16(act * u);
    }
  }
}

/* out[t,:] = bf16(scale * sum_k x[t,k,:]) (moe_sum_reduce.cu:82-103) */
void oracle_moe_sum_reduce(const uint16_t* x, int64_t T, int64_t topk, int64_t H, float scale, uint16_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < T; ++t) {
    for (int64_t h = 0; h < H; ++h) {
      float acc = 0.f;
      for (int64_t k = 0; k < topk; ++k) acc += bf16_to_f32(x[(t * topk + k) * H + h]);
      out[t * H + h] = f32_to_bf16(acc * scale);
    }
  }
}
