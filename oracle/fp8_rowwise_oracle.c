/*
 * Plain-C CPU oracle for the FP8 rowwise-scaled GEMM path.  TEST INFRASTRUCTURE ONLY: it is the
 * checker for tests/ and the timed CPU baseline of bench.py; nothing in the product links it.
 *
 * It is a second, torch-independent restatement of the same arithmetic as fp8_rowwise_oracle.py:
 *   - e4m3fn decode from the format definition (1-4-3, bias 7, no infinities, S.1111.111 = NaN);
 *   - rowwise quantiser, benchmark recipe: scale = max(rowabsmax, 1e-12) / 448 in fp32,
 *     q = e4m3_rne(clamp(x / scale, +-448))       (reference semantics: operator.py:136-145)
 *   - GEMM: y = bf16_rne( sum_k (x[m,k]*xs[m]) * (w[n,k]*ws[n]) (+ bias[n]) ), operands dequantised
 *     first, fp32 products and fp32 accumulation in ascending k (the fp32 dequantise-then-matmul
 *     form, operator.py:237-246).
 *
 * PARITY UNPINNED for the GEMM: the reference's kernels live in FBGEMM, which is not in the reference
 * tree, and the reference has no test vectors for this operator.  The quantiser and the decode table
 * are pinned against fixtures made by running the reference's own quantiser (tests/golden/).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

float oracle_e4m3_to_f32(uint8_t b) {
  const int sign = b >> 7;
  const int e = (b >> 3) & 0xF;
  const int m = b & 0x7;
  float v;
  if (e == 0xF && m == 0x7) {
    v = NAN;
  } else if (e == 0) {
    v = ldexpf((float)m / 8.0f, -6);
  } else {
    v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  }
  return sign ? -v : v;
}

/* round-to-nearest-even of a finite float already clamped to [-448, 448] */
uint8_t oracle_f32_to_e4m3(float x) {
  const uint8_t sign = signbit(x) ? 0x80 : 0x00;
  float a = fabsf(x);
  if (isnan(x)) return (uint8_t)(sign | 0x7F);
  if (a > 448.0f) a = 448.0f;
  if (a == 0.0f) return sign;
  int ex;
  (void)frexpf(a, &ex); /* a = f * 2^ex, f in [0.5, 1) -> unbiased exponent ex - 1 */
  int e = ex - 1;
  if (e < -6) e = -6; /* subnormal range shares the exponent of the smallest normal */
  /* spacing of representable values at this exponent is 2^(e-3) */
  const float step = ldexpf(1.0f, e - 3);
  float q = a / step; /* exact: power-of-two division */
  float r = rintf(q); /* default rounding mode is to nearest even */
  float v = r * step;
  if (v > 448.0f) v = 448.0f;
  /* re-derive the fields from the rounded value */
  if (v < ldexpf(1.0f, -6)) {
    const int m = (int)rintf(v / ldexpf(1.0f, -9));
    return (uint8_t)(sign | m);
  }
  (void)frexpf(v, &ex);
  e = ex - 1;
  const int m = (int)rintf((v / ldexpf(1.0f, e) - 1.0f) * 8.0f);
  return (uint8_t)(sign | ((e + 7) << 3) | m);
}

static uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
  const uint32_t lsb = (u >> 16) & 1u;
  u += 0x7FFFu + lsb;
  return (uint16_t)(u >> 16);
}

static float bf16_to_f32(uint16_t h) {
  const uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

void oracle_row_quantize_f32(const float* x, int64_t rows, int64_t cols, uint8_t* q, float* scale) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    float amax = 0.0f;
    for (int64_t c = 0; c < cols; ++c) {
      const float a = fabsf(xr[c]);
      if (a > amax) amax = a;
    }
    if (amax < 1e-12f) amax = 1e-12f;
    const float s = amax / 448.0f;
    scale[r] = s;
    for (int64_t c = 0; c < cols; ++c) {
      float v = xr[c] / s;
      if (v > 448.0f) v = 448.0f;
      if (v < -448.0f) v = -448.0f;
      q[r * cols + c] = oracle_f32_to_e4m3(v);
    }
  }
}

/* Returns 0 on success, 1 if scratch memory could not be allocated. */
int oracle_gemm_rowwise(const uint8_t* xq, const uint8_t* wq, const float* x_scale, const float* w_scale,
                        const uint16_t* bias_bf16, uint16_t* y_bf16, int64_t M, int64_t N, int64_t K) {
  float table[256];
  for (int i = 0; i < 256; ++i) table[i] = oracle_e4m3_to_f32((uint8_t)i);
  float* w = (float*)malloc((size_t)N * (size_t)K * sizeof(float));
  if (w == NULL) return 1;
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t k = 0; k < K; ++k) w[n * K + k] = table[wq[n * K + k]] * w_scale[n];

  int failed = 0;
#pragma omp parallel
  {
    float* x = (float*)malloc((size_t)K * sizeof(float));
    if (x == NULL) {
#pragma omp atomic write
      failed = 1;
    }
#pragma omp for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
      if (x == NULL) continue;
      for (int64_t k = 0; k < K; ++k) x[k] = table[xq[m * K + k]] * x_scale[m];
      for (int64_t n = 0; n < N; ++n) {
        const float* wn = w + n * K;
        float acc = 0.0f;
        for (int64_t k = 0; k < K; ++k) acc += x[k] * wn[k];
        if (bias_bf16 != NULL) acc += bf16_to_f32(bias_bf16[n]);
        y_bf16[m * N + n] = f32_to_bf16_rne(acc);
      }
    }
    free(x);
  }
  free(w);
  return failed;
}
