/*
 * Scalar C restatement of the reference's INT8 hot-path arithmetic.
 * TEST INFRASTRUCTURE ONLY: linked by tests, the smoke check and the benchmark's
 * CPU-baseline leg; never by the product library.
 *
 * Every function follows the arithmetic of one reference kernel, element by
 * element, with explicit bf16 round-to-nearest-even conversions:
 *   oc_quantize_int8_rowwise   kernels/exact-rowwise-int8/quantizer_kernel.hip:24-106
 *   oc_epilogue                kernels/int8-epilogue/epilogue_kernel.hip:23-56
 *   oc_mod_scale_shift         kernels/mod-scale-shift/mod_kernel.hip:7-22
 *   oc_swiglu_quantize         kernels/swiglu-quant/swiglu_quant_kernel.hip:18-107
 *   oc_int8_gemm               launcher/benchmark_launcher_v14_hires_int8_candidate.py:823
 * It is an independent second statement of the same contract as ref_ops.py; the
 * CPU tests require both to agree bit for bit on the reference's torture vectors.
 *
 * Build: gcc -O2 -fno-fast-math -ffp-contract=off -fopenmp -shared -fPIC
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round-to-nearest-even fp32 -> bf16; NaN stays NaN (quiet) */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

static const float kInv127 = 0.0078740157186985015869140625f;

/* scale + scale_math from a row's absmax / nan flag (quantizer_kernel.hip:67-85) */
static inline float row_scale(float block_max, int block_nan, float *scale_math_out) {
  float scale = block_nan ? NAN : block_max * kInv127;
  if (!isnan(scale) && scale < 1.0e-30f) scale = 1.0e-30f;
  float scale_math = round_bf16(scale);
  if (scale_math == 0.0f) scale_math = round_bf16(1.1754943508222875e-38f);
  *scale_math_out = scale_math;
  return scale;
}

/* one element of pass 2 (quantizer_kernel.hip:91-104) */
static inline int8_t quant_one(float value, float scale_math) {
  float divided = round_bf16(value / scale_math);
  float rounded = nearbyintf(divided);
  if (rounded > 127.0f) rounded = 127.0f;
  else if (rounded < -128.0f) rounded = -128.0f;
  return isfinite(rounded) ? (int8_t)rounded : (int8_t)0;
}

void oc_quantize_int8_rowwise(const uint16_t *x, int8_t *q, float *scales, int64_t rows,
                              int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const uint16_t *xr = x + r * cols;
    float mx = 0.0f;
    int has_nan = 0;
    for (int64_t c = 0; c < cols; ++c) {
      float v = bf16_to_f32(xr[c]);
      if (isnan(v)) has_nan = 1;
      else mx = fmaxf(mx, fabsf(v));
    }
    float sm;
    scales[r] = row_scale(mx, has_nan, &sm);
    for (int64_t c = 0; c < cols; ++c) q[r * cols + c] = quant_one(bf16_to_f32(xr[c]), sm);
  }
}

/* bias_kind: 0 none, 1 bf16, 2 fp32 (epilogue_kernel.hip:13-17) */
void oc_epilogue(const int32_t *acc, const float *rs, const float *cs, const void *bias,
                 int bias_kind, uint16_t *out, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t c = 0; c < cols; ++c) {
      float combined = rs[r] * cs[c];
      float scaled = (float)acc[r * cols + c] * combined;
      uint16_t rounded = f32_to_bf16(scaled);
      if (bias_kind != 0) {
        uint16_t b = bias_kind == 1 ? ((const uint16_t *)bias)[c]
                                    : f32_to_bf16(((const float *)bias)[c]);
        rounded = f32_to_bf16(bf16_to_f32(rounded) + bf16_to_f32(b));
      }
      out[r * cols + c] = rounded;
    }
  }
}

void oc_mod_scale_shift(uint16_t *x, const uint16_t *scale, const uint16_t *shift, int64_t rows,
                        int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t c = 0; c < cols; ++c) {
      float factor = round_bf16(1.0f + bf16_to_f32(scale[c]));
      float product = round_bf16(bf16_to_f32(x[r * cols + c]) * factor);
      x[r * cols + c] = f32_to_bf16(product + bf16_to_f32(shift[c]));
    }
  }
}

static inline uint16_t swiglu_one(uint16_t g16, uint16_t u16) {
  float gate = bf16_to_f32(g16);
  float silu = round_bf16(gate / (1.0f + expf(-gate)));
  return f32_to_bf16(silu * bf16_to_f32(u16));
}

/* x is [rows, 2*cols]; gate = first half of each row */
void oc_swiglu_quantize(const uint16_t *x, int8_t *q, float *scales, int64_t rows, int64_t cols,
                        uint16_t *activated_out /* optional [rows, cols] */) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const uint16_t *xr = x + r * 2 * cols;
    float mx = 0.0f;
    int has_nan = 0;
    for (int64_t c = 0; c < cols; ++c) {
      uint16_t a = swiglu_one(xr[c], xr[cols + c]);
      if (activated_out) activated_out[r * cols + c] = a;
      float v = bf16_to_f32(a);
      if (isnan(v)) has_nan = 1;
      else mx = fmaxf(mx, fabsf(v));
    }
    float sm;
    scales[r] = row_scale(mx, has_nan, &sm);
    for (int64_t c = 0; c < cols; ++c)
      q[r * cols + c] = quant_one(bf16_to_f32(swiglu_one(xr[c], xr[cols + c])), sm);
  }
}

/* acc[M,N] = A[M,K] . W[N,K]^T, exact int32 */
void oc_int8_gemm(const int8_t *a, const int8_t *w, int32_t *acc, int64_t m, int64_t n, int64_t k) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      int32_t s = 0;
      const int8_t *ar = a + i * k, *wr = w + j * k;
      for (int64_t t = 0; t < k; ++t) s += (int32_t)ar[t] * (int32_t)wr[t];
      acc[i * n + j] = s;
    }
  }
}

/*
 * Exhaustive proof obligation for the CUDA quantizer: it replaces the per-element
 * fp32 division `x / scale_math` by `x * rn(1/scale_math)`.  For every bf16 x and
 * every bf16 scale_math in [lo_bits, hi_bits] (bit patterns of positive bf16
 * values), count the pairs whose final int8 differs.  Returns the mismatch count
 * and stores the first offending pair.
 */
int64_t oc_recip_mismatches(uint32_t lo_bits, uint32_t hi_bits, uint32_t *first_x,
                            uint32_t *first_s) {
  int64_t bad = 0;
  uint32_t fx = 0, fs = 0;
#pragma omp parallel for schedule(dynamic, 64) reduction(+ : bad)
  for (uint32_t sb = lo_bits; sb <= hi_bits; ++sb) {
    float sm = bf16_to_f32((uint16_t)sb);
    float r = 1.0f / sm; /* IEEE round-to-nearest reciprocal */
    for (uint32_t xb = 0; xb < 0x10000u; ++xb) {
      float x = bf16_to_f32((uint16_t)xb);
      int8_t want = quant_one(x, sm);
      float divided = round_bf16(x * r);
      float rounded = nearbyintf(divided);
      if (rounded > 127.0f) rounded = 127.0f;
      else if (rounded < -128.0f) rounded = -128.0f;
      int8_t got = isfinite(rounded) ? (int8_t)rounded : (int8_t)0;
      if (got != want) {
        ++bad;
#pragma omp critical
        {
          if (fx == 0 && fs == 0) {
            fx = xb;
            fs = sb;
          }
        }
      }
    }
  }
  if (first_x) *first_x = fx;
  if (first_s) *first_s = fs;
  return bad;
}
