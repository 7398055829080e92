/* Plain-C restatement of the quantised linear-layer math (TEST INFRASTRUCTURE
 * ONLY: second oracle and timed CPU baseline; the CUDA library never links or
 * calls this file).
 *
 * PARITY UNPINNED: the reference project has no AQ4 / FP8 numeric code to
 * follow.  The reference facts that constrain this file are the storage rules
 * of its packed 4-bit descriptor (crates/ullm-core/src/dtype.rs:56-122: two
 * values per U8 byte, ceil(n/2) bytes, one scale per block of consecutive
 * elements) and its e4m3fn dtype tag (crates/ullm-core/src/dtype.rs:6-16).
 * The format itself is the one written in oracle.py's header; this file is an
 * independent implementation of the same rules (bit manipulation here, value
 * grid arithmetic there) so that the two can check each other.
 *
 * Accumulation here is fp32 (the NumPy oracle uses fp64).
 * Build: see the Makefile beside this file (-ffp-contract=off, OpenMP).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- scalar conversions ------------------------------------------------ */

static inline float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)(((u >> 16) & 0x8000u) | 0x7fc0u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* fp32 -> fp16 bits, round to nearest even, written out by hand so that the
 * result does not depend on compiler _Float16 support. */
static uint16_t f32_to_f16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
  if (a >= 0x477ff000u) { /* >= 65520 rounds to infinity */
    return (uint16_t)(sign | 0x7c00u);
  }
  if (a < 0x38800000u) { /* below 2^-14: subnormal half, unit 2^-24 */
    float af;
    memcpy(&af, &a, 4);
    float k = rintf(af * 16777216.0f); /* exact scaling; rintf = ties-to-even */
    return (uint16_t)(sign | (uint16_t)k);
  }
  uint32_t e = (a >> 23) - 127 + 15;
  uint32_t m = a & 0x7fffffu;
  uint32_t keep = m >> 13, rem = m & 0x1fffu;
  uint32_t h = (e << 10) | keep;
  if (rem > 0x1000u || (rem == 0x1000u && (keep & 1u))) h += 1; /* carries into the exponent */
  return (uint16_t)(sign | h);
}

static float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
  float f;
  if (e == 0) {
    f = (float)m * 5.9604644775390625e-08f; /* 2^-24 */
    uint32_t u;
    memcpy(&u, &f, 4);
    u |= sign;
    memcpy(&f, &u, 4);
    return f;
  }
  uint32_t u = sign | ((e == 31 ? 255u : e - 15 + 127) << 23) | (m << 13);
  memcpy(&f, &u, 4);
  return f;
}

static uint8_t f32_to_e4m3(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return 0x7f;
  float af;
  memcpy(&af, &a, 4);
  if (af >= 448.0f) return (uint8_t)(sign | 0x7e);
  if (af < 0.015625f) { /* below 2^-6: unit 2^-9; k == 8 is the first normal code */
    return (uint8_t)(sign | (uint8_t)rintf(af * 512.0f));
  }
  int e = (int)(a >> 23) - 127;
  uint32_t m = a & 0x7fffffu;
  uint32_t keep = m >> 20, rem = m & 0xfffffu;
  uint32_t code = ((uint32_t)(e + 7) << 3) | keep;
  if (rem > 0x80000u || (rem == 0x80000u && (keep & 1u))) code += 1;
  if (code > 0x7eu) code = 0x7eu;
  return (uint8_t)(sign | code);
}

static float e4m3_to_f32(uint8_t c) {
  int e = (c >> 3) & 0xf, m = c & 7;
  float v;
  if (e == 0xf && m == 7) return NAN;
  if (e == 0)
    v = (float)m * 0.001953125f; /* m * 2^-9 */
  else
    v = ldexpf(1.0f + (float)m * 0.125f, e - 7);
  return (c & 0x80) ? -v : v;
}

/* ---- counter-based generator ------------------------------------------- */

static inline uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

uint64_t orc_stream_key(uint64_t seed, uint64_t tensor_id) { return splitmix64(splitmix64(seed) ^ tensor_id); }

static inline float synth_one(uint64_t key, uint64_t i) {
  int64_t s = 0;
  for (int j = 0; j < 3; ++j) {
    uint64_t h = splitmix64(key + 3ull * i + (uint64_t)j);
    s += (int64_t)(h & 0xffff) + (int64_t)((h >> 16) & 0xffff) + (int64_t)((h >> 32) & 0xffff) + (int64_t)(h >> 48);
  }
  return (float)(2 * s - 12 * 65535) * 7.62939453125e-06f; /* 2^-17 */
}

void orc_synth_normal(uint64_t seed, uint64_t tensor_id, uint64_t start, uint64_t count, float *out) {
  uint64_t key = orc_stream_key(seed, tensor_id);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)count; ++i) out[i] = synth_one(key, start + (uint64_t)i);
}

void orc_synth_weights(uint64_t seed, uint64_t tensor_id, uint64_t start, uint64_t count, float std, float *out) {
  uint64_t key = orc_stream_key(seed, tensor_id);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)count; ++i) out[i] = synth_one(key, start + (uint64_t)i) * std;
}

void orc_synth_activations_bf16(uint64_t seed, uint64_t tensor_id, uint64_t start, uint64_t count, uint16_t *out) {
  uint64_t key = orc_stream_key(seed, tensor_id);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)count; ++i) out[i] = f32_to_bf16(synth_one(key, start + (uint64_t)i));
}

/* ---- AQ4 ---------------------------------------------------------------- */

/* returns 0, or 1 for a bad shape, 2 for a non-finite weight */
int orc_aq4_quantize(const float *w, int64_t n, int64_t k, int64_t group, uint8_t *packed, uint16_t *scales) {
  if (group <= 0 || (group & 1) || k % group) return 1;
  int bad = 0;
  int64_t groups = k / group;
#pragma omp parallel for schedule(static) reduction(| : bad)
  for (int64_t r = 0; r < n; ++r) {
    for (int64_t g = 0; g < groups; ++g) {
      const float *src = w + r * k + g * group;
      float amax = 0.0f;
      for (int64_t i = 0; i < group; ++i) {
        float a = fabsf(src[i]);
        if (!(a <= 3.402823466e38f)) bad = 2;
        if (a > amax) amax = a;
      }
      float s = amax / 7.0f;
      if (s > 65504.0f) s = 65504.0f;
      uint16_t hs = f32_to_f16(s);
      scales[r * groups + g] = hs;
      float sf = f16_to_f32(hs);
      uint8_t *dst = packed + r * (k / 2) + g * (group / 2);
      for (int64_t i = 0; i < group; i += 2) {
        int q0 = 0, q1 = 0;
        if (sf != 0.0f) {
          float a0 = rintf(src[i] / sf), a1 = rintf(src[i + 1] / sf);
          a0 = a0 < -7.0f ? -7.0f : (a0 > 7.0f ? 7.0f : a0);
          a1 = a1 < -7.0f ? -7.0f : (a1 > 7.0f ? 7.0f : a1);
          q0 = (int)a0;
          q1 = (int)a1;
        }
        dst[i / 2] = (uint8_t)((q0 + 8) | ((q1 + 8) << 4));
      }
    }
  }
  return bad;
}

void orc_aq4_unpack(const uint8_t *packed, int64_t n, int64_t k, int8_t *q) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n * (k / 2); ++i) {
    q[2 * i] = (int8_t)((int)(packed[i] & 0xf) - 8);
    q[2 * i + 1] = (int8_t)((int)(packed[i] >> 4) - 8);
  }
}

void orc_aq4_dequantize(const uint8_t *packed, const uint16_t *scales, int64_t n, int64_t k, int64_t group,
                        float *out) {
  int64_t groups = k / group;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r)
    for (int64_t g = 0; g < groups; ++g) {
      float sf = f16_to_f32(scales[r * groups + g]);
      const uint8_t *src = packed + r * (k / 2) + g * (group / 2);
      float *dst = out + r * k + g * group;
      for (int64_t i = 0; i < group / 2; ++i) {
        dst[2 * i] = (float)((int)(src[i] & 0xf) - 8) * sf;
        dst[2 * i + 1] = (float)((int)(src[i] >> 4) - 8) * sf;
      }
    }
}

/* ---- FP8 ---------------------------------------------------------------- */

int orc_fp8_quantize(const float *w, int64_t n, int64_t k, uint8_t *codes, float *scale) {
  int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
  for (int64_t r = 0; r < n; ++r) {
    const float *src = w + r * k;
    float amax = 0.0f;
    for (int64_t i = 0; i < k; ++i) {
      float a = fabsf(src[i]);
      if (!(a <= 3.402823466e38f)) bad = 2;
      if (a > amax) amax = a;
    }
    float s = amax / 448.0f;
    scale[r] = s;
    for (int64_t i = 0; i < k; ++i) {
      float v = 0.0f;
      if (s != 0.0f) {
        v = src[i] / s;
        v = v < -448.0f ? -448.0f : (v > 448.0f ? 448.0f : v);
      }
      codes[r * k + i] = f32_to_e4m3(v);
    }
  }
  return bad;
}

void orc_fp8_dequantize(const uint8_t *codes, const float *scale, int64_t n, int64_t k, float *out) {
  float tab[256];
  for (int c = 0; c < 256; ++c) tab[c] = e4m3_to_f32((uint8_t)c);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r)
    for (int64_t i = 0; i < k; ++i) out[r * k + i] = tab[codes[r * k + i]] * scale[r];
}

/* ---- linears (fp32 accumulate; y as fp32 and/or bf16) ------------------- */

static void dot_rows(const float *wrow, const uint16_t *x, int64_t m, int64_t k, float *xf_scratch, float *acc) {
  (void)xf_scratch;
  for (int64_t r = 0; r < m; ++r) {
    const uint16_t *xr = x + r * k;
    float s = 0.0f;
#pragma omp simd reduction(+ : s)
    for (int64_t i = 0; i < k; ++i) s += bf16_to_f32(xr[i]) * wrow[i];
    acc[r] = s;
  }
}

/* y[m][n] = sum_k x[m][k] * w'[n][k]; either output pointer may be NULL */
void orc_linear_aq4(const uint16_t *x, int64_t m, const uint8_t *packed, const uint16_t *scales, int64_t n,
                    int64_t k, int64_t group, float *y_f32, uint16_t *y_bf16) {
  int64_t groups = k / group;
#pragma omp parallel
  {
    float *wrow = (float *)malloc((size_t)k * sizeof(float));
    float *acc = (float *)malloc((size_t)(m > 0 ? m : 1) * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
      for (int64_t g = 0; g < groups; ++g) {
        float sf = f16_to_f32(scales[r * groups + g]);
        const uint8_t *src = packed + r * (k / 2) + g * (group / 2);
        float *dst = wrow + g * group;
        for (int64_t i = 0; i < group / 2; ++i) {
          dst[2 * i] = (float)((int)(src[i] & 0xf) - 8) * sf;
          dst[2 * i + 1] = (float)((int)(src[i] >> 4) - 8) * sf;
        }
      }
      dot_rows(wrow, x, m, k, NULL, acc);
      for (int64_t j = 0; j < m; ++j) {
        if (y_f32) y_f32[j * n + r] = acc[j];
        if (y_bf16) y_bf16[j * n + r] = f32_to_bf16(acc[j]);
      }
    }
    free(wrow);
    free(acc);
  }
}

void orc_linear_fp8(const uint16_t *x, int64_t m, const uint8_t *codes, const float *scale, int64_t n, int64_t k,
                    float *y_f32, uint16_t *y_bf16) {
  float tab[256];
  for (int c = 0; c < 256; ++c) tab[c] = e4m3_to_f32((uint8_t)c);
#pragma omp parallel
  {
    float *wrow = (float *)malloc((size_t)k * sizeof(float));
    float *acc = (float *)malloc((size_t)(m > 0 ? m : 1) * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
      for (int64_t i = 0; i < k; ++i) wrow[i] = tab[codes[r * k + i]] * scale[r];
      dot_rows(wrow, x, m, k, NULL, acc);
      for (int64_t j = 0; j < m; ++j) {
        if (y_f32) y_f32[j * n + r] = acc[j];
        if (y_bf16) y_bf16[j * n + r] = f32_to_bf16(acc[j]);
      }
    }
    free(wrow);
    free(acc);
  }
}

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void orc_set_num_threads(int t) {
#ifdef _OPENMP
  if (t > 0) omp_set_num_threads(t);
#else
  (void)t;
#endif
}
