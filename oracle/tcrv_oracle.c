/*
 * CPU oracle (test infrastructure only; parity unpinned by reference data -- see
 * tcrv_oracle.h).  Build with `-O2 -ffp-contract=off` so every C operator below rounds
 * exactly once; the fused fold is spelled with fmaf() where it is wanted.
 */
#include "tcrv_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ fp16 */

float tcrv_oracle_fp16_to_fp32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      /* subnormal half: renormalise */
      int shift = 0;
      while ((man & 0x400u) == 0) {
        man <<= 1;
        ++shift;
      }
      man &= 0x3ffu;
      bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, sizeof f);
  return f;
}

uint16_t tcrv_oracle_fp32_to_fp16(float f) {
  uint32_t x;
  memcpy(&x, &f, sizeof x);
  uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
  uint32_t absx = x & 0x7fffffffu;
  if (absx >= 0x7f800000u) { /* inf / nan */
    if (absx > 0x7f800000u)
      return (uint16_t)(sign | 0x7e00u | ((absx >> 13) & 0x3ffu));
    return (uint16_t)(sign | 0x7c00u);
  }
  if (absx >= 0x477ff000u) /* >= 65520 rounds to inf */
    return (uint16_t)(sign | 0x7c00u);
  if (absx < 0x33000001u) /* <= 2^-25 rounds to zero (tie goes to even = 0) */
    return sign;
  int32_t e = (int32_t)(absx >> 23) - 127;
  uint32_t man = (absx & 0x7fffffu) | 0x800000u; /* 24-bit significand */
  uint32_t shift;
  uint32_t half_exp;
  if (e < -14) { /* subnormal half */
    shift = (uint32_t)(13 + (-14 - e));
    half_exp = 0;
  } else {
    shift = 13;
    half_exp = (uint32_t)(e + 15);
  }
  uint32_t kept = man >> shift;
  uint32_t rem = man & ((1u << shift) - 1u);
  uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (kept & 1u)))
    ++kept;
  uint32_t out;
  if (half_exp == 0) {
    out = kept; /* a carry into bit 10 lands on the smallest normal, as it should */
  } else {
    out = ((half_exp - 1) << 10) + kept; /* kept has the implicit bit at 0x400 */
  }
  return (uint16_t)(sign | out);
}

static inline float block_scale(const uint8_t *block) {
  uint16_t h = (uint16_t)(block[0] | ((uint16_t)block[1] << 8));
  return tcrv_oracle_fp16_to_fp32(h);
}

/* ------------------------------------------------------------ generators */

static inline uint64_t splitmix64(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

static inline double unit_open(uint64_t seed, uint64_t counter) {
  uint64_t r = splitmix64(seed * 0x2545f4914f6cdd1dull + counter);
  return ((double)(r >> 11) + 0.5) * (1.0 / 9007199254740992.0); /* (0,1) */
}

void tcrv_oracle_fill_uniform(float *out, size_t n, uint64_t seed, float lo, float hi) {
  for (size_t i = 0; i < n; ++i)
    out[i] = (float)((double)lo + ((double)hi - (double)lo) * unit_open(seed, i));
}

void tcrv_oracle_fill_normal(float *out, size_t n, uint64_t seed, float mean, float stddev) {
  for (size_t i = 0; i < n; i += 2) {
    double u1 = unit_open(seed, i);
    double u2 = unit_open(seed, i + 1);
    double r = sqrt(-2.0 * log(u1));
    double a = 6.283185307179586476925286766559 * u2;
    out[i] = (float)((double)mean + (double)stddev * r * cos(a));
    if (i + 1 < n)
      out[i + 1] = (float)((double)mean + (double)stddev * r * sin(a));
  }
}

/* ------------------------------------------------------------ elementwise */

void tcrv_oracle_add_f32(const float *lhs, const float *rhs, float *out, size_t n) {
  for (size_t i = 0; i < n; ++i)
    out[i] = lhs[i] + rhs[i];
}

void tcrv_oracle_add_i32(const int32_t *lhs, const int32_t *rhs, int32_t *out, size_t n) {
  for (size_t i = 0; i < n; ++i)
    out[i] = (int32_t)((uint32_t)lhs[i] + (uint32_t)rhs[i]); /* vadd wraps */
}

void tcrv_oracle_dequantize_i32_f32(const int32_t *lhs, float scale, float *out, size_t n) {
  for (size_t i = 0; i < n; ++i)
    out[i] = (float)lhs[i] * scale; /* vfcvt_f_x_v then vfmul_vf */
}

/* ------------------------------------------------------------- quantizers */

void tcrv_oracle_quantize_row_q8_0(const float *x, uint8_t *vy, size_t n) {
  size_t nb = n / TCRV_QK;
  for (size_t ib = 0; ib < nb; ++ib) {
    const float *xb = x + ib * TCRV_QK;
    uint8_t *yb = vy + ib * TCRV_Q8_0_BLOCK_BYTES;
    float amax = 0.0f; /* vfredmax seeded with 0.0f over vfabs */
    for (int j = 0; j < TCRV_QK; ++j) {
      float a = fabsf(xb[j]);
      if (a > amax)
        amax = a;
    }
    float d = amax / 127.0f;
    float id = 0.0f;
    if (d != 0.0f)
      id = 1.0f / d;
    uint16_t dh = tcrv_oracle_fp32_to_fp16(d);
    yb[0] = (uint8_t)(dh & 0xff);
    yb[1] = (uint8_t)(dh >> 8);
    for (int j = 0; j < TCRV_QK; ++j) {
      float x0 = xb[j] * id;
      /* vfncvt_x_f_w (f32 -> i16, round-to-nearest-even, saturating) */
      float r = nearbyintf(x0); /* default rounding mode is to-nearest-even */
      int32_t i16;
      if (r >= 32767.0f)
        i16 = 32767;
      else if (r <= -32768.0f)
        i16 = -32768;
      else if (r != r)
        i16 = 32767; /* RVV converts NaN to the maximum */
      else
        i16 = (int32_t)r;
      /* vncvt_x_x_w (i16 -> i8) keeps the low byte */
      yb[2 + j] = (uint8_t)(i16 & 0xff);
    }
  }
}

void tcrv_oracle_quantize_row_q4_0(const float *x, uint8_t *vx, size_t n) {
  size_t nb = n / TCRV_QK;
  for (size_t ib = 0; ib < nb; ++ib) {
    const float *xb = x + ib * TCRV_QK;
    uint8_t *wb = vx + ib * TCRV_Q4_0_BLOCK_BYTES;
    float amax = 0.0f, vmax = 0.0f;
    for (int j = 0; j < TCRV_QK; ++j) {
      float a = fabsf(xb[j]);
      if (a > amax) {
        amax = a;
        vmax = xb[j];
      }
    }
    float d = vmax / -8.0f;
    float id = 0.0f;
    if (d != 0.0f)
      id = 1.0f / d;
    uint16_t dh = tcrv_oracle_fp32_to_fp16(d);
    wb[0] = (uint8_t)(dh & 0xff);
    wb[1] = (uint8_t)(dh >> 8);
    for (int j = 0; j < TCRV_QK / 2; ++j) {
      float x0 = xb[j] * id;
      float x1 = xb[j + TCRV_QK / 2] * id;
      int32_t q0 = (int32_t)(int8_t)(x0 + 8.5f);
      int32_t q1 = (int32_t)(int8_t)(x1 + 8.5f);
      if (q0 > 15)
        q0 = 15;
      if (q1 > 15)
        q1 = 15;
      wb[2 + j] = (uint8_t)(q0 | (q1 << 4));
    }
  }
}

/* ------------------------------------------------------------- dequantize */

void tcrv_oracle_decode_nibbles(uint8_t byte, int8_t *lo, int8_t *hi) {
  uint8_t t = (uint8_t)(byte ^ 0x88u);
  int8_t shifted = (int8_t)(uint8_t)(t << 4);
  *lo = (int8_t)(shifted >> 4); /* arithmetic shift on a signed byte */
  *hi = (int8_t)((int8_t)t >> 4);
}

void tcrv_oracle_dequantize_row_q8_0(const uint8_t *vx, float *y, size_t n) {
  size_t nb = n / TCRV_QK;
  for (size_t ib = 0; ib < nb; ++ib) {
    const uint8_t *b = vx + ib * TCRV_Q8_0_BLOCK_BYTES;
    float d = block_scale(b);
    for (int j = 0; j < TCRV_QK; ++j)
      y[ib * TCRV_QK + j] = (float)(int32_t)(int8_t)b[2 + j] * d;
  }
}

void tcrv_oracle_dequantize_row_q4_0(const uint8_t *vx, float *y, size_t n) {
  size_t nb = n / TCRV_QK;
  for (size_t ib = 0; ib < nb; ++ib) {
    const uint8_t *b = vx + ib * TCRV_Q4_0_BLOCK_BYTES;
    float d = block_scale(b);
    for (int j = 0; j < TCRV_QK / 2; ++j) {
      int8_t lo, hi;
      tcrv_oracle_decode_nibbles(b[2 + j], &lo, &hi);
      y[ib * TCRV_QK + j] = (float)(int32_t)lo * d;
      y[ib * TCRV_QK + j + TCRV_QK / 2] = (float)(int32_t)hi * d;
    }
  }
}

/* --------------------------------------------------------------- block dots */

static inline int32_t block_sum_q4_0_q8_0(const uint8_t *xb, const uint8_t *yb) {
  int32_t sumi = 0;
  for (int j = 0; j < TCRV_QK / 2; ++j) {
    int8_t lo, hi;
    tcrv_oracle_decode_nibbles(xb[2 + j], &lo, &hi);
    sumi += (int32_t)lo * (int32_t)(int8_t)yb[2 + j];
    sumi += (int32_t)hi * (int32_t)(int8_t)yb[2 + j + TCRV_QK / 2];
  }
  return sumi;
}

static inline int32_t block_sum_q8_0_q8_0(const uint8_t *xb, const uint8_t *yb) {
  int32_t sumi = 0;
  for (int j = 0; j < TCRV_QK; ++j)
    sumi += (int32_t)(int8_t)xb[2 + j] * (int32_t)(int8_t)yb[2 + j];
  return sumi;
}

void tcrv_oracle_block_sums_q4_0_q8_0(size_t n, int32_t *sumi, const uint8_t *vx, const uint8_t *vy) {
  size_t nb = n / TCRV_QK;
  for (size_t ib = 0; ib < nb; ++ib)
    sumi[ib] = block_sum_q4_0_q8_0(vx + ib * TCRV_Q4_0_BLOCK_BYTES, vy + ib * TCRV_Q8_0_BLOCK_BYTES);
}

void tcrv_oracle_block_sums_q8_0_q8_0(size_t n, int32_t *sumi, const uint8_t *vx, const uint8_t *vy) {
  size_t nb = n / TCRV_QK;
  for (size_t ib = 0; ib < nb; ++ib)
    sumi[ib] = block_sum_q8_0_q8_0(vx + ib * TCRV_Q8_0_BLOCK_BYTES, vy + ib * TCRV_Q8_0_BLOCK_BYTES);
}

static inline float fold_q4(float sumf, int32_t sumi, float dx, float dy, int fold) {
  float t = (float)sumi * dx;
  if (fold == TCRV_FOLD_FMA)
    return fmaf(t, dy, sumf);
  float term = t * dy;
  return sumf + term;
}

static inline float fold_q8(float sumf, int32_t sumi, float dx, float dy, int fold) {
  float scale = dx * dy;
  if (fold == TCRV_FOLD_FMA)
    return fmaf((float)sumi, scale, sumf);
  float term = (float)sumi * scale;
  return sumf + term;
}

static float dot_q4_0_q8_0(size_t n, const uint8_t *vx, const uint8_t *vy, int fold) {
  size_t nb = n / TCRV_QK;
  float sumf = 0.0f;
  for (size_t ib = 0; ib < nb; ++ib) {
    const uint8_t *xb = vx + ib * TCRV_Q4_0_BLOCK_BYTES;
    const uint8_t *yb = vy + ib * TCRV_Q8_0_BLOCK_BYTES;
    sumf = fold_q4(sumf, block_sum_q4_0_q8_0(xb, yb), block_scale(xb), block_scale(yb), fold);
  }
  return sumf;
}

static float dot_q8_0_q8_0(size_t n, const uint8_t *vx, const uint8_t *vy, int fold) {
  size_t nb = n / TCRV_QK;
  float sumf = 0.0f;
  for (size_t ib = 0; ib < nb; ++ib) {
    const uint8_t *xb = vx + ib * TCRV_Q8_0_BLOCK_BYTES;
    const uint8_t *yb = vy + ib * TCRV_Q8_0_BLOCK_BYTES;
    sumf = fold_q8(sumf, block_sum_q8_0_q8_0(xb, yb), block_scale(xb), block_scale(yb), fold);
  }
  return sumf;
}

void tcrv_oracle_vec_dot_q4_0_q8_0(size_t n, float *s, size_t bs, const uint8_t *vx, size_t bx,
                                   const uint8_t *vy, size_t by, int32_t nrc, int fold) {
  (void)bs;
  (void)bx;
  (void)by;
  (void)nrc; /* only n, s, vx, vy are consumed by the reference kernel */
  *s = dot_q4_0_q8_0(n, vx, vy, fold);
}

void tcrv_oracle_vec_dot_q8_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, int fold) {
  *s = dot_q8_0_q8_0(n, vx, vy, fold);
}

/* --------------------------------------------------------------------- GEMM */

typedef struct {
  size_t n;
  float *s;
  const uint8_t *vx;
  const uint8_t *vy;
  size_t by, nr_begin, nr_end, nc, bx, bs;
  int fold;
  int q8_weights;
} gemm_job;

static void *gemm_worker(void *arg) {
  const gemm_job *j = (const gemm_job *)arg;
  for (size_t ir = j->nr_begin; ir < j->nr_end; ++ir) {
    const uint8_t *xr = j->vx + ir * j->bx;
    float *sr = j->s + ir * j->bs;
    for (size_t col = 0; col < j->nc; ++col) {
      const uint8_t *yc = j->vy + col * j->by;
      sr[col] = j->q8_weights ? dot_q8_0_q8_0(j->n, xr, yc, j->fold) : dot_q4_0_q8_0(j->n, xr, yc, j->fold);
    }
  }
  return NULL;
}

static void gemm_run(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr,
                     size_t nc, size_t bx, size_t bs, int fold, int threads, int q8_weights) {
  if (threads < 1)
    threads = 1;
  if ((size_t)threads > nr)
    threads = nr ? (int)nr : 1;
  gemm_job *jobs = (gemm_job *)malloc(sizeof(gemm_job) * (size_t)threads);
  pthread_t *tids = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
  size_t per = (nr + (size_t)threads - 1) / (size_t)threads;
  for (int t = 0; t < threads; ++t) {
    size_t b = (size_t)t * per, e = b + per;
    if (b > nr)
      b = nr;
    if (e > nr)
      e = nr;
    gemm_job j = {n, s, vx, vy, by, b, e, nc, bx, bs, fold, q8_weights};
    jobs[t] = j;
  }
  if (threads == 1) {
    gemm_worker(&jobs[0]);
  } else {
    for (int t = 0; t < threads; ++t)
      pthread_create(&tids[t], NULL, gemm_worker, &jobs[t]);
    for (int t = 0; t < threads; ++t)
      pthread_join(tids[t], NULL);
  }
  free(jobs);
  free(tids);
}

void tcrv_oracle_gemm_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                                size_t nr, size_t nc, size_t bx, size_t bs, int fold, int threads) {
  gemm_run(n, s, vx, vy, by, nr, nc, bx, bs, fold, threads, 0);
}

void tcrv_oracle_gemm_q8_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                                size_t nr, size_t nc, size_t bx, size_t bs, int fold, int threads) {
  gemm_run(n, s, vx, vy, by, nr, nc, bx, bs, fold, threads, 1);
}

/* ------------------------------------------------- CUDA GEMV order restated */

void tcrv_oracle_gemv_lane_order(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                                 size_t nr, size_t nc, size_t bx, size_t bs, int q8_weights) {
  size_t nb = n / TCRV_QK;
  size_t wstride = q8_weights ? TCRV_Q8_0_BLOCK_BYTES : TCRV_Q4_0_BLOCK_BYTES;
  for (size_t ir = 0; ir < nr; ++ir) {
    const uint8_t *xr = vx + ir * bx;
    for (size_t col = 0; col < nc; ++col) {
      const uint8_t *yc = vy + col * by;
      float lane[32];
      for (int l = 0; l < 32; ++l) {
        float acc = 0.0f;
        /* lane l owns block pairs l, l+32, ...: blocks 64i+2l and 64i+2l+1 */
        for (size_t k = 0; 2 * ((size_t)l + 32 * (k / 2)) + (k & 1) < nb; ++k) {
          size_t ib = 2 * ((size_t)l + 32 * (k / 2)) + (k & 1);
          const uint8_t *xb = xr + ib * wstride;
          const uint8_t *yb = yc + ib * TCRV_Q8_0_BLOCK_BYTES;
          if (q8_weights)
            acc = fold_q8(acc, block_sum_q8_0_q8_0(xb, yb), block_scale(xb), block_scale(yb), TCRV_FOLD_FMA);
          else
            acc = fold_q4(acc, block_sum_q4_0_q8_0(xb, yb), block_scale(xb), block_scale(yb), TCRV_FOLD_FMA);
        }
        lane[l] = acc;
      }
      for (int off = 16; off >= 1; off >>= 1) {
        float next[32];
        for (int l = 0; l < 32; ++l)
          next[l] = lane[l] + lane[l ^ off];
        memcpy(lane, next, sizeof lane);
      }
      s[ir * bs + col] = lane[0];
    }
  }
}

void tcrv_oracle_gemv_ksplit_order(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                                   size_t nr, size_t nc, size_t bx, size_t bs, int q8_weights,
                                   size_t chunk_blocks, size_t split) {
  size_t nb = n / TCRV_QK;
  size_t wstride = q8_weights ? TCRV_Q8_0_BLOCK_BYTES : TCRV_Q4_0_BLOCK_BYTES;
  size_t nchunks = (nb + chunk_blocks - 1) / chunk_blocks;
  for (size_t ir = 0; ir < nr; ++ir) {
    const uint8_t *xr = vx + ir * bx;
    for (size_t col = 0; col < nc; ++col) {
      const uint8_t *yc = vy + col * by;
      float total = 0.0f;
      for (size_t w = 0; w < split; ++w) {
        float part = 0.0f; /* warp w: chunks w, w+split, ... ascending, blocks ascending */
        for (size_t c = w; c < nchunks; c += split) {
          for (size_t ib = c * chunk_blocks; ib < (c + 1) * chunk_blocks && ib < nb; ++ib) {
            const uint8_t *xb = xr + ib * wstride;
            const uint8_t *yb = yc + ib * TCRV_Q8_0_BLOCK_BYTES;
            if (q8_weights)
              part = fold_q8(part, block_sum_q8_0_q8_0(xb, yb), block_scale(xb), block_scale(yb), TCRV_FOLD_FMA);
            else
              part = fold_q4(part, block_sum_q4_0_q8_0(xb, yb), block_scale(xb), block_scale(yb), TCRV_FOLD_FMA);
          }
        }
        total = w == 0 ? part : total + part;
      }
      s[ir * bs + col] = total;
    }
  }
}

void tcrv_oracle_gemm_abs_terms(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                                size_t nr, size_t nc, size_t bx, size_t bs, int q8_weights) {
  size_t nb = n / TCRV_QK;
  size_t wstride = q8_weights ? TCRV_Q8_0_BLOCK_BYTES : TCRV_Q4_0_BLOCK_BYTES;
  for (size_t ir = 0; ir < nr; ++ir) {
    const uint8_t *xr = vx + ir * bx;
    for (size_t col = 0; col < nc; ++col) {
      const uint8_t *yc = vy + col * by;
      double acc = 0.0;
      for (size_t ib = 0; ib < nb; ++ib) {
        const uint8_t *xb = xr + ib * wstride;
        const uint8_t *yb = yc + ib * TCRV_Q8_0_BLOCK_BYTES;
        int32_t si = q8_weights ? block_sum_q8_0_q8_0(xb, yb) : block_sum_q4_0_q8_0(xb, yb);
        acc += fabs((double)si * (double)block_scale(xb) * (double)block_scale(yb));
      }
      s[ir * bs + col] = (float)acc;
    }
  }
}

/* ---- forward-pass f32 ops --------------------------------------------------------------- */

void tcrv_oracle_vec_scale_f32(size_t n, float *y, float v) {
  for (size_t i = 0; i < n; ++i)
    y[i] = y[i] * v;
}

void tcrv_oracle_rms_norm_f32(size_t n, const float *x, float *y, float eps) {
  double sum = 0.0;
  for (size_t i = 0; i < n; ++i) {
    const float p = x[i] * x[i]; /* the f32 product rounds before it is widened */
    sum = sum + (double)p;
  }
  const float mean = (float)(sum / (double)n);
  const float scale = 1.0f / sqrtf(mean + eps);
  for (size_t i = 0; i < n; ++i)
    y[i] = x[i] * scale;
}

static float bits_to_float(uint32_t u) {
  float f;
  memcpy(&f, &u, sizeof f);
  return f;
}

static uint32_t float_to_bits(float f) {
  uint32_t u;
  memcpy(&u, &f, sizeof u);
  return u;
}

float tcrv_oracle_expf(float x) {
  const float r = 0x1.8p23f;
  const float z = fmaf(0x1.715476p+0f, x, r);
  const float n = z - r;
  const float b = fmaf(-0x1.7f7d1cp-20f, n, fmaf(-0x1.62e4p-1f, n, x));
  const uint32_t e = float_to_bits(z) << 23;
  const float k = bits_to_float(e + 0x3f800000u);
  const int c = fabsf(n) > 126.0f;
  const float u = b * b;
  const float j_outer = b * 0x1.ffffecp-1f;
  const float j_a = fmaf(0x1.555e66p-3f, b, 0x1.fffdb6p-2f);
  const float j_b = fmaf(0x1.0e4020p-7f, b, 0x1.573e2ep-5f);
  const float j_mid = fmaf(j_b, u, j_a);
  const float j = fmaf(j_mid, u, j_outer);
  const uint32_t d = (n <= 0.0f) ? 0x82000000u : 0u;
  const float s1 = bits_to_float(d + 0x7f000000u);
  const float s2 = bits_to_float(e - d);
  const float r_fast = fmaf(k, j, k);
  const float r_slow = fmaf(s2, j, s2) * s1;
  const float r1 = c ? r_slow : r_fast;
  return (fabsf(n) > 192.0f) ? s1 * s1 : r1;
}

void tcrv_oracle_vec_silu_f32(size_t n, const float *x, float *y) {
  for (size_t i = 0; i < n; ++i)
    y[i] = x[i] / (tcrv_oracle_expf(-x[i]) + 1.0f);
}

double tcrv_oracle_vec_soft_max_f32(size_t n, float *y, const float *x, float max) {
  double sum = 0.0;
  for (size_t i = 0; i < n; ++i) {
    const float v = tcrv_oracle_expf(x[i] - max);
    y[i] = v;
    sum += (double)v;
  }
  return sum;
}

void tcrv_oracle_rope_thetas(size_t n_pairs, float theta_base, float theta_scale, float *theta) {
  float t = theta_base;
  for (size_t p = 0; p < n_pairs; ++p) {
    theta[p] = t;
    t = t * theta_scale;
  }
}

void tcrv_oracle_rope_apply_f32(size_t n_dims, const float *x, float *y, const float *cache, int fold) {
  for (size_t p = 0; p < n_dims / 2; ++p) {
    const float c = cache[2 * p], s = cache[2 * p + 1];
    const float x0 = x[2 * p], x1 = x[2 * p + 1];
    if (fold == TCRV_FOLD_FMA) {
      y[2 * p] = fmaf(x0, c, -(x1 * s));
      y[2 * p + 1] = fmaf(x0, s, x1 * c);
    } else {
      y[2 * p] = x0 * c - x1 * s;
      y[2 * p + 1] = x0 * s + x1 * c;
    }
  }
}

void tcrv_oracle_rope_norm_f32(size_t n_dims, const float *x, float *y, float theta_base, float theta_scale,
                               int fold, float *cache) {
  float theta = theta_base;
  for (size_t p = 0; p < n_dims / 2; ++p) {
    const float pair[2] = {cosf(theta), sinf(theta)};
    if (cache) {
      cache[2 * p] = pair[0];
      cache[2 * p + 1] = pair[1];
    }
    float out[2];
    const float in[2] = {x[2 * p], x[2 * p + 1]};
    tcrv_oracle_rope_apply_f32(2, in, out, pair, fold);
    y[2 * p] = out[0];
    y[2 * p + 1] = out[1];
    theta = theta * theta_scale;
  }
}

void tcrv_oracle_pack_q4_0_to_q4_0x16(size_t nblocks, const uint8_t *src, uint8_t *dst) {
  for (size_t b = 0; b < nblocks; ++b) {
    const size_t sbase = b * 16 * 18, dbase = b * 288;
    for (size_t j = 0; j < 16; ++j)
      for (size_t k = 0; k < 2; ++k)
        dst[dbase + j * 2 + k] = src[sbase + j * 18 + k];
    for (size_t off = 0; off < 16; ++off)
      for (size_t blk = 0; blk < 16; ++blk)
        dst[dbase + 32 + off * 16 + blk] = (uint8_t)(src[sbase + blk * 18 + 2 + off] ^ 0x88);
  }
}

void tcrv_oracle_unpack_q4_0x16_to_q4_0(size_t nblocks, const uint8_t *src, uint8_t *dst) {
  for (size_t b = 0; b < nblocks; ++b) {
    const size_t sbase = b * 288, dbase = b * 16 * 18;
    for (size_t j = 0; j < 16; ++j)
      for (size_t k = 0; k < 2; ++k)
        dst[dbase + j * 18 + k] = src[sbase + j * 2 + k];
    for (size_t off = 0; off < 16; ++off)
      for (size_t blk = 0; blk < 16; ++blk)
        dst[dbase + blk * 18 + 2 + off] = (uint8_t)(src[sbase + 32 + off * 16 + blk] ^ 0x88);
  }
}

/* ---- sibling block formats ------------------------------------------------------------- */

typedef struct {
  size_t wstride, astride, wq, aq, qh, has_min;
} sibling_layout;

static int sibling_get(int format, sibling_layout *l) {
  switch (format) {
    case TCRV_ORACLE_FORMAT_Q4_1_Q8_1: *l = (sibling_layout){20, 36, 4, 4, 0, 1}; return 1;
    case TCRV_ORACLE_FORMAT_Q5_0_Q8_0: *l = (sibling_layout){22, 34, 6, 2, 2, 0}; return 1;
    case TCRV_ORACLE_FORMAT_Q5_1_Q8_1: *l = (sibling_layout){24, 36, 8, 4, 4, 1}; return 1;
    default: return 0;
  }
}

static uint16_t read_u16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

static int32_t sibling_sumi(int format, const sibling_layout *l, const uint8_t *xb, const uint8_t *yb) {
  uint32_t qh = 0;
  if (l->qh)
    qh = (uint32_t)read_u16(xb + l->qh) | ((uint32_t)read_u16(xb + l->qh + 2) << 16);
  int32_t sumi = 0;
  for (int j = 0; j < 16; ++j) {
    int lo = xb[l->wq + j] & 0x0f, hi = xb[l->wq + j] >> 4;
    if (l->qh) {
      lo |= (int)((qh >> j) & 1u) << 4;
      hi |= (int)((qh >> (j + 16)) & 1u) << 4;
    }
    if (format == TCRV_ORACLE_FORMAT_Q5_0_Q8_0) {
      lo -= 16;
      hi -= 16;
    }
    sumi += lo * (int8_t)yb[l->aq + j] + hi * (int8_t)yb[l->aq + 16 + j];
  }
  return sumi;
}

void tcrv_oracle_sibling_block_sums(int format, size_t n, int32_t *sumi, const uint8_t *vx, const uint8_t *vy) {
  sibling_layout l;
  if (!sibling_get(format, &l))
    return;
  for (size_t ib = 0; ib < n / 32; ++ib)
    sumi[ib] = sibling_sumi(format, &l, vx + ib * l.wstride, vy + ib * l.astride);
}

void tcrv_oracle_sibling_vec_dot(int format, size_t n, float *s, const uint8_t *vx, const uint8_t *vy, int fold) {
  sibling_layout l;
  if (!sibling_get(format, &l))
    return;
  float sumf = 0.0f;
  for (size_t ib = 0; ib < n / 32; ++ib) {
    const uint8_t *xb = vx + ib * l.wstride, *yb = vy + ib * l.astride;
    const float dx = tcrv_oracle_fp16_to_fp32(read_u16(xb)), dy = tcrv_oracle_fp16_to_fp32(read_u16(yb));
    const float fs = (float)sibling_sumi(format, &l, xb, yb);
    const float p = dx * dy;
    if (l.has_min) {
      const float mx = tcrv_oracle_fp16_to_fp32(read_u16(xb + 2)), sy = tcrv_oracle_fp16_to_fp32(read_u16(yb + 2));
      const float ms = mx * sy;
      const float t = fold == TCRV_FOLD_FMA ? fmaf(p, fs, ms) : p * fs + ms;
      sumf = sumf + t;
    } else {
      sumf = fold == TCRV_FOLD_FMA ? fmaf(p, fs, sumf) : sumf + p * fs;
    }
  }
  *s = sumf;
}

/* ---- consumers of the 16-row interleaved weight layouts --------------------------------- */

enum { X16_Q4_BYTES = 288, X16_Q8_BYTES = 544, X4_Q8_BYTES = 136 };

void tcrv_oracle_rows_to_q4_0x16(size_t n, size_t nc, const uint8_t *plain, uint8_t *dst) {
  const size_t nb = n / 32;
  uint8_t run[16 * 18];
  for (size_t g = 0; g < nc / 16; ++g)
    for (size_t l = 0; l < nb; ++l) {
      for (size_t r = 0; r < 16; ++r)
        memcpy(run + r * 18, plain + ((g * 16 + r) * nb + l) * 18, 18);
      tcrv_oracle_pack_q4_0_to_q4_0x16(1, run, dst + (g * nb + l) * X16_Q4_BYTES);
    }
}

void tcrv_oracle_rows_to_q8_0x16(size_t n, size_t nc, const uint8_t *plain, uint8_t *dst) {
  const size_t nb = n / 32;
  for (size_t g = 0; g < nc / 16; ++g)
    for (size_t l = 0; l < nb; ++l) {
      uint8_t *out = dst + (g * nb + l) * X16_Q8_BYTES;
      for (size_t r = 0; r < 16; ++r) {
        const uint8_t *in = plain + ((g * 16 + r) * nb + l) * 34;
        out[2 * r] = in[0];
        out[2 * r + 1] = in[1];
        for (size_t i = 0; i < 32; ++i)
          out[32 + i * 16 + r] = in[2 + i];
      }
    }
}

void tcrv_oracle_rows_to_q8_0x4(size_t n, size_t nr, const uint8_t *plain, uint8_t *dst) {
  const size_t nb = n / 32;
  for (size_t y = 0; y < nr / 4; ++y)
    for (size_t l = 0; l < nb; ++l) {
      uint8_t *out = dst + (y * nb + l) * X4_Q8_BYTES;
      for (size_t c = 0; c < 4; ++c) {
        const uint8_t *in = plain + ((y * 4 + c) * nb + l) * 34;
        out[2 * c] = in[0];
        out[2 * c + 1] = in[1];
        for (size_t i = 0; i < 32; ++i)
          out[8 + i * 4 + c] = in[2 + i];
      }
    }
}

/* Integer stage of one x16 block against one activation column, all 16 lanes.  q4: two int16
 * lane accumulators (low / high nibbles, sign-extended by shifts: the xor 0x88 is in the
 * layout), then the widening add; q8: int32 lane accumulators.  `aq` points at the 32
 * activation quants, `astep` is their stride (1 plain, 4 inside block_q8_0x4). */
static void x16_block_sums(int q8w, const uint8_t *bl, const int8_t *aq, size_t astep, int32_t sumi[16]) {
  if (q8w) {
    for (size_t r = 0; r < 16; ++r)
      sumi[r] = 0;
    for (size_t i = 0; i < 32; ++i)
      for (size_t r = 0; r < 16; ++r) {
        const int16_t prod = (int16_t)((int16_t)(int8_t)bl[32 + i * 16 + r] * (int16_t)aq[i * astep]);
        sumi[r] += prod;
      }
  } else {
    int16_t lo[16] = {0}, hi[16] = {0};
    for (size_t i = 0; i < 16; ++i)
      for (size_t r = 0; r < 16; ++r) {
        const uint8_t u = bl[32 + i * 16 + r];
        const int8_t blo = (int8_t)((int8_t)(uint8_t)(u << 4) >> 4), bhi = (int8_t)((int8_t)u >> 4);
        lo[r] = (int16_t)(lo[r] + aq[i * astep] * blo);
        hi[r] = (int16_t)(hi[r] + aq[(16 + i) * astep] * bhi);
      }
    for (size_t r = 0; r < 16; ++r)
      sumi[r] = (int32_t)lo[r] + (int32_t)hi[r];
  }
}

/* vfwmul of two fp16 scales: the exact product, representable in f32. */
static float x16_scale(const uint8_t *bl, size_t r, uint16_t da) {
  return tcrv_oracle_fp16_to_fp32(read_u16(bl + 2 * r)) * tcrv_oracle_fp16_to_fp32(da);
}

static void repack_gemv_strict(int q8w, size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc) {
  const size_t nb = n / 32, wb = q8w ? X16_Q8_BYTES : X16_Q4_BYTES;
  for (size_t x = 0; x < nc / 16; ++x) {
    float sumf[16] = {0};
    for (size_t l = 0; l < nb; ++l) {
      const uint8_t *bl = vx + (x * nb + l) * wb, *al = vy + l * 34;
      int32_t sumi[16];
      x16_block_sums(q8w, bl, (const int8_t *)(al + 2), 1, sumi);
      for (size_t r = 0; r < 16; ++r)
        sumf[r] = fmaf((float)sumi[r], x16_scale(bl, r, read_u16(al)), sumf[r]);
    }
    for (size_t r = 0; r < 16; ++r)
      s[x * 16 + r] = sumf[r];
  }
}

void tcrv_oracle_repack_gemv_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc) {
  repack_gemv_strict(0, n, s, vx, vy, nc);
}

void tcrv_oracle_repack_gemv_q8_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc) {
  repack_gemv_strict(1, n, s, vx, vy, nc);
}

void tcrv_oracle_repack_gemv_split_order(int q8w, size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc,
                                         size_t parts) {
  const size_t nb = n / 32, wb = q8w ? X16_Q8_BYTES : X16_Q4_BYTES;
  const size_t steps = (nb + 7) / 8;
  for (size_t x = 0; x < nc / 16; ++x) {
    float total[16] = {0};
    for (size_t j = 0; j < parts; ++j) {
      const size_t s0 = j * steps / parts, s1 = (j + 1) * steps / parts;
      float chain[8][16];
      memset(chain, 0, sizeof chain);
      for (size_t st = s0; st < s1; ++st)
        for (size_t c = 0; c < 8; ++c) {
          const size_t l = st * 8 + c;
          if (l >= nb)
            continue;
          const uint8_t *bl = vx + (x * nb + l) * wb, *al = vy + l * 34;
          int32_t sumi[16];
          x16_block_sums(q8w, bl, (const int8_t *)(al + 2), 1, sumi);
          for (size_t r = 0; r < 16; ++r)
            chain[c][r] = fmaf((float)sumi[r], x16_scale(bl, r, read_u16(al)), chain[c][r]);
        }
      for (size_t r = 0; r < 16; ++r) {
        const float t0 = chain[0][r] + chain[4][r], t1 = chain[1][r] + chain[5][r];
        const float t2 = chain[2][r] + chain[6][r], t3 = chain[3][r] + chain[7][r];
        const float p = (t0 + t2) + (t1 + t3);
        total[r] = j == 0 ? p : total[r] + p;
      }
    }
    for (size_t r = 0; r < 16; ++r)
      s[x * 16 + r] = total[r];
  }
}

void tcrv_oracle_repack_gemm_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nr, size_t nc,
                                       size_t bs) {
  const size_t nb = n / 32;
  for (size_t y = 0; y < nr / 4; ++y)
    for (size_t x = 0; x < nc / 16; ++x)
      for (size_t c = 0; c < 4; ++c) {
        float sumf[16] = {0};
        for (size_t l = 0; l < nb; ++l) {
          const uint8_t *bl = vx + (x * nb + l) * X16_Q4_BYTES, *al = vy + (y * nb + l) * X4_Q8_BYTES;
          int32_t sumi[16];
          x16_block_sums(0, bl, (const int8_t *)(al + 8 + c), 4, sumi);
          for (size_t r = 0; r < 16; ++r)
            sumf[r] = fmaf((float)sumi[r], x16_scale(bl, r, read_u16(al + 2 * c)), sumf[r]);
        }
        for (size_t r = 0; r < 16; ++r)
          s[(y * 4 + c) * bs + x * 16 + r] = sumf[r];
      }
}

void tcrv_oracle_q4_0_q8_0_integer_core(const int8_t *w, const int8_t *qlo, const int8_t *qhi, const int32_t *acc,
                                        int32_t *out, size_t n) {
  uint32_t total = (uint32_t)acc[0];
  for (size_t j = 0; j < n; ++j) {
    int8_t v0, v1;
    tcrv_oracle_decode_nibbles((uint8_t)w[j], &v0, &v1);
    const int16_t pair = (int16_t)((int16_t)(v0 * qlo[j]) + (int16_t)(v1 * qhi[j]));
    total += (uint32_t)(int32_t)pair;
  }
  out[0] = (int32_t)total;
}
