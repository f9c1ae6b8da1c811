/*
 * CPU oracle for the AM-Simulator hot path (see amsim_oracle.h).
 * TEST INFRASTRUCTURE ONLY — never linked into or called by the product.
 *
 * Every function names the reference file:line it restates.  The arithmetic
 * is integer bit manipulation plus FP32 adds; compile WITHOUT -ffast-math and
 * without FMA contraction (-ffp-contract=off) so that each "acc + product"
 * is one IEEE round-to-nearest add like the reference's GPU code.
 */
#include "amsim_oracle.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <limits.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static int g_threads = 0; /* 0 = OpenMP default */

void am_oracle_set_threads(int n) {
  g_threads = n;
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#endif
}

static inline uint32_t f2u(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
static inline float u2f(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* approx_mul_lut.h:22-25 */
int am_parse_mant_width(const char* path) {
  const char* us = strrchr(path, '_');
  const char* dot = strrchr(path, '.');
  if (!us || !dot || dot <= us + 1) return -1;
  int m = 0;
  for (const char* p = us + 1; p < dot; ++p) {
    if (*p < '0' || *p > '9') return -1;
    m = m * 10 + (*p - '0');
    if (m > 99) return -1;
  }
  /* a_shift = 23 - 2m is held in a uint8_t (approx_mul_lut.h:26,72): m <= 11 */
  if (m < 1 || m > 11) return -1;
  return m;
}

/* approx_mul_lut.h:15-45 */
int am_load_lut(const char* path, uint8_t** out, int* m_out) {
  int m = am_parse_mant_width(path);
  if (m < 0) return 1;
  FILE* f = fopen(path, "rb");
  if (!f) return 2;
  size_t want = (size_t)1 << (2 * m);
  uint8_t* buf = (uint8_t*)malloc(want + 1);
  if (!buf) {
    fclose(f);
    return 3;
  }
  size_t got = fread(buf, 1, want + 1, f);
  fclose(f);
  if (got != want) {
    free(buf);
    return 4;
  }
  *out = buf;
  *m_out = m;
  return 0;
}

/* Direct simulation of the 32-bit multipliers (mantissa width 23: too wide for a
 * table), the reference's cuda/FPmultMBM_fast32.inl:13-126 and cuda/Mitchell_32.inl.
 * Both take sign and exponent from the exact FP32 product, replace its mantissa by
 * an approximate one and move the exponent by the difference between "the exact
 * mantissa product reached 2" and "the approximate one reached 2"; an exact product
 * that is inf/NaN is passed through, one that is zero or subnormal gives +0.
 *
 * Restated arithmetic (not the reference's statement order):
 *  - "the exact mantissa product, rounded to 24 bits, reached 2"
 *    (FPmultMBM_fast32.inl:71-92: a 48-bit integer product, then round-to-nearest-
 *    even by hand) is the FP32 product of 1.ma and 1.mb compared with 2: the
 *    hardware rounding is the same round-to-nearest-even at the same bit;
 *  - MBM mantissa (:13-36): s = ma + mb; carry = s >= 2^23; t = (s mod 2^23) +
 *    (0xA0000 >> carry); if carry and t >= 2^23 the correction is dropped (t = s);
 *    w = (2^23 + t) << carry; Mitchell (Mitchell_32.inl:13-32): t = s mod 2^23;
 *  - approximate "reached 2": w >= 2^24, then w >>= 1; mantissa = w mod 2^23. */
static uint32_t direct_mul_bits(uint32_t at, uint32_t bt, int mbm) {
  const float exact = u2f(at) * u2f(bt);
  const uint32_t eb = f2u(exact);
  const uint32_t eexp = (eb >> 23) & 0xffu;
  if (eexp == 255u) return eb;
  if (eexp == 0u) return 0u;
  const uint32_t ma = at & 0x7fffffu, mb = bt & 0x7fffffu;
  const int exact_two = u2f(0x3f800000u | ma) * u2f(0x3f800000u | mb) >= 2.0f;
  const uint32_t s = ma + mb;
  const uint32_t carry = s >= 0x800000u;
  uint32_t t = s & 0x7fffffu;
  if (mbm) {
    t += 0xA0000u >> carry;
    if (carry && t >= 0x800000u) t = s;
  }
  uint32_t w = (0x800000u + t) << carry;
  const int approx_two = w >= 0x1000000u;
  if (approx_two) w >>= 1;
  const uint32_t e = eexp - (uint32_t)exact_two + (uint32_t)approx_two;
  return (eb & 0x80000000u) + (e << 23) + (w & 0x7fffffu);
}

/* cuda/AMsimulator.inl:13-36.  mant_mask / a_shift / b_shift as derived in
 * approx_mul_lut.h:26-28.  The pseudo-widths AM_DIRECT_MBM32 / AM_DIRECT_MIT32
 * select the direct 32-bit models instead (lut is ignored). */
uint32_t am_mul_bits(uint32_t at, uint32_t bt, const uint8_t* lut, int m) {
  if (m == AM_DIRECT_MBM32) return direct_mul_bits(at, bt, 1);
  if (m == AM_DIRECT_MIT32) return direct_mul_bits(at, bt, 0);
  if (m & AM_WIDE_ENTRIES) {
    /* Format extension (no reference counterpart): 16-bit little-endian entries,
     * carry << 15 | top 15 mantissa bits of the product; everything else as below. */
    const int mw = m & ~AM_WIDE_ENTRIES;
    const uint32_t mask16 = ((1u << mw) - 1u) << (23 - mw);
    const uint32_t idx16 = ((at & mask16) >> (23 - 2 * mw)) | ((bt & mask16) >> (23 - mw));
    const uint32_t v16 = (uint32_t)lut[2 * (size_t)idx16] | ((uint32_t)lut[2 * (size_t)idx16 + 1] << 8);
    uint32_t e16 = ((at & 0x7f800000u) >> 23) + ((bt & 0x7f800000u) >> 23);
    if (e16 <= 127u) return 0u;
    e16 = e16 - 127u + (v16 >> 15);
    return ((at ^ bt) & 0x80000000u) + (e16 << 23) + ((v16 & 0x7fffu) << 8);
  }
  const uint32_t mant_mask = ((1u << m) - 1u) << (23 - m);
  const uint32_t a_shift = (uint32_t)(23 - 2 * m);
  const uint32_t b_shift = (uint32_t)(23 - m);
  const uint32_t idx = ((at & mant_mask) >> a_shift) | ((bt & mant_mask) >> b_shift);
  const uint32_t v = lut[idx];                          /* :21 */
  const uint32_t carry = (v & 0x80u) >> 7;              /* :22 */
  const uint32_t mant = (v & 0x7fu) << (23 - m);        /* :23 */
  const uint32_t sgn = (at ^ bt) & 0x80000000u;         /* :25 */
  uint32_t e = ((at & 0x7f800000u) >> 23) + ((bt & 0x7f800000u) >> 23); /* :26 */
  /* :28 — the two "operand exponent is zero" clauses parse as
   * `at & (EXPONENT_MASK == 0)` and are always false, so only the sum test
   * survives: AM(0, x) is non-zero when the exponent field of x is >= 128. */
  if (e <= 127u) return 0u;
  e = e - 127u + carry;                                 /* :31 */
  return sgn + (e << 23) + mant;                        /* :32, uint32 wrap */
}

float am_mul(float a, float b, const uint8_t* lut, int m) {
  return u2f(am_mul_bits(f2u(a), f2u(b), lut, m));
}

void am_mul_array(const float* a, const float* b, float* out, size_t n,
                  const uint8_t* lut, int m) {
  for (size_t i = 0; i < n; ++i) out[i] = am_mul(a[i], b[i], lut, m);
}

/* cuda/gemm.cu:22-58: value starts at 0, k ascending, single accumulator.
 * The zero-filled k tail of the last 16-wide tile adds AM(0,0) = +0. */
void am_gemm(int m, int n, int k, const float* A, int lda, const float* B,
             int ldb, float* C, int ldc, const uint8_t* lut, int mw) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int i = 0; i < m; ++i) {
    for (int j = 0; j < n; ++j) {
      float acc = 0.0f;
      for (int l = 0; l < k; ++l)
        acc = acc + am_mul(A[(size_t)i * lda + l], B[(size_t)l * ldb + j], lut, mw);
      C[(size_t)i * ldc + j] = acc;
    }
  }
}

/* TF GetWindowedOutputSizeVerbose with dilation 1; the pad-before it yields
 * equals the filter_top/left_offset of convam.cc:557-572. */
static void window_1d(int in, int f, int s, int same, int* out, int* pad_before) {
  if (same) {
    *out = (in + s - 1) / s;
    int total = (*out - 1) * s + f - in;
    if (total < 0) total = 0;
    *pad_before = total / 2;
  } else {
    *out = (in - f + s) / s;
    *pad_before = 0;
  }
}

void am_conv_geometry(int batch, int in_h, int in_w, int in_c, int f_h, int f_w,
                      int out_c, int stride_h, int stride_w, int same,
                      am_conv_geom_t* g) {
  g->batch = batch;
  g->in_h = in_h;
  g->in_w = in_w;
  g->in_c = in_c;
  g->f_h = f_h;
  g->f_w = f_w;
  g->out_c = out_c;
  g->stride_h = stride_h;
  g->stride_w = stride_w;
  window_1d(in_h, f_h, stride_h, same, &g->out_h, &g->pad_top);
  window_1d(in_w, f_w, stride_w, same, &g->out_w, &g->pad_left);
}

/* Forward: patch row (n,oh,ow), patch column (kh,kw,c) — cuda_kernel.cu:39-58;
 * GEMM m = N*OH*OW, n = K, k = KH*KW*C — :163-170.  Padded taps are real
 * zeros pushed through the multiplier, not skipped terms. */
void am_conv2d_fwd(const am_conv_geom_t* g, const float* x, const float* w,
                   float* y, const uint8_t* lut, int m) {
  const int N = g->batch, H = g->in_h, W = g->in_w, C = g->in_c;
  const int KH = g->f_h, KW = g->f_w, K = g->out_c, OH = g->out_h, OW = g->out_w;
#pragma omp parallel for collapse(3) schedule(static)
  for (int n = 0; n < N; ++n)
    for (int oh = 0; oh < OH; ++oh)
      for (int ow = 0; ow < OW; ++ow) {
        float* yo = y + (((size_t)n * OH + oh) * OW + ow) * K;
        for (int ko = 0; ko < K; ++ko) {
          float acc = 0.0f;
          for (int kh = 0; kh < KH; ++kh) {
            const int ih = oh * g->stride_h - g->pad_top + kh;
            for (int kw = 0; kw < KW; ++kw) {
              const int iw = ow * g->stride_w - g->pad_left + kw;
              const int inside = ih >= 0 && iw >= 0 && ih < H && iw < W;
              const float* xp = inside ? x + (((size_t)n * H + ih) * W + iw) * C : NULL;
              const float* wp = w + ((size_t)(kh * KW + kw) * C) * K + ko;
              for (int c = 0; c < C; ++c) {
                const float a = inside ? xp[c] : 0.0f;
                acc = acc + am_mul(a, wp[(size_t)c * K], lut, m);
              }
            }
          }
          yo[ko] = acc;
        }
      }
}

/* Filter gradient: patch row (kh,kw,c), patch column (n,oh,ow) —
 * cuda_kernel.cu:331-350; GEMM m = KH*KW*C, n = K, k = N*OH*OW with the
 * gathered input as A and the output gradient as B — :417-425. */
void am_conv2d_bwd_filter(const am_conv_geom_t* g, const float* x,
                          const float* dy, float* dw, const uint8_t* lut, int m) {
  const int N = g->batch, H = g->in_h, W = g->in_w, C = g->in_c;
  const int KH = g->f_h, KW = g->f_w, K = g->out_c, OH = g->out_h, OW = g->out_w;
#pragma omp parallel for collapse(3) schedule(static)
  for (int kh = 0; kh < KH; ++kh)
    for (int kw = 0; kw < KW; ++kw)
      for (int c = 0; c < C; ++c) {
        float* out = dw + ((size_t)(kh * KW + kw) * C + c) * K;
        for (int ko = 0; ko < K; ++ko) {
          float acc = 0.0f;
          for (int n = 0; n < N; ++n)
            for (int oh = 0; oh < OH; ++oh) {
              const int ih = oh * g->stride_h + kh - g->pad_top;
              for (int ow = 0; ow < OW; ++ow) {
                const int iw = ow * g->stride_w + kw - g->pad_left;
                const int inside = ih >= 0 && iw >= 0 && ih < H && iw < W;
                const float a = inside ? x[(((size_t)n * H + ih) * W + iw) * C + c] : 0.0f;
                const float b = dy[(((size_t)n * OH + oh) * OW + ow) * K + ko];
                acc = acc + am_mul(a, b, lut, m);
              }
            }
          out[ko] = acc;
        }
      }
}

/* Input gradient: the output gradient is dilated by the stride into a
 * "hole" grid of (OH-1)*sh+1 rows (convam.cc:1066-1067), padded by
 * KH-1-pad_top (convam.cc:1083-1084) and gathered per input position with
 * column order (kh,kw,ko) — cuda_kernel.cu:467-500; the filter is flipped
 * spatially with C and K swapped — cuda/reverseNswapdim23.cu:16; GEMM
 * m = N*H*W, n = C, k = KH*KW*K — cuda_kernel.cu:569-583. */
void am_conv2d_bwd_input(const am_conv_geom_t* g, const float* w,
                         const float* dy, float* dx, const uint8_t* lut, int m) {
  const int N = g->batch, H = g->in_h, W = g->in_w, C = g->in_c;
  const int KH = g->f_h, KW = g->f_w, K = g->out_c, OH = g->out_h, OW = g->out_w;
  const int sh = g->stride_h, sw = g->stride_w;
  const int hole_h = (OH - 1) * sh + 1, hole_w = (OW - 1) * sw + 1;
  const int bpt = KH - 1 - g->pad_top, bpl = KW - 1 - g->pad_left;
#pragma omp parallel for collapse(3) schedule(static)
  for (int n = 0; n < N; ++n)
    for (int yy = 0; yy < H; ++yy)
      for (int xx = 0; xx < W; ++xx) {
        float* out = dx + (((size_t)n * H + yy) * W + xx) * C;
        for (int c = 0; c < C; ++c) {
          float acc = 0.0f;
          for (int kh = 0; kh < KH; ++kh) {
            const int u = yy - bpt + kh;
            for (int kw = 0; kw < KW; ++kw) {
              const int v = xx - bpl + kw;
              const int hit = u >= 0 && v >= 0 && u < hole_h && v < hole_w &&
                              (u % sh) == 0 && (v % sw) == 0;
              const float* gp =
                  hit ? dy + (((size_t)n * OH + u / sh) * OW + v / sw) * K : NULL;
              const float* wp =
                  w + (((size_t)(KH - 1 - kh) * KW + (KW - 1 - kw)) * C + c) * K;
              for (int ko = 0; ko < K; ++ko) {
                const float a = hit ? gp[ko] : 0.0f;
                acc = acc + am_mul(a, wp[ko], lut, m);
              }
            }
          }
          out[c] = acc;
        }
      }
}

/* cuda/denseam_kernel.cu:32-41 */
void am_dense_fwd(const float* x, const float* w, float* y, int batch,
                  int units, int in_w, const uint8_t* lut, int m) {
  am_gemm(batch, units, in_w, x, in_w, w, units, y, units, lut, m);
}

/* cuda/denseam_kernel.cu:58-67: dw[k,u] = sum_b AM(x[b,k], g[b,u]) */
void am_dense_bwd_weight(const float* x, const float* g, float* dw, int batch,
                         int units, int in_w, const uint8_t* lut, int m) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int k = 0; k < in_w; ++k)
    for (int u = 0; u < units; ++u) {
      float acc = 0.0f;
      for (int b = 0; b < batch; ++b)
        acc = acc + am_mul(x[(size_t)b * in_w + k], g[(size_t)b * units + u], lut, m);
      dw[(size_t)k * units + u] = acc;
    }
}

/* cuda/denseam_kernel.cu:84-94: dx[b,k] = sum_u AM(w[k,u], g[b,u]) — the
 * weight is the first (LUT-row) operand. */
void am_dense_bwd_input(const float* w, const float* g, float* dx, int batch,
                        int units, int in_w, const uint8_t* lut, int m) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < batch; ++b)
    for (int k = 0; k < in_w; ++k) {
      float acc = 0.0f;
      for (int u = 0; u < units; ++u)
        acc = acc + am_mul(w[(size_t)k * units + u], g[(size_t)b * units + u], lut, m);
      dx[(size_t)b * in_w + k] = acc;
    }
}

/* cuda/matmulam_kernel.cu:30-96; output shapes matmulam.cc:122-147. */
void am_matmul(const float* a, const float* b, float* c, int batch_a,
               int batch_b, int row_a, int col_a, int col_b, const uint8_t* lut,
               int m) {
  int nb = batch_a > batch_b ? batch_a : batch_b;
  if (nb == 0) nb = 1;
  const size_t sa = (batch_a > 1) ? (size_t)row_a * col_a : 0;
  const size_t sb = (batch_b > 1) ? (size_t)col_a * col_b : 0;
  for (int i = 0; i < nb; ++i)
    am_gemm(row_a, col_b, col_a, a + i * sa, col_a, b + i * sb, col_b,
            c + (size_t)i * row_a * col_b, col_b, lut, m);
}

/* ---------------- T = int32 ------------------------------------------------ */

/* float -> int32 as the GPU's cvt.rzi.s32.f32 does it: truncate, saturate, NaN -> 0 */
static inline int32_t f2i_sat(float f) {
  if (f != f) return 0;
  if (f >= 2147483648.0f) return INT32_MAX;
  if (f <= -2147483648.0f) return INT32_MIN;
  return (int32_t)f;
}

/* one accumulation step of gemm<int32> (cuda/gemm.cu:49 with T = int32) */
static inline int32_t step_i32(int32_t acc, int32_t a, int32_t b, const uint8_t* lut, int m) {
  return f2i_sat((float)acc + am_mul((float)a, (float)b, lut, m));
}

void am_gemm_i32(int m, int n, int k, const int32_t* A, int lda, const int32_t* B,
                 int ldb, int32_t* C, int ldc, const uint8_t* lut, int mw) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      int32_t acc = 0;
      for (int l = 0; l < k; ++l) acc = step_i32(acc, A[(size_t)i * lda + l], B[(size_t)l * ldb + j], lut, mw);
      C[(size_t)i * ldc + j] = acc;
    }
}

void am_conv2d_fwd_i32(const am_conv_geom_t* g, const int32_t* x, const int32_t* w,
                       int32_t* y, const uint8_t* lut, int m) {
  const int N = g->batch, H = g->in_h, W = g->in_w, C = g->in_c;
  const int KH = g->f_h, KW = g->f_w, K = g->out_c, OH = g->out_h, OW = g->out_w;
#pragma omp parallel for collapse(3) schedule(static)
  for (int n = 0; n < N; ++n)
    for (int oh = 0; oh < OH; ++oh)
      for (int ow = 0; ow < OW; ++ow)
        for (int ko = 0; ko < K; ++ko) {
          int32_t acc = 0;
          for (int kh = 0; kh < KH; ++kh)
            for (int kw = 0; kw < KW; ++kw) {
              const int ih = oh * g->stride_h - g->pad_top + kh, iw = ow * g->stride_w - g->pad_left + kw;
              const int inside = ih >= 0 && iw >= 0 && ih < H && iw < W;
              for (int c = 0; c < C; ++c) {
                const int32_t a = inside ? x[(((size_t)n * H + ih) * W + iw) * C + c] : 0;
                acc = step_i32(acc, a, w[(((size_t)kh * KW + kw) * C + c) * K + ko], lut, m);
              }
            }
          y[(((size_t)n * OH + oh) * OW + ow) * K + ko] = acc;
        }
}

void am_conv2d_bwd_filter_i32(const am_conv_geom_t* g, const int32_t* x,
                              const int32_t* dy, int32_t* dw, const uint8_t* lut, int m) {
  const int N = g->batch, H = g->in_h, W = g->in_w, C = g->in_c;
  const int KH = g->f_h, KW = g->f_w, K = g->out_c, OH = g->out_h, OW = g->out_w;
#pragma omp parallel for collapse(3) schedule(static)
  for (int kh = 0; kh < KH; ++kh)
    for (int kw = 0; kw < KW; ++kw)
      for (int c = 0; c < C; ++c)
        for (int ko = 0; ko < K; ++ko) {
          int32_t acc = 0;
          for (int n = 0; n < N; ++n)
            for (int oh = 0; oh < OH; ++oh)
              for (int ow = 0; ow < OW; ++ow) {
                const int ih = oh * g->stride_h + kh - g->pad_top, iw = ow * g->stride_w + kw - g->pad_left;
                const int inside = ih >= 0 && iw >= 0 && ih < H && iw < W;
                const int32_t a = inside ? x[(((size_t)n * H + ih) * W + iw) * C + c] : 0;
                acc = step_i32(acc, a, dy[(((size_t)n * OH + oh) * OW + ow) * K + ko], lut, m);
              }
          dw[(((size_t)kh * KW + kw) * C + c) * K + ko] = acc;
        }
}

void am_conv2d_bwd_input_i32(const am_conv_geom_t* g, const int32_t* w,
                             const int32_t* dy, int32_t* dx, const uint8_t* lut, int m) {
  const int N = g->batch, H = g->in_h, W = g->in_w, C = g->in_c;
  const int KH = g->f_h, KW = g->f_w, K = g->out_c, OH = g->out_h, OW = g->out_w;
  const int sh = g->stride_h, sw = g->stride_w;
  const int hole_h = (OH - 1) * sh + 1, hole_w = (OW - 1) * sw + 1;
  const int bpt = KH - 1 - g->pad_top, bpl = KW - 1 - g->pad_left;
#pragma omp parallel for collapse(3) schedule(static)
  for (int n = 0; n < N; ++n)
    for (int yy = 0; yy < H; ++yy)
      for (int xx = 0; xx < W; ++xx)
        for (int c = 0; c < C; ++c) {
          int32_t acc = 0;
          for (int kh = 0; kh < KH; ++kh)
            for (int kw = 0; kw < KW; ++kw) {
              const int u = yy - bpt + kh, v = xx - bpl + kw;
              const int hit = u >= 0 && v >= 0 && u < hole_h && v < hole_w && (u % sh) == 0 && (v % sw) == 0;
              for (int ko = 0; ko < K; ++ko) {
                const int32_t a = hit ? dy[(((size_t)n * OH + u / sh) * OW + v / sw) * K + ko] : 0;
                acc = step_i32(acc, a, w[((((size_t)(KH - 1 - kh)) * KW + (KW - 1 - kw)) * C + c) * K + ko], lut, m);
              }
            }
          dx[(((size_t)n * H + yy) * W + xx) * C + c] = acc;
        }
}

/* ---------------- reference CPU op path: exact multiply ------------------ */

/* convam.cc:452-491 */
void cpu_conv2d_fwd(const am_conv_geom_t* g, const float* x, const float* w,
                    float* y) {
  const int H = g->in_h, W = g->in_w, C = g->in_c, K = g->out_c;
  for (int n = 0; n < g->batch; ++n)
    for (int oy = 0; oy < g->out_h; ++oy)
      for (int ox = 0; ox < g->out_w; ++ox)
        for (int ko = 0; ko < K; ++ko) {
          const int x0 = ox * g->stride_w - g->pad_left;
          const int y0 = oy * g->stride_h - g->pad_top;
          float total = 0.0f;
          for (int fy = 0; fy < g->f_h; ++fy)
            for (int fx = 0; fx < g->f_w; ++fx)
              for (int c = 0; c < C; ++c) {
                const int ix = x0 + fx, iy = y0 + fy;
                float xv = 0.0f;
                if (ix >= 0 && ix < W && iy >= 0 && iy < H)
                  xv = x[(((size_t)n * H + iy) * W + ix) * C + c];
                const float wv = w[(((size_t)fy * g->f_w + fx) * C + c) * K + ko];
                total += xv * wv;
              }
          y[(((size_t)n * g->out_h + oy) * g->out_w + ox) * K + ko] = total;
        }
}

/* convam.cc:639-686: walks the stride-dilated gradient grid with the batch
 * innermost; positions that are not multiples of the stride contribute 0. */
void cpu_conv2d_bwd_filter(const am_conv_geom_t* g, const float* x,
                           const float* dy, float* dw) {
  const int H = g->in_h, W = g->in_w, C = g->in_c, K = g->out_c;
  const int gh = (g->out_h - 1) * g->stride_h + 1;
  const int gw = (g->out_w - 1) * g->stride_w + 1;
  for (int fy = 0; fy < g->f_h; ++fy)
    for (int fx = 0; fx < g->f_w; ++fx)
      for (int c = 0; c < C; ++c)
        for (int ko = 0; ko < K; ++ko) {
          const int x0 = fx - g->pad_left, y0 = fy - g->pad_top;
          float total = 0.0f;
          for (int gy = 0; gy < gh; ++gy)
            for (int gx = 0; gx < gw; ++gx)
              for (int n = 0; n < g->batch; ++n) {
                const int ix = x0 + gx, iy = y0 + gy;
                float xv = 0.0f;
                if (ix >= 0 && ix < W && iy >= 0 && iy < H)
                  xv = x[(((size_t)n * H + iy) * W + ix) * C + c];
                float gv = 0.0f;
                if (gy % g->stride_h == 0 && gx % g->stride_w == 0)
                  gv = dy[(((size_t)n * g->out_h + gy / g->stride_h) * g->out_w +
                           gx / g->stride_w) * K + ko];
                total += xv * gv;
              }
          dw[(((size_t)fy * g->f_w + fx) * C + c) * K + ko] = total;
        }
}

/* convam.cc:910-954.  The reference indexes the gradient with `batch`
 * instead of the loop variable (:931, out of bounds); the loop variable is
 * used here. */
void cpu_conv2d_bwd_input(const am_conv_geom_t* g, const float* w,
                          const float* dy, float* dx) {
  const int H = g->in_h, W = g->in_w, C = g->in_c, K = g->out_c;
  const int gh = (g->out_h - 1) * g->stride_h + 1;
  const int gw = (g->out_w - 1) * g->stride_w + 1;
  const int bpt = g->f_h - 1 - g->pad_top, bpl = g->f_w - 1 - g->pad_left;
  for (int n = 0; n < g->batch; ++n)
    for (int oy = 0; oy < H; ++oy)
      for (int ox = 0; ox < W; ++ox)
        for (int c = 0; c < C; ++c) {
          const int x0 = ox - bpl, y0 = oy - bpt;
          float total = 0.0f;
          for (int fy = 0; fy < g->f_h; ++fy)
            for (int fx = 0; fx < g->f_w; ++fx)
              for (int ko = 0; ko < K; ++ko) {
                const int ix = x0 + fx, iy = y0 + fy;
                float gv = 0.0f;
                if (ix >= 0 && ix < gw && iy >= 0 && iy < gh &&
                    iy % g->stride_h == 0 && ix % g->stride_w == 0)
                  gv = dy[(((size_t)n * g->out_h + iy / g->stride_h) * g->out_w +
                           ix / g->stride_w) * K + ko];
                const float wv = w[((((size_t)(g->f_h - 1 - fy)) * g->f_w +
                                     (g->f_w - 1 - fx)) * C + c) * K + ko];
                total += gv * wv;
              }
          dx[(((size_t)n * H + oy) * W + ox) * C + c] = total;
        }
}

/* denseam.cc:64-71 */
void cpu_dense_fwd(const float* x, const float* w, float* y, int batch,
                   int units, int in_w) {
  for (int i = 0; i < batch; ++i)
    for (int j = 0; j < units; ++j) {
      y[(size_t)i * units + j] = 0.0f;
      for (int k = 0; k < in_w; ++k)
        y[(size_t)i * units + j] += x[(size_t)i * in_w + k] * w[(size_t)k * units + j];
    }
}

/* denseam.cc:151-157 — the reference accumulates into an output it never
 * clears; it is zero-filled here. */
void cpu_dense_bwd_weight(const float* x, const float* g, float* dw, int batch,
                          int units, int in_w) {
  memset(dw, 0, sizeof(float) * (size_t)in_w * units);
  for (int i = 0; i < batch; ++i)
    for (int j = 0; j < units; ++j)
      for (int k = 0; k < in_w; ++k)
        dw[(size_t)k * units + j] += x[(size_t)i * in_w + k] * g[(size_t)i * units + j];
}

/* denseam.cc:166-173 — same uncleared output; the duplicated outer `for`
 * (:166-167) would run the body batch times, it runs once here. */
void cpu_dense_bwd_input(const float* w, const float* g, float* dx, int batch,
                         int units, int in_w) {
  memset(dx, 0, sizeof(float) * (size_t)batch * in_w);
  for (int i = 0; i < batch; ++i)
    for (int j = 0; j < units; ++j)
      for (int k = 0; k < in_w; ++k)
        dx[(size_t)i * in_w + k] += w[(size_t)k * units + j] * g[(size_t)i * units + j];
}

/* matmulam.cc:178-208: column-outer loop order, one total per output. */
void cpu_gemm(int m, int n, int k, const float* a, int lda, const float* b,
              int ldb, float* c, int ldc) {
  for (size_t j = 0; j < (size_t)n; ++j)
    for (size_t i = 0; i < (size_t)m; ++i) {
      float total = 0.0f;
      for (size_t l = 0; l < (size_t)k; ++l) total += a[i * lda + l] * b[l * ldb + j];
      c[i * ldc + j] = total;
    }
}
