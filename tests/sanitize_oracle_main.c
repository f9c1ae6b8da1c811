/* Runs every entry point of the CPU oracle on small ragged shapes.  Built by
 * tests/test_sanitizers.py with -fsanitize=address,undefined: any out-of-bounds
 * access, misaligned access or signed overflow in the restated index maps aborts
 * the program.  Prints a checksum so the work cannot be optimised away. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "amsim_oracle.h"

static float* rnd(size_t n, unsigned* s) {
  float* p = (float*)malloc(n * sizeof(float) + 4);
  for (size_t i = 0; i < n; ++i) {
    *s = *s * 1664525u + 1013904223u;
    p[i] = (i % 7 == 3) ? 0.0f : ((float)(int)((*s >> 9) & 0xFFFF) - 32768.0f) / 8192.0f;
  }
  return p;
}

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  uint8_t* lut = NULL;
  int m = 0;
  if (am_load_lut(argv[1], &lut, &m)) return 3;
  unsigned seed = 1;
  double sum = 0;
  /* batch, h, w, c, fh, fw, k, stride, same */
  const int cases[][9] = {{2, 7, 6, 3, 3, 3, 5, 1, 1}, {1, 9, 9, 4, 5, 5, 6, 2, 1}, {2, 8, 8, 2, 3, 2, 7, 2, 0},
                          {3, 5, 5, 8, 5, 5, 4, 1, 0}, {1, 6, 7, 5, 1, 1, 9, 1, 0}, {2, 11, 4, 1, 4, 3, 2, 3, 1}};
  for (size_t ci = 0; ci < sizeof(cases) / sizeof(cases[0]); ++ci) {
    const int* c = cases[ci];
    am_conv_geom_t g;
    am_conv_geometry(c[0], c[1], c[2], c[3], c[4], c[5], c[6], c[7], c[7], c[8], &g);
    const size_t nx = (size_t)g.batch * g.in_h * g.in_w * g.in_c, nw = (size_t)g.f_h * g.f_w * g.in_c * g.out_c,
                 ny = (size_t)g.batch * g.out_h * g.out_w * g.out_c;
    float *x = rnd(nx, &seed), *w = rnd(nw, &seed), *dy = rnd(ny, &seed);
    float *y = (float*)malloc(ny * 4 + 4), *dw = (float*)malloc(nw * 4 + 4), *dx = (float*)malloc(nx * 4 + 4);
    am_conv2d_fwd(&g, x, w, y, lut, m);
    am_conv2d_bwd_filter(&g, x, dy, dw, lut, m);
    am_conv2d_bwd_input(&g, w, dy, dx, lut, m);
    for (size_t i = 0; i < ny; ++i) sum += y[i];
    for (size_t i = 0; i < nw; ++i) sum += dw[i];
    for (size_t i = 0; i < nx; ++i) sum += dx[i];
    cpu_conv2d_fwd(&g, x, w, y);
    cpu_conv2d_bwd_filter(&g, x, dy, dw);
    cpu_conv2d_bwd_input(&g, w, dy, dx);
    for (size_t i = 0; i < ny; ++i) sum += y[i];
    am_conv2d_fwd(&g, x, w, y, NULL, AM_DIRECT_MBM32);
    am_conv2d_bwd_filter(&g, x, dy, dw, NULL, AM_DIRECT_MIT32);
    for (size_t i = 0; i < nw; ++i) sum += dw[i];
    free(x); free(w); free(dy); free(y); free(dw); free(dx);
  }
  {
    const int b = 5, kin = 13, u = 7;
    float *x = rnd((size_t)b * kin, &seed), *w = rnd((size_t)kin * u, &seed), *gy = rnd((size_t)b * u, &seed);
    float *y = (float*)malloc(b * u * 4), *dw = (float*)malloc(kin * u * 4), *dx = (float*)malloc(b * kin * 4);
    am_dense_fwd(x, w, y, b, u, kin, lut, m);
    am_dense_bwd_weight(x, gy, dw, b, u, kin, lut, m);
    am_dense_bwd_input(w, gy, dx, b, u, kin, lut, m);
    cpu_dense_fwd(x, w, y, b, u, kin);
    cpu_dense_bwd_weight(x, gy, dw, b, u, kin);
    cpu_dense_bwd_input(w, gy, dx, b, u, kin);
    for (int i = 0; i < b * u; ++i) sum += y[i];
    for (int i = 0; i < kin * u; ++i) sum += dw[i];
    for (int i = 0; i < b * kin; ++i) sum += dx[i];
    float* c = (float*)malloc(3 * b * u * 4);
    float* a3 = rnd((size_t)3 * b * kin, &seed);
    am_matmul(a3, w, c, 3, 0, b, kin, u, lut, m); /* rank-3 x rank-2 */
    for (int i = 0; i < 3 * b * u; ++i) sum += c[i];
    am_gemm(b, u, kin, x, kin, w, u, y, u, lut, m);
    cpu_gemm(b, u, kin, x, kin, w, u, y, u);
    free(x); free(w); free(gy); free(y); free(dw); free(dx); free(c); free(a3);
  }
  /* special operand classes through the primitive */
  const uint32_t specials[] = {0u, 0x80000000u, 1u, 0x007FFFFFu, 0x00800000u, 0x3F800000u, 0x40000000u, 0x7F7FFFFFu,
                               0x7F800000u, 0x7FC00000u, 0xFF800000u, 0x7E967699u};
  for (size_t i = 0; i < sizeof(specials) / 4; ++i)
    for (size_t j = 0; j < sizeof(specials) / 4; ++j) sum += (double)(am_mul_bits(specials[i], specials[j], lut, m) & 0xFFFF);
  free(lut);
  printf("checksum %.6e\n", sum);
  return 0;
}
