/* A plain C program over the C ABI of libamsim.so: no Python, no torch, no C++.
 * It is what a host in another language binds: open a LUT, run the primitive and one
 * convolution in all three directions on device buffers of its own, and check the
 * convolution against sums of the primitive's products accumulated on the host in the
 * reference order (cuda/gemm.cu:30-53: one ascending chain per output).
 *
 *   abi_driver <lut file>        exit code 0 = all checks passed
 *
 * Built by approxtrain_b200/_build.py (gcc + the CUDA runtime for the buffers). */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "amsim.h"

#define CK(call)                                                                   \
  do {                                                                             \
    int rc_ = (call);                                                              \
    if (rc_ != 0) {                                                                \
      fprintf(stderr, "%s:%d: %s -> %d (%s)\n", __FILE__, __LINE__, #call, rc_,    \
              amsim_last_error());                                                 \
      return 1;                                                                    \
    }                                                                              \
  } while (0)

static float frand(unsigned* s) {
  *s = *s * 1664525u + 1013904223u;
  return ((float)((*s >> 8) & 0xFFFF) / 32768.0f) - 1.0f; /* [-1, 1) */
}

int main(int argc, char** argv) {
  if (argc != 2) {
    fprintf(stderr, "usage: %s <MODEL>_<m>.bin\n", argv[0]);
    return 2;
  }
  enum { N = 2, H = 6, W = 5, C = 4, KH = 3, KW = 3, K = 8 };
  int oh, ow, pt, pl;
  CK(amsim_conv2d_geometry(H, W, KH, KW, 1, 1, /*same=*/1, &oh, &ow, &pt, &pl));
  const size_t nx = (size_t)N * H * W * C, nw = (size_t)KH * KW * C * K, ny = (size_t)N * oh * ow * K;
  float *x = malloc(nx * 4), *w = malloc(nw * 4), *dy = malloc(ny * 4), *y = malloc(ny * 4), *dx = malloc(nx * 4),
        *dw = malloc(nw * 4);
  unsigned seed = 7;
  for (size_t i = 0; i < nx; ++i) x[i] = frand(&seed);
  for (size_t i = 0; i < nw; ++i) w[i] = frand(&seed);
  for (size_t i = 0; i < ny; ++i) dy[i] = frand(&seed);

  amsim_lut* lut = NULL;
  CK(amsim_lut_open(argv[1], 0, &lut));
  float *d_x, *d_w, *d_dy, *d_y, *d_dx, *d_dw;
  CK(cudaMalloc((void**)&d_x, nx * 4));
  CK(cudaMalloc((void**)&d_w, nw * 4));
  CK(cudaMalloc((void**)&d_dy, ny * 4));
  CK(cudaMalloc((void**)&d_y, ny * 4));
  CK(cudaMalloc((void**)&d_dx, nx * 4));
  CK(cudaMalloc((void**)&d_dw, nw * 4));
  CK(cudaMemcpy(d_x, x, nx * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(d_w, w, nw * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(d_dy, dy, ny * 4, cudaMemcpyHostToDevice));

  /* forward, deterministic mode: must equal the host-side chain of primitive products bit for bit */
  CK(amsim_conv2d_fwd(NULL, lut, d_x, d_w, d_y, N, H, W, C, KH, KW, K, oh, ow, 1, 1, pt, pl, AMSIM_DETERMINISTIC));
  CK(cudaMemcpy(y, d_y, ny * 4, cudaMemcpyDeviceToHost));
  /* products of one output through the primitive entry point */
  const int n0 = 1, oy = 2, ox = 3, k0 = 5, taps = KH * KW * C;
  float a[KH * KW * C], b[KH * KW * C], prod[KH * KW * C];
  for (int kh = 0; kh < KH; ++kh)
    for (int kw = 0; kw < KW; ++kw)
      for (int c = 0; c < C; ++c) {
        const int iy = oy - pt + kh, ix = ox - pl + kw, t = (kh * KW + kw) * C + c;
        a[t] = (iy >= 0 && iy < H && ix >= 0 && ix < W) ? x[((n0 * H + iy) * W + ix) * C + c] : 0.0f;
        b[t] = w[((kh * KW + kw) * C + c) * K + k0];
      }
  float *d_a, *d_b, *d_p;
  CK(cudaMalloc((void**)&d_a, sizeof a));
  CK(cudaMalloc((void**)&d_b, sizeof b));
  CK(cudaMalloc((void**)&d_p, sizeof prod));
  CK(cudaMemcpy(d_a, a, sizeof a, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(d_b, b, sizeof b, cudaMemcpyHostToDevice));
  CK(amsim_mul(NULL, lut, d_a, d_b, d_p, (size_t)taps));
  CK(cudaMemcpy(prod, d_p, sizeof prod, cudaMemcpyDeviceToHost));
  volatile float acc = 0.0f;
  for (int t = 0; t < taps; ++t) acc = acc + prod[t];
  const float got = y[((n0 * oh + oy) * ow + ox) * K + k0];
  if (memcmp((const void*)&acc, &got, 4) != 0) {
    fprintf(stderr, "forward output differs from the chain of primitive products: %.9g vs %.9g\n", got, acc);
    return 1;
  }

  /* gradients: fast mode runs, deterministic mode runs, and the two agree to 1e-5 relative L2 */
  const size_t ws_bytes = amsim_conv2d_bwd_filter_workspace(N, H, W, C, KH, KW, K, oh, ow, AMSIM_FAST);
  void* ws = NULL;
  if (ws_bytes) CK(cudaMalloc(&ws, ws_bytes));
  float* ref = malloc((nx > nw ? nx : nw) * 4);
  for (int pass = 0; pass < 2; ++pass) {
    const unsigned flags = pass ? AMSIM_FAST : AMSIM_DETERMINISTIC;
    CK(amsim_conv2d_bwd_input(NULL, lut, d_w, d_dy, d_dx, N, H, W, C, KH, KW, K, oh, ow, 1, 1, pt, pl, flags));
    CK(amsim_conv2d_bwd_filter(NULL, lut, d_x, d_dy, d_dw, N, H, W, C, KH, KW, K, oh, ow, 1, 1, pt, pl, ws,
                               pass ? ws_bytes : 0, flags));
    CK(cudaMemcpy(dx, d_dx, nx * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(dw, d_dw, nw * 4, cudaMemcpyDeviceToHost));
    if (!pass) {
      memcpy(ref, dw, nw * 4);
    } else {
      double num = 0, den = 0;
      for (size_t i = 0; i < nw; ++i) {
        num += ((double)dw[i] - ref[i]) * ((double)dw[i] - ref[i]);
        den += (double)ref[i] * ref[i];
      }
      if (sqrt(num / den) > 1e-5) {
        fprintf(stderr, "fast filter gradient is %.3g away from the deterministic one\n", sqrt(num / den));
        return 1;
      }
    }
  }
  /* error path: a NULL handle is refused with a message, nothing is launched */
  if (amsim_conv2d_fwd(NULL, NULL, d_x, d_w, d_y, N, H, W, C, KH, KW, K, oh, ow, 1, 1, pt, pl, AMSIM_FAST) == AMSIM_OK ||
      strlen(amsim_last_error()) == 0) {
    fprintf(stderr, "a NULL lut handle was accepted\n");
    return 1;
  }
  CK(cudaDeviceSynchronize());
  CK(amsim_lut_close(lut));
  printf("abi_driver ok: %s, %s\n", argv[1], amsim_version());
  return 0;
}
