/*
 * CPU oracle for the AM-Simulator hot path of ApproxTrain.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of what the
 * reference's GPU kernels compute (LUT approximate multiply + FP32
 * accumulation in the reference's order) and of the reference's CPU op path
 * (exact multiply) used as a timed baseline.  The product library never links
 * or calls anything in this directory; only the tests, the smoke check and
 * the benchmark's CPU-baseline leg do.
 *
 * Parity pin: am_mul_bits() is compared exhaustively against the reference's
 * own cuda/AMsimulator.inl (compiled as host C++ by oracle/build.sh) and
 * the LUT bytes against lut/lut_gen.cc output and the shipped lut/ *.bin md5s.
 */
#ifndef AMSIM_ORACLE_H_
#define AMSIM_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* LUT descriptor: bytes[2^(2m)] and the mantissa width m parsed from the file
 * name "<MODEL>_<m>.bin" (approx_mul_lut.h:22-28). */
typedef struct {
  const uint8_t* bytes;
  int m;
} am_lut_t;

/* approx_mul_lut.h:22-25 — m is the integer between the last '_' and the last
 * '.' of the path.  Returns -1 when it cannot be parsed or is outside 1..11. */
int am_parse_mant_width(const char* path);

/* approx_mul_lut.h:15-45 — read 2^(2m) bytes.  Unlike the reference (which
 * asks for 4x as many bytes and stops at EOF) the file must hold exactly
 * 2^(2m) bytes.  Returns 0 on success; *out is malloc'ed, caller frees. */
int am_load_lut(const char* path, uint8_t** out, int* m);

/* Pseudo mantissa widths: every function below that takes (lut, m) runs the
 * reference's direct 32-bit model instead of a table when m is one of these
 * (cuda/FPmultMBM_fast32.inl:41-126, cuda/Mitchell_32.inl; lut may be NULL). */
#define AM_DIRECT_MBM32 132
#define AM_DIRECT_MIT32 123
/* m | AM_WIDE_ENTRIES: the table holds 2^(2m) 16-bit little-endian entries
 * (carry << 15 | top 15 mantissa bits) instead of bytes: a format extension of this
 * repository that makes m = 8..11 numerically meaningful; no reference counterpart. */
#define AM_WIDE_ENTRIES 0x100

/* cuda/AMsimulator.inl:13-36 on raw bit patterns. */
uint32_t am_mul_bits(uint32_t at, uint32_t bt, const uint8_t* lut, int m);
float am_mul(float a, float b, const uint8_t* lut, int m);
void am_mul_array(const float* a, const float* b, float* out, size_t n,
                  const uint8_t* lut, int m);

/* cuda/gemm.cu:16-58 — C[m x n] = sum_k AM(A[i,k], B[k,j]), one ascending-k
 * FP32 chain per output, row-major with leading dimensions. */
void am_gemm(int m, int n, int k, const float* A, int lda, const float* B,
             int ldb, float* C, int ldc, const uint8_t* lut, int mw);

/* Convolution geometry shared by the three conv entry points.  NHWC
 * activations, HWIO filters.  pad_top/pad_left are the forward pad-before
 * amounts (convam.cc:557-572), 0 for VALID. */
typedef struct {
  int batch, in_h, in_w, in_c;
  int f_h, f_w, out_c;
  int out_h, out_w;
  int stride_h, stride_w;
  int pad_top, pad_left;
} am_conv_geom_t;

/* TF window arithmetic (GetWindowedOutputSizeVerbose): same = 1 -> SAME. */
void am_conv_geometry(int batch, int in_h, int in_w, int in_c, int f_h, int f_w,
                      int out_c, int stride_h, int stride_w, int same,
                      am_conv_geom_t* g);

/* cuda/cuda_kernel.cu:34-60 (im2col) + gemm: order (kh,kw,c). */
void am_conv2d_fwd(const am_conv_geom_t* g, const float* x, const float* w,
                   float* y, const uint8_t* lut, int m);
/* cuda/cuda_kernel.cu:326-353 + gemm :417-427: x is the A operand, the
 * reduction runs over (n,oh,ow) ascending. */
void am_conv2d_bwd_filter(const am_conv_geom_t* g, const float* x,
                          const float* dy, float* dw, const uint8_t* lut, int m);
/* cuda/cuda_kernel.cu:462-502 + cuda/reverseNswapdim23.cu:9-19 + gemm: dy is
 * the A operand, the flipped filter the B operand, order (kh,kw,ko). */
void am_conv2d_bwd_input(const am_conv_geom_t* g, const float* w,
                         const float* dy, float* dx, const uint8_t* lut, int m);

/* cuda/denseam_kernel.cu:18-96 */
void am_dense_fwd(const float* x, const float* w, float* y, int batch,
                  int units, int in_w, const uint8_t* lut, int m);
void am_dense_bwd_weight(const float* x, const float* g, float* dw, int batch,
                         int units, int in_w, const uint8_t* lut, int m);
void am_dense_bwd_input(const float* w, const float* g, float* dx, int batch,
                        int units, int in_w, const uint8_t* lut, int m);

/* cuda/matmulam_kernel.cu:11-99 — batch 0 means "rank-2 operand", batch 1
 * broadcasts.  Every output batch is computed (the reference leaves all but
 * the first uninitialised when batch_a == 1 < batch_b). */
void am_matmul(const float* a, const float* b, float* c, int batch_a,
               int batch_b, int row_a, int col_a, int col_b, const uint8_t* lut,
               int m);

/* ---- T = int32 (cuda/gemm.cu:64-67, cuda/denseam_kernel.cu:146-151) ---------
 * The reference instantiates its kernels for int32 as well: operands are
 * converted to float for the multiplier and the int32 accumulator is updated
 * as  acc = (int32)((float)acc + product)  at every step (float -> int
 * conversion truncates toward zero and, on the GPU, saturates; NaN -> 0). */
void am_gemm_i32(int m, int n, int k, const int32_t* A, int lda, const int32_t* B,
                 int ldb, int32_t* C, int ldc, const uint8_t* lut, int mw);
void am_conv2d_fwd_i32(const am_conv_geom_t* g, const int32_t* x, const int32_t* w,
                       int32_t* y, const uint8_t* lut, int m);
void am_conv2d_bwd_filter_i32(const am_conv_geom_t* g, const int32_t* x,
                              const int32_t* dy, int32_t* dw, const uint8_t* lut, int m);
void am_conv2d_bwd_input_i32(const am_conv_geom_t* g, const int32_t* w,
                             const int32_t* dy, int32_t* dx, const uint8_t* lut, int m);

/* ---- reference CPU op path (exact multiply), the timed baseline ---------- */
/* convam.cc:452-491 */
void cpu_conv2d_fwd(const am_conv_geom_t* g, const float* x, const float* w,
                    float* y);
/* convam.cc:639-686 (loop over the dilated gradient, batch innermost) */
void cpu_conv2d_bwd_filter(const am_conv_geom_t* g, const float* x,
                           const float* dy, float* dw);
/* convam.cc:910-954 (with the batch index defect at :931 corrected) */
void cpu_conv2d_bwd_input(const am_conv_geom_t* g, const float* w,
                          const float* dy, float* dx);
/* denseam.cc:64-71, :151-157, :166-173 (outputs zero-filled first) */
void cpu_dense_fwd(const float* x, const float* w, float* y, int batch,
                   int units, int in_w);
void cpu_dense_bwd_weight(const float* x, const float* g, float* dw, int batch,
                          int units, int in_w);
void cpu_dense_bwd_input(const float* w, const float* g, float* dx, int batch,
                         int units, int in_w);
/* matmulam.cc:178-208 */
void cpu_gemm(int m, int n, int k, const float* a, int lda, const float* b,
              int ldb, float* c, int ldc);

/* Number of OpenMP threads the AM oracle functions use (results do not depend
 * on it: every output keeps its own serial chain).  The cpu_* baseline loops
 * are always single-threaded like the reference functors. */
void am_oracle_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif /* AMSIM_ORACLE_H_ */
