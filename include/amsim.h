/*
 * amsim — C ABI of the B200 (sm_100a) AM-Simulator kernels.
 *
 * Drop-in boundary for ApproxTrain's GPU functors: each entry point below
 * replaces one functor that the reference's TensorFlow op hosts call
 * (convam.h / denseam.h / matmulam.h / approx_mul_lut.h), with the same
 * argument meaning.  Differences that hold for every call:
 *
 *   - plain C types only; all tensor pointers are DEVICE pointers to FP32
 *     data owned by the caller (NHWC activations, HWIO filters, row-major
 *     matrices), the LUT handle owns its own device memory;
 *   - `stream` is a cudaStream_t passed as void*; calls are stream-ordered,
 *     never synchronise the device and never exit the process (the reference
 *     calls cudaDeviceSynchronize after every launch and exit(1) on error,
 *     cuda/error.cuh:11-27);
 *   - the return value is an AMSIM_* status; amsim_last_error() gives the text
 *     of the calling thread's last failure;
 *   - no im2col or reversed-filter scratch is needed (convam.h:69-105 take
 *     `im2col` and `rsfilter` buffers): the gathers are index maps inside the
 *     kernels.  Only the split-K gradient kernels use caller-provided scratch.
 *
 * `flags`:
 *   AMSIM_FAST           default.  Products equal the reference primitive
 *                        except where an operand has a zero exponent field
 *                        (product taken as 0) or the exponent sum is <= 127
 *                        (reference returns 0, here the exact tiny product,
 *                        < 2^-125); each forward / input-gradient output is one
 *                        ascending-k FP32 chain like the reference kernel, the
 *                        filter / weight gradients are split along the
 *                        reduction and summed in a fixed order, and so are
 *                        forward / input-gradient outputs of shapes with too
 *                        few output tiles to fill the GPU (thread-block clusters
 *                        share a tile's reduction).  Run-to-run identical.
 *   AMSIM_DETERMINISTIC  every product is the reference primitive bit for bit
 *                        (cuda/AMsimulator.inl:13-36) and every output is one
 *                        ascending chain in the reference's order
 *                        (cuda/gemm.cu:30-53): results are bit-identical to the
 *                        reference GPU kernels.  Slower.
 */
#ifndef AMSIM_H_
#define AMSIM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AMSIM_OK 0
#define AMSIM_ERR_INVALID 1      /* null pointer, bad shape, bad flag */
#define AMSIM_ERR_LUT_NAME 2     /* mantissa width not parseable / out of 1..11 */
#define AMSIM_ERR_LUT_IO 3       /* file cannot be opened or read */
#define AMSIM_ERR_LUT_SIZE 4     /* file is not exactly 2^(2m) bytes */
#define AMSIM_ERR_CUDA 5         /* a CUDA runtime call failed */
#define AMSIM_ERR_WORKSPACE 6    /* scratch buffer missing or too small */
#define AMSIM_ERR_UNSUPPORTED 7  /* valid request this build cannot serve */

#define AMSIM_FAST 0u
#define AMSIM_DETERMINISTIC 1u
/* Tensors are int32 instead of float (the reference registers Convam*, Denseam*
 * for T in {float, int32}: convam.cc:604-621, denseam.cc:126-143).  Pass the
 * int32 pointers through the float* parameters.  Semantics of the reference's
 * int32 kernels (cuda/gemm.cu:49,64-67): operands converted to float for the
 * multiplier, accumulator updated as (int)((float)acc + product) per step.
 * Unoptimised (one thread per output); implies the reference's order. */
#define AMSIM_INT32 2u

typedef struct amsim_lut amsim_lut; /* opaque, immutable after open */

/* Text of the calling thread's most recent failure ("" if none). */
const char* amsim_last_error(void);

/* Library version string and the SM architecture the kernels were built for. */
const char* amsim_version(void);

/* ---- LUT ------------------------------------------------------------------
 * Replaces approx_mul_lut_base::load_lut_binary (approx_mul_lut.h:15-45) and
 * approx_mul_lut<GpuDevice> (cuda/approx_mul_lut.cu:24-53).  `path` is the
 * op's `mant_mul_lut` attribute: "<MODEL>_<m>.bin", m = digits between the
 * last '_' and the last '.', file = 2^(2m) raw bytes.  Handles are cached per
 * (real path, device) and reference counted; close drops one reference.
 * The file must hold exactly 2^(2m) bytes (the reference reads "up to").
 * For m <= 7 the GEMM kernels keep the table in shared memory; for m = 8..11
 * (up to 4 MiB) they look it up in global memory, where it stays L2-resident.
 * A table whose entries satisfy (carry << m) + mantissa == i + j for every
 * index pair (Mitchell's logarithmic multiplier, e.g. MIT_7) needs no lookups:
 * the kernels add the operands' mantissa fields instead, with identical bits
 * (set AMSIM_NO_ADDITIVE in the environment before opening to force the table).
 *
 * Format extension (no reference counterpart): a file of exactly 2 * 2^(2m) bytes
 * under the same name holds 16-bit little-endian entries, carry << 15 | top 15
 * mantissa bits of the product.  A byte keeps 7 mantissa bits, so byte tables for
 * m = 8..11 drop the product's leading bits; 16-bit entries keep them
 * (approxtrain_b200/lutgen.py writes both formats).  Looked up in global memory,
 * FP32 ops only; amsim_lut_info reports the same m, mask and shifts.
 *
 * Two pseudo-paths select the reference's direct C simulation of its 32-bit
 * multipliers (mantissa width 23, README.md:107: "for multipliers with mantissa
 * bit-width greater or equal to 12, direct C simulation should be used"):
 *   "direct:MBM32"  cuda/FPmultMBM_fast32.inl:41-126 (FMBM32_MULTIPLIER)
 *   "direct:MIT32"  cuda/Mitchell_32.inl (MITCHEL23_MULTIPLIER)
 * No file is read; every product is computed arithmetically inside the same GEMM
 * kernels (sign/exponent of the exact FP32 product, approximate mantissa, inf/NaN
 * passed through, zero/subnormal products flushed to +0).  Both accumulate in the
 * reference's order whatever the mode flag says; FP32 only. */
int amsim_lut_open(const char* path, int device, amsim_lut** out);
/* Same, from bytes already in host memory (m given explicitly). */
int amsim_lut_open_bytes(const uint8_t* bytes, int m, int device, amsim_lut** out);
int amsim_lut_close(amsim_lut* lut);
/* approx_mul_lut.h:53-70 getters: mantissa width, mask, shifts; the raw LUT
 * bytes on the device (what the reference binds to its texture object). */
int amsim_lut_info(const amsim_lut* lut, int* mant_width, uint32_t* mant_mask,
                   int* a_shift, int* b_shift, const uint8_t** device_bytes);

/* ---- the primitive ----------------------------------------------------------
 * out[i] = AMsimulator(a[i], b[i]) — cuda/AMsimulator.inl:13-36, bit-exact,
 * every m in 1..11.  The reference has no elementwise op; this exposes the
 * primitive the GEMM kernels are built on so it can be checked on its own. */
int amsim_mul(void* stream, const amsim_lut* lut, const float* a, const float* b,
              float* out, size_t n);

/* ---- convolution geometry -----------------------------------------------------
 * TF window arithmetic used by ConvamOp::Compute (convam.cc:315-407) and the
 * filter_left/top_offset derivation (convam.cc:557-572): same != 0 -> SAME.
 * pad_top / pad_left are the forward pad-before amounts (0 for VALID). */
int amsim_conv2d_geometry(int in_h, int in_w, int f_h, int f_w, int stride_h,
                          int stride_w, int same, int* out_h, int* out_w,
                          int* pad_top, int* pad_left);

/* ---- AMConv2D -------------------------------------------------------------------
 * Forward: replaces ConvamFunctor<GPUDevice> (convam.h:69-80,
 * cuda/cuda_kernel.cu:100-321).  y[n,oh,ow,k] = sum over (kh,kw,c) of
 * AM(x[n, oh*sh - pad_top + kh, ow*sw - pad_left + kw, c] or 0, w[kh,kw,c,k]). */
int amsim_conv2d_fwd(void* stream, const amsim_lut* lut, const float* x,
                     const float* w, float* y, int batch, int in_h, int in_w,
                     int in_c, int f_h, int f_w, int out_c, int out_h, int out_w,
                     int stride_h, int stride_w, int pad_top, int pad_left,
                     unsigned flags);

/* Forward with the layer's exact epilogue fused in: y = act(conv(x, w) + bias).
 * In the reference the bias add and the activation are separate TensorFlow ops
 * after Convam / Denseam (python/keras/layers/am_convolutional.py:267-292,
 * amdenselayer.py:222-226); here they run in the kernel's epilogue with the
 * same arithmetic (one FP32 add per output, then max with 0), so the result
 * equals the unfused sequence bit for bit.  `bias` (out_c floats) may be NULL;
 * `act`: 0 = none, 1 = ReLU.  FP32 only. */
#define AMSIM_ACT_NONE 0
#define AMSIM_ACT_RELU 1
int amsim_conv2d_fwd_bias_act(void* stream, const amsim_lut* lut, const float* x,
                              const float* w, const float* bias, float* y, int batch,
                              int in_h, int in_w, int in_c, int f_h, int f_w, int out_c,
                              int out_h, int out_w, int stride_h, int stride_w,
                              int pad_top, int pad_left, int act, unsigned flags);
int amsim_dense_fwd_bias_act(void* stream, const amsim_lut* lut, const float* x,
                             const float* w, const float* bias, float* y, int batch,
                             int units, int input_width, int act, unsigned flags);

/* The same with a per-output-channel factor first: y = act(conv(x, w) * scale[k] + bias[k]),
 * one FP32 multiply, one FP32 add, then the activation.  This is an inference-time
 * BatchNormalization folded behind the convolution (the reference applies Keras
 * BatchNormalization as a separate exact layer after AMConv2D, e.g.
 * profile/resnet50_lut.py:568-718): scale = gamma / sqrt(var + eps),
 * bias = beta - mean * scale.  `scale` and `bias` (out_c floats each) may be NULL.  No
 * reference counterpart as a fused op; equals the unfused sequence bit for bit. */
int amsim_conv2d_fwd_scale_bias_act(void* stream, const amsim_lut* lut, const float* x,
                                    const float* w, const float* scale, const float* bias,
                                    float* y, int batch, int in_h, int in_w, int in_c,
                                    int f_h, int f_w, int out_c, int out_h, int out_w,
                                    int stride_h, int stride_w, int pad_top, int pad_left,
                                    int act, unsigned flags);

/* Input gradient: replaces ConvamInputGradFunctor<GPUDevice> (convam.h:82-93,
 * cuda/cuda_kernel.cu:462-657) including cuda/reverseNswapdim23.cu.  The
 * functor's hole_grad_* and back-pad arguments are derived here from the
 * forward geometry (convam.cc:1066-1084). */
int amsim_conv2d_bwd_input(void* stream, const amsim_lut* lut, const float* w,
                           const float* dy, float* dx, int batch, int in_h,
                           int in_w, int in_c, int f_h, int f_w, int out_c,
                           int out_h, int out_w, int stride_h, int stride_w,
                           int pad_top, int pad_left, unsigned flags);

/* Filter gradient: replaces ConvamFilterGradFunctor<GPUDevice>
 * (convam.h:95-105, cuda/cuda_kernel.cu:326-461).  AMSIM_FAST splits the
 * N*OH*OW reduction over thread blocks and needs `workspace` of at least
 * amsim_conv2d_bwd_filter_workspace(...) bytes (device memory, 256-byte
 * aligned, contents irrelevant on entry, clobbered on return; 0 bytes means
 * none needed and NULL is accepted). */
size_t amsim_conv2d_bwd_filter_workspace(int batch, int in_h, int in_w, int in_c,
                                         int f_h, int f_w, int out_c, int out_h,
                                         int out_w, unsigned flags);
int amsim_conv2d_bwd_filter(void* stream, const amsim_lut* lut, const float* x,
                            const float* dy, float* dw, int batch, int in_h,
                            int in_w, int in_c, int f_h, int f_w, int out_c,
                            int out_h, int out_w, int stride_h, int stride_w,
                            int pad_top, int pad_left, void* workspace,
                            size_t workspace_bytes, unsigned flags);

/* Filter gradient for callers that cannot hand over scratch memory.
 * (No counterpart in the reference: its functor takes the scratch from the
 * TensorFlow allocator.)
 *
 * Same computation, same split plan and therefore bit-identical results as
 * amsim_conv2d_bwd_filter, but the split-K partial sums live in a buffer that
 * is part of the library image on the device (AMSIM_STATIC_SCRATCH_BYTES,
 * resident on every GPU that loads the library until the process exits)
 * instead of a caller-supplied workspace.  It is meant for hosts that have no
 * way to allocate at the point of the call: a plain C driver without a device
 * allocator, an op host whose framework offers no temporary tensors there, or
 * stream-ordered code that must not call cudaMalloc because that call
 * synchronises the whole device.  The call itself performs no cudaMalloc /
 * cudaFree and calls nothing that allocates device memory.
 *
 *  - A shape whose plan needs more than AMSIM_STATIC_SCRATCH_BYTES is refused
 *    with AMSIM_ERR_WORKSPACE (nothing is launched); use the workspace variant.
 *  - The first call on a device looks up the buffer's device address
 *    (cudaGetSymbolAddress); make that first call before starting any stream
 *    capture on that device.
 *  - The buffer is shared by every call in the process and keeps whatever the
 *    previous call left in it.  Nothing in it has to start at zero: every
 *    partial sum a call reads back was written by that same call.  Two calls
 *    that may run at the same time on one GPU (different streams or threads)
 *    would overwrite each other's partial sums: serialise them. */
#define AMSIM_STATIC_SCRATCH_BYTES (8u << 20)
int amsim_conv2d_bwd_filter_static(void* stream, const amsim_lut* lut, const float* x,
                                   const float* dy, float* dw, int batch, int in_h,
                                   int in_w, int in_c, int f_h, int f_w, int out_c,
                                   int out_h, int out_w, int stride_h, int stride_w,
                                   int pad_top, int pad_left, unsigned flags);

/* ---- denseam ---------------------------------------------------------------------
 * Replace DenseamFunctor / DenseamWeightGradFunctor / DenseamInputGradFunctor
 * (denseam.h:7-28, cuda/denseam_kernel.cu:18-145).  x[batch,input_width],
 * w[input_width,units], y and g [batch,units], all row-major. */
int amsim_dense_fwd(void* stream, const amsim_lut* lut, const float* x,
                    const float* w, float* y, int batch, int units,
                    int input_width, unsigned flags);
size_t amsim_dense_bwd_weight_workspace(int batch, int units, int input_width,
                                        unsigned flags);
int amsim_dense_bwd_weight(void* stream, const amsim_lut* lut, const float* x,
                           const float* g, float* dw, int batch, int units,
                           int input_width, void* workspace,
                           size_t workspace_bytes, unsigned flags);
int amsim_dense_bwd_input(void* stream, const amsim_lut* lut, const float* w,
                          const float* g, float* dx, int batch, int units,
                          int input_width, unsigned flags);

/* ---- MatMulAM ----------------------------------------------------------------------
 * Replaces LaunchMatMul<GpuDevice> (matmulam.h:10-18,
 * cuda/matmulam_kernel.cu:11-99) with one launch for all batches.
 * batch_* == 0 means the operand is rank 2; batch 1 broadcasts; when both are
 * > 1 they must be equal (matmulam.cc:93).  col_a must equal row_b.  Output is
 * [max(batch_a,batch_b,1)] x row_a x col_b.  Every output batch is computed
 * (the reference computes only the first when batch_a == 1 < batch_b). */
int amsim_matmul(void* stream, const amsim_lut* lut, const float* a,
                 const float* b, float* c, int batch_a, int batch_b, int row_a,
                 int col_a, int row_b, int col_b, unsigned flags);

/* MatMulAM with the transposes done by the kernel's index maps and an optional scalar
 * factor.  The reference op declares transpose_a / transpose_b but its kernel ignores them
 * (matmulam.cc:48-56, cuda/matmulam_kernel.cu:11-99), so its Python wrapper materialises the
 * transposed operand first (python/ops/math_ops.py:82-93); here row_* / col_* describe the
 * operands AS STORED and transpose_* says to read them transposed in place:
 *   C = alpha * op(A) x op(B),  op(X) = X^T when transpose_x != 0.
 * Products are AM(op(A)[i,k], op(B)[k,j]) summed over ascending k as in amsim_matmul.
 * `alpha` (host pointer, may be NULL) multiplies every finished sum once in FP32: the
 * 1/sqrt(d_k) of scaled dot-product attention (ammha/multihead_attention.py:18-30). */
int amsim_matmul_ex(void* stream, const amsim_lut* lut, const float* a, const float* b,
                    float* c, int batch_a, int batch_b, int row_a, int col_a, int row_b,
                    int col_b, int transpose_a, int transpose_b, const float* alpha,
                    unsigned flags);

/* Bias gradient: dbias[c] = sum over rows of grad[row][c] for a row-major rows x cols gradient
 * (NHWC output gradient: rows = batch * out_h * out_w, cols = channels; dense: rows = batch).  An
 * exact FP32 sum in a fixed order (the same bits on every run), bound by one read of `grad`.  In
 * the reference this is TensorFlow's stock BiasAddGrad behind the Keras layers' bias add
 * (python/keras/layers/am_convolutional.py:267-292, amdenselayer.py:222-226), not part of its
 * custom ops; it is here because it sits between the AM ops of every training step.
 * `workspace`: amsim_bias_grad_workspace(rows, cols) bytes of device scratch, 16-byte aligned. */
size_t amsim_bias_grad_workspace(long long rows, int cols);
int amsim_bias_grad(void* stream, const float* grad, float* dbias, long long rows, int cols,
                    void* workspace, size_t workspace_bytes);

/* Number of kernels this library has launched since it was loaded (all devices, all
 * streams).  For benchmarks that report their launch count; no reference counterpart. */
unsigned long long amsim_debug_launch_count(void);

/* The debug switches (environment variables AMSIM_*, listed in INTEGRATION.md) are read once,
 * when an entry point first needs one; they are never read on the launch path, so a *_workspace
 * query and the launch that follows it see the same plan.  This call re-reads them.  Meant for
 * tests that change a switch between two calls; not safe against launches running in other
 * threads.  No reference counterpart. */
void amsim_debug_reload_env(void);

/* Bounds-checking debug build (compiled with -DAMSIM_BOUNDS_CHECK; the stand-in for a device-side
 * memory checker): every access of the kernels to a caller's tensor or to scratch is compared with
 * the buffer's extent and alignment before it is made; a bad one is skipped and the first is
 * recorded.  This call waits for the device, returns that record in *word (0 = every access since
 * the last call was in bounds; otherwise source line << 44 | (buffer + 1) << 40 | byte offset, buffers
 * 0 lane operand, 1 uniform operand, 2 output, 3 scratch) and clears it.  A normal build returns
 * AMSIM_ERR_UNSUPPORTED and *word = 0.  No reference counterpart. */
int amsim_debug_bounds_report(unsigned long long* word);

/* Host-side check of the kernels' constant-divisor arithmetic (no GPU work):
 * returns n / d computed the way the device code does.  For tests. */
uint32_t amsim_debug_fastdiv(uint32_t n, uint32_t d);

#ifdef __cplusplus
}
#endif
#endif /* AMSIM_H_ */
