// C entry points over the reference's OWN GPU functors (ConvamFunctor, ConvamFilterGradFunctor,
// ConvamInputGradFunctor: convam.h:69-105; Denseam*Functor: denseam.h:7-28; LaunchMatMul:
// matmulam.h:10-18), whose translation units are compiled unmodified from a reference checkout
// by oracle/build_ref_cuda.sh against the stand-in headers in oracle/tf_stub.  Device pointers
// in, device pointers out; every functor synchronises the device itself (cuda_kernel.cu:91-92).
// TEST INFRASTRUCTURE ONLY: the GPU tests use this library to show that the deterministic mode
// of the product is bit-identical to the reference's GPU kernels, and the benchmark times it as
// an extra baseline.  The product never links or loads it.
#define GOOGLE_CUDA 1
#include "convam.h"
#include "denseam.h"
#include "matmulam.h"

using GPUDevice = Eigen::GpuDevice;

// cuda/approx_mul_lut.cu specialises the class inside its own translation unit; the same
// declaration is repeated here so that this unit sees the specialisation it links against.
template <>
class approx_mul_lut<Eigen::GpuDevice> : public approx_mul_lut_base {
 public:
  explicit approx_mul_lut(tensorflow::OpKernelConstruction* context);
  ~approx_mul_lut();
  auto get_mant_mul_lut_text_() -> cudaTextureObject_t& { return mant_mul_lut_text_; }
  auto get_mant_mul_lut_() -> uint8_t* { return mant_mul_lut_cuda_; }
};

extern "C" {

void* ref_cuda_lut_open(const char* path) {
  tensorflow::OpKernelConstruction ctx(path);
  return new approx_mul_lut<GPUDevice>(&ctx);
}

void ref_cuda_lut_close(void* lut) { delete static_cast<approx_mul_lut<GPUDevice>*>(lut); }

// convam.cc:502-595: the op passes an im2col scratch of batch*out_h*out_w * f_h*f_w*in_c elements
void ref_cuda_conv2d_fwd(void* lut, const float* x, const float* w, float* y, float* im2col, int batch, int in_h, int in_w,
                         int in_c, int f_h, int f_w, int out_c, int out_h, int out_w, int stride_h, int stride_w,
                         int pad_top, int pad_left, int padding_enum) {
  GPUDevice d;
  ConvamFunctor<GPUDevice, float>()(d, x, y, batch, out_h, out_w, out_c, stride_w, stride_h, pad_left, pad_top, f_h, f_w,
                                    in_c, in_w, in_h, w, im2col, padding_enum, *static_cast<approx_mul_lut<GPUDevice>*>(lut));
}

// convam.cc:751-866: im2col scratch of f_h*f_w*in_c * batch*out_h*out_w elements
void ref_cuda_conv2d_bwd_filter(void* lut, const float* x, const float* dy, float* dw, float* im2col, int batch, int in_h,
                                int in_w, int in_c, int f_h, int f_w, int out_c, int out_h, int out_w, int stride_h,
                                int stride_w, int pad_top, int pad_left) {
  GPUDevice d;
  ConvamFilterGradFunctor<GPUDevice, float>()(d, x, dy, im2col, in_h, in_w, batch, in_c, out_w, out_h, out_c, pad_left, pad_top,
                                              stride_h, stride_w, f_w, f_h, dw, *static_cast<approx_mul_lut<GPUDevice>*>(lut));
}

// convam.cc:1018-1136: hole = (out - 1) * stride + 1, back pads = f - 1 - pad; scratch: im2col of
// batch*in_h*in_w * f_h*f_w*out_c elements and the reversed filter of f_h*f_w*in_c*out_c
void ref_cuda_conv2d_bwd_input(void* lut, const float* w, const float* dy, float* dx, float* im2col, float* rsfilter,
                               int batch, int in_h, int in_w, int in_c, int f_h, int f_w, int out_c, int out_h, int out_w,
                               int stride_h, int stride_w, int pad_top, int pad_left) {
  GPUDevice d;
  const int hole_h = (out_h - 1) * stride_h + 1, hole_w = (out_w - 1) * stride_w + 1;
  ConvamInputGradFunctor<GPUDevice, float>()(d, dy, im2col, hole_w, hole_h, f_h - 1 - pad_top, f_w - 1 - pad_left, w, rsfilter,
                                             f_h, f_w, out_c, stride_h, stride_w, batch, in_h, in_w, in_c, dx, out_h, out_w,
                                             *static_cast<approx_mul_lut<GPUDevice>*>(lut));
}

void ref_cuda_dense_fwd(void* lut, const float* x, const float* w, float* y, int batch, int units, int input_width) {
  GPUDevice d;
  DenseamFunctor<GPUDevice, float>()(d, x, w, y, batch, units, input_width, *static_cast<approx_mul_lut<GPUDevice>*>(lut));
}

void ref_cuda_dense_bwd_weight(void* lut, const float* x, const float* g, float* dw, int batch, int units, int input_width) {
  GPUDevice d;
  DenseamWeightGradFunctor<GPUDevice, float>()(d, x, g, dw, batch, units, input_width,
                                               *static_cast<approx_mul_lut<GPUDevice>*>(lut));
}

void ref_cuda_dense_bwd_input(void* lut, const float* w, const float* g, float* dx, int batch, int units, int input_width) {
  GPUDevice d;
  DenseamInputGradFunctor<GPUDevice, float>()(d, w, g, dx, batch, units, input_width,
                                              *static_cast<approx_mul_lut<GPUDevice>*>(lut));
}

void ref_cuda_matmul(void* lut, const float* a, const float* b, float* c, int batch_a, int batch_b, int row_a, int col_a,
                     int row_b, int col_b) {
  GPUDevice d;
  LaunchMatMul<GPUDevice, float>()(d, a, b, batch_a, batch_b, row_a, col_a, row_b, col_b, c,
                                   *static_cast<approx_mul_lut<GPUDevice>*>(lut));
}

}  // extern "C"
