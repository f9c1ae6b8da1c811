/* Stand-in for the few TensorFlow / Eigen names the reference's CUDA translation units
 * mention (cuda/gemm.cu, cuda/cuda_kernel.cu, cuda/denseam_kernel.cu, cuda/matmulam_kernel.cu,
 * cuda/approx_mul_lut.cu, approx_mul_lut.h): the int32 typedef, an OpKernelConstruction that
 * hands out the "mant_mul_lut" attribute, and a GpuDevice that carries a stream.  With these
 * the reference's own kernels and launchers compile with nvcc straight from a reference
 * checkout (oracle/build_ref_cuda.sh); nothing of TensorFlow itself is needed or used.
 * TEST INFRASTRUCTURE ONLY. */
#ifndef AMSIM_ORACLE_TF_STUB_H_
#define AMSIM_ORACLE_TF_STUB_H_
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <cmath>
#include <iostream>
#include <string>
#include <vector>

namespace tensorflow {
typedef int int32;
typedef unsigned int uint32;
struct Status {
  bool ok() const { return true; }
};
class OpKernelConstruction {
 public:
  explicit OpKernelConstruction(const std::string& lut_file) : lut_file_(lut_file) {}
  Status GetAttr(const char*, std::string* value) const {
    *value = lut_file_;
    return Status();
  }

 private:
  std::string lut_file_;
};
}  // namespace tensorflow

#define OP_REQUIRES_OK(CTX, EXPR) \
  do {                            \
    (void)(CTX);                  \
    (void)(EXPR);                 \
  } while (0)

namespace Eigen {
struct GpuDevice {
  cudaStream_t stream_ = 0;
  cudaStream_t stream() const { return stream_; }
};
struct ThreadPoolDevice {};
}  // namespace Eigen
#endif
