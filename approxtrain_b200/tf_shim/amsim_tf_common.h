// Shared pieces of the TensorFlow op hosts that put libamsim.so behind the
// reference's op names.  NOT built by default: TensorFlow headers are needed
// (see Makefile in this directory).  The ops keep the reference's
// registrations byte for byte (names, inputs, attrs, shape functions), so
// python/ops/amnn_ops.py, python/keras/layers/amdenselayer.py and
// python/ops/math_ops.py load these libraries unchanged.
#ifndef AMSIM_TF_COMMON_H_
#define AMSIM_TF_COMMON_H_

#define EIGEN_USE_GPU
#include <stdlib.h>

#include <string>

#include "amsim.h"
#include "tensorflow/core/framework/op.h"
#include "tensorflow/core/framework/op_kernel.h"
#include "tensorflow/core/framework/shape_inference.h"
#include "tensorflow/core/util/padding.h"
#include "tensorflow/core/util/tensor_format.h"

namespace amsim_tf {

using tensorflow::OpKernelConstruction;
using tensorflow::OpKernelContext;
using tensorflow::errors::Internal;
using tensorflow::errors::InvalidArgument;

// Owns one reference to the device LUT named by the op's `mant_mul_lut` attr
// (the role of approx_mul_lut<GPUDevice>, approx_mul_lut.h:75-80).
class LutAttr {
 public:
  explicit LutAttr(OpKernelConstruction* ctx) {
    std::string path;
    OP_REQUIRES_OK(ctx, ctx->GetAttr("mant_mul_lut", &path));
    int device = 0;
    cudaGetDevice(&device);
    const int rc = amsim_lut_open(path.c_str(), device, &lut_);
    OP_REQUIRES(ctx, rc == AMSIM_OK, InvalidArgument("mant_mul_lut: ", amsim_last_error()));
  }
  ~LutAttr() { amsim_lut_close(lut_); }
  LutAttr(const LutAttr&) = delete;
  LutAttr& operator=(const LutAttr&) = delete;
  const amsim_lut* get() const { return lut_; }

 private:
  amsim_lut* lut_ = nullptr;
};

// AMSIM_FAST unless the process environment holds AMSIM_TF_DETERMINISTIC=1 when the first op runs:
// then every op takes the reference's exact summation order (AMSIM_DETERMINISTIC), bit-identical
// to the reference's GPU kernels.  Read once; the ops are registered for T = float only (the
// reference's int32 registrations are served by the C ABI's AMSIM_INT32 flag, not by these hosts).
inline unsigned ModeFlag() {
  static const unsigned flag = [] {
    const char* e = getenv("AMSIM_TF_DETERMINISTIC");
    return (e && *e && *e != '0') ? (unsigned)AMSIM_DETERMINISTIC : (unsigned)AMSIM_FAST;
  }();
  return flag;
}

inline void* StreamOf(OpKernelContext* ctx) {
  return reinterpret_cast<void*>(ctx->eigen_device<Eigen::GpuDevice>().stream());
}

inline tensorflow::Status FromAmsim(int rc) {
  if (rc == AMSIM_OK) return tensorflow::Status::OK();
  if (rc == AMSIM_ERR_INVALID) return InvalidArgument(amsim_last_error());
  return Internal(amsim_last_error());
}

}  // namespace amsim_tf
#endif  // AMSIM_TF_COMMON_H_
