// TensorFlow op host for MatMulAM on top of libamsim.so (GPU, float).
// Registration as in the reference (matmulam.cc:48-56); rank rules and error
// texts follow matmulam.cc:86-147.  Builds into matmulam.so
// (python/ops/math_ops.py:8).  Not compiled in this repository's test runs.
#include "amsim_tf_common.h"
#include "tensorflow/core/framework/common_shape_fns.h"

using namespace tensorflow;  // NOLINT
using amsim_tf::FromAmsim;
using amsim_tf::LutAttr;
using amsim_tf::StreamOf;

REGISTER_OP("MatMulAM")
    .Input("a: T")
    .Input("b: T")
    .Output("product: T")
    .Attr("transpose_a: bool = false")
    .Attr("transpose_b: bool = false")
    .Attr("T: {float, int32}")
    .Attr("mant_mul_lut: string")
    .SetShapeFn(shape_inference::MatMulShape);

class AmsimMatMulOp : public OpKernel {
 public:
  explicit AmsimMatMulOp(OpKernelConstruction* ctx) : OpKernel(ctx), lut_(ctx) {}
  void Compute(OpKernelContext* ctx) override {
    const Tensor& a = ctx->input(0);
    const Tensor& b = ctx->input(1);
    OP_REQUIRES(ctx, (a.dims() == 2 || a.dims() == 3) && (b.dims() == 2 || b.dims() == 3),
                errors::InvalidArgument(
                    "Input a and b should be 2 dimensional or 3 dimensional and compitable batch size"));
    const int ba = a.dims() == 3 ? a.dim_size(0) : 0, bb = b.dims() == 3 ? b.dim_size(0) : 0;
    const int m = a.dim_size(a.dims() - 2), k = a.dim_size(a.dims() - 1);
    const int kb = b.dim_size(b.dims() - 2), n = b.dim_size(b.dims() - 1);
    OP_REQUIRES(ctx, k == kb, errors::InvalidArgument("Does not meet cols of mat a is equal rows of mat b"));
    OP_REQUIRES(ctx, ba == 0 || bb == 0 || ba == bb || ba == 1 || bb == 1,
                errors::InvalidArgument("Does not meet batch of mat a is equal batch of matb"));
    const int nb = std::max(ba, bb);
    Tensor* out = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, nb ? TensorShape({nb, m, n}) : TensorShape({m, n}), &out));
    if (out->NumElements() == 0) return;
    OP_REQUIRES_OK(ctx, FromAmsim(amsim_matmul(StreamOf(ctx), lut_.get(), a.flat<float>().data(),
                                               b.flat<float>().data(), out->flat<float>().data(), ba, bb, m, k, kb, n,
                                               AMSIM_FAST)));
  }

 private:
  LutAttr lut_;
};

REGISTER_KERNEL_BUILDER(Name("MatMulAM").Device(DEVICE_GPU).TypeConstraint<float>("T"), AmsimMatMulOp);
