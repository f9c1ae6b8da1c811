// TensorFlow op host for MatMulAM on top of libamsim.so (GPU, float).
// Inputs, output and attrs as in the reference's registration (matmulam.cc:48-56); error
// texts follow matmulam.cc:86-147.  Builds into matmulam.so (python/ops/math_ops.py:8).
// Not compiled in this repository's test runs.
//
// Two things go beyond the reference's kernel, both supersets of its behaviour:
//  * transpose_a / transpose_b are honoured (the reference's kernel ignores them and its
//    Python wrapper materialises the transposes before the op, math_ops.py:82-93, so the
//    unmodified wrapper always passes false and sees no difference);
//  * operands of rank > 3 with equal leading axes are accepted and folded into the batch
//    (ammha/multihead_attention.py:18,30 passes [batch, heads, seq, depth]); the shape
//    function below equals MatMulShape for rank-2 operands.
#include <algorithm>

#include "amsim_tf_common.h"
#include "tensorflow/core/framework/common_shape_fns.h"

using namespace tensorflow;  // NOLINT
using amsim_tf::FromAmsim;
using amsim_tf::LutAttr;
using amsim_tf::ModeFlag;
using amsim_tf::StreamOf;

static Status MatMulAMShape(shape_inference::InferenceContext* c) {
  using shape_inference::DimensionHandle;
  using shape_inference::ShapeHandle;
  ShapeHandle a = c->input(0), b = c->input(1);
  if (!c->RankKnown(a) || !c->RankKnown(b)) {
    c->set_output(0, c->UnknownShape());
    return Status::OK();
  }
  const int ra = c->Rank(a), rb = c->Rank(b);
  if (ra < 2 || rb < 2) return errors::InvalidArgument("Input a and b should be 2 dimensional or 3 dimensional and compitable batch size");
  bool ta = false, tb = false;
  TF_RETURN_IF_ERROR(c->GetAttr("transpose_a", &ta));
  TF_RETURN_IF_ERROR(c->GetAttr("transpose_b", &tb));
  DimensionHandle m = c->Dim(a, ta ? ra - 1 : ra - 2), ka = c->Dim(a, ta ? ra - 2 : ra - 1);
  DimensionHandle kb = c->Dim(b, tb ? rb - 1 : rb - 2), n = c->Dim(b, tb ? rb - 2 : rb - 1);
  DimensionHandle merged;
  TF_RETURN_IF_ERROR(c->Merge(ka, kb, &merged));
  ShapeHandle lead;
  TF_RETURN_IF_ERROR(c->Subshape(ra >= rb ? a : b, 0, -2, &lead));
  ShapeHandle out;
  TF_RETURN_IF_ERROR(c->Concatenate(lead, c->Matrix(m, n), &out));
  c->set_output(0, out);
  return Status::OK();
}

REGISTER_OP("MatMulAM")
    .Input("a: T")
    .Input("b: T")
    .Output("product: T")
    .Attr("transpose_a: bool = false")
    .Attr("transpose_b: bool = false")
    .Attr("T: {float, int32}")
    .Attr("mant_mul_lut: string")
    .SetShapeFn(MatMulAMShape);

class AmsimMatMulOp : public OpKernel {
 public:
  explicit AmsimMatMulOp(OpKernelConstruction* ctx) : OpKernel(ctx), lut_(ctx) {
    OP_REQUIRES_OK(ctx, ctx->GetAttr("transpose_a", &ta_));
    OP_REQUIRES_OK(ctx, ctx->GetAttr("transpose_b", &tb_));
  }
  void Compute(OpKernelContext* ctx) override {
    const Tensor& a = ctx->input(0);
    const Tensor& b = ctx->input(1);
    const int ra = a.dims(), rb = b.dims();
    OP_REQUIRES(ctx, ra >= 2 && rb >= 2,
                errors::InvalidArgument(
                    "Input a and b should be 2 dimensional or 3 dimensional and compitable batch size"));
    // leading axes fold into one batch count; 0 = rank-2 operand (broadcast)
    auto batch_of = [](const Tensor& t) {
      int64 n = 1;
      for (int i = 0; i + 2 < t.dims(); ++i) n *= t.dim_size(i);
      return t.dims() > 2 ? static_cast<int>(n) : 0;
    };
    const int ba = batch_of(a), bb = batch_of(b);
    if (ra > 3 || rb > 3) {
      bool same = ra == rb;
      for (int i = 0; same && i + 2 < ra; ++i) same = a.dim_size(i) == b.dim_size(i);
      OP_REQUIRES(ctx, same, errors::InvalidArgument("operands of rank > 3 need equal leading axes"));
    }
    const int row_a = a.dim_size(ra - 2), col_a = a.dim_size(ra - 1);
    const int row_b = b.dim_size(rb - 2), col_b = b.dim_size(rb - 1);
    const int m = ta_ ? col_a : row_a, k = ta_ ? row_a : col_a;
    const int kb = tb_ ? col_b : row_b, n = tb_ ? row_b : col_b;
    OP_REQUIRES(ctx, k == kb, errors::InvalidArgument("Does not meet cols of mat a is equal rows of mat b"));
    OP_REQUIRES(ctx, ba == 0 || bb == 0 || ba == bb || ba == 1 || bb == 1,
                errors::InvalidArgument("Does not meet batch of mat a is equal batch of matb"));
    TensorShape shape;
    const Tensor& lead = ra >= rb ? a : b;
    for (int i = 0; i + 2 < lead.dims(); ++i) shape.AddDim(lead.dim_size(i));
    shape.AddDim(m);
    shape.AddDim(n);
    Tensor* out = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, shape, &out));
    if (out->NumElements() == 0) return;
    OP_REQUIRES_OK(ctx, FromAmsim(amsim_matmul_ex(StreamOf(ctx), lut_.get(), a.flat<float>().data(),
                                                  b.flat<float>().data(), out->flat<float>().data(), ba, bb, row_a,
                                                  col_a, row_b, col_b, ta_ ? 1 : 0, tb_ ? 1 : 0, /*alpha=*/nullptr,
                                                  ModeFlag())));
  }

 private:
  LutAttr lut_;
  bool ta_ = false, tb_ = false;
};

REGISTER_KERNEL_BUILDER(Name("MatMulAM").Device(DEVICE_GPU).TypeConstraint<float>("T"), AmsimMatMulOp);
