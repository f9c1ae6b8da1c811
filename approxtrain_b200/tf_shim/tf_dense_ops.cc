// TensorFlow op hosts for Denseam / DenseamGrad on top of libamsim.so (GPU,
// float).  Registrations as in the reference (denseam.cc:36-57, :177-184).
// Builds into denseam_gpu.so (python/keras/layers/amdenselayer.py:46).
// Not compiled in this repository's test runs: TensorFlow is required.
#include "amsim_tf_common.h"

using namespace tensorflow;  // NOLINT
using amsim_tf::FromAmsim;
using amsim_tf::LutAttr;
using amsim_tf::ModeFlag;
using amsim_tf::StreamOf;

REGISTER_OP("Denseam")
    .Input("input: T")
    .Input("weights: T")
    .Output("output: T")
    .Attr("T: {float, int32}")
    .Attr("mant_mul_lut: string")
    .SetShapeFn([](shape_inference::InferenceContext* c) {
      shape_inference::ShapeHandle in, w;
      TF_RETURN_IF_ERROR(c->WithRank(c->input(0), 2, &in));
      TF_RETURN_IF_ERROR(c->WithRank(c->input(1), 2, &w));
      c->set_output(0, c->Matrix(c->Dim(in, 0), c->Dim(w, 1)));
      return Status::OK();
    });

REGISTER_OP("DenseamGrad")
    .Input("grad: T")
    .Input("input: T")
    .Input("weights: T")
    .Output("grad_input: T")
    .Output("grad_weights: T")
    .Attr("T: {float, int32}")
    .Attr("mant_mul_lut: string");

class AmsimDenseOp : public OpKernel {
 public:
  explicit AmsimDenseOp(OpKernelConstruction* ctx) : OpKernel(ctx), lut_(ctx) {}
  void Compute(OpKernelContext* ctx) override {
    const Tensor& x = ctx->input(0);
    const Tensor& w = ctx->input(1);
    OP_REQUIRES(ctx, x.dims() == 2 && w.dims() == 2 && x.dim_size(1) == w.dim_size(0),
                errors::InvalidArgument("Denseam takes input [batch, width] and weights [width, units]"));
    const int batch = x.dim_size(0), width = x.dim_size(1), units = w.dim_size(1);
    Tensor* y = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({batch, units}), &y));
    if (y->NumElements() == 0) return;
    OP_REQUIRES_OK(ctx, FromAmsim(amsim_dense_fwd(StreamOf(ctx), lut_.get(), x.flat<float>().data(),
                                                  w.flat<float>().data(), y->flat<float>().data(), batch, units, width,
                                                  ModeFlag())));
  }

 private:
  LutAttr lut_;
};

class AmsimDenseGradOp : public OpKernel {
 public:
  explicit AmsimDenseGradOp(OpKernelConstruction* ctx) : OpKernel(ctx), lut_(ctx) {}
  void Compute(OpKernelContext* ctx) override {
    const Tensor& g = ctx->input(0);
    const Tensor& x = ctx->input(1);
    const Tensor& w = ctx->input(2);
    OP_REQUIRES(ctx, x.dims() == 2 && w.dims() == 2 && g.dims() == 2,
                errors::InvalidArgument("DenseamGrad takes rank-2 tensors"));
    const int batch = x.dim_size(0), width = x.dim_size(1), units = w.dim_size(1);
    Tensor *dx = nullptr, *dw = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, x.shape(), &dx));
    OP_REQUIRES_OK(ctx, ctx->allocate_output(1, w.shape(), &dw));
    const size_t ws_bytes = amsim_dense_bwd_weight_workspace(batch, units, width, ModeFlag());
    Tensor ws;
    void* ws_ptr = nullptr;
    if (ws_bytes > 0) {
      OP_REQUIRES_OK(ctx, ctx->allocate_temp(DT_UINT8, TensorShape({static_cast<int64>(ws_bytes) + 256}), &ws));
      uintptr_t p = reinterpret_cast<uintptr_t>(ws.flat<uint8>().data());
      ws_ptr = reinterpret_cast<void*>((p + 255) & ~static_cast<uintptr_t>(255));
    }
    OP_REQUIRES_OK(ctx, FromAmsim(amsim_dense_bwd_weight(StreamOf(ctx), lut_.get(), x.flat<float>().data(),
                                                         g.flat<float>().data(), dw->flat<float>().data(), batch, units,
                                                         width, ws_ptr, ws_bytes, ModeFlag())));
    OP_REQUIRES_OK(ctx, FromAmsim(amsim_dense_bwd_input(StreamOf(ctx), lut_.get(), w.flat<float>().data(),
                                                        g.flat<float>().data(), dx->flat<float>().data(), batch, units,
                                                        width, ModeFlag())));
  }

 private:
  LutAttr lut_;
};

REGISTER_KERNEL_BUILDER(Name("Denseam").Device(DEVICE_GPU).TypeConstraint<float>("T"), AmsimDenseOp);
REGISTER_KERNEL_BUILDER(Name("DenseamGrad").Device(DEVICE_GPU).TypeConstraint<float>("T"), AmsimDenseGradOp);
