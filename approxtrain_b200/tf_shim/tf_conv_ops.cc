// TensorFlow op hosts for Convam / ConvamInputGrad / ConvamFilterGrad on top of
// libamsim.so (GPU, float).  Registrations are those of the reference
// (convam.cc:427-437, :690-707, :958-975); the kernels only derive the window
// geometry and call the C ABI.  Builds into convam_gpu.so (the name
// python/ops/amnn_ops.py:40 loads).  Not compiled in this repository's test
// runs: TensorFlow is required.
#include "amsim_tf_common.h"
#include "tensorflow/core/framework/common_shape_fns.h"

using namespace tensorflow;  // NOLINT
using amsim_tf::FromAmsim;
using amsim_tf::LutAttr;
using amsim_tf::ModeFlag;
using amsim_tf::StreamOf;

namespace {

struct Window {
  int stride_h = 1, stride_w = 1;
  bool same = false;
};

// strides / dilations / padding / data_format attrs, NHWC only, no dilation.
Status ReadWindow(OpKernelConstruction* ctx, Window* w) {
  std::vector<int32> strides, dilations;
  std::string format;
  Padding padding;
  TF_RETURN_IF_ERROR(ctx->GetAttr("strides", &strides));
  TF_RETURN_IF_ERROR(ctx->GetAttr("dilations", &dilations));
  TF_RETURN_IF_ERROR(ctx->GetAttr("data_format", &format));
  TF_RETURN_IF_ERROR(ctx->GetAttr("padding", &padding));
  if (format != "NHWC") return errors::InvalidArgument("AM convolution supports NHWC only");
  if (strides.size() != 4 || strides[0] != 1 || strides[3] != 1 || strides[1] < 1 || strides[2] < 1)
    return errors::InvalidArgument("strides must be [1, sh, sw, 1] with positive sh, sw");
  if (dilations.size() != 4 || dilations[1] != 1 || dilations[2] != 1)
    return errors::InvalidArgument("Dilation is not supported in current implementation");
  w->stride_h = strides[1];
  w->stride_w = strides[2];
  w->same = padding == Padding::SAME;
  return Status::OK();
}

struct Geometry {
  int n, h, w, c, kh, kw, k, oh, ow, pt, pl;
};

Status MakeGeometry(const Window& win, const TensorShape& in, const TensorShape& filter, Geometry* g) {
  if (in.dims() != 4) return errors::InvalidArgument("input must be 4-dimensional", in.DebugString());
  if (filter.dims() != 4) return errors::InvalidArgument("filter must be 4-dimensional: ", filter.DebugString());
  g->n = in.dim_size(0); g->h = in.dim_size(1); g->w = in.dim_size(2); g->c = in.dim_size(3);
  g->kh = filter.dim_size(0); g->kw = filter.dim_size(1); g->k = filter.dim_size(3);
  if (filter.dim_size(2) != g->c) return errors::InvalidArgument("input depth must match filter depth");
  return FromAmsim(amsim_conv2d_geometry(g->h, g->w, g->kh, g->kw, win.stride_h, win.stride_w, win.same ? 1 : 0,
                                         &g->oh, &g->ow, &g->pt, &g->pl));
}

Status ShapeFromInt32Vector(const Tensor& t, TensorShape* out) {
  if (!TensorShapeUtils::IsVector(t.shape()) || t.NumElements() != 4)
    return errors::InvalidArgument("sizes input must be a 1-D tensor with 4 elements");
  auto v = t.vec<int32>();
  *out = TensorShape({v(0), v(1), v(2), v(3)});
  return Status::OK();
}

}  // namespace

REGISTER_OP("Convam")
    .Input("input: T")
    .Input("filter: T")
    .Output("output: T")
    .Attr("T: {float, int32}")
    .Attr("strides: list(int)")
    .Attr("dilations: list(int) = [1, 1, 1, 1]")
    .Attr("mant_mul_lut: string")
    .Attr(GetPaddingAttrString())
    .Attr(GetConvnetDataFormatAttrString())
    .SetShapeFn(shape_inference::Conv2DShape);

REGISTER_OP("ConvamFilterGrad")
    .Input("filter_sizes: int32")
    .Input("input: T")
    .Input("out_backprop: T")
    .Output("grad_filter: T")
    .Attr("T: {float, int32}")
    .Attr("strides: list(int)")
    .Attr("dilations: list(int) = [1, 1, 1, 1]")
    .Attr("mant_mul_lut: string")
    .Attr(GetPaddingAttrString())
    .Attr(GetConvnetDataFormatAttrString())
    .SetShapeFn([](shape_inference::InferenceContext* c) {
      shape_inference::ShapeHandle s;
      TF_RETURN_IF_ERROR(c->MakeShapeFromShapeTensor(0, &s));
      TF_RETURN_IF_ERROR(c->WithRank(s, 4, &s));
      c->set_output(0, s);
      return Status::OK();
    });

REGISTER_OP("ConvamInputGrad")
    .Input("input_sizes: int32")
    .Input("filter: T")
    .Input("out_backprop: T")
    .Output("grad_input: T")
    .Attr("T: {float, int32}")
    .Attr("strides: list(int)")
    .Attr(GetPaddingAttrString())
    .Attr(GetConvnetDataFormatAttrString())
    .Attr("dilations: list(int) = [1, 1, 1, 1]")
    .Attr("mant_mul_lut: string")
    .SetShapeFn([](shape_inference::InferenceContext* c) {
      shape_inference::ShapeHandle s;
      TF_RETURN_IF_ERROR(c->MakeShapeFromShapeTensor(0, &s));
      TF_RETURN_IF_ERROR(c->WithRank(s, 4, &s));
      c->set_output(0, s);
      return Status::OK();
    });

class AmsimConvOp : public OpKernel {
 public:
  explicit AmsimConvOp(OpKernelConstruction* ctx) : OpKernel(ctx), lut_(ctx) { OP_REQUIRES_OK(ctx, ReadWindow(ctx, &win_)); }
  void Compute(OpKernelContext* ctx) override {
    const Tensor& x = ctx->input(0);
    const Tensor& f = ctx->input(1);
    Geometry g;
    OP_REQUIRES_OK(ctx, MakeGeometry(win_, x.shape(), f.shape(), &g));
    Tensor* y = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({g.n, g.oh, g.ow, g.k}), &y));
    if (y->NumElements() == 0) return;
    OP_REQUIRES_OK(ctx, FromAmsim(amsim_conv2d_fwd(StreamOf(ctx), lut_.get(), x.flat<float>().data(),
                                                   f.flat<float>().data(), y->flat<float>().data(), g.n, g.h, g.w, g.c,
                                                   g.kh, g.kw, g.k, g.oh, g.ow, win_.stride_h, win_.stride_w, g.pt,
                                                   g.pl, ModeFlag())));
  }

 private:
  LutAttr lut_;
  Window win_;
};

class AmsimConvInputGradOp : public OpKernel {
 public:
  explicit AmsimConvInputGradOp(OpKernelConstruction* ctx) : OpKernel(ctx), lut_(ctx) {
    OP_REQUIRES_OK(ctx, ReadWindow(ctx, &win_));
  }
  void Compute(OpKernelContext* ctx) override {
    TensorShape in_shape;
    OP_REQUIRES_OK(ctx, ShapeFromInt32Vector(ctx->input(0), &in_shape));
    const Tensor& f = ctx->input(1);
    const Tensor& dy = ctx->input(2);
    Tensor* dx = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, in_shape, &dx));
    if (dx->NumElements() == 0) return;
    Geometry g;
    OP_REQUIRES_OK(ctx, MakeGeometry(win_, in_shape, f.shape(), &g));
    OP_REQUIRES(ctx, dy.shape() == TensorShape({g.n, g.oh, g.ow, g.k}),
                errors::InvalidArgument("out_backprop shape does not match the forward output"));
    OP_REQUIRES_OK(ctx, FromAmsim(amsim_conv2d_bwd_input(StreamOf(ctx), lut_.get(), f.flat<float>().data(),
                                                         dy.flat<float>().data(), dx->flat<float>().data(), g.n, g.h,
                                                         g.w, g.c, g.kh, g.kw, g.k, g.oh, g.ow, win_.stride_h,
                                                         win_.stride_w, g.pt, g.pl, ModeFlag())));
  }

 private:
  LutAttr lut_;
  Window win_;
};

class AmsimConvFilterGradOp : public OpKernel {
 public:
  explicit AmsimConvFilterGradOp(OpKernelConstruction* ctx) : OpKernel(ctx), lut_(ctx) {
    OP_REQUIRES_OK(ctx, ReadWindow(ctx, &win_));
  }
  void Compute(OpKernelContext* ctx) override {
    TensorShape f_shape;
    OP_REQUIRES_OK(ctx, ShapeFromInt32Vector(ctx->input(0), &f_shape));
    const Tensor& x = ctx->input(1);
    const Tensor& dy = ctx->input(2);
    Tensor* dw = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, f_shape, &dw));
    if (dw->NumElements() == 0) return;
    Geometry g;
    OP_REQUIRES_OK(ctx, MakeGeometry(win_, x.shape(), f_shape, &g));
    const size_t ws_bytes =
        amsim_conv2d_bwd_filter_workspace(g.n, g.h, g.w, g.c, g.kh, g.kw, g.k, g.oh, g.ow, ModeFlag());
    Tensor ws;
    void* ws_ptr = nullptr;
    if (ws_bytes > 0) {
      OP_REQUIRES_OK(ctx, ctx->allocate_temp(DT_UINT8, TensorShape({static_cast<int64>(ws_bytes) + 256}), &ws));
      uintptr_t p = reinterpret_cast<uintptr_t>(ws.flat<uint8>().data());
      ws_ptr = reinterpret_cast<void*>((p + 255) & ~static_cast<uintptr_t>(255));
    }
    OP_REQUIRES_OK(ctx, FromAmsim(amsim_conv2d_bwd_filter(StreamOf(ctx), lut_.get(), x.flat<float>().data(),
                                                          dy.flat<float>().data(), dw->flat<float>().data(), g.n, g.h,
                                                          g.w, g.c, g.kh, g.kw, g.k, g.oh, g.ow, win_.stride_h,
                                                          win_.stride_w, g.pt, g.pl, ws_ptr, ws_bytes, ModeFlag())));
  }

 private:
  LutAttr lut_;
  Window win_;
};

REGISTER_KERNEL_BUILDER(Name("Convam").Device(DEVICE_GPU).TypeConstraint<float>("T"), AmsimConvOp);
REGISTER_KERNEL_BUILDER(
    Name("ConvamInputGrad").Device(DEVICE_GPU).TypeConstraint<float>("T").HostMemory("input_sizes"),
    AmsimConvInputGradOp);
REGISTER_KERNEL_BUILDER(
    Name("ConvamFilterGrad").Device(DEVICE_GPU).TypeConstraint<float>("T").HostMemory("filter_sizes"),
    AmsimConvFilterGradOp);
