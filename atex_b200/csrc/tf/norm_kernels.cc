// TensorFlow GPU OpKernels of the four fused norm ops.  Thin glue: validate,
// view the tensors as [N, D] / [N, C, D], allocate outputs and scratch from the
// OpKernelContext, and call libnvnorms through its C ABI on the context's
// compute stream.  Not compiled in environments without TensorFlow.
//
// Takes the place of FusedLayerNormOp / FusedLayerNormGradOp
// (atex/nv_norms/cc/kernels/fused_layer_norm_op.cc:285-484) and
// FusedInstanceNormOp / FusedInstanceNormGradOp
// (atex/nv_norms/cc/kernels/fused_instance_norm_op.cc:311-560).  Only GPU kernels
// are registered: this build has no CPU implementation.
#define EIGEN_USE_GPU

#include <string>
#include <vector>

#include "nvnorms.h"
#include "tensorflow/core/framework/op_kernel.h"
#include "tensorflow/core/framework/register_types.h"
#include "tensorflow/core/framework/tensor.h"
#include "tensorflow/core/util/gpu_kernel_helper.h"

namespace tensorflow {
namespace {

using GPUDevice = Eigen::GpuDevice;

template <typename T>
struct NvnType;
template <>
struct NvnType<float> {
  static constexpr int value = NVN_F32;
};
template <>
struct NvnType<Eigen::half> {
  static constexpr int value = NVN_F16;
};
template <>
struct NvnType<Eigen::bfloat16> {
  static constexpr int value = NVN_BF16;
};

Status FromNvn(int st, const char* what) {
  if (st == NVN_OK) return OkStatus();
  if (st == NVN_ERR_CUDA)
    return errors::Internal(what, ": CUDA error ", nvn_last_cuda_error());
  if (st == NVN_ERR_WORKSPACE || st == NVN_ERR_UNSUPPORTED || st == NVN_ERR_LIMIT)
    return errors::Internal(what, ": ", nvn_status_string(st));
  return errors::InvalidArgument(nvn_status_string(st));
}

std::vector<int64_t> DimsOf(const Tensor& t) {
  std::vector<int64_t> d(t.dims());
  for (int i = 0; i < t.dims(); ++i) d[i] = t.dim_size(i);
  return d;
}

// Scratch for one call: a uint8 temp tensor whose lifetime TF ties to the stream.
Status Scratch(OpKernelContext* ctx, size_t bytes, Tensor* holder, void** ptr) {
  *ptr = nullptr;
  if (bytes == 0) return OkStatus();
  TF_RETURN_IF_ERROR(
      ctx->allocate_temp(DT_UINT8, TensorShape({static_cast<int64_t>(bytes)}), holder));
  *ptr = holder->flat<uint8>().data();
  return OkStatus();
}

void* StreamOf(OpKernelContext* ctx) {
  return reinterpret_cast<void*>(ctx->eigen_device<GPUDevice>().stream());
}

// ----------------------------------------------------------------------------
// LayerNorm
// ----------------------------------------------------------------------------
template <typename T>
class FusedLayerNormOp : public OpKernel {
 public:
  explicit FusedLayerNormOp(OpKernelConstruction* c) : OpKernel(c) {
    OP_REQUIRES_OK(c, c->GetAttr("epsilon", &epsilon_));
    OP_REQUIRES_OK(c, c->GetAttr("axis", &axis_));
  }

  void Compute(OpKernelContext* ctx) override {
    const Tensor& x = ctx->input(0);
    const Tensor& scale = ctx->input(1);
    const Tensor& offset = ctx->input(2);
    OP_REQUIRES(ctx, x.dims() > 0,
                errors::InvalidArgument("input must be at least 1-dimensional",
                                        x.shape().DebugString()));
    const std::vector<int64_t> dims = DimsOf(x);
    int64_t N = 0, D = 0;
    OP_REQUIRES_OK(ctx, FromNvn(nvn_ln_dims(x.dims(), dims.data(), static_cast<int>(axis_.size()),
                                            axis_.data(), &N, &D),
                                "nvn_ln_dims"));
    OP_REQUIRES(ctx, scale.NumElements() == D,
                errors::InvalidArgument("scale must have the same number of elements as the "
                                        "features of x, got ",
                                        scale.NumElements(), " and ", D));
    OP_REQUIRES(ctx, offset.NumElements() == D,
                errors::InvalidArgument("offset must have the same number of elements as the "
                                        "features of x, got ",
                                        offset.NumElements(), " and ", D));
    Tensor* y = nullptr;  // may share x's buffer: the kernels allow y == x
    OP_REQUIRES_OK(ctx, ctx->forward_input_or_allocate_output({0}, 0, x.shape(), &y));
    Tensor *mean = nullptr, *inv_std = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(1, TensorShape({N}), &mean));
    OP_REQUIRES_OK(ctx, ctx->allocate_output(2, TensorShape({N}), &inv_std));
    if (x.NumElements() == 0) return;
    Tensor holder;
    void* ws = nullptr;
    const size_t ws_bytes = nvn_ln_fwd_workspace_bytes(NvnType<T>::value, N, D);
    OP_REQUIRES_OK(ctx, Scratch(ctx, ws_bytes, &holder, &ws));
    OP_REQUIRES_OK(
        ctx, FromNvn(nvn_ln_fwd(NvnType<T>::value, x.flat<T>().data(), scale.flat<float>().data(),
                                offset.flat<float>().data(), N, D, epsilon_, y->flat<T>().data(),
                                mean->flat<float>().data(), inv_std->flat<float>().data(), ws,
                                ws_bytes, StreamOf(ctx)),
                     "nvn_ln_fwd"));
  }

 private:
  float epsilon_;
  std::vector<int> axis_;
};

template <typename T>
class FusedLayerNormGradOp : public OpKernel {
 public:
  explicit FusedLayerNormGradOp(OpKernelConstruction* c) : OpKernel(c) {
    OP_REQUIRES_OK(c, c->GetAttr("axis", &axis_));
  }

  void Compute(OpKernelContext* ctx) override {
    const Tensor& dy = ctx->input(0);
    const Tensor& x = ctx->input(1);
    const Tensor& scale = ctx->input(2);
    const Tensor& mean = ctx->input(3);
    const Tensor& inv_std = ctx->input(4);
    OP_REQUIRES(ctx, dy.dims() > 0 && x.dims() > 0,
                errors::InvalidArgument("input must be at least 1-dimensional",
                                        x.shape().DebugString()));
    OP_REQUIRES(ctx, mean.dims() == 1,
                errors::InvalidArgument("saved mean must be 1-dimensional",
                                        mean.shape().DebugString()));
    OP_REQUIRES(ctx, inv_std.dims() == 1,
                errors::InvalidArgument("saved inverted variance must be 1-dimensional",
                                        inv_std.shape().DebugString()));
    OP_REQUIRES(ctx, x.shape() == dy.shape(),
                errors::InvalidArgument("x and y_backprop must have same shape, but x has shape ",
                                        x.shape(), " and y_backprop has shape ", dy.shape()));
    const std::vector<int64_t> dims = DimsOf(x);
    int64_t N = 0, D = 0;
    OP_REQUIRES_OK(ctx, FromNvn(nvn_ln_dims(x.dims(), dims.data(), static_cast<int>(axis_.size()),
                                            axis_.data(), &N, &D),
                                "nvn_ln_dims"));
    OP_REQUIRES(ctx, scale.NumElements() == D,
                errors::InvalidArgument("scale must have the same number of elements as the "
                                        "features of x, got ",
                                        scale.NumElements(), " and ", D));
    OP_REQUIRES(ctx, mean.NumElements() == N,
                errors::InvalidArgument("reserve_space_1 must have the same number of elements "
                                        "as the batches of x, got ",
                                        mean.NumElements(), " and ", N));
    OP_REQUIRES(ctx, inv_std.NumElements() == N,
                errors::InvalidArgument("reserve_space_2 must have the same number of elements "
                                        "as the channels of x, got ",
                                        inv_std.NumElements(), " and ", N));
    Tensor *dx = nullptr, *dgamma = nullptr, *dbeta = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, x.shape(), &dx));
    OP_REQUIRES_OK(ctx, ctx->allocate_output(1, scale.shape(), &dgamma));
    OP_REQUIRES_OK(ctx, ctx->allocate_output(2, scale.shape(), &dbeta));
    Tensor holder;
    void* ws = nullptr;
    const size_t ws_bytes =
        x.NumElements() == 0 ? 0 : nvn_ln_bwd_workspace_bytes(NvnType<T>::value, N, D);
    OP_REQUIRES_OK(ctx, Scratch(ctx, ws_bytes, &holder, &ws));
    // Empty inputs: the library zero-fills dgamma / dbeta and launches nothing else.
    OP_REQUIRES_OK(
        ctx, FromNvn(nvn_ln_bwd(NvnType<T>::value, dy.flat<T>().data(), x.flat<T>().data(),
                                scale.flat<float>().data(), mean.flat<float>().data(),
                                inv_std.flat<float>().data(), N, D, dx->flat<T>().data(),
                                dgamma->flat<float>().data(), dbeta->flat<float>().data(), ws,
                                ws_bytes, StreamOf(ctx)),
                     "nvn_ln_bwd"));
  }

 private:
  std::vector<int> axis_;
};

// ----------------------------------------------------------------------------
// InstanceNorm
// ----------------------------------------------------------------------------
struct InDims {
  int64_t N = 0, C = 0, D = 0;
  int channel_first = 0;
};

Status InstanceDims(const Tensor& x, const std::string& data_format, InDims* d) {
  if (x.dims() < 4)
    return errors::InvalidArgument("input must be at least 4-dimensional",
                                   x.shape().DebugString());
  const std::vector<int64_t> dims = DimsOf(x);
  const int st = nvn_in_dims(x.dims(), dims.data(), data_format.c_str(), &d->N, &d->C, &d->D,
                             &d->channel_first);
  if (st == NVN_ERR_DATA_FORMAT) return errors::InvalidArgument("Invalid data format");
  return FromNvn(st, "nvn_in_dims");
}

template <typename T>
class FusedInstanceNormOp : public OpKernel {
 public:
  explicit FusedInstanceNormOp(OpKernelConstruction* c) : OpKernel(c) {
    if (!c->GetAttr("data_format", &data_format_).ok()) data_format_ = "N...C";
    OP_REQUIRES_OK(c, c->GetAttr("epsilon", &epsilon_));
  }

  void Compute(OpKernelContext* ctx) override {
    const Tensor& x = ctx->input(0);
    const Tensor& scale = ctx->input(1);
    const Tensor& offset = ctx->input(2);
    InDims d;
    OP_REQUIRES_OK(ctx, InstanceDims(x, data_format_, &d));
    OP_REQUIRES(ctx, scale.dims() == 1,
                errors::InvalidArgument("scale must be 1-dimensional",
                                        scale.shape().DebugString()));
    OP_REQUIRES(ctx, offset.dims() == 1,
                errors::InvalidArgument("offset must be 1-dimensional",
                                        offset.shape().DebugString()));
    OP_REQUIRES(ctx, scale.NumElements() == d.C,
                errors::InvalidArgument("scale must have the same number of elements as the "
                                        "channels of x, got ",
                                        scale.NumElements(), " and ", d.C));
    OP_REQUIRES(ctx, offset.NumElements() == d.C,
                errors::InvalidArgument("offset must have the same number of elements as the "
                                        "channels of x, got ",
                                        offset.NumElements(), " and ", d.C));
    Tensor* y = nullptr;
    OP_REQUIRES_OK(ctx, ctx->forward_input_or_allocate_output({0}, 0, x.shape(), &y));
    Tensor *mean = nullptr, *inv_std = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(1, TensorShape({d.N, d.C}), &mean));
    OP_REQUIRES_OK(ctx, ctx->allocate_output(2, TensorShape({d.N, d.C}), &inv_std));
    if (x.NumElements() == 0) return;
    Tensor holder;
    void* ws = nullptr;
    const size_t ws_bytes =
        nvn_in_fwd_workspace_bytes(NvnType<T>::value, d.N, d.C, d.D, d.channel_first);
    OP_REQUIRES_OK(ctx, Scratch(ctx, ws_bytes, &holder, &ws));
    OP_REQUIRES_OK(
        ctx, FromNvn(nvn_in_fwd(NvnType<T>::value, x.flat<T>().data(), scale.flat<float>().data(),
                                offset.flat<float>().data(), d.N, d.C, d.D, d.channel_first,
                                epsilon_, y->flat<T>().data(), mean->flat<float>().data(),
                                inv_std->flat<float>().data(), ws, ws_bytes, StreamOf(ctx)),
                     "nvn_in_fwd"));
  }

 private:
  std::string data_format_;
  float epsilon_;
};

template <typename T>
class FusedInstanceNormGradOp : public OpKernel {
 public:
  explicit FusedInstanceNormGradOp(OpKernelConstruction* c) : OpKernel(c) {
    if (!c->GetAttr("data_format", &data_format_).ok()) data_format_ = "N...C";
  }

  void Compute(OpKernelContext* ctx) override {
    const Tensor& dy = ctx->input(0);
    const Tensor& x = ctx->input(1);
    const Tensor& scale = ctx->input(2);
    const Tensor& mean = ctx->input(3);
    const Tensor& inv_std = ctx->input(4);
    OP_REQUIRES(ctx, dy.dims() > 3,
                errors::InvalidArgument("input must be at least 4-dimensional",
                                        dy.shape().DebugString()));
    OP_REQUIRES(ctx, scale.dims() == 1,
                errors::InvalidArgument("scale must be 1-dimensional",
                                        scale.shape().DebugString()));
    OP_REQUIRES(ctx, mean.dims() == 2,
                errors::InvalidArgument("saved mean must be 2-dimensional",
                                        mean.shape().DebugString()));
    OP_REQUIRES(ctx, inv_std.dims() == 2,
                errors::InvalidArgument("saved inverted variance must be 2-dimensional",
                                        inv_std.shape().DebugString()));
    OP_REQUIRES(ctx, x.shape() == dy.shape(),
                errors::InvalidArgument("x and y_backprop must have same shape, but x has shape ",
                                        x.shape(), " and y_backprop has shape ", dy.shape()));
    InDims d;
    OP_REQUIRES_OK(ctx, InstanceDims(x, data_format_, &d));
    OP_REQUIRES(ctx, scale.NumElements() == d.C,
                errors::InvalidArgument("scale must have the same number of elements as the "
                                        "channels of x, got ",
                                        scale.NumElements(), " and ", d.C));
    OP_REQUIRES(ctx, mean.NumElements() == d.N * d.C,
                errors::InvalidArgument("reserve_space_1 must have the same number of elements "
                                        "as the batches*channels of x, got ",
                                        mean.NumElements(), " and ", d.N * d.C));
    OP_REQUIRES(ctx, inv_std.NumElements() == d.N * d.C,
                errors::InvalidArgument("reserve_space_2 must have the same number of elements "
                                        "as the batches * channels of x, got ",
                                        inv_std.NumElements(), " and ", d.N * d.C));
    Tensor *dx = nullptr, *dgamma = nullptr, *dbeta = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, x.shape(), &dx));
    OP_REQUIRES_OK(ctx, ctx->allocate_output(1, scale.shape(), &dgamma));
    OP_REQUIRES_OK(ctx, ctx->allocate_output(2, scale.shape(), &dbeta));
    Tensor holder;
    void* ws = nullptr;
    const size_t ws_bytes =
        x.NumElements() == 0
            ? 0
            : nvn_in_bwd_workspace_bytes(NvnType<T>::value, d.N, d.C, d.D, d.channel_first);
    OP_REQUIRES_OK(ctx, Scratch(ctx, ws_bytes, &holder, &ws));
    OP_REQUIRES_OK(
        ctx, FromNvn(nvn_in_bwd(NvnType<T>::value, dy.flat<T>().data(), x.flat<T>().data(),
                                scale.flat<float>().data(), mean.flat<float>().data(),
                                inv_std.flat<float>().data(), d.N, d.C, d.D, d.channel_first,
                                dx->flat<T>().data(), dgamma->flat<float>().data(),
                                dbeta->flat<float>().data(), ws, ws_bytes, StreamOf(ctx)),
                     "nvn_in_bwd"));
  }

 private:
  std::string data_format_;
};

#define NVN_REGISTER(T)                                                                      \
  REGISTER_KERNEL_BUILDER(                                                                   \
      Name("FusedLayerNorm").Device(DEVICE_GPU).TypeConstraint<T>("T").TypeConstraint<float>("U"), \
      FusedLayerNormOp<T>);                                                                  \
  REGISTER_KERNEL_BUILDER(Name("FusedLayerNormGrad")                                         \
                              .Device(DEVICE_GPU)                                            \
                              .TypeConstraint<T>("T")                                        \
                              .TypeConstraint<float>("U"),                                   \
                          FusedLayerNormGradOp<T>);                                          \
  REGISTER_KERNEL_BUILDER(Name("FusedInstanceNorm")                                          \
                              .Device(DEVICE_GPU)                                            \
                              .TypeConstraint<T>("T")                                        \
                              .TypeConstraint<float>("U"),                                   \
                          FusedInstanceNormOp<T>);                                           \
  REGISTER_KERNEL_BUILDER(Name("FusedInstanceNormGrad")                                      \
                              .Device(DEVICE_GPU)                                            \
                              .TypeConstraint<T>("T")                                        \
                              .TypeConstraint<float>("U"),                                   \
                          FusedInstanceNormGradOp<T>);

NVN_REGISTER(float)
NVN_REGISTER(Eigen::half)
NVN_REGISTER(Eigen::bfloat16)
#undef NVN_REGISTER

}  // namespace
}  // namespace tensorflow
