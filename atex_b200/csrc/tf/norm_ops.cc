// TensorFlow op schema of the four fused norm ops, for building
// _fused_nv_norm_ops.so against a TensorFlow installation (see CMakeLists.txt in
// this directory).  Not compiled in environments without TensorFlow.
//
// Same op names, inputs, outputs and attrs as the reference registrations
// (atex/nv_norms/cc/ops/norm_ops.cc:148-202) so graphs and the registered
// gradients keep working; `T` additionally admits bfloat16.  Shape inference
// delegates the axis / data_format rules to libnvnorms (nvn_ln_dims,
// nvn_in_dims), which is also what the kernels use.
#include <string>
#include <vector>

#include "nvnorms.h"
#include "tensorflow/core/framework/op.h"
#include "tensorflow/core/framework/shape_inference.h"

namespace tensorflow {
namespace {

using shape_inference::DimensionHandle;
using shape_inference::InferenceContext;
using shape_inference::ShapeHandle;

Status StatusFromNvn(int st, const std::string& detail = "") {
  if (st == NVN_OK) return OkStatus();
  return errors::InvalidArgument(nvn_status_string(st), detail);
}

// Static dims of `shape` (unknown dims as 1 so that products stay defined; the
// affected outputs are then marked unknown by the callers).
bool StaticDims(InferenceContext* c, ShapeHandle shape, std::vector<int64_t>* dims) {
  bool known = true;
  const int rank = c->Rank(shape);
  dims->resize(rank);
  for (int i = 0; i < rank; ++i) {
    const int64_t v = c->Value(c->Dim(shape, i));
    known = known && v >= 0;
    (*dims)[i] = v >= 0 ? v : 1;
  }
  return known;
}

// grad == false: outputs (x shape, [N], [N]);  grad == true: (x shape, [D], [D]).
Status LayerNormShapes(InferenceContext* c, int x_input, bool grad) {
  ShapeHandle x;
  TF_RETURN_IF_ERROR(c->WithRankAtLeast(c->input(x_input), 1, &x));
  std::vector<int> axis;
  TF_RETURN_IF_ERROR(c->GetAttr("axis", &axis));
  std::vector<int64_t> dims;
  const bool known = StaticDims(c, x, &dims);
  int64_t N = 0, D = 0;
  TF_RETURN_IF_ERROR(StatusFromNvn(nvn_ln_dims(static_cast<int>(dims.size()), dims.data(),
                                               static_cast<int>(axis.size()), axis.data(), &N, &D)));
  const DimensionHandle vec = known ? c->MakeDim(grad ? D : N) : c->UnknownDim();
  c->set_output(0, x);
  c->set_output(1, c->Vector(vec));
  c->set_output(2, c->Vector(vec));
  return OkStatus();
}

// grad == false: outputs (x shape, [N, C], [N, C]);  grad == true: (x shape, [C], [C]).
Status InstanceNormShapes(InferenceContext* c, int x_input, bool grad) {
  ShapeHandle x;
  TF_RETURN_IF_ERROR(c->WithRankAtLeast(c->input(x_input), 4, &x));
  std::string data_format;
  TF_RETURN_IF_ERROR(c->GetAttr("data_format", &data_format));
  std::vector<int64_t> dims;
  StaticDims(c, x, &dims);
  int64_t N = 0, C = 0, D = 0;
  int channel_first = 0;
  TF_RETURN_IF_ERROR(StatusFromNvn(
      nvn_in_dims(static_cast<int>(dims.size()), dims.data(), data_format.c_str(), &N, &C, &D,
                  &channel_first),
      ", but got" + data_format));
  const int rank = c->Rank(x);
  const DimensionHandle batch = c->Dim(x, 0);
  const DimensionHandle channels = c->Dim(x, channel_first ? 1 : rank - 1);
  c->set_output(0, x);
  if (grad) {
    c->set_output(1, c->Vector(channels));
    c->set_output(2, c->Vector(channels));
  } else {
    c->set_output(1, c->MakeShape({batch, channels}));
    c->set_output(2, c->MakeShape({batch, channels}));
  }
  return OkStatus();
}

}  // namespace

#define NVN_NORM_IO_FWD   \
  .Input("x: T")          \
  .Input("scale: U")      \
  .Input("offset: U")     \
  .Output("y: T")         \
  .Output("reserve_space_1: U") \
  .Output("reserve_space_2: U")

#define NVN_NORM_IO_GRAD        \
  .Input("y_backprop: T")       \
  .Input("x: T")                \
  .Input("scale: U")            \
  .Input("reserve_space_1: U")  \
  .Input("reserve_space_2: U")  \
  .Output("x_backprop: T")      \
  .Output("scale_backprop: U")  \
  .Output("offset_backprop: U")

#define NVN_NORM_TYPES                  \
  .Attr("T: {half, bfloat16, float}")   \
  .Attr("U: {float}")                   \
  .Attr("epsilon: float = 0.001")

REGISTER_OP("FusedLayerNorm")
NVN_NORM_IO_FWD NVN_NORM_TYPES.Attr("axis: list(int) = [-1]")
    .SetShapeFn([](InferenceContext* c) { return LayerNormShapes(c, 0, false); });

REGISTER_OP("FusedLayerNormGrad")
NVN_NORM_IO_GRAD NVN_NORM_TYPES.Attr("axis: list(int) = [-1]")
    .SetShapeFn([](InferenceContext* c) { return LayerNormShapes(c, 1, true); });

REGISTER_OP("FusedInstanceNorm")
NVN_NORM_IO_FWD NVN_NORM_TYPES.Attr("data_format: string = 'N...C'")
    .SetShapeFn([](InferenceContext* c) { return InstanceNormShapes(c, 0, false); });

REGISTER_OP("FusedInstanceNormGrad")
NVN_NORM_IO_GRAD NVN_NORM_TYPES.Attr("data_format: string = 'N...C'")
    .SetShapeFn([](InferenceContext* c) { return InstanceNormShapes(c, 1, true); });

}  // namespace tensorflow
