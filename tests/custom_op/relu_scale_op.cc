// Test operators written against paddle/extension.h: a differentiable scaled ReLU, a list-input concat-sum with an
// optional bias, and a shape / dtype inference pair.
#include "paddle/extension.h"

#include <vector>

template <typename data_t>
void relu_scale_fwd(const data_t* x, data_t* y, int64_t n, float scale) {
  for (int64_t i = 0; i < n; ++i) y[i] = x[i] > static_cast<data_t>(0) ? static_cast<data_t>(x[i] * scale) : static_cast<data_t>(0);
}

std::vector<paddle::Tensor> ReluScaleForward(const paddle::Tensor& x, float scale) {
  CHECK_CPU_INPUT(x);
  auto xc = x.contiguous();
  auto out = paddle::empty_like(xc);
  PD_DISPATCH_FLOATING_TYPES(xc.type(), "relu_scale_fwd", ([&] { relu_scale_fwd<data_t>(xc.data<data_t>(), out.data<data_t>(), xc.numel(), scale); }));
  return {out};
}

std::vector<paddle::Tensor> ReluScaleBackward(const paddle::Tensor& x, const paddle::Tensor& out, const paddle::Tensor& grad_out, float scale) {
  auto gx = paddle::zeros_like(x);
  PD_DISPATCH_FLOATING_TYPES(x.type(), "relu_scale_bwd", ([&] {
    const data_t* o = out.data<data_t>();
    const data_t* g = grad_out.data<data_t>();
    data_t* r = gx.data<data_t>();
    for (int64_t i = 0; i < x.numel(); ++i) r[i] = o[i] > static_cast<data_t>(0) ? static_cast<data_t>(g[i] * scale) : static_cast<data_t>(0);
  }));
  return {gx};
}

std::vector<std::vector<int64_t>> ReluScaleInferShape(std::vector<int64_t> x_shape) { return {x_shape}; }
std::vector<paddle::DataType> ReluScaleInferDtype(paddle::DataType x_dtype) { return {x_dtype}; }

PD_BUILD_OP(relu_scale)
    .Inputs({"X"})
    .Outputs({"Out"})
    .Attrs({"scale: float"})
    .SetKernelFn(PD_KERNEL(ReluScaleForward))
    .SetInferShapeFn(PD_INFER_SHAPE(ReluScaleInferShape))
    .SetInferDtypeFn(PD_INFER_DTYPE(ReluScaleInferDtype));

PD_BUILD_GRAD_OP(relu_scale)
    .Inputs({"X", "Out", paddle::Grad("Out")})
    .Outputs({paddle::Grad("X")})
    .Attrs({"scale: float"})
    .SetKernelFn(PD_KERNEL(ReluScaleBackward));

// sum of a list of tensors (+ optional bias), returning the sum and the number of terms as an int64 scalar tensor
std::vector<paddle::Tensor> SumListForward(const std::vector<paddle::Tensor>& xs, const paddle::optional<paddle::Tensor>& bias,
                                           const std::vector<int64_t>& repeat, bool negate) {
  PD_CHECK(!xs.empty(), "sum_list needs at least one tensor");
  at::Tensor acc = at::zeros_like(xs[0].aten());
  for (size_t i = 0; i < xs.size(); ++i) acc = acc + xs[i].aten() * static_cast<double>(i < repeat.size() ? repeat[i] : 1);
  if (bias) acc = acc + bias->aten();
  if (negate) acc = -acc;
  return {paddle::Tensor(acc), paddle::full({1}, static_cast<int64_t>(xs.size()), paddle::DataType::INT64)};
}

std::vector<std::vector<paddle::Tensor>> SumListBackward(const std::vector<paddle::Tensor>& xs, const paddle::Tensor& grad_out,
                                                         const std::vector<int64_t>& repeat, bool negate);

PD_BUILD_OP(sum_list)
    .Inputs({paddle::Vec("X"), paddle::Optional("Bias")})
    .Outputs({"Out", "Count"})
    .Attrs({"repeat: std::vector<int64_t>", "negate: bool"})
    .SetKernelFn(PD_KERNEL(SumListForward));
