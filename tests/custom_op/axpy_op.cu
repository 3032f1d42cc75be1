// CUDA test operator written against paddle/extension.h: out = a * x + y on the tensor's current stream.
#include "paddle/extension.h"

template <typename data_t>
__global__ void axpy_kernel(const data_t* x, const data_t* y, data_t* out, int64_t n, float a) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = static_cast<data_t>(a * static_cast<float>(x[i]) + static_cast<float>(y[i]));
}

std::vector<paddle::Tensor> AxpyForward(const paddle::Tensor& x, const paddle::Tensor& y, float a) {
  CHECK_INPUT(x);
  CHECK_INPUT(y);
  PD_CHECK(x.shape() == y.shape(), "axpy: x and y must have the same shape");
  auto out = paddle::empty_like(x);
  const int64_t n = x.numel();
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((n + threads - 1) / threads);
  if (n == 0) return {out};
  PD_DISPATCH_FLOATING_AND_HALF_TYPES(x.type(), "axpy", ([&] {
    axpy_kernel<data_t><<<blocks, threads, 0, x.stream()>>>(x.data<data_t>(), y.data<data_t>(), out.data<data_t>(), n, a);
  }));
  return {out};
}

std::vector<paddle::Tensor> AxpyBackward(const paddle::Tensor& grad_out, float a) {
  return {paddle::Tensor(grad_out.aten() * a), grad_out};
}

PD_BUILD_OP(axpy).Inputs({"X", "Y"}).Outputs({"Out"}).Attrs({"a: float"}).SetKernelFn(PD_KERNEL(AxpyForward));
PD_BUILD_GRAD_OP(axpy).Inputs({paddle::Grad("Out")}).Outputs({paddle::Grad("X"), paddle::Grad("Y")}).Attrs({"a: float"}).SetKernelFn(PD_KERNEL(AxpyBackward));
