// Custom-operator header: the subset of the reference's `paddle/extension.h` an out-of-tree operator uses
// (paddle/phi/api/ext/op_meta_info.h: PD_BUILD_OP / PD_BUILD_GRAD_OP / PD_KERNEL / PD_INFER_SHAPE / PD_INFER_DTYPE,
// paddle/phi/api/include/tensor.h: paddle::Tensor), implemented over ATen so that a custom kernel receives the same
// device memory, stream and allocator as the rest of the framework.  An operator source that sticks to this subset
// compiles unchanged; `paddle.utils.cpp_extension.load` builds it (CUDA sources for sm_100a) and turns every
// registered operator into a Python function with autograd wired to its PD_BUILD_GRAD_OP.
#pragma once

#include <torch/extension.h>

#include <cstdint>
#include <functional>
#include <map>
#include <optional>
#include <string>
#include <type_traits>
#include <vector>

#ifdef __CUDACC__
#include <ATen/cuda/CUDAContext.h>
#endif

namespace paddle {

enum class DataType { UNDEFINED = 0, BOOL, INT8, UINT8, INT16, INT32, INT64, FLOAT16, BFLOAT16, FLOAT32, FLOAT64, COMPLEX64, COMPLEX128 };

inline at::ScalarType to_aten(DataType d) {
  switch (d) {
    case DataType::BOOL: return at::kBool;
    case DataType::INT8: return at::kChar;
    case DataType::UINT8: return at::kByte;
    case DataType::INT16: return at::kShort;
    case DataType::INT32: return at::kInt;
    case DataType::INT64: return at::kLong;
    case DataType::FLOAT16: return at::kHalf;
    case DataType::BFLOAT16: return at::kBFloat16;
    case DataType::FLOAT32: return at::kFloat;
    case DataType::FLOAT64: return at::kDouble;
    case DataType::COMPLEX64: return at::kComplexFloat;
    case DataType::COMPLEX128: return at::kComplexDouble;
    default: TORCH_CHECK(false, "undefined paddle::DataType");
  }
}
inline DataType from_aten(at::ScalarType t) {
  switch (t) {
    case at::kBool: return DataType::BOOL;
    case at::kChar: return DataType::INT8;
    case at::kByte: return DataType::UINT8;
    case at::kShort: return DataType::INT16;
    case at::kInt: return DataType::INT32;
    case at::kLong: return DataType::INT64;
    case at::kHalf: return DataType::FLOAT16;
    case at::kBFloat16: return DataType::BFLOAT16;
    case at::kFloat: return DataType::FLOAT32;
    case at::kDouble: return DataType::FLOAT64;
    case at::kComplexFloat: return DataType::COMPLEX64;
    case at::kComplexDouble: return DataType::COMPLEX128;
    default: return DataType::UNDEFINED;
  }
}

using float16 = at::Half;
using bfloat16 = at::BFloat16;

class Place {
 public:
  Place() = default;
  explicit Place(c10::Device d) : dev_(d) {}
  bool is_gpu() const { return dev_.is_cuda(); }
  int GetDeviceId() const { return dev_.has_index() ? dev_.index() : 0; }
  c10::Device device() const { return dev_; }
  bool operator==(const Place& o) const { return dev_ == o.dev_; }

 private:
  c10::Device dev_{c10::kCPU};
};
inline Place CPUPlace() { return Place(c10::Device(c10::kCPU)); }
inline Place GPUPlace(int id = 0) { return Place(c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(id))); }

class Tensor {
 public:
  Tensor() = default;
  Tensor(at::Tensor t) : t_(std::move(t)) {}  // NOLINT: implicit on purpose, kernels return ATen results directly
  std::vector<int64_t> shape() const { return t_.sizes().vec(); }
  std::vector<int64_t> dims() const { return shape(); }
  int64_t numel() const { return t_.numel(); }
  int64_t size() const { return t_.numel(); }
  DataType dtype() const { return from_aten(t_.scalar_type()); }
  DataType type() const { return dtype(); }
  Place place() const { return Place(t_.device()); }
  bool is_gpu() const { return t_.is_cuda(); }
  bool is_cpu() const { return t_.is_cpu(); }
  bool defined() const { return t_.defined(); }
  bool initialized() const { return t_.defined(); }
  bool is_initialized() const { return t_.defined(); }
  template <typename T>
  T* data() const { return t_.data_ptr<T>(); }
  template <typename T>
  T* mutable_data() { return t_.data_ptr<T>(); }
  void* data() const { return t_.data_ptr(); }
  Tensor copy_to(const Place& p, bool blocking = true) const { return Tensor(t_.to(p.device(), /*non_blocking=*/!blocking)); }
  Tensor cast(DataType d) const { return Tensor(t_.to(to_aten(d))); }
  Tensor contiguous() const { return Tensor(t_.contiguous()); }
  Tensor reshape(const std::vector<int64_t>& s) const { return Tensor(t_.reshape(s)); }
  void reshape_(const std::vector<int64_t>& s) { t_ = t_.reshape(s); }
#ifdef __CUDACC__
  cudaStream_t stream() const { return at::cuda::getCurrentCUDAStream(t_.device().index()).stream(); }
#endif
  const at::Tensor& aten() const { return t_; }
  at::Tensor& aten() { return t_; }

 private:
  at::Tensor t_;
};

template <typename T>
using optional = std::optional<T>;

inline at::TensorOptions opts(DataType d, const Place& p) { return at::TensorOptions().dtype(to_aten(d)).device(p.device()); }
inline Tensor empty(const std::vector<int64_t>& shape, DataType d = DataType::FLOAT32, const Place& p = CPUPlace()) {
  return Tensor(at::empty(shape, opts(d, p)));
}
inline Tensor zeros(const std::vector<int64_t>& shape, DataType d = DataType::FLOAT32, const Place& p = CPUPlace()) {
  return Tensor(at::zeros(shape, opts(d, p)));
}
inline Tensor ones(const std::vector<int64_t>& shape, DataType d = DataType::FLOAT32, const Place& p = CPUPlace()) {
  return Tensor(at::ones(shape, opts(d, p)));
}
template <typename S>
inline Tensor full(const std::vector<int64_t>& shape, S value, DataType d = DataType::FLOAT32, const Place& p = CPUPlace()) {
  return Tensor(at::full(shape, value, opts(d, p)));
}
inline Tensor empty_like(const Tensor& x) { return Tensor(at::empty_like(x.aten())); }
inline Tensor zeros_like(const Tensor& x) { return Tensor(at::zeros_like(x.aten())); }

// names of gradient / list / optional slots in Inputs({...}) and Outputs({...})
inline std::string Grad(const std::string& name) { return name + "@GRAD"; }
inline std::string Vec(const std::string& name) { return name + "@VECTOR"; }
inline std::string Optional(const std::string& name) { return name + "@OPTIONAL"; }

// hidden like pybind11's own types: the registry is private to each extension's shared object
namespace detail __attribute__((visibility("hidden"))) {

namespace py = pybind11;

template <typename T>
struct ArgCaster {
  static T cast(py::handle h) { return py::cast<T>(h); }
};
template <>
struct ArgCaster<Tensor> {
  static Tensor cast(py::handle h) { return Tensor(py::cast<at::Tensor>(h)); }
};
template <>
struct ArgCaster<std::vector<Tensor>> {
  static std::vector<Tensor> cast(py::handle h) {
    std::vector<Tensor> out;
    for (auto item : py::cast<py::sequence>(h)) out.emplace_back(py::cast<at::Tensor>(item));
    return out;
  }
};
template <>
struct ArgCaster<optional<Tensor>> {
  static optional<Tensor> cast(py::handle h) {
    if (h.is_none()) return std::nullopt;
    return Tensor(py::cast<at::Tensor>(h));
  }
};
template <>
struct ArgCaster<optional<std::vector<Tensor>>> {
  static optional<std::vector<Tensor>> cast(py::handle h) {
    if (h.is_none()) return std::nullopt;
    return ArgCaster<std::vector<Tensor>>::cast(h);
  }
};

inline py::object to_py(const Tensor& t) { return t.defined() ? py::cast(t.aten()) : py::none(); }
inline py::object to_py(const std::vector<Tensor>& v) {
  py::list out;
  for (const auto& t : v) out.append(to_py(t));
  return out;
}
inline py::object to_py(const std::vector<std::vector<int64_t>>& v) { return py::cast(v); }
inline py::object to_py(const std::vector<DataType>& v) {
  py::list out;
  for (auto d : v) out.append(static_cast<int>(d));
  return out;
}
template <>
struct ArgCaster<DataType> {
  static DataType cast(py::handle h) { return static_cast<DataType>(py::cast<int>(h)); }
};
template <>
struct ArgCaster<std::vector<DataType>> {
  static std::vector<DataType> cast(py::handle h) {
    std::vector<DataType> out;
    for (auto item : py::cast<py::sequence>(h)) out.push_back(static_cast<DataType>(py::cast<int>(item)));
    return out;
  }
};

using ErasedFn = std::function<py::object(const py::list&)>;

template <typename F>
struct Erase;
template <typename R, typename... Args>
struct Erase<R (*)(Args...)> {
  template <R (*fn)(Args...), size_t... I>
  static py::object call(const py::list& args, std::index_sequence<I...>) {
    TORCH_CHECK(args.size() == sizeof...(Args), "custom operator expects ", sizeof...(Args), " arguments, got ", args.size());
    return to_py(fn(ArgCaster<std::decay_t<Args>>::cast(args[I])...));
  }
  template <R (*fn)(Args...)>
  static ErasedFn make() {
    return [](const py::list& args) { return call<fn>(args, std::index_sequence_for<Args...>{}); };
  }
};

struct OpMeta {
  std::vector<std::string> inputs, outputs, attrs;
  std::map<std::string, std::string> inplace;
  ErasedFn kernel, infer_shape, infer_dtype;
};

inline std::map<std::string, OpMeta>& registry() {
  static std::map<std::string, OpMeta> r;
  return r;
}

}  // namespace detail

class __attribute__((visibility("hidden"))) OpMetaInfoBuilder {
 public:
  explicit OpMetaInfoBuilder(std::string name) : name_(std::move(name)) { detail::registry()[name_]; }
  OpMetaInfoBuilder& Inputs(std::vector<std::string> v) { meta().inputs = std::move(v); return *this; }
  OpMetaInfoBuilder& Outputs(std::vector<std::string> v) { meta().outputs = std::move(v); return *this; }
  OpMetaInfoBuilder& Attrs(std::vector<std::string> v) { meta().attrs = std::move(v); return *this; }
  OpMetaInfoBuilder& SetInplaceMap(std::map<std::string, std::string> m) { meta().inplace = std::move(m); return *this; }
  OpMetaInfoBuilder& SetKernelFn(detail::ErasedFn f) { meta().kernel = std::move(f); return *this; }
  OpMetaInfoBuilder& SetInferShapeFn(detail::ErasedFn f) { meta().infer_shape = std::move(f); return *this; }
  OpMetaInfoBuilder& SetInferDtypeFn(detail::ErasedFn f) { meta().infer_dtype = std::move(f); return *this; }

 private:
  detail::OpMeta& meta() { return detail::registry()[name_]; }
  std::string name_;
};

// Called from the generated binding source: exposes the registry of this shared object to Python.
inline void bind_ops(pybind11::module_& m) {
  namespace py = pybind11;
  m.def("op_names", []() {
    std::vector<std::string> out;
    for (auto& kv : detail::registry()) out.push_back(kv.first);
    return out;
  });
  m.def("op_meta", [](const std::string& name) {
    auto it = detail::registry().find(name);
    TORCH_CHECK(it != detail::registry().end(), "no custom operator named ", name);
    py::dict d;
    d["inputs"] = it->second.inputs;
    d["outputs"] = it->second.outputs;
    d["attrs"] = it->second.attrs;
    d["inplace"] = it->second.inplace;
    d["has_infer_shape"] = static_cast<bool>(it->second.infer_shape);
    d["has_infer_dtype"] = static_cast<bool>(it->second.infer_dtype);
    return d;
  });
  m.def("run", [](const std::string& name, const py::list& args) {
    auto it = detail::registry().find(name);
    TORCH_CHECK(it != detail::registry().end() && it->second.kernel, "custom operator ", name, " has no kernel");
    return it->second.kernel(args);
  });
  m.def("infer_shape", [](const std::string& name, const py::list& args) { return detail::registry().at(name).infer_shape(args); });
  m.def("infer_dtype", [](const std::string& name, const py::list& args) { return detail::registry().at(name).infer_dtype(args); });
}

}  // namespace paddle

#define PD_CONCAT_(a, b) a##b
#define PD_CONCAT(a, b) PD_CONCAT_(a, b)
#define PD_BUILD_OP(op_name) \
  static ::paddle::OpMetaInfoBuilder PD_CONCAT(__pd_op_builder_##op_name##_, __COUNTER__) = ::paddle::OpMetaInfoBuilder(#op_name)
#define PD_BUILD_GRAD_OP(op_name) \
  static ::paddle::OpMetaInfoBuilder PD_CONCAT(__pd_grad_op_builder_##op_name##_, __COUNTER__) = ::paddle::OpMetaInfoBuilder(#op_name "_grad")
#define PD_BUILD_DOUBLE_GRAD_OP(op_name) \
  static ::paddle::OpMetaInfoBuilder PD_CONCAT(__pd_grad2_op_builder_##op_name##_, __COUNTER__) = \
      ::paddle::OpMetaInfoBuilder(#op_name "_grad_grad")
#define PD_KERNEL(...) ::paddle::detail::Erase<decltype(&__VA_ARGS__)>::make<&__VA_ARGS__>()
#define PD_INFER_SHAPE(...) ::paddle::detail::Erase<decltype(&__VA_ARGS__)>::make<&__VA_ARGS__>()
#define PD_INFER_DTYPE(...) ::paddle::detail::Erase<decltype(&__VA_ARGS__)>::make<&__VA_ARGS__>()

#define PD_CHECK(cond, ...) TORCH_CHECK(cond, ##__VA_ARGS__)
#define PD_THROW(...) TORCH_CHECK(false, ##__VA_ARGS__)
#define CHECK_INPUT(x) PD_CHECK((x).is_gpu(), #x " must be a GPU Tensor.")
#define CHECK_CPU_INPUT(x) PD_CHECK((x).is_cpu(), #x " must be a CPU Tensor.")

#define PD_PRIVATE_CASE(enum_type, cpp_type, ...) \
  case enum_type: {                               \
    using data_t = cpp_type;                      \
    return __VA_ARGS__();                         \
  }
#define PD_DISPATCH_FLOATING_TYPES(TYPE, NAME, ...)                              \
  [&] {                                                                          \
    switch (TYPE) {                                                              \
      PD_PRIVATE_CASE(::paddle::DataType::FLOAT32, float, __VA_ARGS__)           \
      PD_PRIVATE_CASE(::paddle::DataType::FLOAT64, double, __VA_ARGS__)          \
      default: PD_THROW("function " #NAME " is not implemented for this data type"); \
    }                                                                            \
  }()
#define PD_DISPATCH_FLOATING_AND_HALF_TYPES(TYPE, NAME, ...)                     \
  [&] {                                                                          \
    switch (TYPE) {                                                              \
      PD_PRIVATE_CASE(::paddle::DataType::FLOAT32, float, __VA_ARGS__)           \
      PD_PRIVATE_CASE(::paddle::DataType::FLOAT64, double, __VA_ARGS__)          \
      PD_PRIVATE_CASE(::paddle::DataType::FLOAT16, ::paddle::float16, __VA_ARGS__) \
      PD_PRIVATE_CASE(::paddle::DataType::BFLOAT16, ::paddle::bfloat16, __VA_ARGS__) \
      default: PD_THROW("function " #NAME " is not implemented for this data type"); \
    }                                                                            \
  }()
#define PD_DISPATCH_INTEGRAL_TYPES(TYPE, NAME, ...)                              \
  [&] {                                                                          \
    switch (TYPE) {                                                              \
      PD_PRIVATE_CASE(::paddle::DataType::INT32, int, __VA_ARGS__)               \
      PD_PRIVATE_CASE(::paddle::DataType::INT64, int64_t, __VA_ARGS__)           \
      PD_PRIVATE_CASE(::paddle::DataType::INT8, int8_t, __VA_ARGS__)             \
      PD_PRIVATE_CASE(::paddle::DataType::UINT8, uint8_t, __VA_ARGS__)           \
      PD_PRIVATE_CASE(::paddle::DataType::INT16, int16_t, __VA_ARGS__)           \
      default: PD_THROW("function " #NAME " is not implemented for this data type"); \
    }                                                                            \
  }()
