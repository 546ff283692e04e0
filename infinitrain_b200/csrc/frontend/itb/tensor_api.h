// The reference's Tensor method names on torch::Tensor, for code that is carried over from it
// (reference: infini_train/include/tensor.h:62-223 -- the reference passes std::shared_ptr<Tensor> and
// spells its methods in PascalCase; here a tensor is a torch::Tensor value and these are free
// functions of the same names and argument orders).  Arithmetic operators, comparison operators and
// printing come with torch::Tensor itself.
#pragma once
#include <torch/torch.h>

#include <fstream>
#include <iostream>

namespace itb {
namespace tensor_api {
using Tensor = torch::Tensor;

// ---- construction / metadata
inline Tensor MakeTensor(const std::vector<int64_t>& dims, torch::Dtype dtype, torch::Device device, bool requires_grad = false) {
  return torch::empty(dims, torch::dtype(dtype).device(device).requires_grad(requires_grad));
}
inline Tensor FromData(const float* data, const std::vector<int64_t>& dims, torch::Dtype dtype, torch::Device device) {
  return torch::from_blob(const_cast<float*>(data), dims, torch::kFloat32).clone().to(device, dtype);
}
inline const std::vector<int64_t> Dims(const Tensor& t) { return t.sizes().vec(); }
inline size_t NumElements(const Tensor& t) { return static_cast<size_t>(t.numel()); }
inline size_t SizeInBytes(const Tensor& t) { return static_cast<size_t>(t.nbytes()); }
inline torch::Dtype Dtype(const Tensor& t) { return t.scalar_type(); }
inline torch::Device GetDevice(const Tensor& t) { return t.device(); }
inline void* DataPtr(const Tensor& t) { return t.data_ptr(); }
inline bool IsContiguous(const Tensor& t) { return t.is_contiguous(); }

// ---- value semantics of the reference
inline Tensor Detach(const Tensor& t) { return t.detach(); }
inline void Fill(Tensor& t, const torch::Scalar& v) {
  torch::NoGradGuard g;
  t.fill_(v);
}
inline Tensor To(const Tensor& t, torch::Device device) { return t.to(device); }
inline Tensor To(const Tensor& t, torch::Dtype dtype) { return t.to(dtype); }
inline void CopyFrom(Tensor& dst, const Tensor& src) {   // across devices and dtypes, shapes must agree
  torch::NoGradGuard g;
  dst.copy_(src);
}

// ---- comparisons and logic (results are boolean tensors; the reference returns them in the input dtype)
inline Tensor Equals(const Tensor& a, const Tensor& b) { return a.eq(b); }
inline Tensor Equals(const Tensor& a, float s) { return a.eq(s); }
inline Tensor Lt(const Tensor& a, const Tensor& b) { return a.lt(b); }
inline Tensor Lt(const Tensor& a, float s) { return a.lt(s); }
inline Tensor Le(const Tensor& a, const Tensor& b) { return a.le(b); }
inline Tensor Le(const Tensor& a, float s) { return a.le(s); }
inline Tensor Gt(const Tensor& a, const Tensor& b) { return a.gt(b); }
inline Tensor Gt(const Tensor& a, float s) { return a.gt(s); }
inline Tensor Ge(const Tensor& a, const Tensor& b) { return a.ge(b); }
inline Tensor Ge(const Tensor& a, float s) { return a.ge(s); }
inline Tensor And(const Tensor& a, const Tensor& b) { return a.logical_and(b); }
inline Tensor Or(const Tensor& a, const Tensor& b) { return a.logical_or(b); }

// ---- arithmetic
inline Tensor Add(const Tensor& a, const Tensor& b) { return a + b; }
inline Tensor Add(const Tensor& a, float s) { return a + s; }
inline Tensor Sub(const Tensor& a, const Tensor& b) { return a - b; }
inline Tensor Mul(const Tensor& a, const Tensor& b) { return a * b; }
inline Tensor Mul(const Tensor& a, float s) { return a * s; }
inline Tensor Div(const Tensor& a, const Tensor& b) { return a / b; }
inline Tensor Neg(const Tensor& a) { return a.neg(); }
inline Tensor Reciprocal(const Tensor& a) { return a.reciprocal(); }
inline Tensor Sin(const Tensor& a) { return a.sin(); }
inline Tensor Cos(const Tensor& a) { return a.cos(); }
inline Tensor Tanh(const Tensor& a) { return a.tanh(); }
inline Tensor Pow(const Tensor& a, float e) { return a.pow(e); }
inline Tensor Rsqrt(const Tensor& a) { return a.rsqrt(); }
inline Tensor Exp(const Tensor& a) { return a.exp(); }
inline Tensor Log(const Tensor& a) { return a.log(); }

// ---- reductions along one dimension
inline Tensor Mean(const Tensor& a, int64_t dim, bool keep_dim = false) { return a.mean(dim, keep_dim); }
inline Tensor Sum(const Tensor& a, int64_t dim, bool keep_dim = false) { return a.sum(dim, keep_dim); }
inline Tensor Min(const Tensor& a, int64_t dim, bool keep_dim = false) { return std::get<0>(a.min(dim, keep_dim)); }
inline Tensor Max(const Tensor& a, int64_t dim, bool keep_dim = false) { return std::get<0>(a.max(dim, keep_dim)); }

// ---- shape
inline std::vector<Tensor> Split(const Tensor& a, int64_t split_size, int64_t dim = 0) { return a.split(split_size, dim); }
inline Tensor Gather(const Tensor& a, int64_t dim, const Tensor& index) { return a.gather(dim, index); }
inline Tensor Transpose(const Tensor& a, int64_t d0, int64_t d1) { return a.transpose(d0, d1); }
inline Tensor Slice(const Tensor& a, int64_t dim, int64_t start, int64_t end, int64_t step = 1) { return a.slice(dim, start, end, step); }
inline Tensor RepeatInterleave(const Tensor& a, int64_t repeat, int64_t dim) { return a.repeat_interleave(repeat, dim); }
inline Tensor View(const Tensor& a, const std::vector<int64_t>& dims) { return a.view(dims); }
inline Tensor Contiguous(const Tensor& a) { return a.contiguous(); }
inline Tensor Flatten(const Tensor& a, int64_t start = 0, int64_t end = -1) { return a.flatten(start, end); }
inline Tensor Squeeze(const Tensor& a, int64_t dim) { return a.squeeze(dim); }
inline Tensor Unsqueeze(const Tensor& a, int64_t dim) { return a.unsqueeze(dim); }
inline Tensor Matmul(const Tensor& a, const Tensor& b) { return a.matmul(b); }
inline Tensor Outer(const Tensor& a, const Tensor& b) { return a.outer(b); }
inline Tensor MaskedFill(const Tensor& a, const Tensor& mask, float value) { return a.masked_fill(mask.to(torch::kBool), value); }

// ---- autograd
inline Tensor RequiresGrad(Tensor t) { return t.set_requires_grad(true); }
inline void Backward(const Tensor& t, const Tensor& gradient = Tensor(), bool retain_graph = false, bool create_graph = false) {
  t.backward(gradient, retain_graph, create_graph);
}
inline void ZeroGrad(Tensor& t) { t.mutable_grad() = Tensor(); }

// ---- IO: NumPy .npy version 1.0, little-endian fp32, C order (what the reference's SaveAsNpy writes)
inline void SaveAsNpy(const Tensor& t, const std::string& path) {
  Tensor f = t.detach().to(torch::kCPU, torch::kFloat32).contiguous();
  std::string shape = "(";
  for (int64_t i = 0; i < f.dim(); ++i) shape += std::to_string(f.size(i)) + (f.dim() == 1 || i + 1 < f.dim() ? "," : "");
  shape += ")";
  std::string header = "{'descr': '<f4', 'fortran_order': False, 'shape': " + shape + ", }";
  while ((10 + header.size() + 1) % 64) header += ' ';
  header += '\n';
  std::ofstream out(path, std::ios::binary);
  TORCH_CHECK(out.is_open(), "cannot write ", path);
  const char magic[8] = {'\x93', 'N', 'U', 'M', 'P', 'Y', 1, 0};
  out.write(magic, 8);
  const uint16_t hl = static_cast<uint16_t>(header.size());
  out.write(reinterpret_cast<const char*>(&hl), 2);
  out.write(header.data(), static_cast<std::streamsize>(header.size()));
  out.write(static_cast<const char*>(f.data_ptr()), static_cast<std::streamsize>(f.nbytes()));
}
inline void Print(const Tensor& t, std::ostream& os = std::cout) { os << t << std::endl; }

}  // namespace tensor_api
}  // namespace itb
