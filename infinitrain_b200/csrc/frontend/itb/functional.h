// itb::nn::function: the reference's functional wrappers (infini_train/include/nn/functional.h:25-184)
// under the same names and argument orders, on torch::Tensor.  Where the reference's result differs from
// libtorch's default the reference's is kept: comparisons give 0/1 in the INPUT's dtype (its kernels write
// the input type, src/autograd/elementwise.cc), Slice takes per-dimension start / end / step lists.
#pragma once
#include <vector>

#include "module.h"

namespace itb {
namespace nn {
namespace function {

// Lower / upper triangle of the last two dimensions; `diagonal` shifts the kept band.
inline Tensor Tril(const Tensor& input, int64_t diagonal = 0) { return input.tril(diagonal); }
inline Tensor Triu(const Tensor& input, int64_t diagonal = 0) { return input.triu(diagonal); }
// fp32 tensor of ones on the CPU (the reference allocates on its default device, the CPU).
inline Tensor Ones(const std::vector<int64_t>& size) { return torch::ones(size, torch::kFloat32); }

inline Tensor Reciprocal(const Tensor& input) { return input.reciprocal(); }
inline Tensor Sin(const Tensor& input) { return input.sin(); }
inline Tensor Cos(const Tensor& input) { return input.cos(); }
inline Tensor Tanh(const Tensor& input) { return input.tanh(); }
inline Tensor Pow(const Tensor& input, float exponent) { return input.pow(exponent); }
inline Tensor Pow(float base, const Tensor& input) { return torch::pow(torch::Scalar(base), input); }
inline Tensor Rsqrt(const Tensor& input) { return input.rsqrt(); }
inline Tensor Exp(const Tensor& input) { return input.exp(); }
inline Tensor Log(const Tensor& input) { return input.log(); }
inline Tensor Sigmoid(const Tensor& input) { return input.sigmoid(); }
inline Tensor Softmax(const Tensor& input, int64_t dim = -1) { return input.softmax(dim); }

inline Tensor Mean(const Tensor& input, int64_t dim, bool keep_dim = false) { return input.mean(dim, keep_dim); }
inline Tensor Sum(const Tensor& input, int64_t dim, bool keep_dim = false) { return input.sum(dim, keep_dim); }
inline Tensor Min(const Tensor& input, int64_t dim, bool keep_dim = false) { return std::get<0>(input.min(dim, keep_dim)); }
inline Tensor Max(const Tensor& input, int64_t dim, bool keep_dim = false) { return std::get<0>(input.max(dim, keep_dim)); }

// One (start, end, step) per dimension of `input`; end is exclusive.
inline Tensor Slice(const Tensor& input, const std::vector<int64_t>& starts, const std::vector<int64_t>& ends,
                    const std::vector<int64_t>& steps) {
  TORCH_CHECK(static_cast<int64_t>(starts.size()) == input.dim() && starts.size() == ends.size() &&
                  starts.size() == steps.size(),
              "Slice: one start / end / step per dimension of the input");
  Tensor out = input;
  for (int64_t d = 0; d < input.dim(); ++d) {
    TORCH_CHECK(steps[d] > 0, "Slice: steps are positive");
    out = out.slice(d, starts[d], ends[d], steps[d]);
  }
  return out;
}
inline Tensor Stack(const TensorList& inputs, int64_t dim = 0) { return torch::stack(inputs, dim); }
inline Tensor Concat(const TensorList& inputs, int64_t dim = 0) { return torch::cat(inputs, dim); }

// ---- comparisons and logic: forward only, 0 / 1 in the dtype of the first operand
inline Tensor as_input_dtype(const Tensor& mask, const Tensor& like) { return mask.to(like.scalar_type()); }
inline Tensor Equals(const Tensor& a, const Tensor& b) { return as_input_dtype(a.eq(b), a); }
inline Tensor Equals(const Tensor& a, float s) { return as_input_dtype(a.eq(s), a); }
inline Tensor Lt(const Tensor& a, const Tensor& b) { return as_input_dtype(a.lt(b), a); }
inline Tensor Lt(const Tensor& a, float s) { return as_input_dtype(a.lt(s), a); }
inline Tensor Le(const Tensor& a, const Tensor& b) { return as_input_dtype(a.le(b), a); }
inline Tensor Le(const Tensor& a, float s) { return as_input_dtype(a.le(s), a); }
inline Tensor Gt(const Tensor& a, const Tensor& b) { return as_input_dtype(a.gt(b), a); }
inline Tensor Gt(const Tensor& a, float s) { return as_input_dtype(a.gt(s), a); }
inline Tensor Ge(const Tensor& a, const Tensor& b) { return as_input_dtype(a.ge(b), a); }
inline Tensor Ge(const Tensor& a, float s) { return as_input_dtype(a.ge(s), a); }
inline Tensor And(const Tensor& a, const Tensor& b) { return as_input_dtype(a.ne(0).logical_and(b.ne(0)), a); }
inline Tensor Or(const Tensor& a, const Tensor& b) { return as_input_dtype(a.ne(0).logical_or(b.ne(0)), a); }

// masked_fill with a mask of the input's shape, or one aligned to its leading or trailing dimensions
// (the reference's Mask kernel accepts both alignments, src/autograd/transform.cc).  Non-zero = fill.
inline Tensor Mask(const Tensor& input, const Tensor& mask, float value) {
  Tensor m = mask.ne(0);
  if (m.dim() < input.dim()) {
    bool tail = true;
    for (int64_t i = 0; i < m.dim(); ++i) tail = tail && m.size(m.dim() - 1 - i) == input.size(input.dim() - 1 - i);
    if (!tail) {
      // leading alignment: mask [d0..dk] against input [d0..dk, ...]
      for (int64_t i = 0; i < m.dim(); ++i)
        TORCH_CHECK(m.size(i) == input.size(i), "Mask: the mask matches neither the leading nor the trailing dimensions");
      std::vector<int64_t> shape = m.sizes().vec();
      shape.resize(input.dim(), 1);
      m = m.view(shape);
    }
  }
  return input.masked_fill(m, value);
}

// out[dims] = 0 except out[..., indices[..., k]] = values[..., k] along the last dimension (the top-k
// scatter of the reference, src/kernels/cuda/scatter.cu:17-29).
inline Tensor Scatter(const Tensor& values, const Tensor& indices, const std::vector<int64_t>& out_dims) {
  Tensor out = torch::zeros(out_dims, values.options());
  return out.scatter(-1, indices.to(torch::kLong), values);
}
inline Tensor Gather(const Tensor& input, int64_t dim, const Tensor& index) { return input.gather(dim, index.to(torch::kLong)); }
inline Tensor RepeatInterleave(const Tensor& input, int64_t repeat, int64_t dim) { return input.repeat_interleave(repeat, dim); }
inline Tensor Outer(const Tensor& a, const Tensor& b) { return a.outer(b); }

}  // namespace function
}  // namespace nn
}  // namespace itb
