// The reference's element-type names for the C++ frontend: the DataType enumeration with sizes,
// descriptions and the promotion rule, mapped both ways onto torch dtypes, and the tagged host Scalar.
//
// Reference: infini_train/include/datatype.h:86-132 (13 types, kDataTypeToSize, kDataTypeToDesc,
// PromoteDataTypes: equal -> itself, fp16 with bf16 -> fp32, floating point beats integer, else the wider
// one) and include/scalar.h:12-82 (a value tagged bool / double / int64 / uint64 with checked casts).
// The reference's software FP16 / BF16 structs have no counterpart: tensors hold c10::Half / c10::BFloat16.
#pragma once
#include <torch/torch.h>

#include <cstdint>
#include <string>

namespace itb {

enum class DataType : int8_t {
  kBOOL, kUINT8, kINT8, kUINT16, kINT16, kUINT32, kINT32, kUINT64, kINT64, kBFLOAT16, kFLOAT16, kFLOAT32, kFLOAT64
};

inline size_t DataTypeSize(DataType t) {
  switch (t) {
    case DataType::kBOOL: case DataType::kUINT8: case DataType::kINT8: return 1;
    case DataType::kUINT16: case DataType::kINT16: case DataType::kBFLOAT16: case DataType::kFLOAT16: return 2;
    case DataType::kUINT32: case DataType::kINT32: case DataType::kFLOAT32: return 4;
    default: return 8;
  }
}
inline const char* DataTypeDesc(DataType t) {
  static const char* kNames[] = {"bool", "uint8", "int8", "uint16", "int16", "uint32", "int32", "uint64", "int64",
                                 "bfloat16", "float16", "float32", "float64"};
  return kNames[static_cast<int>(t)];
}
inline bool IsFloatingPoint(DataType t) { return t >= DataType::kBFLOAT16; }

inline DataType PromoteDataTypes(DataType a, DataType b) {
  if (a == b) return a;
  if ((a == DataType::kFLOAT16 && b == DataType::kBFLOAT16) || (a == DataType::kBFLOAT16 && b == DataType::kFLOAT16))
    return DataType::kFLOAT32;
  const bool af = IsFloatingPoint(a), bf = IsFloatingPoint(b);
  if (af != bf) return af ? a : b;
  return DataTypeSize(a) >= DataTypeSize(b) ? a : b;
}

inline torch::Dtype ToTorch(DataType t) {
  switch (t) {
    case DataType::kBOOL: return torch::kBool;
    case DataType::kUINT8: return torch::kUInt8;
    case DataType::kINT8: return torch::kInt8;
    case DataType::kUINT16: return torch::kUInt16;
    case DataType::kINT16: return torch::kInt16;
    case DataType::kUINT32: return torch::kUInt32;
    case DataType::kINT32: return torch::kInt32;
    case DataType::kUINT64: return torch::kUInt64;
    case DataType::kINT64: return torch::kInt64;
    case DataType::kBFLOAT16: return torch::kBFloat16;
    case DataType::kFLOAT16: return torch::kFloat16;
    case DataType::kFLOAT32: return torch::kFloat32;
    default: return torch::kFloat64;
  }
}
inline DataType FromTorch(torch::Dtype d) {
  switch (d) {
    case torch::kBool: return DataType::kBOOL;
    case torch::kUInt8: return DataType::kUINT8;
    case torch::kInt8: return DataType::kINT8;
    case torch::kUInt16: return DataType::kUINT16;
    case torch::kInt16: return DataType::kINT16;
    case torch::kUInt32: return DataType::kUINT32;
    case torch::kInt32: return DataType::kINT32;
    case torch::kUInt64: return DataType::kUINT64;
    case torch::kInt64: return DataType::kINT64;
    case torch::kBFloat16: return DataType::kBFLOAT16;
    case torch::kFloat16: return DataType::kFLOAT16;
    case torch::kFloat32: return DataType::kFLOAT32;
    case torch::kFloat64: return DataType::kFLOAT64;
    default: TORCH_CHECK(false, "dtype ", d, " has no DataType");
  }
}

// A host value tagged with its kind; To<T>() converts between kinds the way the reference does (bool ->
// 0 / 1, integers truncate doubles), ToTorch() hands it to libtorch.
class Scalar {
 public:
  enum class Kind { kBool, kDouble, kInt64, kUInt64 };
  Scalar() : kind_(Kind::kInt64) { v_.i = 0; }
  Scalar(bool b) : kind_(Kind::kBool) { v_.b = b; }
  Scalar(double d) : kind_(Kind::kDouble) { v_.d = d; }
  Scalar(float f) : kind_(Kind::kDouble) { v_.d = f; }
  Scalar(int i) : kind_(Kind::kInt64) { v_.i = i; }
  Scalar(int64_t i) : kind_(Kind::kInt64) { v_.i = i; }
  Scalar(uint64_t u) : kind_(Kind::kUInt64) { v_.u = u; }
  Kind kind() const { return kind_; }
  template <typename T>
  T To() const {
    switch (kind_) {
      case Kind::kBool: return static_cast<T>(v_.b);
      case Kind::kDouble: return static_cast<T>(v_.d);
      case Kind::kInt64: return static_cast<T>(v_.i);
      default: return static_cast<T>(v_.u);
    }
  }
  torch::Scalar ToTorch() const {
    switch (kind_) {
      case Kind::kBool: return torch::Scalar(v_.b);
      case Kind::kDouble: return torch::Scalar(v_.d);
      case Kind::kInt64: return torch::Scalar(v_.i);
      default: return torch::Scalar(static_cast<int64_t>(v_.u));
    }
  }

 private:
  Kind kind_;
  union {
    bool b;
    double d;
    int64_t i;
    uint64_t u;
  } v_;
};

}  // namespace itb
