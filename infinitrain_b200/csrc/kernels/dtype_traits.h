// Element types of the C launch interface as C++ types: ItbDtypeOf<T>::value is the dtype code the
// launchers take (kItbF32 / kItbBF16).  An element type the kernels do not implement is a COMPILE
// error, not a run-time one -- the single-backend counterpart of the reference's dtype dispatch, which
// static_asserts on a dtype that a kernel did not register (include/dtype_dispatch.h:230-336,
// tests/dtype/test_dtype_dispatch_compile_fail.cc).
#pragma once
#include <type_traits>

#include "kernels.h"

struct __nv_bfloat16;
namespace c10 {
struct BFloat16;
}

template <typename T>
struct ItbDtypeOf {
  // dependent on T so that it fires only when this primary template is instantiated
  static_assert(!std::is_same<T, T>::value,
                "infinitrain_b200: the sm_100a kernels take float and bfloat16 elements only");
  static constexpr int value = -1;
};
template <>
struct ItbDtypeOf<float> {
  static constexpr int value = kItbF32;
};
template <>
struct ItbDtypeOf<__nv_bfloat16> {
  static constexpr int value = kItbBF16;
};
template <>
struct ItbDtypeOf<c10::BFloat16> {
  static constexpr int value = kItbBF16;
};

// Typed front of the untyped launchers, e.g. itb_cast_typed(src, dst, n, stream) for any supported pair.
template <typename TS, typename TD>
inline int itb_cast_typed(const TS* src, TD* dst, long long n, cudaStream_t stream) {
  return itb_cast(src, ItbDtypeOf<TS>::value, dst, ItbDtypeOf<TD>::value, n, stream);
}
