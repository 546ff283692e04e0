// MUST NOT COMPILE: double is not an element type of the sm_100a kernels, so the typed launch front
// rejects it with a static_assert.  The build system registers a test that tries to build this file
// and passes only when the compiler refuses (the reference's negative compile test:
// tests/dtype/test_dtype_dispatch_compile_fail.cc, CMakeLists.txt:222-234).
#include "dtype_traits.h"

int main() {
  double* p = nullptr;
  float* q = nullptr;
  return itb_cast_typed(p, q, 0, nullptr);
}
