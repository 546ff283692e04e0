// The positive control of compile_fail_dtype.cc: the same call with supported element types
// compiles (so that the negative test fails for the reason it names and not for a missing header).
#include "dtype_traits.h"

static_assert(ItbDtypeOf<float>::value == kItbF32, "float maps to kItbF32");
static_assert(ItbDtypeOf<__nv_bfloat16>::value == kItbBF16, "bf16 maps to kItbBF16");

int main() { return 0; }
