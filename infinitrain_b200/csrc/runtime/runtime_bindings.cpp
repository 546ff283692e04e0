// Python bindings of the host runtime.
#include <torch/extension.h>

#include "runtime.h"

void bind_runtime(pybind11::module_& m) { (void)m; }
