// Python bindings of the multi-GPU kernels.
#include <torch/extension.h>

#include "comm.h"

void bind_comm(pybind11::module_& m) { (void)m; }
