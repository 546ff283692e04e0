// C launch interface of the multi-GPU (NVLink / NVSwitch) kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
