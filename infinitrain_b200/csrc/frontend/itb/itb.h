// infinitrain_b200 C++ frontend: one include for programs written against the reference's C++ API shape.
//
//   #include "itb/itb.h"
//   auto model = std::make_shared<itb::nn::TransformerModel>(itb::nn::TransformerConfig::GPT2());
//   itb::optim::Adam opt(model->Parameters(), 1e-4);
//   auto loss = itb::ops::cross_entropy(model->forward(x), y);  loss.backward();  opt.Step();
//
// Build: g++ -std=c++17 -I infinitrain_b200/csrc/frontend against libtorch (examples/cpp/build.py);
// add -DITB_WITH_CUDA and link infinitrain_b200/_C.so for the sm_100a kernels.
#pragma once
#include "data.h"
#include "data_parallel.h"
#include "datatype.h"
#include "ddp.h"
#include "fault_tolerance.h"
#include "functional.h"
#include "io.h"
#include "layers.h"
#include "lora.h"
#include "module.h"
#include "ops.h"
#include "optim.h"
#include "parallel_env.h"
#include "pipeline.h"
#include "precision.h"
#include "profiler.h"
#include "process_group.h"
#include "runtime.h"
#include "tensor_api.h"
#include "tensor_parallel.h"
#include "tokenizer.h"
#include "transformer.h"
