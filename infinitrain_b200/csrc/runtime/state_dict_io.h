// Checkpoint state-dict files, shared by the Python bindings and the C++ frontend.
// Layout (little endian): uint32 magic 0x54504B43, uint32 version 1, uint32 count, then per tensor
// { uint32 name_len, name, int8 dtype code, uint32 ndim, int64 dims[ndim], uint64 bytes, raw data }
// (the reference's format: infini_train/src/checkpoint/checkpoint.cc:112-140).
#pragma once
#include <algorithm>
#include <torch/torch.h>

#include <cstdio>
#include <fstream>
#include <string>
#include <utility>
#include <vector>

namespace itb {

inline constexpr uint32_t kCkptMagic = 0x54504B43, kCkptVersion = 1;

inline int8_t dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kBool: return 0;
    case at::kByte: return 1;
    case at::kChar: return 2;
    case at::kUInt16: return 3;
    case at::kShort: return 4;
    case at::kUInt32: return 5;
    case at::kInt: return 6;
    case at::kUInt64: return 7;
    case at::kLong: return 8;
    case at::kBFloat16: return 9;
    case at::kHalf: return 10;
    case at::kFloat: return 11;
    case at::kDouble: return 12;
    default: TORCH_CHECK(false, "checkpoint: unsupported dtype ", t);
  }
}
inline at::ScalarType dtype_from_code(int8_t c) {
  static const at::ScalarType table[13] = {at::kBool,  at::kByte,   at::kChar, at::kUInt16,   at::kShort,
                                           at::kUInt32, at::kInt,   at::kUInt64, at::kLong,   at::kBFloat16,
                                           at::kHalf,  at::kFloat, at::kDouble};
  TORCH_CHECK(c >= 0 && c < 13, "checkpoint: bad dtype code ", int(c));
  return table[c];
}

inline void save_state_dict(const std::string& path, const std::vector<std::string>& names,
                     const std::vector<at::Tensor>& tensors) {
  TORCH_CHECK(names.size() == tensors.size(), "save_state_dict: names / tensors mismatch");
  const std::string tmp = path + ".tmp";
  {
    std::ofstream ofs(tmp, std::ios::binary);
    TORCH_CHECK(ofs.is_open(), "Failed to open checkpoint file: ", tmp);
    uint32_t count = static_cast<uint32_t>(names.size());
    ofs.write(reinterpret_cast<const char*>(&kCkptMagic), 4);
    ofs.write(reinterpret_cast<const char*>(&kCkptVersion), 4);
    ofs.write(reinterpret_cast<const char*>(&count), 4);
    for (size_t i = 0; i < names.size(); ++i) {
      at::Tensor t = tensors[i].detach().to(at::kCPU).contiguous();
      uint32_t len = static_cast<uint32_t>(names[i].size());
      ofs.write(reinterpret_cast<const char*>(&len), 4);
      ofs.write(names[i].data(), len);
      int8_t code = dtype_code(t.scalar_type());
      ofs.write(reinterpret_cast<const char*>(&code), 1);
      uint32_t ndim = static_cast<uint32_t>(t.dim());
      ofs.write(reinterpret_cast<const char*>(&ndim), 4);
      for (int64_t d : t.sizes()) ofs.write(reinterpret_cast<const char*>(&d), 8);
      uint64_t bytes = static_cast<uint64_t>(t.numel()) * t.element_size();
      ofs.write(reinterpret_cast<const char*>(&bytes), 8);
      ofs.write(static_cast<const char*>(t.data_ptr()), static_cast<std::streamsize>(bytes));
    }
    TORCH_CHECK(ofs.good(), "write failed: ", tmp);
  }
  TORCH_CHECK(std::rename(tmp.c_str(), path.c_str()) == 0, "rename failed: ", path);
}

inline std::vector<std::pair<std::string, at::Tensor>> load_state_dict(const std::string& path) {
  std::ifstream ifs(path, std::ios::binary);
  TORCH_CHECK(ifs.is_open(), "Failed to open checkpoint file: ", path);
  ifs.seekg(0, std::ios::end);
  const uint64_t file_size = static_cast<uint64_t>(ifs.tellg());
  ifs.seekg(0, std::ios::beg);
  uint32_t magic = 0, version = 0, count = 0;
  ifs.read(reinterpret_cast<char*>(&magic), 4);
  ifs.read(reinterpret_cast<char*>(&version), 4);
  ifs.read(reinterpret_cast<char*>(&count), 4);
  TORCH_CHECK(ifs.good() && magic == kCkptMagic, "Invalid checkpoint magic: ", path);
  TORCH_CHECK(version == kCkptVersion, "Unsupported checkpoint version: ", path);
  std::vector<std::pair<std::string, at::Tensor>> out;
  for (uint32_t i = 0; i < count; ++i) {
    uint32_t len = 0;
    ifs.read(reinterpret_cast<char*>(&len), 4);
    TORCH_CHECK(ifs.good() && len < (1u << 20), "Corrupt checkpoint (name length): ", path);
    std::string name(len, '\0');
    ifs.read(name.data(), len);
    int8_t code = 0;
    ifs.read(reinterpret_cast<char*>(&code), 1);
    uint32_t ndim = 0;
    ifs.read(reinterpret_cast<char*>(&ndim), 4);
    TORCH_CHECK(ifs.good() && ndim <= 16, "Corrupt checkpoint (rank): ", path);
    std::vector<int64_t> dims(ndim);
    for (auto& d : dims) ifs.read(reinterpret_cast<char*>(&d), 8);
    uint64_t bytes = 0;
    ifs.read(reinterpret_cast<char*>(&bytes), 8);
    TORCH_CHECK(ifs.good(), "Truncated checkpoint: ", path);
    // validate the record against itself and against the file BEFORE allocating: a corrupt dims or
    // bytes field must give a clear error, not a huge allocation
    const auto dtype = dtype_from_code(code);
    uint64_t numel = 1;
    for (int64_t d : dims) {
      TORCH_CHECK(d >= 0, "Corrupt checkpoint (negative dimension) for key: ", name);
      TORCH_CHECK(d == 0 || numel <= (uint64_t{1} << 56) / static_cast<uint64_t>(d),
                  "Corrupt checkpoint (dimensions overflow) for key: ", name);
      numel *= static_cast<uint64_t>(d);
    }
    TORCH_CHECK(bytes == numel * c10::elementSize(dtype), "Tensor bytes mismatch for key: ", name);
    TORCH_CHECK(bytes <= file_size - std::min<uint64_t>(file_size, static_cast<uint64_t>(ifs.tellg())),
                "Truncated checkpoint: ", path);
    at::Tensor t = torch::empty(dims, torch::dtype(dtype));
    ifs.read(static_cast<char*>(t.data_ptr()), static_cast<std::streamsize>(bytes));
    TORCH_CHECK(ifs.good() || (ifs.eof() && i + 1 == count && ifs.gcount() == (std::streamsize)bytes),
                "Truncated checkpoint: ", path);
    out.emplace_back(std::move(name), std::move(t));
  }
  return out;
}

}  // namespace itb
