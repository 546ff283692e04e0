// A small device-parameterised test harness for the native tests (no third-party test library is
// installed).  It plays the role of the reference's gtest fixtures (tests/common/test_utils.h:14-66:
// every test class instantiated for CPU and, when built with CUDA, for CUDA; SKIP_CPU / ONLY_CUDA /
// REQUIRE_MIN_DEVICES macros):
//
//   ITB_TEST_P(Suite, Name) { ... device() ... }   runs once per device the binary is asked for
//   ITB_TEST(Suite, Name) { ... }                  device-independent (runs in the cpu pass only)
//   ITB_ONLY_CUDA(); ITB_ONLY_CPU(); ITB_REQUIRE_MIN_DEVICES(n);     skip the current case
//   EXPECT(cond); EXPECT_NEAR(a, b, tol); EXPECT_THROWS(stmt);
//
//   <binary> --device cpu|cuda [--filter substring] [--list]
//
// Exit code 0: all selected cases passed (skipped ones are listed); 1: a case failed; 77: nothing
// could run (for example --device cuda without a visible GPU), which ctest reports as "skipped".
#pragma once
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <stdexcept>
#include <string>
#include <vector>

#include <unistd.h>

namespace itbtest {

enum class Dev { kCPU, kCUDA };

struct Skip : std::exception {
  std::string why;
  explicit Skip(std::string w) : why(std::move(w)) {}
  const char* what() const noexcept override { return why.c_str(); }
};
struct Failure : std::exception {
  std::string msg;
  explicit Failure(std::string m) : msg(std::move(m)) {}
  const char* what() const noexcept override { return msg.c_str(); }
};

// A fresh directory under $TMPDIR (or /tmp) for the files of one case; it is left for the system to clean.
inline std::string temp_dir(const std::string& tag) {
  const char* base = std::getenv("TMPDIR");
  std::string pattern = std::string(base && *base ? base : "/tmp") + "/itb_" + tag + "_XXXXXX";
  std::vector<char> buf(pattern.begin(), pattern.end());
  buf.push_back('\0');
  if (!mkdtemp(buf.data())) throw std::runtime_error("cannot create a temporary directory from " + pattern);
  return std::string(buf.data());
}

struct Case {
  std::string suite, name;
  bool parameterised;
  std::function<void()> fn;
};
inline std::vector<Case>& registry() {
  static std::vector<Case> r;
  return r;
}
inline Dev& current_device() {
  static Dev d = Dev::kCPU;
  return d;
}
inline int& visible_cuda_devices() {
  static int n = 0;
  return n;
}
struct Registrar {
  Registrar(const char* suite, const char* name, bool parameterised, std::function<void()> fn) {
    registry().push_back({suite, name, parameterised, std::move(fn)});
  }
};

inline void fail(const char* file, int line, const std::string& what) {
  throw Failure(std::string(file) + ":" + std::to_string(line) + ": " + what);
}

// How many CUDA devices the process can use; binaries without libtorch_cuda or the CUDA runtime
// override nothing and get 0.  Tests built on libtorch define ITB_TEST_WITH_TORCH before including.
inline int count_cuda_devices();

inline int run_all(int argc, char** argv) {
  std::string device = "cpu", filter;
  bool list = false;
  for (int i = 1; i < argc; ++i) {
    if (!std::strcmp(argv[i], "--device") && i + 1 < argc) device = argv[++i];
    else if (!std::strcmp(argv[i], "--filter") && i + 1 < argc) filter = argv[++i];
    else if (!std::strcmp(argv[i], "--list")) list = true;
  }
  if (device != "cpu" && device != "cuda") {
    std::fprintf(stderr, "unknown --device %s (cpu | cuda)\n", device.c_str());
    return 2;
  }
  current_device() = device == "cuda" ? Dev::kCUDA : Dev::kCPU;
  visible_cuda_devices() = count_cuda_devices();
  if (current_device() == Dev::kCUDA && visible_cuda_devices() == 0) {
    std::printf("SKIPPED: no CUDA device is visible\n");
    return 77;
  }
  int passed = 0, failed = 0, skipped = 0;
  for (const Case& c : registry()) {
    const std::string full = c.suite + "." + c.name + (c.parameterised ? "/" + device : std::string());
    if (!c.parameterised && current_device() == Dev::kCUDA) continue;   // device-independent: cpu pass only
    if (!filter.empty() && full.find(filter) == std::string::npos) continue;
    if (list) {
      std::printf("%s\n", full.c_str());
      continue;
    }
    try {
      c.fn();
      std::printf("[ ok      ] %s\n", full.c_str());
      ++passed;
    } catch (const Skip& s) {
      std::printf("[ skipped ] %s: %s\n", full.c_str(), s.what());
      ++skipped;
    } catch (const Failure& f) {
      std::printf("[ FAILED  ] %s\n    %s\n", full.c_str(), f.what());
      ++failed;
    } catch (const std::exception& e) {
      std::printf("[ FAILED  ] %s\n    unexpected exception: %s\n", full.c_str(), e.what());
      ++failed;
    }
  }
  if (list) return 0;
  std::printf("%d passed, %d failed, %d skipped (%s)\n", passed, failed, skipped, device.c_str());
  if (failed) return 1;
  return passed == 0 && skipped > 0 ? 77 : 0;
}

}  // namespace itbtest

#define ITB_TEST_IMPL(Suite, Name, Param)                                                       \
  static void itb_test_##Suite##_##Name();                                                      \
  static ::itbtest::Registrar itb_reg_##Suite##_##Name(#Suite, #Name, Param, itb_test_##Suite##_##Name); \
  static void itb_test_##Suite##_##Name()
#define ITB_TEST_P(Suite, Name) ITB_TEST_IMPL(Suite, Name, true)
#define ITB_TEST(Suite, Name) ITB_TEST_IMPL(Suite, Name, false)

#define ITB_ONLY_CUDA()                                                                        \
  do {                                                                                         \
    if (::itbtest::current_device() != ::itbtest::Dev::kCUDA) throw ::itbtest::Skip("CUDA only"); \
  } while (0)
#define ITB_ONLY_CPU()                                                                        \
  do {                                                                                        \
    if (::itbtest::current_device() != ::itbtest::Dev::kCPU) throw ::itbtest::Skip("CPU only"); \
  } while (0)
#define ITB_REQUIRE_MIN_DEVICES(n)                                                          \
  do {                                                                                      \
    if (::itbtest::visible_cuda_devices() < (n))                                            \
      throw ::itbtest::Skip("needs " #n " CUDA devices");                                   \
  } while (0)

#define EXPECT(cond)                                                  \
  do {                                                                \
    if (!(cond)) ::itbtest::fail(__FILE__, __LINE__, "EXPECT(" #cond ")"); \
  } while (0)
#define EXPECT_NEAR(a, b, tol)                                                                      \
  do {                                                                                              \
    const double itb_a = static_cast<double>(a), itb_b = static_cast<double>(b);                    \
    if (!(std::fabs(itb_a - itb_b) <= (tol)))                                                       \
      ::itbtest::fail(__FILE__, __LINE__, "EXPECT_NEAR(" #a ", " #b "): " + std::to_string(itb_a) + \
                                              " vs " + std::to_string(itb_b));                      \
  } while (0)
#define EXPECT_THROWS(stmt)                                                        \
  do {                                                                             \
    bool itb_threw = false;                                                        \
    try {                                                                          \
      stmt;                                                                        \
    } catch (const ::itbtest::Failure&) {                                          \
      throw;                                                                       \
    } catch (...) {                                                                \
      itb_threw = true;                                                            \
    }                                                                              \
    if (!itb_threw) ::itbtest::fail(__FILE__, __LINE__, "expected an exception: " #stmt); \
  } while (0)

#ifdef ITB_TEST_WITH_TORCH
#include <torch/torch.h>
namespace itbtest {
inline int count_cuda_devices() { return torch::cuda::is_available() ? static_cast<int>(torch::cuda::device_count()) : 0; }
// The torch device of the current pass.
inline torch::Device device() {
  return current_device() == Dev::kCUDA ? torch::Device(torch::kCUDA, 0) : torch::Device(torch::kCPU);
}
}  // namespace itbtest
#else
namespace itbtest {
inline int count_cuda_devices() { return 0; }
}  // namespace itbtest
#endif

#define ITB_TEST_MAIN() \
  int main(int argc, char** argv) { return ::itbtest::run_all(argc, argv); }
