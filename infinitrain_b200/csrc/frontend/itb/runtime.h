// Device runtime of the C++ frontend: devices, streams with priorities, events, raw device memory and
// copies, memory-pool high-water marks, and the RAII device guard.
//
// Reference: infini_train/include/core/runtime/device_guard.h:59-143 (DeviceGuardImpl: SetDevice /
// GetStream / CreateStreamWithPriority / EventRecord / StreamWaitEvent / EventElapsedTime /
// Malloc(Async) / Memcpy(Async) / GetMemPoolPeakMB), :107-143 (DeviceGuard), and the per-backend
// registry behind them (:145-199).  There is ONE accelerator backend here, so the registry collapses
// into `Runtime::For(device)`: a CUDA runtime on c10's streams, events and caching allocator (raw
// allocations come out of the same pool as the tensors, so a custom kernel's scratch memory shows
// up in the same statistics), and a CPU runtime with the same surface for code that is written
// against it and runs in CPU tests.
#pragma once
#include <torch/torch.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <utility>

#ifdef ITB_WITH_CUDA
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAFunctions.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>
#endif

namespace itb {
namespace core {

enum class MemcpyKind { kH2D, kD2H, kD2D, kH2H };
enum class RuntimeStatus { kSuccess, kNotReady, kError };
enum class EventFlag { kDefault, kDisableTiming, kBlockingSync };

// A queue of device work.  On the CPU there is one, and everything on it has completed by the time
// the call that enqueued it returns.
class Stream {
 public:
  explicit Stream(torch::Device device) : device_(device) {}
#ifdef ITB_WITH_CUDA
  Stream(torch::Device device, c10::cuda::CUDAStream s) : device_(device), cuda_(s) {}
  cudaStream_t handle() const { return cuda_.has_value() ? cuda_->stream() : nullptr; }
  const c10::optional<c10::cuda::CUDAStream>& cuda() const { return cuda_; }
  int priority() const { return cuda_.has_value() ? cuda_->priority() : 0; }
#else
  int priority() const { return 0; }
#endif
  torch::Device device() const { return device_; }

 private:
  torch::Device device_;
#ifdef ITB_WITH_CUDA
  c10::optional<c10::cuda::CUDAStream> cuda_;
#endif
};

class Event {
 public:
  explicit Event(EventFlag flags = EventFlag::kDefault) : flags_(flags) {
#ifdef ITB_WITH_CUDA
    unsigned f = cudaEventDefault;
    if (flags == EventFlag::kDisableTiming) f = cudaEventDisableTiming;
    if (flags == EventFlag::kBlockingSync) f = cudaEventBlockingSync;
    cuda_ = std::make_unique<at::cuda::CUDAEvent>(f);
#endif
  }
  EventFlag flags() const { return flags_; }

 private:
  friend class Runtime;
  EventFlag flags_;
  bool recorded_ = false, on_cuda_ = false;
  std::chrono::steady_clock::time_point host_time_;
#ifdef ITB_WITH_CUDA
  std::unique_ptr<at::cuda::CUDAEvent> cuda_;
#endif
};

class Runtime {
 public:
  // The runtime of a device type (the index of `device` is ignored: calls take the device they mean).
  static Runtime& For(torch::Device device) {
    static Runtime cpu(torch::kCPU), cuda(torch::kCUDA);
    if (device.is_cuda()) {
#ifndef ITB_WITH_CUDA
      TORCH_CHECK(false, "this build has no CUDA runtime (compile with -DITB_WITH_CUDA)");
#else
      // the caching allocator and the stream pools exist only after libtorch's lazy CUDA initialisation
      static const bool ready = (at::globalContext().lazyInitDevice(c10::DeviceType::CUDA), true);
      (void)ready;
#endif
      return cuda;
    }
    return cpu;
  }
  torch::DeviceType Type() const { return type_; }
  bool is_cuda() const { return type_ == torch::kCUDA; }

  // ---- devices
  int DeviceCount() const {
#ifdef ITB_WITH_CUDA
    if (is_cuda()) return static_cast<int>(c10::cuda::device_count());
#endif
    return 1;
  }
  torch::Device GetDevice() const {
#ifdef ITB_WITH_CUDA
    if (is_cuda()) return torch::Device(torch::kCUDA, c10::cuda::current_device());
#endif
    return torch::Device(torch::kCPU);
  }
  void SetDevice(torch::Device device) const {
    TORCH_CHECK(device.type() == type_, "SetDevice: device of another runtime");
#ifdef ITB_WITH_CUDA
    if (is_cuda()) c10::cuda::set_device(device.has_index() ? device.index() : 0);
#endif
  }

  // ---- streams
  Stream GetStream(torch::Device device) const {   // the stream kernels of this thread launch on
#ifdef ITB_WITH_CUDA
    if (is_cuda()) return Stream(device, c10::cuda::getCurrentCUDAStream(index_of(device)));
#endif
    return Stream(device);
  }
  Stream CreateStream(torch::Device device) const { return CreateStreamWithPriority(device, 0); }
  // priority: 0 = default, negative = higher (as the CUDA runtime counts).  Streams come from c10's
  // pools (32 per priority and device, handed out round robin), so "destroying" one is a no-op; c10
  // keeps fewer priority levels than the device offers and clamps the request to the highest it has.
  Stream CreateStreamWithPriority(torch::Device device, int priority) const {
#ifdef ITB_WITH_CUDA
    if (is_cuda()) return Stream(device, c10::cuda::getStreamFromPool(priority, index_of(device)));
#endif
    (void)priority;
    return Stream(device);
  }
  void DestroyStream(Stream*) const {}
  void GetStreamPriorityRange(int* low, int* high) const {
    *low = *high = 0;
#ifdef ITB_WITH_CUDA
    if (is_cuda()) {
      int least = 0, greatest = 0;
      TORCH_CHECK(cudaDeviceGetStreamPriorityRange(&least, &greatest) == cudaSuccess, "cudaDeviceGetStreamPriorityRange");
      *low = least, *high = greatest;   // numerically: high priority <= low priority
    }
#endif
  }
  // Makes `stream` the current stream of this thread until the returned guard dies (kernels of the
  // frontend and of libtorch launch on the current stream).
#ifdef ITB_WITH_CUDA
  std::unique_ptr<c10::cuda::CUDAStreamGuard> UseStream(const Stream& stream) const {
    TORCH_CHECK(stream.cuda().has_value(), "UseStream: not a CUDA stream");
    return std::make_unique<c10::cuda::CUDAStreamGuard>(*stream.cuda());
  }
#endif

  // ---- events
  void EventRecord(Event* event, const Stream& stream) const {
    event->recorded_ = true;
#ifdef ITB_WITH_CUDA
    if (is_cuda()) {
      event->on_cuda_ = true;
      event->cuda_->record(*stream.cuda());
      return;
    }
#endif
    (void)stream;
    event->host_time_ = std::chrono::steady_clock::now();
  }
  void StreamWaitEvent(const Stream& stream, Event* event) const {
    TORCH_CHECK(event->recorded_, "StreamWaitEvent: the event was never recorded");
#ifdef ITB_WITH_CUDA
    if (is_cuda()) event->cuda_->block(*stream.cuda());
#endif
    (void)stream;
  }
  RuntimeStatus EventSynchronize(Event* event) const {
    if (!event->recorded_) return RuntimeStatus::kError;
#ifdef ITB_WITH_CUDA
    if (event->on_cuda_) event->cuda_->synchronize();
#endif
    return RuntimeStatus::kSuccess;
  }
  RuntimeStatus EventQuery(Event* event) const {
    if (!event->recorded_) return RuntimeStatus::kError;
#ifdef ITB_WITH_CUDA
    if (event->on_cuda_) return event->cuda_->query() ? RuntimeStatus::kSuccess : RuntimeStatus::kNotReady;
#endif
    return RuntimeStatus::kSuccess;
  }
  // milliseconds between two recorded events (both must have completed; not for kDisableTiming events)
  float EventElapsedTime(Event* start, Event* stop) const {
    TORCH_CHECK(start->recorded_ && stop->recorded_, "EventElapsedTime: both events must have been recorded");
    TORCH_CHECK(start->flags_ != EventFlag::kDisableTiming && stop->flags_ != EventFlag::kDisableTiming,
                "EventElapsedTime: events created without timing");
#ifdef ITB_WITH_CUDA
    if (start->on_cuda_ && stop->on_cuda_) return start->cuda_->elapsed_time(*stop->cuda_);
#endif
    return std::chrono::duration<float, std::milli>(stop->host_time_ - start->host_time_).count();
  }

  // ---- synchronisation
  void SynchronizeDevice(torch::Device device) const {
#ifdef ITB_WITH_CUDA
    if (is_cuda()) {
      c10::cuda::CUDAGuard g(index_of(device));
      c10::cuda::device_synchronize();
    }
#endif
    (void)device;
  }
  void SynchronizeStream(const Stream& stream) const {
#ifdef ITB_WITH_CUDA
    if (is_cuda()) stream.cuda()->synchronize();
#endif
    (void)stream;
  }

  // ---- memory: raw blocks from the pool the tensors use (CUDA) or the C heap, 64-byte aligned (CPU)
  void Malloc(void** ptr, size_t size) const {
#ifdef ITB_WITH_CUDA
    if (is_cuda()) {
      *ptr = c10::cuda::CUDACachingAllocator::raw_alloc(size);
      return;
    }
#endif
    *ptr = size ? std::aligned_alloc(64, (size + 63) / 64 * 64) : nullptr;
    TORCH_CHECK(size == 0 || *ptr, "out of host memory");
  }
  // The block may be reused by later work of `stream` as soon as it is freed, without a device synchronisation.
  void MallocAsync(void** ptr, size_t size, const Stream& stream) const {
#ifdef ITB_WITH_CUDA
    if (is_cuda()) {
      *ptr = c10::cuda::CUDACachingAllocator::raw_alloc_with_stream(size, stream.handle());
      return;
    }
#endif
    (void)stream;
    Malloc(ptr, size);
  }
  void Free(void* ptr) const {
    if (!ptr) return;
#ifdef ITB_WITH_CUDA
    if (is_cuda()) {
      c10::cuda::CUDACachingAllocator::raw_delete(ptr);
      return;
    }
#endif
    std::free(ptr);
  }
  void FreeAsync(void* ptr, const Stream&) const { Free(ptr); }   // the caching pool defers reuse by stream itself
  void Memcpy(void* dst, const void* src, size_t count, MemcpyKind kind) const {
#ifdef ITB_WITH_CUDA
    if (is_cuda() && kind != MemcpyKind::kH2H) {
      auto s = c10::cuda::getCurrentCUDAStream();
      TORCH_CHECK(cudaMemcpyAsync(dst, src, count, ToCuda(kind), s.stream()) == cudaSuccess, "cudaMemcpyAsync failed");
      s.synchronize();
      return;
    }
#endif
    (void)kind;
    std::memcpy(dst, src, count);
  }
  void MemcpyAsync(void* dst, const void* src, size_t count, MemcpyKind kind, const Stream& stream) const {
#ifdef ITB_WITH_CUDA
    if (is_cuda() && kind != MemcpyKind::kH2H) {
      TORCH_CHECK(cudaMemcpyAsync(dst, src, count, ToCuda(kind), stream.handle()) == cudaSuccess, "cudaMemcpyAsync failed");
      return;
    }
#endif
    (void)kind, (void)stream;
    std::memcpy(dst, src, count);
  }
  void ResetMemPoolHighWatermarks(torch::Device device) const {
#ifdef ITB_WITH_CUDA
    if (is_cuda()) c10::cuda::CUDACachingAllocator::resetPeakStats(index_of(device));
#endif
    (void)device;
  }
  // (peak allocated, peak reserved) in MB since the last reset
  std::pair<size_t, size_t> GetMemPoolPeakMB(torch::Device device) const {
#ifdef ITB_WITH_CUDA
    if (is_cuda()) {
      const auto st = c10::cuda::CUDACachingAllocator::getDeviceStats(index_of(device));
      const size_t used = static_cast<size_t>(st.allocated_bytes[0].peak), reserved = static_cast<size_t>(st.reserved_bytes[0].peak);
      return {used >> 20, reserved >> 20};
    }
#endif
    (void)device;
    return {0, 0};
  }

 private:
  explicit Runtime(torch::DeviceType type) : type_(type) {}
#ifdef ITB_WITH_CUDA
  static c10::DeviceIndex index_of(torch::Device d) { return d.has_index() ? d.index() : c10::cuda::current_device(); }
  static cudaMemcpyKind ToCuda(MemcpyKind k) {
    switch (k) {
      case MemcpyKind::kH2D: return cudaMemcpyHostToDevice;
      case MemcpyKind::kD2H: return cudaMemcpyDeviceToHost;
      case MemcpyKind::kD2D: return cudaMemcpyDeviceToDevice;
      default: return cudaMemcpyHostToHost;
    }
  }
#endif
  torch::DeviceType type_;
};

// Switches this thread to `device` and back to where it was when the guard dies.
class DeviceGuard {
 public:
  explicit DeviceGuard(torch::Device device) : runtime_(Runtime::For(device)), original_(runtime_.GetDevice()), current_(device) {
    runtime_.SetDevice(device);
  }
  ~DeviceGuard() { runtime_.SetDevice(original_); }
  DeviceGuard(const DeviceGuard&) = delete;
  DeviceGuard& operator=(const DeviceGuard&) = delete;
  void SetDevice(torch::Device device) {
    runtime_.SetDevice(device);
    current_ = device;
  }
  torch::Device original_device() const { return original_; }
  torch::Device current_device() const { return current_; }

 private:
  Runtime& runtime_;
  torch::Device original_, current_;
};

}  // namespace core
}  // namespace itb
