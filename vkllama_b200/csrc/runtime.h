// Private C++ side of the C ABI: device, pooled allocator, tensors, commands.
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>

#include <atomic>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/vkllama_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace vkl {

int fail(int code, const char *fmt, ...);
void count_launches(uint64_t n);

#define VKL_CUDA(expr)                                                                   \
  do {                                                                                   \
    cudaError_t e__ = (expr);                                                            \
    if (e__ != cudaSuccess)                                                              \
      return ::vkl::fail(VKL_INTERNAL, "%s: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                         __FILE__, __LINE__);                                            \
  } while (0)
#define VKL_OKAY(expr)              \
  do {                              \
    int s__ = (expr);               \
    if (s__ != VKL_OK) return s__;  \
  } while (0)
// Launch + count (n kernels).
#define VKL_LAUNCH(n, expr) \
  do {                      \
    VKL_CUDA(expr);         \
    ::vkl::count_launches(n); \
  } while (0)

}  // namespace vkl

// Device memory comes from a pool of free blocks in size classes. Ops enqueue work and return
// without synchronising, and every command and model has its own non-blocking stream, so a block
// that is released may still be in use by queued kernels. release() therefore records an event on
// every stream of the device, and alloc() hands a pooled block out only when all of its events
// have completed (otherwise it takes another block or allocates a new one). The pool is capped:
// beyond `pool_cap` bytes a released block goes back to the driver (cudaFree synchronises).
struct vkl_device {
  struct FreeBlock {
    void *ptr;
    std::vector<cudaEvent_t> fences;  // work queued on the device's streams when the block was released
  };
  int ordinal = 0;
  cudaDeviceProp prop;
  std::mutex mu;
  std::multimap<size_t, FreeBlock> pool;  // free blocks by size class
  size_t pooled_bytes = 0, pool_cap = 0;
  std::vector<cudaStream_t> streams;       // streams of the live commands and models
  std::vector<cudaEvent_t> spare_events;
  std::atomic<int> live_buffers{0};    // tensors' buffers still referencing this device
  std::atomic<bool> closed{false};     // destroy was requested; the last buffer frees the device
  static size_t size_class(size_t bytes);
  int alloc(size_t bytes, void **out);
  void release(void *p, size_t bytes);
  void add_stream(cudaStream_t s);
  void remove_stream(cudaStream_t s);
  size_t pool_bytes();
  ~vkl_device();
};

namespace vkl {
struct Buffer {
  vkl_device *dev;
  void *ptr;
  size_t bytes;
  Buffer(vkl_device *d, void *p, size_t b) : dev(d), ptr(p), bytes(b) { dev->live_buffers.fetch_add(1); }
  Buffer(const Buffer &) = delete;
  ~Buffer() {
    dev->release(ptr, bytes);
    if (dev->live_buffers.fetch_sub(1) == 1 && dev->closed.load()) delete dev;
  }
};
size_t dtype_elem_bytes(int dtype);
// The command's device error word (allocated and zeroed on first use); wait() reports it.
int command_error_word(vkl_command *cmd, uint32_t **out);
}  // namespace vkl

struct vkl_tensor {
  std::atomic<int> ref{1};
  vkl_device *dev = nullptr;
  std::shared_ptr<vkl::Buffer> buf;
  int dtype = VKL_FP32;
  size_t c = 0, h = 0, w = 0;
  size_t cs = 0, hs = 0, ws = 0;  // bytes, as in the reference (host layout for Q8_0)
  void update_strides();
  size_t size() const { return c * h * w; }
  size_t rows() const { return c * h; }
  size_t host_bytes() const;    // dense host copy (34-byte blocks for Q8_0)
  size_t device_bytes() const;  // private device layout
  bool dense() const;
  uint8_t *data() const { return static_cast<uint8_t *>(buf->ptr); }
  // Q8_0 planes
  const uint8_t *codes() const { return data(); }
  const uint8_t *scales() const { return data() + vkl::q8_layout((uint32_t)rows(), (uint32_t)w).codes_bytes(); }
};

struct vkl_command {
  vkl_device *dev = nullptr;
  cudaStream_t stream = nullptr;
  bool recording = false;
  bool submitted = false;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;  // recorded by begin() and end()
  std::vector<std::function<void()>> deferred;  // run by wait()
  uint32_t *err_word = nullptr;  // device word raised by a kernel whose bounded wait ran out; read by wait()
  bool err_used = false;
};

namespace vkl {
int tensor_new(vkl_device *dev, size_t c, size_t h, size_t w, int dtype, vkl_tensor **out);
// Make *slot a dense tensor of this shape, reusing it when it already matches.
int ensure_tensor(vkl_device *dev, vkl_tensor **slot, size_t c, size_t h, size_t w, int dtype);
int recording(vkl_command *cmd, const char *who);
}  // namespace vkl
