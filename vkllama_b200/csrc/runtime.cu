// Device, pooled allocator, tensors, commands and the host quantizer behind the
// C ABI. Replaces src/core of the reference (Vulkan device, VMA tensors,
// command buffers) with a CUDA device, a size-bucketed block pool and streams.
#include "runtime.h"

#include <math.h>
#include <stdio.h>

#include <algorithm>
#include <string.h>

namespace vkl {

static thread_local std::string g_err;
static std::atomic<uint64_t> g_launches{0};

int fail(int code, const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}
void count_launches(uint64_t n) { g_launches += n; }

size_t dtype_elem_bytes(int dtype) {
  switch (dtype) {
    case VKL_FP32: return 4;
    case VKL_FP16: return 2;
    case VKL_UINT32: return 4;
    case VKL_INT8: return 1;
    case VKL_Q8_0: return 1;
  }
  return 0;
}

int recording(vkl_command *cmd, const char *who) {
  if (!cmd) return fail(VKL_INVALID_ARGUMENT, "%s: null command", who);
  if (!cmd->recording)
    return fail(VKL_FAILED_PRECONDITION, "%s: command is not recording (call begin first)", who);
  return VKL_OK;
}

int tensor_new(vkl_device *dev, size_t c, size_t h, size_t w, int dtype, vkl_tensor **out) {
  if (!dev || !out) return fail(VKL_INVALID_ARGUMENT, "tensor: null device or output");
  if (dtype < VKL_FP32 || dtype > VKL_Q8_0) return fail(VKL_INVALID_ARGUMENT, "tensor: dtype %d is unknown", dtype);
  vkl_tensor *t = new vkl_tensor();
  t->dev = dev;
  t->dtype = dtype;
  t->c = c;
  t->h = h;
  t->w = w;
  t->update_strides();
  const size_t bytes = t->device_bytes();
  void *p = nullptr;
  if (int s = dev->alloc(bytes ? bytes : 16, &p)) {
    delete t;
    return s;
  }
  t->buf = std::make_shared<Buffer>(dev, p, bytes ? bytes : 16);
  *out = t;
  return VKL_OK;
}

int ensure_tensor(vkl_device *dev, vkl_tensor **slot, size_t c, size_t h, size_t w, int dtype) {
  vkl_tensor *t = *slot;
  if (t && t->c == c && t->h == h && t->w == w && t->dtype == dtype) return VKL_OK;
  if (t) vkl_tensor_release(t);
  *slot = nullptr;
  return tensor_new(dev, c, h, w, dtype, slot);
}

}  // namespace vkl

using namespace vkl;

// ------------------------------------------------------------------ device
// Size classes: multiples of 256 bytes up to 64 KiB, then four classes per power of two (at most
// 25 % over the request), so that calls with varying row counts land in a bounded set of sizes.
size_t vkl_device::size_class(size_t bytes) {
  if (bytes <= 65536) return (bytes + 255) & ~(size_t)255;
  size_t p2 = 65536;
  while (p2 * 2 < bytes) p2 *= 2;  // p2 < bytes <= 2 * p2
  const size_t step = p2 / 4;
  return (bytes + step - 1) / step * step;
}
static bool fences_done(vkl_device::FreeBlock &b, std::vector<cudaEvent_t> &spare) {
  while (!b.fences.empty()) {
    const cudaError_t q = cudaEventQuery(b.fences.back());
    if (q == cudaErrorNotReady) return false;
    (void)cudaGetLastError();  // a failed query (sticky error elsewhere) is not this block's problem: treat as done
    spare.push_back(b.fences.back());
    b.fences.pop_back();
  }
  return true;
}
int vkl_device::alloc(size_t bytes, void **out) {
  bytes = size_class(bytes);
  {
    std::lock_guard<std::mutex> lk(mu);
    auto range = pool.equal_range(bytes);
    for (auto it = range.first; it != range.second; ++it) {
      if (!fences_done(it->second, spare_events)) continue;  // queued work may still touch it
      *out = it->second.ptr;
      pool.erase(it);
      pooled_bytes -= bytes;
      return VKL_OK;
    }
  }
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) {
    // Give pooled blocks back to the driver once and retry (cudaFree waits for queued work).
    {
      std::lock_guard<std::mutex> lk(mu);
      for (auto &kv : pool) {
        cudaFree(kv.second.ptr);
        for (cudaEvent_t ev : kv.second.fences) spare_events.push_back(ev);
      }
      pool.clear();
      pooled_bytes = 0;
    }
    (void)cudaGetLastError();
    e = cudaMalloc(out, bytes);
  }
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(VKL_RESOURCE_EXHAUSTED, "device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
  }
  return VKL_OK;
}
void vkl_device::release(void *p, size_t bytes) {
  bytes = size_class(bytes);
  std::lock_guard<std::mutex> lk(mu);
  if (pooled_bytes + bytes > pool_cap) {
    cudaFree(p);  // synchronises with everything queued on the device
    return;
  }
  FreeBlock b{p, {}};
  int cur = -1;
  cudaGetDevice(&cur);
  if (cur != ordinal) cudaSetDevice(ordinal);
  for (cudaStream_t s : streams) {
    // a stream that is being captured runs nothing now (its work is being recorded into a graph):
    // no fence, and no event record that would become a node of that graph
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cs) != cudaSuccess) (void)cudaGetLastError();
    if (cs != cudaStreamCaptureStatusNone) continue;
    cudaEvent_t ev = nullptr;
    if (!spare_events.empty()) {
      ev = spare_events.back();
      spare_events.pop_back();
    } else if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) {
      (void)cudaGetLastError();
      ev = nullptr;
    }
    if (ev && cudaEventRecord(ev, s) == cudaSuccess) {
      b.fences.push_back(ev);
    } else {  // no fence could be set: wait for the stream instead
      (void)cudaGetLastError();
      if (ev) spare_events.push_back(ev);
      cudaStreamSynchronize(s);
      (void)cudaGetLastError();
    }
  }
  if (cur != ordinal && cur >= 0) cudaSetDevice(cur);
  pool.emplace(bytes, std::move(b));
  pooled_bytes += bytes;
}
void vkl_device::add_stream(cudaStream_t s) {
  std::lock_guard<std::mutex> lk(mu);
  streams.push_back(s);
}
void vkl_device::remove_stream(cudaStream_t s) {
  std::lock_guard<std::mutex> lk(mu);
  // blocks fenced on this stream: the caller has synchronised it, the events are complete
  streams.erase(std::remove(streams.begin(), streams.end(), s), streams.end());
}
size_t vkl_device::pool_bytes() {
  std::lock_guard<std::mutex> lk(mu);
  return pooled_bytes;
}
vkl_device::~vkl_device() {
  for (auto &kv : pool) {
    cudaFree(kv.second.ptr);
    for (cudaEvent_t ev : kv.second.fences) cudaEventDestroy(ev);
  }
  for (cudaEvent_t ev : spare_events) cudaEventDestroy(ev);
}

extern "C" {

const char *vkl_last_error(void) { return g_err.c_str(); }
uint64_t vkl_kernel_launches(void) { return g_launches.load(); }

int vkl_device_create(int ordinal, vkl_device **out) {
  if (!out) return fail(VKL_INVALID_ARGUMENT, "device_create: null output");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    (void)cudaGetLastError();
    return fail(VKL_FAILED_PRECONDITION, "no CUDA device is available (%s); this library has no CPU fallback",
                e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
  }
  if (ordinal < 0 || ordinal >= n) return fail(VKL_INVALID_ARGUMENT, "device %d does not exist (%d devices)", ordinal, n);
  VKL_CUDA(cudaSetDevice(ordinal));
  vkl_device *d = new vkl_device();
  d->ordinal = ordinal;
  cudaError_t pe = cudaGetDeviceProperties(&d->prop, ordinal);
  if (pe != cudaSuccess) {
    delete d;
    return fail(VKL_INTERNAL, "cudaGetDeviceProperties: %s", cudaGetErrorString(pe));
  }
  if (d->prop.major < 10) {
    const int major = d->prop.major, minor = d->prop.minor;
    delete d;
    return fail(VKL_FAILED_PRECONDITION, "device %d is sm_%d%d; this library is built for sm_100a only", ordinal, major, minor);
  }
  // free blocks kept for reuse: at most an eighth of the device memory
  d->pool_cap = d->prop.totalGlobalMem / 8;
  *out = d;
  return VKL_OK;
}
int vkl_device_pool_bytes(vkl_device *dev, size_t *bytes) {
  if (!dev || !bytes) return fail(VKL_INVALID_ARGUMENT, "device_pool_bytes: null argument");
  *bytes = dev->pool_bytes();
  return VKL_OK;
}
int vkl_device_destroy(vkl_device *dev) {
  if (!dev) return VKL_OK;
  cudaSetDevice(dev->ordinal);
  cudaDeviceSynchronize();
  // Tensors may outlive the handle (they are reference counted); the last
  // buffer to go frees the device record.
  dev->closed.store(true);
  if (dev->live_buffers.load() == 0) delete dev;
  return VKL_OK;
}
int vkl_device_info(vkl_device *dev, char *name, int *sm_count, size_t *total_mem) {
  if (!dev) return fail(VKL_INVALID_ARGUMENT, "device_info: null device");
  if (name) snprintf(name, 256, "%s", dev->prop.name);
  if (sm_count) *sm_count = dev->prop.multiProcessorCount;
  if (total_mem) *total_mem = dev->prop.totalGlobalMem;
  return VKL_OK;
}

}  // extern "C"

// ------------------------------------------------------------------ tensor
void vkl_tensor::update_strides() {
  // src/core/tensor.cpp:248-258, with the 34-byte block of the device/GGUF layout.
  const size_t items = dtype == VKL_Q8_0 ? 32 : 1;
  const size_t bpb = dtype == VKL_Q8_0 ? 34 : dtype_elem_bytes(dtype);
  ws = dtype_elem_bytes(dtype);
  hs = ((w + items - 1) / items) * bpb;
  cs = h * hs;
}
size_t vkl_tensor::host_bytes() const {
  const size_t items = dtype == VKL_Q8_0 ? 32 : 1;
  const size_t bpb = dtype == VKL_Q8_0 ? 34 : dtype_elem_bytes(dtype);
  return c * h * ((w + items - 1) / items) * bpb;
}
size_t vkl_tensor::device_bytes() const {
  if (dtype == VKL_Q8_0) return q8_layout((uint32_t)rows(), (uint32_t)w).total_bytes();
  return host_bytes();
}
bool vkl_tensor::dense() const {
  const size_t items = dtype == VKL_Q8_0 ? 32 : 1;
  const size_t bpb = dtype == VKL_Q8_0 ? 34 : dtype_elem_bytes(dtype);
  const size_t dhs = ((w + items - 1) / items) * bpb;
  return hs == dhs && cs == h * dhs;
}

namespace vkl {
int command_error_word(vkl_command *cmd, uint32_t **out) {
  if (!cmd->err_word) {
    void *p = nullptr;
    VKL_OKAY(cmd->dev->alloc(256, &p));
    VKL_CUDA(cudaMemsetAsync(p, 0, 256, cmd->stream));
    cmd->err_word = (uint32_t *)p;
  }
  cmd->err_used = true;
  *out = cmd->err_word;
  return VKL_OK;
}
}  // namespace vkl

extern "C" {

int vkl_tensor_create(vkl_device *dev, int c, int h, int w, int dtype, vkl_tensor **out) {
  if (c < 0 || h < 0 || w < 0) return fail(VKL_INVALID_ARGUMENT, "tensor_create: negative extent (%d, %d, %d)", c, h, w);
  return tensor_new(dev, (size_t)c, (size_t)h, (size_t)w, dtype, out);
}
int vkl_tensor_retain(vkl_tensor *t) {
  if (!t) return fail(VKL_INVALID_ARGUMENT, "tensor_retain: null tensor");
  t->ref.fetch_add(1);
  return VKL_OK;
}
int vkl_tensor_release(vkl_tensor *t) {
  if (!t) return VKL_OK;
  if (t->ref.fetch_sub(1) == 1) delete t;
  return VKL_OK;
}
int vkl_tensor_view(vkl_tensor *t, size_t c, size_t h, size_t w, vkl_tensor **out) {
  if (!t || !out) return fail(VKL_INVALID_ARGUMENT, "tensor_view: null argument");
  if (t->dtype == VKL_Q8_0) return fail(VKL_UNIMPLEMENTED, "tensor_view: Q8_0 tensors cannot be viewed");
  if (c > t->c || h > t->h || w > t->w)
    return fail(VKL_OUT_OF_RANGE, "view (%zu, %zu, %zu) exceeds tensor (%zu, %zu, %zu)", c, h, w, t->c, t->h, t->w);
  vkl_tensor *v = new vkl_tensor();
  v->dev = t->dev;
  v->buf = t->buf;
  v->dtype = t->dtype;
  v->c = c;
  v->h = h;
  v->w = w;
  v->cs = t->cs;  // a view keeps the parent's strides (tensor.cpp:294-302)
  v->hs = t->hs;
  v->ws = t->ws;
  *out = v;
  return VKL_OK;
}
int vkl_tensor_reshape(vkl_tensor *t, size_t c, size_t h, size_t w) {
  if (!t) return fail(VKL_INVALID_ARGUMENT, "tensor_reshape: null tensor");
  if (c * h * w != t->c * t->h * t->w)
    return fail(VKL_OUT_OF_RANGE, "reshape from (%zu, %zu, %zu) to (%zu, %zu, %zu) error.", t->c, t->h, t->w, c, h, w);
  if (t->dtype == VKL_Q8_0 && (w != t->w)) return fail(VKL_UNIMPLEMENTED, "reshape: Q8_0 rows cannot change width");
  t->c = c;
  t->h = h;
  t->w = w;
  t->update_strides();
  return VKL_OK;
}
int vkl_tensor_shape(vkl_tensor *t, uint32_t o[6]) {
  if (!t || !o) return fail(VKL_INVALID_ARGUMENT, "tensor_shape: null argument");
  o[0] = (uint32_t)t->c; o[1] = (uint32_t)t->h; o[2] = (uint32_t)t->w;
  o[3] = (uint32_t)t->cs; o[4] = (uint32_t)t->hs; o[5] = (uint32_t)t->ws;
  return VKL_OK;
}
int vkl_tensor_dtype(vkl_tensor *t, int *dtype) {
  if (!t || !dtype) return fail(VKL_INVALID_ARGUMENT, "tensor_dtype: null argument");
  *dtype = t->dtype;
  return VKL_OK;
}
int vkl_tensor_bytes(vkl_tensor *t, size_t *bytes) {
  if (!t || !bytes) return fail(VKL_INVALID_ARGUMENT, "tensor_bytes: null argument");
  *bytes = t->host_bytes();
  return VKL_OK;
}
int vkl_tensor_device_ptr(vkl_tensor *t, void **ptr) {
  if (!t || !ptr) return fail(VKL_INVALID_ARGUMENT, "tensor_device_ptr: null argument");
  *ptr = t->data();
  return VKL_OK;
}

// ----------------------------------------------------------------- command
int vkl_command_create(vkl_device *dev, vkl_command **out) {
  if (!dev || !out) return fail(VKL_INVALID_ARGUMENT, "command_create: null argument");
  VKL_CUDA(cudaSetDevice(dev->ordinal));
  vkl_command *c = new vkl_command();
  c->dev = dev;
  cudaError_t e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    delete c;
    return fail(VKL_INTERNAL, "cudaStreamCreate: %s", cudaGetErrorString(e));
  }
  cudaEventCreate(&c->ev0);
  cudaEventCreate(&c->ev1);
  dev->add_stream(c->stream);
  *out = c;
  return VKL_OK;
}
int vkl_command_destroy(vkl_command *cmd) {
  if (!cmd) return VKL_OK;
  cudaStreamSynchronize(cmd->stream);
  for (auto &f : cmd->deferred) f();
  if (cmd->err_word) cmd->dev->release(cmd->err_word, 256);
  cmd->dev->remove_stream(cmd->stream);
  cudaStreamDestroy(cmd->stream);
  if (cmd->ev0) cudaEventDestroy(cmd->ev0);
  if (cmd->ev1) cudaEventDestroy(cmd->ev1);
  delete cmd;
  return VKL_OK;
}
int vkl_command_begin(vkl_command *cmd) {
  if (!cmd) return fail(VKL_INVALID_ARGUMENT, "command_begin: null command");
  if (cmd->recording) return fail(VKL_FAILED_PRECONDITION, "command_begin: already recording");
  VKL_CUDA(cudaSetDevice(cmd->dev->ordinal));
  cmd->recording = true;
  cmd->submitted = false;
  VKL_CUDA(cudaEventRecord(cmd->ev0, cmd->stream));
  return VKL_OK;
}
int vkl_command_end(vkl_command *cmd) {
  if (!cmd) return fail(VKL_INVALID_ARGUMENT, "command_end: null command");
  if (!cmd->recording) return fail(VKL_FAILED_PRECONDITION, "command_end: not recording");
  cmd->recording = false;
  VKL_CUDA(cudaEventRecord(cmd->ev1, cmd->stream));
  return VKL_OK;
}
int vkl_command_submit(vkl_command *cmd) {
  if (!cmd) return fail(VKL_INVALID_ARGUMENT, "command_submit: null command");
  if (cmd->recording) return fail(VKL_FAILED_PRECONDITION, "command_submit: still recording (call end first)");
  cmd->submitted = true;  // work is already queued on the stream in order
  return VKL_OK;
}
int vkl_command_wait(vkl_command *cmd) {
  if (!cmd) return fail(VKL_INVALID_ARGUMENT, "command_wait: null command");
  cudaError_t e = cudaStreamSynchronize(cmd->stream);
  auto tasks = std::move(cmd->deferred);
  cmd->deferred.clear();
  for (auto &f : tasks) f();
  if (e != cudaSuccess) return fail(VKL_INTERNAL, "command_wait: %s", cudaGetErrorString(e));
  if (cmd->err_used) {
    uint32_t err = 0;
    cmd->err_used = false;
    VKL_CUDA(cudaMemcpy(&err, cmd->err_word, 4, cudaMemcpyDeviceToHost));
    if (err) {
      cudaMemset(cmd->err_word, 0, 4);
      return fail(VKL_INTERNAL, "command_wait: a bounded wait inside a kernel ran out (code %u)", err);
    }
  }
  return VKL_OK;
}
int vkl_command_elapsed_us(vkl_command *cmd, float *usec) {
  if (!cmd || !usec) return fail(VKL_INVALID_ARGUMENT, "command_elapsed_us: null argument");
  float ms = 0.f;
  cudaError_t e = cudaEventElapsedTime(&ms, cmd->ev0, cmd->ev1);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(VKL_FAILED_PRECONDITION, "command_elapsed_us: the command has not been recorded and waited on");
  }
  *usec = ms * 1000.f;
  return VKL_OK;
}
int vkl_command_stream(vkl_command *cmd, void **cuda_stream) {
  if (!cmd || !cuda_stream) return fail(VKL_INVALID_ARGUMENT, "command_stream: null argument");
  *cuda_stream = cmd->stream;
  return VKL_OK;
}
int vkl_command_submit_and_wait(vkl_command *cmd) {
  VKL_OKAY(vkl_command_submit(cmd));
  return vkl_command_wait(cmd);
}

int vkl_command_upload(vkl_command *cmd, const void *host, size_t bytes, vkl_tensor *to) {
  VKL_OKAY(recording(cmd, "upload"));
  if (!host || !to) return fail(VKL_INVALID_ARGUMENT, "upload: null argument");
  if (!to->dense()) return fail(VKL_UNIMPLEMENTED, "upload: destination must be dense");
  if (bytes > to->host_bytes())
    return fail(VKL_OUT_OF_RANGE, "upload: %zu bytes exceed the tensor's %zu", bytes, to->host_bytes());
  if (to->dtype == VKL_Q8_0) {
    if (bytes != to->host_bytes())
      return fail(VKL_INVALID_ARGUMENT, "upload: a Q8_0 tensor takes exactly %zu bytes of 34-byte blocks, got %zu",
                  to->host_bytes(), bytes);
    void *tmp = nullptr;
    VKL_OKAY(cmd->dev->alloc(bytes, &tmp));
    vkl_device *dev = cmd->dev;
    cmd->deferred.push_back([dev, tmp, bytes]() { dev->release(tmp, bytes); });
    VKL_CUDA(cudaMemcpyAsync(tmp, host, bytes, cudaMemcpyHostToDevice, cmd->stream));
    VKL_LAUNCH(1, launch_q8_repack((const uint8_t *)tmp, to->data(), (uint32_t)to->rows(), (uint32_t)to->w, cmd->stream));
    return VKL_OK;
  }
  VKL_CUDA(cudaMemcpyAsync(to->data(), host, bytes, cudaMemcpyHostToDevice, cmd->stream));
  return VKL_OK;
}

int vkl_command_download(vkl_command *cmd, vkl_tensor *from, void *host, size_t bytes) {
  VKL_OKAY(recording(cmd, "download"));
  if (!host || !from) return fail(VKL_INVALID_ARGUMENT, "download: null argument");
  if (bytes > from->host_bytes())
    return fail(VKL_OUT_OF_RANGE, "download: %zu bytes exceed the tensor's %zu", bytes, from->host_bytes());
  if (from->dtype == VKL_Q8_0) {
    const size_t full = from->host_bytes();
    void *tmp = nullptr;
    VKL_OKAY(cmd->dev->alloc(full, &tmp));
    vkl_device *dev = cmd->dev;
    cmd->deferred.push_back([dev, tmp, full]() { dev->release(tmp, full); });
    VKL_LAUNCH(1, launch_q8_unpack(from->data(), (uint8_t *)tmp, (uint32_t)from->rows(), (uint32_t)from->w, cmd->stream));
    VKL_CUDA(cudaMemcpyAsync(host, tmp, bytes, cudaMemcpyDeviceToHost, cmd->stream));
    return VKL_OK;
  }
  if (from->dense()) {
    VKL_CUDA(cudaMemcpyAsync(host, from->data(), bytes, cudaMemcpyDeviceToHost, cmd->stream));
    return VKL_OK;
  }
  // Strided view: copy row by row groups with a pitched copy per channel.
  const size_t row = from->w * from->ws;
  size_t left = bytes;
  uint8_t *dst = (uint8_t *)host;
  for (size_t c = 0; c < from->c && left; ++c) {
    const size_t rows = std::min(from->h, left / row);
    if (rows)
      VKL_CUDA(cudaMemcpy2DAsync(dst, row, from->data() + c * from->cs, from->hs, row, rows,
                                 cudaMemcpyDeviceToHost, cmd->stream));
    dst += rows * row;
    left -= rows * row;
    if (rows < from->h) break;
  }
  return VKL_OK;
}

// ---------------------------------------------------------- host quantizer
// src/core/quants.h:37-96: scale = absmax/127.0f; inverse = scale > 0 ?
// 127.0f/absmax : 0; code = (int8)roundf(x*inverse); tail codes are 0.
static void quantize_block(const float *src, size_t start, size_t n, float *scale_out, int8_t *codes) {
  float amax = fabsf(src[start]);
  for (size_t i = start; i < start + 32 && i < n; ++i) amax = std::max(fabsf(src[i]), amax);
  const float scale = amax / 127.0f;
  const float inv = scale > 0 ? 127.0f / amax : .0f;
  *scale_out = scale;
  for (size_t i = start; i < start + 32; ++i) codes[i - start] = i >= n ? (int8_t)0 : (int8_t)roundf(src[i] * inv);
}
static uint16_t host_f2h(float f) {
  const __half h = __float2half_rn(f);
  uint16_t u;
  memcpy(&u, &h, 2);
  return u;
}

int vkl_q8_0_quantize(const float *src, void *blocks34, size_t h, size_t w) {
  if (!src || !blocks34) return fail(VKL_INVALID_ARGUMENT, "q8_0_quantize: null argument");
  const size_t nb = (w + 31) / 32;
  uint8_t *dst = (uint8_t *)blocks34;
  for (size_t r = 0; r < h; ++r)
    for (size_t b = 0; b < nb; ++b) {
      float scale;
      uint8_t *blk = dst + (r * nb + b) * 34;
      quantize_block(src + r * w, b * 32, w, &scale, (int8_t *)(blk + 2));
      const uint16_t hs = host_f2h(scale);
      memcpy(blk, &hs, 2);
    }
  return VKL_OK;
}
int vkl_q8_0_quantize36(const float *src, void *blocks36, size_t h, size_t w) {
  if (!src || !blocks36) return fail(VKL_INVALID_ARGUMENT, "q8_0_quantize36: null argument");
  const size_t nb = (w + 31) / 32;
  uint8_t *dst = (uint8_t *)blocks36;
  for (size_t r = 0; r < h; ++r)
    for (size_t b = 0; b < nb; ++b) {
      float scale;
      uint8_t *blk = dst + (r * nb + b) * 36;
      quantize_block(src + r * w, b * 32, w, &scale, (int8_t *)(blk + 4));
      memcpy(blk, &scale, 4);
    }
  return VKL_OK;
}
int vkl_q8_0_dequantize(const void *blocks34, float *dst, size_t h, size_t w) {
  if (!dst || !blocks34) return fail(VKL_INVALID_ARGUMENT, "q8_0_dequantize: null argument");
  const size_t nb = (w + 31) / 32;
  const uint8_t *src = (const uint8_t *)blocks34;
  for (size_t r = 0; r < h; ++r)
    for (size_t b = 0; b < nb; ++b) {
      const uint8_t *blk = src + (r * nb + b) * 34;
      __half hs;
      memcpy(&hs, blk, 2);
      const float d = __half2float(hs);
      for (size_t i = 0; i < 32 && b * 32 + i < w; ++i) dst[r * w + b * 32 + i] = (float)(int8_t)blk[2 + i] * d;
    }
  return VKL_OK;
}
int vkl_q8_0_blocks36_to_34(const void *blocks36, void *blocks34, size_t n) {
  if (!blocks36 || !blocks34) return fail(VKL_INVALID_ARGUMENT, "blocks36_to_34: null argument");
  const uint8_t *s = (const uint8_t *)blocks36;
  uint8_t *d = (uint8_t *)blocks34;
  for (size_t b = 0; b < n; ++b) {
    float scale;
    memcpy(&scale, s + b * 36, 4);
    const uint16_t hs = host_f2h(scale);
    memcpy(d + b * 34, &hs, 2);
    memcpy(d + b * 34 + 2, s + b * 36 + 4, 32);
  }
  return VKL_OK;
}

int vkl_q8_0_quantize_device(vkl_command *cmd, vkl_tensor *src, vkl_tensor *dst) {
  VKL_OKAY(recording(cmd, "q8_0_quantize_device"));
  if (!src || !dst) return fail(VKL_INVALID_ARGUMENT, "q8_0_quantize_device: null tensor");
  if (src->dtype != VKL_FP32 || dst->dtype != VKL_Q8_0 || src->rows() != dst->rows() || src->w != dst->w)
    return fail(VKL_INVALID_ARGUMENT, "q8_0_quantize_device: need FP32 and Q8_0 tensors of one shape");
  const size_t bytes = dst->host_bytes();
  void *tmp = nullptr;
  VKL_OKAY(cmd->dev->alloc(bytes, &tmp));
  vkl_device *dev = cmd->dev;
  cmd->deferred.push_back([dev, tmp, bytes]() { dev->release(tmp, bytes); });
  VKL_LAUNCH(1, launch_q8_quantize((const float *)src->data(), (uint8_t *)tmp, (uint32_t)src->rows(), (uint32_t)src->w, cmd->stream));
  VKL_LAUNCH(1, launch_q8_repack((const uint8_t *)tmp, dst->data(), (uint32_t)dst->rows(), (uint32_t)dst->w, cmd->stream));
  return VKL_OK;
}

int vkl_tensor_fill_synthetic(vkl_command *cmd, vkl_tensor *t, uint64_t seed, uint64_t id, float mean, float stdv) {
  VKL_OKAY(recording(cmd, "fill_synthetic"));
  if (!t) return fail(VKL_INVALID_ARGUMENT, "fill_synthetic: null tensor");
  if (!t->dense()) return fail(VKL_UNIMPLEMENTED, "fill_synthetic: tensor must be dense");
  if (t->dtype == VKL_FP32) {
    VKL_LAUNCH(1, launch_synth_f32((float *)t->data(), seed, id, 0, t->size(), mean, stdv, cmd->stream));
  } else if (t->dtype == VKL_FP16) {
    VKL_LAUNCH(1, launch_synth_f16((__half *)t->data(), seed, id, 0, t->size(), mean, stdv, cmd->stream));
  } else if (t->dtype == VKL_Q8_0) {
    const size_t bytes = t->host_bytes();
    void *tmp = nullptr;
    VKL_OKAY(cmd->dev->alloc(bytes, &tmp));
    vkl_device *dev = cmd->dev;
    cmd->deferred.push_back([dev, tmp, bytes]() { dev->release(tmp, bytes); });
    VKL_LAUNCH(1, launch_synth_q8((uint8_t *)tmp, seed, id, (uint32_t)t->rows(), (uint32_t)t->w, mean, stdv, 0, 0, (uint32_t)t->w, cmd->stream));
    VKL_LAUNCH(1, launch_q8_repack((const uint8_t *)tmp, t->data(), (uint32_t)t->rows(), (uint32_t)t->w, cmd->stream));
  } else {
    return fail(VKL_UNIMPLEMENTED, "fill_synthetic: dtype %d", t->dtype);
  }
  return VKL_OK;
}

}  // extern "C"
