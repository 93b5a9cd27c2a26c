/* dispatch.cu -- the host side of libvx_cuda_dispatch.so for B200.
 *
 * Exports the vx_plugin_*, vx_collective_*, vx_host_worker_*, vx_cuda_*_stream
 * entry points that a compiled Vx program binds (include/vx_hardware_runtime.h)
 * and serves them with this repository's own sm_100a kernels: a `kind=matmul`
 * region runs a hand-written GEMM (kernels.h), a region that carries a PTX
 * image is loaded and launched through the driver API, placements are
 * cudaMalloc / cudaMallocAsync memory, collectives are NCCL on the caller's
 * stream.  It replaces the reference's runtime/cuda_dispatch.cpp; the entry
 * point each function stands in for is named at the function.
 *
 * Differences from the reference that are deliberate:
 *   - no cuBLAS anywhere;
 *   - no host fallback: a region placed on a GPU that this library cannot run
 *     on the GPU stops the program with a message (the reference runs it on
 *     CPU threads through libffi);
 *   - no remote-worker routing (a fleet manifest is not read).
 */
#include "kernels.h"
#include "vx_arrival_counts.h"
#include "vx_collective.h"
#include "vx_device_pool.h"
#include "vx_dispatch_plan.h"
#include "vx_kernel_launch.h"
#include "vx_stream_policy.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

/* ---------------------------------------------------------------- messages */
bool env_on(const char *name) {
  const char *v = getenv(name);
  return v && *v && strcmp(v, "0") != 0;
}
bool verbose() {
  static const bool on = env_on("VX_DISPATCH_VERBOSE");
  return on;
}
void say(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  fputs("[Vx CUDA] ", stderr);
  vfprintf(stderr, fmt, ap);
  fputc('\n', stderr);
  va_end(ap);
}
[[noreturn]] void fatal(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  fputs("[Vx CUDA] FATAL: ", stderr);
  vfprintf(stderr, fmt, ap);
  fputc('\n', stderr);
  va_end(ap);
  abort();
}
#define CUDA_OK(expr)                                                          \
  do {                                                                         \
    const cudaError_t e_ = (expr);                                             \
    if (e_ != cudaSuccess)                                                     \
      fatal("%s failed: %s", #expr, cudaGetErrorString(e_));                   \
  } while (0)

/* ------------------------------------------------------------- driver API
 * libcuda.so.1 is opened at run time: a build machine has the toolkit but no
 * driver, and every program must still link there. */
struct Driver {
  CUresult (*GetErrorName)(CUresult, const char **);
  CUresult (*ModuleLoadData)(CUmodule *, const void *);
  CUresult (*ModuleLoadDataEx)(CUmodule *, const void *, unsigned,
                               CUjit_option *, void **);
  CUresult (*ModuleGetFunction)(CUfunction *, CUmodule, const char *);
  CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int);
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned,
                           unsigned, unsigned, unsigned, CUstream, void **,
                           void **);
  CUresult (*CtxGetCurrent)(CUcontext *);
  CUresult (*CtxGetDevice)(CUdevice *);
  CUresult (*DevicePrimaryCtxRetain)(CUcontext *, CUdevice);
  CUresult (*DevicePrimaryCtxRelease)(CUdevice);
  CUresult (*OccupancyMaxActiveBlocksPerMultiprocessor)(int *, CUfunction, int,
                                                        size_t);
  CUresult (*TensorMapEncodeTiled)(
      CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
      const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
      const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
};

const Driver *driver_or_null() {
  static const Driver *api = []() -> const Driver * {
    void *lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) {
      say("cannot open libcuda.so.1: %s", dlerror());
      return nullptr;
    }
    static Driver d;
    bool whole = true;
    auto bind = [&](auto &fn, const char *name, bool required) {
      fn = reinterpret_cast<std::decay_t<decltype(fn)>>(dlsym(lib, name));
      if (!fn && required) {
        say("libcuda.so.1 has no %s", name);
        whole = false;
      }
    };
    bind(d.GetErrorName, "cuGetErrorName", true);
    bind(d.ModuleLoadData, "cuModuleLoadData", true);
    bind(d.ModuleLoadDataEx, "cuModuleLoadDataEx", true);
    bind(d.ModuleGetFunction, "cuModuleGetFunction", true);
    bind(d.FuncSetAttribute, "cuFuncSetAttribute", true);
    bind(d.LaunchKernel, "cuLaunchKernel", true);
    bind(d.CtxGetCurrent, "cuCtxGetCurrent", true);
    bind(d.CtxGetDevice, "cuCtxGetDevice", true);
    bind(d.DevicePrimaryCtxRetain, "cuDevicePrimaryCtxRetain", true);
    bind(d.DevicePrimaryCtxRelease, "cuDevicePrimaryCtxRelease_v2", true);
    bind(d.OccupancyMaxActiveBlocksPerMultiprocessor,
         "cuOccupancyMaxActiveBlocksPerMultiprocessor", true);
    bind(d.TensorMapEncodeTiled, "cuTensorMapEncodeTiled", false);
    return whole ? &d : nullptr;
  }();
  return api;
}

/* Whether this machine has a GPU this library can use. Said once. */
bool have_gpu() {
  static const bool yes = [] {
    int n = 0;
    const cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
      say("no CUDA device (%s)",
          e == cudaSuccess ? "none present" : cudaGetErrorString(e));
      cudaGetLastError();
      return false;
    }
    return driver_or_null() != nullptr;
  }();
  return yes;
}

const Driver &driver() {
  const Driver *d = driver_or_null();
  if (!d)
    fatal("the driver API was used on a machine where libcuda.so.1 did not "
          "load");
  return *d;
}

/* ------------------------------------------------ streams, waits, recording
 * (reference cuda_dispatch.cpp:188-325) */
thread_local cudaStream_t t_stream = nullptr;      /* vx_cuda_set_stream */
thread_local const char *t_last_on_stream = nullptr;

std::mutex g_unwaited_mu;
std::unordered_map<int, std::string> g_unwaited; /* device -> last kernel */

bool recording() {
  if (!t_stream)
    return false;
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  const cudaError_t e = cudaStreamIsCapturing(t_stream, &st);
  if (e != cudaSuccess)
    fatal("Vx could not ask whether the stream from vx_cuda_set_stream records "
          "a CUDA graph: %s.",
          cudaGetErrorString(e));
  return st != cudaStreamCaptureStatusNone;
}

[[noreturn]] void refuse_in_recording(
    const char *what,
    const char *fix = "Give the function only tensors in device memory, and "
                      "read its results after the recording ends.") {
  fatal("%s, while the stream from vx_cuda_set_stream records a CUDA graph.\n"
        "          A graph cannot hold this. %s",
        what, fix);
}

void wait_for_device() {
  std::unordered_map<int, std::string> started;
  {
    std::lock_guard<std::mutex> lock(g_unwaited_mu);
    started.swap(g_unwaited);
  }
  if (started.empty())
    return;
  int was = 0;
  cudaGetDevice(&was);
  for (const auto &entry : started) {
    cudaSetDevice(entry.first);
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess)
      fatal("a kernel faulted on GPU %d: %s.\n"
            "          The last kernel started there is %s. Set VX_CUDA_SYNC=1 "
            "to name the kernel that faulted.",
            entry.first, cudaGetErrorString(e), entry.second.c_str());
  }
  cudaSetDevice(was);
}

void wait_for_kernels(const char *why) {
  switch (vx_wait_action_for(t_stream != nullptr, recording())) {
  case VX_WAIT_DEVICE:
    wait_for_device();
    return;
  case VX_WAIT_REFUSE:
    refuse_in_recording(why);
  case VX_WAIT_STREAM:
    break;
  }
  const cudaError_t e = cudaStreamSynchronize(t_stream);
  if (e != cudaSuccess)
    fatal("a kernel faulted on the stream from vx_cuda_set_stream: %s.\n"
          "          The last kernel started there is %s. Set VX_CUDA_SYNC=1 to "
          "name the kernel that faulted.",
          cudaGetErrorString(e),
          t_last_on_stream ? t_last_on_stream : "unknown");
}

void started_kernel(const char *name) {
  static const bool sync_each = getenv("VX_CUDA_SYNC") != nullptr;
  int device = 0;
  cudaGetDevice(&device);
  if (sync_each) {
    if (recording())
      refuse_in_recording("VX_CUDA_SYNC=1 waits after each launch",
                          "Unset VX_CUDA_SYNC for a recording.");
    const cudaError_t e =
        t_stream ? cudaStreamSynchronize(t_stream) : cudaDeviceSynchronize();
    if (e != cudaSuccess)
      fatal("%s faulted on GPU %d: %s", name, device, cudaGetErrorString(e));
    return;
  }
  if (t_stream)
    t_last_on_stream = name;
  std::lock_guard<std::mutex> lock(g_unwaited_mu);
  static const bool at_exit = atexit(wait_for_device) == 0;
  (void)at_exit;
  g_unwaited[device] = name;
}

/* --------------------------------------------------------- device memory
 * (reference :327-340, :575-600) */
std::mutex g_on_stream_mu;
std::unordered_map<void *, cudaStream_t> g_on_stream; /* cudaMallocAsync'd */

/* Stream-ordered temporaries come from a pool of this library's own, one per
   device, that keeps what is freed (the default pool gives its memory back to
   the driver at the next synchronisation, and a product that needs 100 MB of
   scratch on every call then pays for the allocation every time). */
cudaMemPool_t stream_pool() {
  static std::mutex mu;
  static cudaMemPool_t pools[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!pools[dev]) {
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    cudaMemPool_t pool = nullptr;
    if (cudaMemPoolCreate(&pool, &props) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    uint64_t keep = UINT64_MAX;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    pools[dev] = pool;
  }
  return pools[dev];
}

cudaError_t device_alloc(void **ptr, size_t bytes) {
  if (!t_stream)
    return cudaMalloc(ptr, bytes);
  cudaMemPool_t pool = stream_pool();
  const cudaError_t e = pool ? cudaMallocFromPoolAsync(ptr, bytes, pool, t_stream)
                             : cudaMallocAsync(ptr, bytes, t_stream);
  if (e == cudaSuccess) {
    std::lock_guard<std::mutex> lock(g_on_stream_mu);
    g_on_stream[*ptr] = t_stream;
  }
  return e;
}

/* transfer_async copies that may still be running: device pointer -> event
   (reference :342-404). */
std::mutex g_copies_mu;
std::unordered_map<void *, cudaEvent_t> g_copies;

void stream_waits_for_copy(cudaStream_t stream, void *ptr) {
  cudaEvent_t ev = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_copies_mu);
    auto it = g_copies.find(ptr);
    if (it != g_copies.end())
      ev = it->second;
  }
  if (ev)
    CUDA_OK(cudaStreamWaitEvent(stream, ev, 0));
}

void finish_copy_into(void *ptr) {
  cudaEvent_t ev = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_copies_mu);
    auto it = g_copies.find(ptr);
    if (it == g_copies.end())
      return;
    ev = it->second;
    g_copies.erase(it);
  }
  CUDA_OK(cudaEventSynchronize(ev));
  CUDA_OK(cudaEventDestroy(ev));
}

void forget_ended_copies() {
  std::lock_guard<std::mutex> lock(g_copies_mu);
  for (auto it = g_copies.begin(); it != g_copies.end();) {
    if (cudaEventQuery(it->second) == cudaSuccess) {
      cudaEventDestroy(it->second);
      it = g_copies.erase(it);
    } else {
      ++it;
    }
  }
}

void device_free(void *ptr) {
  finish_copy_into(ptr);
  cudaStream_t from = nullptr;
  bool stream_ordered = false;
  {
    std::lock_guard<std::mutex> lock(g_on_stream_mu);
    auto it = g_on_stream.find(ptr);
    if (it != g_on_stream.end()) {
      from = it->second;
      stream_ordered = true;
      g_on_stream.erase(it);
    }
  }
  switch (vx_free_action_for(t_stream != nullptr, recording(), stream_ordered)) {
  case VX_FREE_ON_STREAM:
    cudaFreeAsync(ptr, from);
    return;
  case VX_FREE_REFUSE:
    refuse_in_recording("Vx freed device memory that needs a wait first");
  case VX_FREE_AFTER_DEVICE_WAIT:
  case VX_FREE_AFTER_STREAM_WAIT:
    wait_for_kernels("Vx freed device memory");
    cudaFree(ptr);
    return;
  }
}

bool is_device_ptr(const void *ptr) {
  if (!ptr)
    return false;
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, ptr) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

/* ------------------------------------------------ pinned staging for
 * transfer_async (reference :406-572): the caller may reuse its memory as soon
 * as the call returns, so the bytes go through pinned chunks of the runtime;
 * the GPU copies one chunk while host threads fill the next. */
constexpr size_t kChunkBytes = size_t(8) << 20;
constexpr int kChunks = 4;
constexpr size_t kStagingMinBytes = size_t(1) << 20;

struct Staging {
  std::mutex mu;
  void *host[kChunks] = {};
  cudaEvent_t copied[kChunks] = {};
  int next = 0;
  bool ok = false;
};

Staging *staging_for_current_device() {
  static std::mutex mu;
  static std::unordered_map<int, Staging *> all;
  int device = 0;
  CUDA_OK(cudaGetDevice(&device));
  std::lock_guard<std::mutex> lock(mu);
  Staging *&s = all[device];
  if (s)
    return s->ok ? s : nullptr;
  s = new Staging();
  s->ok = true;
  for (int i = 0; i < kChunks && s->ok; ++i) {
    if (cudaHostAlloc(&s->host[i], kChunkBytes, cudaHostAllocDefault) !=
            cudaSuccess ||
        cudaEventCreateWithFlags(&s->copied[i], cudaEventDisableTiming) !=
            cudaSuccess) {
      cudaGetLastError();
      s->ok = false;
    }
  }
  if (!s->ok)
    for (int i = 0; i < kChunks; ++i) {
      if (s->host[i])
        cudaFreeHost(s->host[i]);
      if (s->copied[i])
        cudaEventDestroy(s->copied[i]);
      s->host[i] = nullptr;
      s->copied[i] = nullptr;
    }
  return s->ok ? s : nullptr;
}

/* memcpy split over a few threads: one thread moves ~11 GB/s, the link ~54. */
void parallel_memcpy(void *dst, const void *src, size_t bytes) {
  static const unsigned parts =
      std::max(1u, std::min(4u, std::thread::hardware_concurrency() / 4));
  if (parts == 1 || bytes < (size_t(1) << 20)) {
    memcpy(dst, src, bytes);
    return;
  }
  const size_t each = ((bytes / parts) + 63) & ~size_t(63);
  std::vector<std::thread> helpers;
  for (unsigned i = 1; i < parts; ++i) {
    const size_t lo = std::min(bytes, each * i);
    const size_t hi = i + 1 == parts ? bytes : std::min(bytes, lo + each);
    helpers.emplace_back([=] {
      memcpy((char *)dst + lo, (const char *)src + lo, hi - lo);
    });
  }
  memcpy(dst, src, std::min(bytes, each));
  for (auto &t : helpers)
    t.join();
}

void copy_to_device_async(void *dev, const void *host, size_t bytes,
                          cudaStream_t stream) {
  Staging *s = bytes >= kStagingMinBytes ? staging_for_current_device() : nullptr;
  if (!s) {
    CUDA_OK(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, stream));
    return;
  }
  if (verbose())
    say("copy of %zu bytes through pinned memory", bytes);
  std::lock_guard<std::mutex> lock(s->mu);
  for (size_t done = 0; done < bytes; done += kChunkBytes) {
    const size_t n = std::min(kChunkBytes, bytes - done);
    const int c = s->next;
    s->next = (c + 1) % kChunks;
    CUDA_OK(cudaEventSynchronize(s->copied[c]));
    parallel_memcpy(s->host[c], (const char *)host + done, n);
    CUDA_OK(cudaMemcpyAsync((char *)dev + done, s->host[c], n,
                            cudaMemcpyHostToDevice, stream));
    CUDA_OK(cudaEventRecord(s->copied[c], stream));
  }
}

cudaStream_t copy_stream_of_current_device() {
  static std::mutex mu;
  static std::unordered_map<int, cudaStream_t> streams;
  int device = 0;
  CUDA_OK(cudaGetDevice(&device));
  std::lock_guard<std::mutex> lock(mu);
  cudaStream_t &s = streams[device];
  if (!s)
    CUDA_OK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  return s;
}

/* -------------------------------------------------------- which GPU
 * (reference :636-729) */
struct Declared {
  int32_t declared, builtin;
};
Declared g_local[64];
std::atomic<size_t> g_local_count{0};
std::mutex g_local_mu;

int gpu_index(int32_t topology_id) {
  const size_t n = g_local_count.load(std::memory_order_acquire);
  for (size_t i = 0; i < n; ++i)
    if (g_local[i].declared == topology_id) {
      topology_id = g_local[i].builtin;
      break;
    }
  return vx_topology_device_index(topology_id, VX_TOPO_GPU_BASE);
}

void require_primary_context(const char *why) {
  const Driver *d = driver_or_null();
  CUcontext cur = nullptr, primary = nullptr;
  CUdevice dev = 0;
  if (!d || d->CtxGetCurrent(&cur) != CUDA_SUCCESS || !cur)
    return;
  if (d->CtxGetDevice(&dev) != CUDA_SUCCESS ||
      d->DevicePrimaryCtxRetain(&primary, dev) != CUDA_SUCCESS)
    return;
  d->DevicePrimaryCtxRelease(dev);
  if (cur != primary)
    fatal("a %s found a CUDA context that is not the primary context of GPU "
          "%d.\n"
          "          Vx uses the primary context. Make it current with "
          "cuDevicePrimaryCtxRetain and\n"
          "          cuCtxSetCurrent, and allocate the buffers that you give Vx "
          "in it.",
          why, (int)dev);
}

/* Make the GPU that `topology_id` names current. An id that is not a GPU's
   leaves the current device alone. */
void select_device(int32_t topology_id, const char *why) {
  if (have_gpu())
    require_primary_context(why);
  const int index = gpu_index(topology_id);
  if (index < 0)
    return;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || index >= count)
    fatal("launch targets GPU %d, but this machine has %d", index, count);
  CUDA_OK(cudaSetDevice(index));
  if (verbose())
    say("device %d %s", index, why);
}

[[noreturn]] void no_gpu_for(const char *what, const char *name) {
  fatal("%s%s%s needs a GPU, and this machine has none that CUDA can use.\n"
        "          This dispatch library has no host fallback for tensors "
        "placed on a GPU.",
        what, name ? " " : "", name ? name : "");
}

/* ---------------------------------------------------- operand staging
 * (reference :843-980) */
using Pool = vx::DevicePool<void *(*)(size_t), void (*)(void *, size_t)>;
Pool &pool() {
  static Pool p(
      [](size_t bytes) -> void * {
        void *ptr = nullptr;
        if (cudaMalloc(&ptr, bytes) != cudaSuccess) {
          cudaGetLastError();
          return nullptr;
        }
        return ptr;
      },
      [](void *ptr, size_t) { cudaFree(ptr); }, vx::vx_pool_capacity_bytes());
  return p;
}

/* A matrix on the device: either the caller's own memory or a temporary that
   goes back to where it came from when this object dies. */
class Staged {
public:
  Staged() = default;
  Staged(const Staged &) = delete;
  Staged &operator=(const Staged &) = delete;
  Staged(Staged &&o) noexcept { *this = std::move(o); }
  Staged &operator=(Staged &&o) noexcept {
    if (this != &o) {
      drop();
      ptr = o.ptr;
      row_stride = o.row_stride;
      bytes_ = o.bytes_;
      kind_ = o.kind_;
      o.kind_ = Borrowed;
      o.ptr = nullptr;
    }
    return *this;
  }
  ~Staged() { drop(); }

  static Staged borrowed(void *p, int64_t stride) {
    Staged s;
    s.ptr = p;
    s.row_stride = stride;
    return s;
  }
  /* A temporary of `bytes`: stream-ordered under a caller stream, else pooled
     (pooled == false forces cudaMalloc: results are not pooled). */
  static Staged temporary(size_t bytes, int64_t stride, bool pooled) {
    Staged s;
    s.bytes_ = bytes;
    s.row_stride = stride;
    if (t_stream || !pooled) {
      if (device_alloc(&s.ptr, bytes) != cudaSuccess) {
        cudaGetLastError();
        s.ptr = nullptr;
      }
      s.kind_ = FromAlloc;
    } else {
      s.ptr = pool().acquire(bytes);
      s.kind_ = FromPool;
    }
    return s;
  }

  void *ptr = nullptr;
  int64_t row_stride = 0;

private:
  enum Kind { Borrowed, FromPool, FromAlloc };
  void drop() {
    if (ptr && kind_ == FromPool)
      pool().release(ptr, bytes_);
    else if (ptr && kind_ == FromAlloc)
      device_free(ptr);
    ptr = nullptr;
    kind_ = Borrowed;
  }
  size_t bytes_ = 0;
  Kind kind_ = Borrowed;
};

Staged stage(const void *data, int64_t rows, int64_t cols, int64_t row_stride,
             size_t elem) {
  if (is_device_ptr(data))
    return Staged::borrowed(const_cast<void *>(data), row_stride);
  if (recording())
    refuse_in_recording("Vx copied a tensor in host memory to the GPU");
  const size_t width = (size_t)cols * elem;
  Staged s = Staged::temporary((size_t)rows * width, cols, true);
  if (!s.ptr)
    fatal("out of device memory staging %zu bytes (%lld x %lld).",
          (size_t)rows * width, (long long)rows, (long long)cols);
  if (t_stream)
    CUDA_OK(cudaMemcpy2DAsync(s.ptr, width, data, (size_t)row_stride * elem,
                              width, (size_t)rows, cudaMemcpyHostToDevice,
                              t_stream));
  else
    CUDA_OK(cudaMemcpy2D(s.ptr, width, data, (size_t)row_stride * elem, width,
                         (size_t)rows, cudaMemcpyHostToDevice));
  return s;
}

/* ------------------------------------------------------------- the GEMM
 * (reference :988-1120, with this library's kernels where it calls cuBLAS) */
void gemm_on_device(const vx_gemm_plan &p, const Staged &a, const Staged &b,
                    void *c, int64_t ldc) {
  const char *why = nullptr;
  switch (p.dtype) {
  case VX_DTYPE_F32: {
    /* on the tensor cores as exact bf16 terms where the shape is for it
       (VXB_F32_TENSOR=0: always the FP32 pipe), else the FP32 kernel */
    const char *off = getenv("VXB_F32_TENSOR");
    const size_t need = (off && off[0] == '0')
                            ? 0
                            : vxb::gemm_f32_split_scratch_bytes(p.m, p.n, p.k, ldc);
    if (need) {
      Staged scratch = Staged::temporary(need, 0, true);
      if (scratch.ptr) {
        why = vxb::gemm_f32_split((const float *)a.ptr, a.row_stride,
                                  (const float *)b.ptr, b.row_stride, (float *)c,
                                  ldc, p.m, p.n, p.k, scratch.ptr, t_stream);
        break;
      }
    }
    why = vxb::gemm_f32((const float *)a.ptr, a.row_stride,
                        (const float *)b.ptr, b.row_stride, (float *)c, ldc,
                        p.m, p.n, p.k, t_stream);
    break;
  }
  case VX_DTYPE_F64:
    why = vxb::gemm_f64((const double *)a.ptr, a.row_stride,
                        (const double *)b.ptr, b.row_stride, (double *)c, ldc,
                        p.m, p.n, p.k, t_stream);
    break;
  case VX_DTYPE_F16:
  case VX_DTYPE_BF16:
    why = vxb::gemm_16(p.dtype == VX_DTYPE_BF16, a.ptr, a.row_stride, b.ptr,
                       b.row_stride, c, ldc, p.m, p.n, p.k, t_stream);
    break;
  default:
    fatal("unsupported GEMM element type %d", (int)p.dtype);
  }
  if (why)
    fatal("a GEMM %lldx%lldx%lld %s did not start: %s", (long long)p.m,
          (long long)p.n, (long long)p.k, vx_dtype_name(p.dtype), why);
}

void run_gemm(const vx_gemm_plan &p) {
  const size_t elem = vx_dtype_bytes(p.dtype);
  if (verbose())
    say("GEMM %lldx%lldx%lld %s -> %s", (long long)p.m, (long long)p.n,
        (long long)p.k, vx_dtype_name(p.dtype),
        p.out_kind == VX_GEMM_OUT_SLOT ? "slot" : "buffer");

  Staged a = stage(p.a_data, p.m, p.k, p.a_row_stride, elem);
  Staged b = stage(p.b_data, p.k, p.n, p.b_row_stride, elem);
  const bool in_place =
      p.out_kind == VX_GEMM_OUT_BUFFER && is_device_ptr(p.out_data);
  Staged c = in_place ? Staged::borrowed(p.out_data, p.out_row_stride)
                      : Staged::temporary((size_t)p.m * p.n * elem, p.n, false);
  if (!c.ptr)
    fatal("out of device memory for a %lldx%lld result", (long long)p.m,
          (long long)p.n);

  const bool timed = getenv("VX_TIME_KERNEL") != nullptr;
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  if (timed) {
    if (recording())
      refuse_in_recording("VX_TIME_KERNEL waits for each kernel",
                          "Unset VX_TIME_KERNEL for a recording.");
    cudaEventCreate(&t0);
    cudaEventCreate(&t1);
    cudaEventRecord(t0, t_stream);
  }
  gemm_on_device(p, a, b, c.ptr, c.row_stride);
  if (timed) {
    float ms = 0;
    cudaEventRecord(t1, t_stream);
    cudaEventSynchronize(t1);
    cudaEventElapsedTime(&ms, t0, t1);
    say("GEMM device time %.3f ms (%lldx%lldx%lld)", ms, (long long)p.m,
        (long long)p.n, (long long)p.k);
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
  }
  started_kernel("a GEMM");
  if (in_place)
    return;

  wait_for_kernels("Vx copied a GEMM result to host memory");
  const size_t width = (size_t)p.n * elem;
  if (p.out_kind == VX_GEMM_OUT_SLOT) {
    /* The program's allocator frees what a slot publishes: malloc memory. */
    void *result = malloc((size_t)p.m * width);
    if (!result)
      fatal("out of memory for a %lldx%lld result", (long long)p.m,
            (long long)p.n);
    CUDA_OK(cudaMemcpy(result, c.ptr, (size_t)p.m * width,
                       cudaMemcpyDeviceToHost));
    vx_gemm_publish_slot(&p, result);
  } else {
    CUDA_OK(cudaMemcpy2D(p.out_data, (size_t)p.out_row_stride * elem, c.ptr,
                         width, width, (size_t)p.m, cudaMemcpyDeviceToHost));
  }
}

/* ------------------------------------------- a compiler-emitted PTX image
 * (reference :1340-1674) */
unsigned dynamic_shared_bytes(const void *payload, size_t size) {
  const char *v = vx_payload_field(payload, size, "shared=");
  return v ? (unsigned)strtoul(v, nullptr, 10) : 0;
}

bool payload_is_ptx(const void *payload, size_t size) {
  const char *f = vx_payload_field(payload, size, "format=");
  return !f || strcmp(f, "ptx") == 0;
}

struct LoadedKernel {
  CUfunction fn;
  int params;
  std::vector<long> align;
};

bool run_device_image(const void *payload, size_t size, void **args,
                      const int32_t *tags, int64_t num_args) {
  const char *image = vx_payload_field(payload, size, "image=");
  const char *name = (const char *)payload;
  if (!image || !*image)
    return false;

  /* A module belongs to one context, and two libraries may both have a kernel
     of this name: the key has the kernel, the GPU and the library that holds
     the payload. */
  static std::unordered_map<std::string, LoadedKernel> cache;
  static std::mutex cache_mu;
  int device = 0;
  cudaGetDevice(&device);
  Dl_info where;
  const void *library = dladdr(payload, &where) ? where.dli_fbase : nullptr;
  char key_tail[64];
  snprintf(key_tail, sizeof key_tail, "@%d@%p", device, library);
  const std::string key = std::string(name) + key_tail;

  LoadedKernel k;
  {
    std::lock_guard<std::mutex> lock(cache_mu);
    auto hit = cache.find(key);
    if (hit != cache.end()) {
      k = hit->second;
    } else {
      if (recording()) {
        char what[256];
        snprintf(what, sizeof what,
                 "The first call of %s loaded its kernel image", name);
        refuse_in_recording(what,
                            "Call the function once before the recording.");
      }
      cudaFree(nullptr); /* make the primary context current */
      CUmodule mod = nullptr;
      CUresult rc;
      const char *cap = getenv("VX_MAXRREG");
      if (cap && *cap) {
        CUjit_option opt[1] = {CU_JIT_MAX_REGISTERS};
        void *val[1] = {(void *)(uintptr_t)(unsigned)atoi(cap)};
        rc = driver().ModuleLoadDataEx(&mod, image, 1, opt, val);
      } else {
        rc = driver().ModuleLoadData(&mod, image);
      }
      if (rc != CUDA_SUCCESS) {
        const char *err = nullptr;
        driver().GetErrorName(rc, &err);
        const bool sticky =
            rc == CUDA_ERROR_ILLEGAL_ADDRESS || rc == CUDA_ERROR_LAUNCH_FAILED ||
            rc == CUDA_ERROR_MISALIGNED_ADDRESS ||
            rc == CUDA_ERROR_ILLEGAL_INSTRUCTION ||
            rc == CUDA_ERROR_HARDWARE_STACK_ERROR ||
            rc == CUDA_ERROR_INVALID_ADDRESS_SPACE ||
            rc == CUDA_ERROR_INVALID_PC || rc == CUDA_ERROR_ASSERT;
        if (sticky)
          fatal("an earlier kernel failed on the GPU: %s.\n"
                "          The error showed when the device image for %s "
                "loaded. A common cause is a kernel\n"
                "          that uses memory the GPU cannot reach, such as a "
                "pointer to host memory.",
                err ? err : "?", name);
        const char *chip = vx_payload_field(payload, size, "chip=");
        fatal("the device image for %s did not load: %s.\n"
              "          It was compiled for %s. A known cause is an unresolved "
              "`__nv_` symbol\n"
              "          (libdevice was not linked -- set VX_LIBDEVICE).",
              name, err ? err : "?", chip ? chip : "sm_80");
      }
      if (driver().ModuleGetFunction(&k.fn, mod, name) != CUDA_SUCCESS)
        fatal("the device image loaded but has no entry named %s.", name);
      const unsigned shared = dynamic_shared_bytes(payload, size);
      if (shared > 48 * 1024) {
        rc = driver().FuncSetAttribute(
            k.fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)shared);
        if (rc != CUDA_SUCCESS) {
          int most = 0;
          const char *err = nullptr;
          cudaDeviceGetAttribute(&most, cudaDevAttrMaxSharedMemoryPerBlockOptin,
                                 device);
          driver().GetErrorName(rc, &err);
          fatal("%s needs %u bytes of shared memory, and GPU %d gives a block "
                "at most %d: %s.",
                name, shared, device, most, err ? err : "?");
        }
      }
      k.params = vx_launch_entry_param_count(image, name);
      k.align.assign(k.params > 0 ? k.params : 0, 0);
      vx_launch_param_aligns(image, name, k.align.data(), (int)k.align.size());
      cache.emplace(key, k);
    }
  }

  vx_launch_params params;
  if (!vx_launch_build_params(args, tags, num_args, &params))
    return false; /* a publication slot: no device form exists for it */

  /* `assert_flag=1` (reference runtime/vx_kernel_launch.h:379-393): the kernel
     takes one parameter more than the dispatch carries, a pointer to a 4-byte
     integer in device memory that a failed `assert` sets; the kernel then
     runs on to its end. The integer is cleared on the stream before the
     launch and read after it; a value other than 0 stops the program, as a
     failed assert on the host does. One integer per GPU, kept for the life of
     the process. Reading it waits for the kernel, which a recording graph
     cannot hold. */
  int32_t *assert_word = nullptr;
  void *assert_param = nullptr;
  if (vx_launch_takes_assert_flag(payload, size)) {
    if (recording())
      refuse_in_recording("A kernel built with asserts is checked after it ran",
                          "Build the kernel without asserts for a recording.");
    static std::mutex mu;
    static std::unordered_map<int, int32_t *> words;
    std::lock_guard<std::mutex> lock(mu);
    int32_t *&word = words[device];
    if (!word)
      CUDA_OK(cudaMalloc((void **)&word, sizeof(int32_t)));
    assert_word = word;
    if (params.count >= VX_LAUNCH_MAX_PARAMS)
      fatal("%s has more parameters than a launch can carry", name);
    assert_param = assert_word;
    params.params[params.count++] = &assert_param;
    CUDA_OK(cudaMemsetAsync(assert_word, 0, sizeof(int32_t), t_stream));
  }

  if (k.params != params.count)
    fatal("%s declares %d parameters and its arguments produced %d.\n"
          "          Launching would read past what was supplied. The compiler's "
          "idea of this kernel's\n"
          "          signature and the runtime's have diverged.",
          name, k.params, params.count);

  const int bad =
      vx_launch_misaligned(&params, k.align.data(), (int)k.align.size());
  if (bad >= 0) {
    uintptr_t at;
    memcpy(&at, params.params[bad], sizeof at);
    int64_t arg = 0;
    for (int first = 0; arg < num_args; ++arg) {
      first += vx_launch_param_width(tags[arg]);
      if (bad < first)
        break;
    }
    fatal("argument %lld of %s is at address %p. The machine file gives its "
          "memory space\n"
          "          `alignment: %ld B`, and the address is not a multiple of "
          "%ld. A tensor view over\n"
          "          memory from elsewhere must start at a multiple of the "
          "alignment of its space.",
          (long long)arg, name, (void *)at, k.align[bad], k.align[bad]);
  }

  /* Launch shape: what the `across` loops gave; else a grid-strided loop's trip
     count (one iteration per thread, blocks of up to 128, at most 4096 blocks);
     else one thread, because an unannotated region is a serial loop nest. */
  unsigned shape[3] = {1, 1, 1}, block = 1;
  char why[160];
  const int given =
      vx_launch_shape(payload, size, args, tags, num_args, shape, &block, why,
                      sizeof why);
  if (given < 0)
    fatal("%s: %s", name, why);
  if (!given) {
    long threads = 0;
    const long trip =
        vx_launch_trip(payload, size, args, tags, num_args, &threads);
    if (trip < 0 || threads < 0)
      fatal("%s: `launch=` names a launch value that is not an i32", name);
    if (threads != 0) {
      if (trip > 0) {
        shape[0] = (unsigned)std::min(trip, 4096L);
        block = (unsigned)std::min(threads, 1024L);
      }
    } else if (trip > 1) {
      block = (unsigned)std::min(trip, 128L);
      shape[0] = (unsigned)std::min(((unsigned long)trip + block - 1) / block,
                                    4096UL);
    }
  }

  const bool timed = getenv("VX_TIME_KERNEL") != nullptr;
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  if (timed) {
    if (recording())
      refuse_in_recording("VX_TIME_KERNEL waits for each kernel",
                          "Unset VX_TIME_KERNEL for a recording.");
    int resident = 0;
    if (driver().OccupancyMaxActiveBlocksPerMultiprocessor(
            &resident, k.fn, (int)block, 0) == CUDA_SUCCESS)
      say("%s occupancy: %d block(s) of %u threads per SM", name, resident,
          block);
    cudaEventCreate(&t0);
    cudaEventCreate(&t1);
    cudaEventRecord(t0, t_stream);
  }
  const CUresult rc = driver().LaunchKernel(
      k.fn, shape[0], shape[1], shape[2], block, 1, 1,
      dynamic_shared_bytes(payload, size), (CUstream)t_stream, params.params,
      nullptr);
  if (rc != CUDA_SUCCESS) {
    const char *err = nullptr;
    driver().GetErrorName(rc, &err);
    fatal("launching %s failed: %s", name, err ? err : "?");
  }
  started_kernel(name);
  if (assert_word) {
    int32_t failed = 0;
    const cudaError_t e = cudaMemcpyAsync(&failed, assert_word, sizeof failed,
                                          cudaMemcpyDeviceToHost, t_stream);
    const cudaError_t w =
        e == cudaSuccess ? cudaStreamSynchronize(t_stream) : e;
    if (w != cudaSuccess)
      fatal("%s faulted on GPU %d: %s", name, device, cudaGetErrorString(w));
    if (failed != 0)
      fatal("an assert failed in %s", name);
  }
  if (timed) {
    float ms = 0;
    cudaEventRecord(t1, t_stream);
    cudaEventSynchronize(t1);
    cudaEventElapsedTime(&ms, t0, t1);
    say("%s device time %.3f ms (%ux%u threads)", name, ms, shape[0], block);
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
  }
  if (verbose())
    say("%s ran on GPU %d from its own image (%d params, %ux%u threads)", name,
        device, params.count, shape[0], block);
  return true;
}

/* ---------------------------------------------------------- collectives */
vx::NcclCollective &job() {
  static vx::NcclCollective c(vx::CollectiveDevice{
      [] { return (void *)t_stream; },
      [] { return recording(); },
      [](const void *p) { return is_device_ptr(p); },
      [] {
        int d = 0;
        CUDA_OK(cudaGetDevice(&d));
        return d;
      },
      [](int d) { CUDA_OK(cudaSetDevice(d)); },
  });
  return c;
}
vx::OneRankCollective g_one_rank;

void collective_check(const std::string &why) {
  if (!why.empty())
    fatal("%s", why.c_str());
}

void warn_space_access_contradiction(uint32_t topology_id, size_t bytes) {
  static std::mutex mu;
  static std::unordered_map<uint32_t, bool> told;
  const bool strict = getenv("VX_STRICT_SPACES") != nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (told[topology_id] && !strict)
      return;
    told[topology_id] = true;
  }
  say("staging %zu bytes onto topology %u as device memory, but the program's "
      "machine model says the host may read that space (`managed:` is absent "
      "or `cached`).\n"
      "  Nothing here can honour that: this is cudaMalloc memory. A host read "
      "of it -- `print` on the result, most likely -- will fault.\n"
      "  Declare the space `managed: explicit` and the compiler will require "
      "the transfer home, or keep the operands in a space the host can read.",
      bytes, topology_id);
  if (strict)
    fatal("VX_STRICT_SPACES is set; refusing to stage.");
}

vx::ArrivalCounts &arrival_counts() {
  static vx::ArrivalCounts counts;
  return counts;
}

} // namespace

/* What the tensor-parallel helpers (nn_api.cu) need from this file. */
namespace vxb {
cudaStream_t caller_stream() { return t_stream; }
void note_kernel(const char *name) { started_kernel(name); }
vx::NcclCollective *nccl_job() { return have_gpu() ? &job() : nullptr; }
} // namespace vxb

extern "C" {

/* reference cuda_dispatch.cpp:1199-1254 */
void *vx_plugin_alloc_and_transfer(size_t bytes, void *host_ptr,
                                   uint32_t topology_id,
                                   uint32_t space_access) {
  if (gpu_index((int32_t)topology_id) < 0) {
    /* Not a GPU's memory: host memory, as for every backend. */
    void *p = malloc(bytes);
    if (p && host_ptr)
      memcpy(p, host_ptr, bytes);
    return p;
  }
  if (!have_gpu())
    no_gpu_for("a transfer to GPU memory", nullptr);
  select_device((int32_t)topology_id, "stage");
  if (space_access == VX_SPACE_ACCESS_HOST_READABLE)
    warn_space_access_contradiction(topology_id, bytes);
  void *dev = nullptr;
  CUDA_OK(device_alloc(&dev, bytes));
  if (host_ptr) {
    if (recording())
      refuse_in_recording("Vx copied a tensor in host memory to the GPU");
    if (t_stream)
      CUDA_OK(cudaMemcpyAsync(dev, host_ptr, bytes, cudaMemcpyHostToDevice,
                              t_stream));
    else
      CUDA_OK(cudaMemcpy(dev, host_ptr, bytes, cudaMemcpyHostToDevice));
  }
  return dev;
}

/* reference :1256-1281 */
void *vx_plugin_alloc_and_transfer_async(size_t bytes, void *host_ptr,
                                         uint32_t topology_id,
                                         uint32_t space_access) {
  if (!host_ptr || gpu_index((int32_t)topology_id) < 0 || !have_gpu() ||
      t_stream)
    return vx_plugin_alloc_and_transfer(bytes, host_ptr, topology_id,
                                        space_access);
  select_device((int32_t)topology_id, "stage");
  if (space_access == VX_SPACE_ACCESS_HOST_READABLE)
    warn_space_access_contradiction(topology_id, bytes);
  forget_ended_copies();
  void *dev = nullptr;
  CUDA_OK(device_alloc(&dev, bytes));
  cudaStream_t s = copy_stream_of_current_device();
  copy_to_device_async(dev, host_ptr, bytes, s);
  cudaEvent_t done = nullptr;
  CUDA_OK(cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
  CUDA_OK(cudaEventRecord(done, s));
  std::lock_guard<std::mutex> lock(g_copies_mu);
  g_copies[dev] = done;
  return dev;
}

/* reference :1283-1337 */
void *vx_plugin_transfer_peer(void *src, uint32_t src_topology_id,
                              uint32_t dst_topology_id, size_t bytes) {
  if (!have_gpu() || !is_device_ptr(src)) {
    void *dst = malloc(bytes);
    if (dst && src)
      memcpy(dst, src, bytes);
    return dst;
  }
  const int from = gpu_index((int32_t)src_topology_id);
  const int to = gpu_index((int32_t)dst_topology_id);
  if (from < 0 || to < 0)
    fatal("peer transfer between topologies %u and %u, which are not both GPUs",
          src_topology_id, dst_topology_id);
  finish_copy_into(src);
  select_device((int32_t)dst_topology_id, "peer");
  void *dst = nullptr;
  CUDA_OK(device_alloc(&dst, bytes));
  if (t_stream)
    CUDA_OK(cudaMemcpyPeerAsync(dst, to, src, from, bytes, t_stream));
  else
    CUDA_OK(cudaMemcpyPeer(dst, to, src, from, bytes));
  if (verbose())
    say("peer %d -> %d, %zu bytes", from, to, bytes);
  return dst;
}

/* reference :1676-1861 */
uint64_t vx_plugin_dispatch_async(const void *payload, size_t payload_size,
                                  void **device_args, const int32_t *arg_tags,
                                  int64_t num_args) {
  const char *name = (const char *)payload;
  const bool gpu = have_gpu();

  if (gpu)
    for (int64_t i = 0; i < num_args; ++i) {
      if (VX_ABI_KIND(arg_tags[i]) != VX_ABI_KIND_MEMREF || !device_args[i])
        continue;
      void *desc = *(void **)device_args[i];
      if (desc && VX_ABI_IS_SLOT(arg_tags[i]))
        desc = vx_memref_aligned(desc);
      if (desc)
        stream_waits_for_copy(t_stream, vx_memref_aligned(desc));
    }

  vx_gemm_plan plan;
  if (vx_gemm_plan_decode(payload, payload_size, device_args, arg_tags,
                          num_args, &plan)) {
    if (!gpu)
      no_gpu_for("the matrix product", name);
    select_device(vx_payload_topology(payload, payload_size), "dispatch");
    run_gemm(plan);
    return 1;
  }
  if (vx_payload_field(payload, payload_size, "image=") &&
      payload_is_ptx(payload, payload_size)) {
    if (!gpu)
      no_gpu_for("the kernel", name);
    select_device(vx_payload_topology(payload, payload_size), "dispatch");
    if (run_device_image(payload, payload_size, device_args, arg_tags,
                         num_args))
      return 1;
    fatal("%s has an argument that a GPU launch cannot carry (a publication "
          "slot), and this dispatch\n"
          "          library has no host fallback.",
          name ? name : "a kernel");
  }
  const char *kind = vx_payload_field(payload, payload_size, "kind=");
  fatal("%s (kind=%s) carries no PTX image and is not a matrix product, so "
        "there is nothing to run on\n"
        "          the GPU, and this dispatch library has no host fallback.",
        name ? name : "a kernel", kind ? kind : "<unclassified>");
}

/* reference :1863-1908 */
uint64_t vx_plugin_dispatch_async_flat(float *xout, float *x, float *w, int n,
                                       int d) {
  if (n <= 0 || d <= 0)
    return 1;
  if (!have_gpu())
    no_gpu_for("a matrix-vector product", nullptr);
  for (void *operand : {(void *)xout, (void *)x, (void *)w})
    stream_waits_for_copy(t_stream, operand);
  Staged dw = stage(w, d, n, n, sizeof(float));
  Staged dx = stage(x, 1, n, n, sizeof(float));
  const bool in_place = is_device_ptr(xout);
  Staged dy = in_place ? Staged::borrowed(xout, d)
                       : Staged::temporary((size_t)d * sizeof(float), d, false);
  if (!dy.ptr)
    fatal("out of device memory for a vector of %d values", d);
  if (const char *why =
          vxb::matvec_f32((float *)dy.ptr, (const float *)dx.ptr,
                          (const float *)dw.ptr, n, d, t_stream))
    fatal("a matrix-vector product did not start: %s", why);
  started_kernel("a matrix-vector product");
  if (!in_place) {
    wait_for_kernels("Vx copied a matrix-vector product to host memory");
    CUDA_OK(cudaMemcpy(xout, dy.ptr, (size_t)d * sizeof(float),
                       cudaMemcpyDeviceToHost));
  }
  return 1;
}

/* reference :1910-1914 */
void vx_plugin_await_future(uint64_t) {
  if (have_gpu())
    wait_for_kernels("Vx waited for a GPU region to finish");
}
void vx_plugin_release_future(uint64_t) {}

/* reference :1916-1938 */
int32_t vx_plugin_transfer_device_to_host(void *device_ptr, void *host_ptr,
                                          size_t bytes, uint32_t topology_id) {
  if (is_device_ptr(device_ptr)) {
    select_device((int32_t)topology_id, "fetch");
    finish_copy_into(device_ptr);
    wait_for_kernels("Vx copied a tensor to host memory");
    CUDA_OK(cudaMemcpy(host_ptr, device_ptr, bytes, cudaMemcpyDeviceToHost));
  } else {
    memcpy(host_ptr, device_ptr, bytes);
  }
  return 1;
}

/* reference :1940-1954 */
void vx_plugin_free(void *device_ptr, uint32_t topology_id) {
  if (!device_ptr)
    return;
  if (is_device_ptr(device_ptr)) {
    select_device((int32_t)topology_id, "free");
    device_free(device_ptr);
  } else {
    free(device_ptr);
  }
}

/* reference :1966-2026: a TMA descriptor for compiled code's lanes::copy_async,
   kept in device memory, one per distinct (descriptor, GPU). 0 = no map. */
int64_t vx_plugin_tensor_map(int64_t base, int64_t rank, int64_t elem_bytes,
                             int64_t d0, int64_t d1, int64_t d2, int64_t d3,
                             int64_t d4, int64_t s0, int64_t s1, int64_t s2,
                             int64_t s3, int64_t s4, int64_t b0, int64_t b1,
                             int64_t b2, int64_t b3, int64_t b4) {
  const int64_t dims[5] = {d0, d1, d2, d3, d4};
  const int64_t strides[5] = {s0, s1, s2, s3, s4};
  const int64_t box[5] = {b0, b1, b2, b3, b4};
  if (!have_gpu() || rank < 1 || rank > 5 || base % 16 != 0 ||
      (elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8) ||
      strides[rank - 1] != 1 || !is_device_ptr((void *)base))
    return 0;
  const Driver *api = driver_or_null();
  if (!api || !api->TensorMapEncodeTiled)
    return 0;
  /* The descriptor counts dimensions from the innermost one. */
  cuuint64_t gdim[5], gstride[4];
  cuuint32_t bdim[5], estride[5];
  for (int64_t r = 0; r < rank; ++r) {
    const int64_t d = rank - 1 - r;
    if (dims[d] < 1 || box[d] < 1 || box[d] > 256)
      return 0;
    gdim[r] = (cuuint64_t)dims[d];
    bdim[r] = (cuuint32_t)box[d];
    estride[r] = 1;
    if (r > 0) {
      const int64_t bytes = strides[d] * elem_bytes;
      if (bytes % 16 != 0)
        return 0;
      gstride[r - 1] = (cuuint64_t)bytes;
    }
  }
  CUtensorMap map;
  const CUtensorMapDataType type = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                   : elem_bytes == 4
                                       ? CU_TENSOR_MAP_DATA_TYPE_UINT32
                                       : CU_TENSOR_MAP_DATA_TYPE_UINT64;
  if (api->TensorMapEncodeTiled(&map, type, (cuuint32_t)rank, (void *)base,
                                gdim, gstride, bdim, estride,
                                CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_NONE,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return 0;
  int device = 0;
  CUDA_OK(cudaGetDevice(&device));
  std::string key((const char *)&map, sizeof map);
  key.append((const char *)&device, sizeof device);
  static std::mutex mu;
  static std::unordered_map<std::string, void *> maps;
  std::lock_guard<std::mutex> lock(mu);
  void *&on_device = maps[key];
  if (!on_device) {
    CUDA_OK(cudaMalloc(&on_device, sizeof map));
    CUDA_OK(cudaMemcpy(on_device, &map, sizeof map, cudaMemcpyHostToDevice));
  }
  return (int64_t)on_device;
}

/* reference :2030-2035 */
void vx_cuda_set_stream(void *stream) { t_stream = (cudaStream_t)stream; }
void *vx_cuda_get_stream(void) { return t_stream; }

/* A launch here never runs on host worker threads. */
int64_t vx_host_worker_id(void) { return 0; }
int64_t vx_host_worker_count(void) { return 1; }

/* reference :2064-2123 */
void vx_collective_init(int32_t rank, int32_t ranks) {
  if (!have_gpu()) {
    collective_check(g_one_rank.init(rank, ranks));
    return;
  }
  const char *lib = getenv("VX_NCCL_LIB");
  collective_check(job().init(rank, ranks, lib && *lib ? lib : "libnccl.so.2",
                              getenv("VX_NCCL_ID_FILE"),
                              std::chrono::seconds(300)));
}
void vx_collective_finish(void) {
  collective_check(have_gpu() ? job().finish() : g_one_rank.finish());
}
int32_t vx_collective_rank(void) {
  return have_gpu() ? job().rank() : g_one_rank.rank();
}
int32_t vx_collective_ranks(void) {
  return have_gpu() ? job().ranks() : g_one_rank.ranks();
}
void vx_collective_all_reduce_sum_f32(const float *in, float *out,
                                      int64_t count) {
  const char *fn = "vx_collective_all_reduce_sum_f32";
  collective_check(have_gpu() ? job().all_reduce_sum(in, out, count,
                                                     vx::NcclFloat32, fn)
                              : g_one_rank.copy(in, out, count, 4, fn));
}
void vx_collective_all_reduce_sum_bf16(const uint16_t *in, uint16_t *out,
                                       int64_t count) {
  const char *fn = "vx_collective_all_reduce_sum_bf16";
  collective_check(have_gpu() ? job().all_reduce_sum(in, out, count,
                                                     vx::NcclBfloat16, fn)
                              : g_one_rank.copy(in, out, count, 2, fn));
}
void vx_collective_all_gather_f32(const float *in, float *out, int64_t count) {
  const char *fn = "vx_collective_all_gather_f32";
  collective_check(have_gpu()
                       ? job().all_gather(in, out, count, vx::NcclFloat32, fn)
                       : g_one_rank.copy(in, out, count, 4, fn));
}
void vx_collective_all_gather_bf16(const uint16_t *in, uint16_t *out,
                                   int64_t count) {
  const char *fn = "vx_collective_all_gather_bf16";
  collective_check(have_gpu()
                       ? job().all_gather(in, out, count, vx::NcclBfloat16, fn)
                       : g_one_rank.copy(in, out, count, 2, fn));
}

/* reference :2130-2149 */
void *vx_plugin_arrivals_take(const void *site, size_t bytes, void *zeros,
                              uint32_t topology_id, uint32_t space_access) {
  if (void *kept = arrival_counts().take(site, topology_id, t_stream, bytes))
    return kept;
  return vx_plugin_alloc_and_transfer(bytes, zeros, topology_id, space_access);
}
void vx_plugin_arrivals_give(const void *site, void *count, size_t bytes,
                             uint32_t topology_id) {
  if (void *spare =
          arrival_counts().give(site, topology_id, t_stream, count, bytes))
    vx_plugin_free(spare, topology_id);
}

/* reference :2151-2207 */
int32_t vx_plugin_control(uint32_t opcode, void *payload) {
  switch (opcode) {
  case VX_CTRL_GET_DEVICE_COUNT: {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    return n;
  }
  case VX_CTRL_INIT_DEVICE:
    return have_gpu() ? 1 : 0;
  case VX_CTRL_WAIT:
  case VX_CTRL_WAIT_FOR_TENSORS:
  case VX_CTRL_WAIT_FOR_THREAD:
    if (have_gpu())
      wait_for_kernels("a read of GPU memory in place");
    return 1;
  case VX_CTRL_SHUTDOWN:
    if (have_gpu())
      cudaDeviceReset();
    return 1;
  case VX_CTRL_LOCAL_DEVICE: {
    const int32_t *pair = (const int32_t *)payload;
    if (!pair)
      return 0;
    std::lock_guard<std::mutex> lock(g_local_mu);
    const size_t n = g_local_count.load(std::memory_order_relaxed);
    for (size_t i = 0; i < n; ++i)
      if (g_local[i].declared == pair[0]) {
        if (g_local[i].builtin != pair[1])
          fatal("the topology %d is declared as two local devices, %d and %d",
                pair[0], g_local[i].builtin, pair[1]);
        return 1;
      }
    if (n == sizeof g_local / sizeof g_local[0])
      fatal("more than %zu declared local devices", n);
    g_local[n] = {pair[0], pair[1]};
    g_local_count.store(n + 1, std::memory_order_release);
    return 1;
  }
  default:
    return 0;
  }
}

} /* extern "C" */
