/* static_scratch.cu -- decode attention for callers that must not allocate.
 *
 * The split-KV attention kernel needs scratch memory: one partial result per
 * (head, block of positions) and a counter per head.  vx_nn_attention takes
 * the partials from the caller (`part`) and keeps its counters in memory that
 * the library allocates on first use.  Some hosts cannot have that: a serving
 * process that gave every byte of device memory to its own pool at start-up
 * has nothing left for a later cudaMalloc, and a host inside a latency-bound
 * loop cannot take the device-wide synchronisation that cudaMalloc and
 * cudaFree imply.  For them this file offers the same attention with its
 * scratch in a fixed array that is part of the library image: every GPU that
 * loads the library holds kStaticScratchBytes of it until the process exits,
 * and nothing is ever allocated or freed here.
 *
 * The array is shared by every call on a device and keeps what the last call
 * left in it.  The counters region must be zero when a launch starts; each
 * launch leaves it zero again, and the first call on a device clears it.  Two
 * calls that overlap on the GPU (different streams) would write the same
 * partials and counters and race: keep calls on one device in stream order.
 * The array is kStaticScratchBytes = 68 KiB + 2 MiB.
 */
#include "kernels.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

namespace vxb {
cudaStream_t caller_stream();
void note_kernel(const char *name);
void set_last_error(const char *why);
} // namespace vxb

namespace {

/* Layout of the array, in bytes:
     [0, 64 Ki)          int32 table, entry i holds i: the kernel reads the
                         position from device memory, and `table + pos` is
                         that memory without a copy per call;
     [64 Ki, 65 Ki)      int32 counters, one per head tile;
     [68 Ki, 68 Ki + 2 Mi) the partial results. */
constexpr int kMaxPositions = 16384;
constexpr int kMaxHeads = 256;
constexpr size_t kCountersAt = (size_t)kMaxPositions * 4;
constexpr size_t kPartialsAt = kCountersAt + 4096;
constexpr size_t kMaxPartialFloats = (size_t)1 << 19; /* 2 MiB of partials */
constexpr size_t kStaticScratchBytes = kPartialsAt + kMaxPartialFloats * 4;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

/* Device code may name the array directly. */
__global__ void static_scratch_setup_kernel() {
  int32_t *table = reinterpret_cast<int32_t *>(g_static_scratch);
  int32_t *counters = reinterpret_cast<int32_t *>(g_static_scratch + kCountersAt);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < kMaxPositions;
       i += gridDim.x * blockDim.x)
    table[i] = i;
  if (blockIdx.x == 0 && threadIdx.x < kMaxHeads)
    counters[threadIdx.x] = 0;
}

struct DeviceSetup {
  unsigned char *base = nullptr; /* the array's address on this device */
};
constexpr int kMaxDevices = 64;
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mu;

/* The device address of the array for the current device. In host code the
   array's name stands for a host-side shadow, not for device memory, so the
   address comes from cudaGetSymbolAddress, once per device, with that device
   current. The same first call fills the position table and clears the
   counters (the partials need no clearing: every row that is read was written
   by the same launch). */
const char *scratch_for_current_device(unsigned char **base,
                                       cudaStream_t stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return "cannot tell which GPU is current";
  std::lock_guard<std::mutex> lock(g_setup_mu);
  if (!g_setup[dev].base) {
    void *p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      static thread_local char msg[160];
      snprintf(msg, sizeof msg, "cudaGetSymbolAddress failed: %s",
               cudaGetErrorString(e));
      return msg;
    }
    static_scratch_setup_kernel<<<16, 256, 0, stream>>>();
    if (cudaGetLastError() != cudaSuccess)
      return "could not set up the static scratch";
    g_setup[dev].base = (unsigned char *)p;
  }
  *base = g_setup[dev].base;
  return nullptr;
}

} // namespace

extern "C" {

/* Attention of the token at position `pos` over rows 0..pos of the KV cache:
 * the computation of vx_nn_attention (stdlib/std/nn.vx:349) on plain device
 * pointers -- q and out [q_heads, head_dim], caches [max_seq, kv_heads,
 * head_dim], all f32 -- with no allocation of any kind.  It has no counterpart
 * in the reference.
 *
 * It always runs the split kernel (one block per 32 positions below position
 * 640, per 64 from there on, as the reference cuts them), whose partial
 * results and per-head counters live in the array above.
 *
 * Limit: pos < 16384, q_heads <= 256 and
 * q_heads * (pos / n + 1) * (head_dim + 2) <= 2^19 with n = 32 or 64 as above
 * (for 32 heads of 128 that is every position below 8064).  Beyond it the
 * call returns -1 and vx_b200_last_error() says so.
 *
 * The first call on a GPU looks up the array's device address, fills its
 * position table and clears its counters; make that call before any stream
 * capture begins.  Every call on a GPU shares the array and each launch
 * leaves the counters at zero for the next; two calls that overlap on the GPU
 * (different streams) race on the partials and the counters.
 * Runs on the stream of vx_cuda_set_stream. Returns 0 when queued. */
int32_t vx_b200_attention_decode_static(float *out, const float *q,
                                        const float *k_cache,
                                        const float *v_cache, int32_t pos,
                                        int32_t q_heads, int32_t kv_heads,
                                        int32_t head_dim) {
  auto refuse = [](const char *why) {
    vxb::set_last_error(why);
    return -1;
  };
  if (pos < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 ||
      head_dim <= 0 || head_dim % 4 != 0 || head_dim > 128)
    return refuse("vx_b200_attention_decode_static: needs pos >= 0, q_heads a "
                  "multiple of kv_heads, head_dim a multiple of 4 up to 128");
  const int n_pos = pos >= 640 ? 64 : 32;
  const size_t need =
      (size_t)q_heads * ((size_t)pos / n_pos + 1) * ((size_t)head_dim + 2);
  if (q_heads > kMaxHeads || pos >= kMaxPositions || need > kMaxPartialFloats) {
    static thread_local char msg[256];
    snprintf(msg, sizeof msg,
             "vx_b200_attention_decode_static: %d heads at position %d need "
             "%zu floats of scratch, and the static scratch holds %zu (at "
             "most %d heads, positions below %d); use vx_nn_attention with "
             "its own scratch",
             q_heads, pos, need, kMaxPartialFloats, kMaxHeads, kMaxPositions);
    return refuse(msg);
  }
  cudaStream_t stream = vxb::caller_stream();
  unsigned char *base = nullptr;
  if (const char *why = scratch_for_current_device(&base, stream))
    return refuse(why);

  vxb::AttnArgs a{};
  a.q = q;
  a.k_cache = k_cache;
  a.v_cache = v_cache;
  a.cache_batch_stride = 0;
  a.out = out;
  a.q_heads = q_heads;
  a.kv_heads = kv_heads;
  a.head_dim = head_dim;
  a.batch = 1;
  a.positions = (const int32_t *)base + pos;
  a.max_pos = pos;
  a.counters = (int32_t *)(base + kCountersAt);
  a.scratch = (float *)(base + kPartialsAt);
  a.split = n_pos;
  a.kernel = vxb::kAttnSplit; /* the kernel that uses the scratch */
  if (const char *why = vxb::attention_decode(a, stream))
    return refuse(why);
  vxb::note_kernel("attention (static scratch)");
  return 0;
}

} /* extern "C" */
