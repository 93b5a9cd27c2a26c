/* launch.cuh -- launching kernels of a chain with programmatic dependent launch.
 *
 * The decode step is a chain of ~160 short kernels, each of which needs the
 * output of the one before.  Launched the plain way, an SM that finishes its
 * share of kernel N idles until the whole grid has drained and kernel N+1 has
 * been dispatched.  With the programmatic-serialization attribute the blocks of
 * N+1 start as soon as blocks of N leave, run the part of their work that does
 * not depend on N (for a projection: filling their shared-memory ring with
 * weights), and only then wait for N (griddepcontrol.wait).  Every kernel
 * launched through launch_chained() calls chain_wait() before it touches
 * anything an earlier kernel wrote.
 *
 * VXB_PDL=0 in the environment turns the attribute off (plain stream order).
 */
#ifndef VXB_LAUNCH_CUH
#define VXB_LAUNCH_CUH

#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>

namespace vxb {

/* All earlier kernels of the chain have finished and their writes are visible.
   A no-op for a kernel launched the plain way. */
__device__ __forceinline__ void chain_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
/* The next kernel of the chain may start its independent part. */
__device__ __forceinline__ void chain_release() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

/* A kernel that wants more than 48 KiB of dynamic shared memory has to opt in,
   and the opt-in belongs to the (kernel, device) pair: a process that places
   regions on several GPUs (spawn on(Topology::GPU[i]) switches the current
   device) needs it on each of them. Asked once per pair, for the current
   device; the answer of that one call is what every later call returns. */
inline cudaError_t allow_dynamic_smem(const void *kernel, int bytes) {
  static std::mutex mu;
  static std::map<std::pair<const void *, int>, cudaError_t> asked;
  int dev = 0;
  const cudaError_t which = cudaGetDevice(&dev);
  if (which != cudaSuccess)
    return which;
  std::lock_guard<std::mutex> lock(mu);
  const auto key = std::make_pair(kernel, dev);
  const auto hit = asked.find(key);
  if (hit != asked.end())
    return hit->second;
  const cudaError_t e = cudaFuncSetAttribute(
      kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  asked[key] = e;
  return e;
}

inline bool chain_enabled() {
  static const bool on = [] {
    const char *v = getenv("VXB_PDL");
    return !(v && strcmp(v, "0") == 0);
  }();
  return on;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block,
                           size_t smem, cudaStream_t stream, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chain_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

/* The same for a kernel whose blocks form clusters of `cluster_x` along x
   (grid.x a multiple of it): the blocks of a cluster run together and can read
   one another's shared memory. */
template <typename... KArgs, typename... Args>
cudaError_t launch_chained_cluster_smem(void (*kernel)(KArgs...), dim3 grid,
                                        dim3 block, unsigned cluster_x, size_t smem,
                                        cudaStream_t stream, Args &&...args);

template <typename... KArgs, typename... Args>
cudaError_t launch_chained_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                   unsigned cluster_x, cudaStream_t stream,
                                   Args &&...args) {
  return launch_chained_cluster_smem(kernel, grid, block, cluster_x, 0, stream,
                                     std::forward<Args>(args)...);
}

template <typename... KArgs, typename... Args>
cudaError_t launch_chained_cluster_smem(void (*kernel)(KArgs...), dim3 grid,
                                        dim3 block, unsigned cluster_x, size_t smem,
                                        cudaStream_t stream, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chain_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

} // namespace vxb

#endif /* VXB_LAUNCH_CUH */
