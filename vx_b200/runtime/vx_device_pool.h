/* vx_device_pool.h -- keep freed device buffers for the next dispatch of the
 * same size.
 *
 * A dispatch whose operands sit in host memory needs scratch device buffers,
 * and cudaMalloc/cudaFree cost more than a small GEMM.  Buffers are kept by
 * exact byte size (the same program asks for the same sizes again), up to a
 * byte budget; beyond it a release goes straight back to the allocator.
 * Interface and accounting follow the reference's runtime/vx_device_pool.h
 * :52-161 (its device_pool_test.cpp runs against this file).
 */
#ifndef VX_DEVICE_POOL_H
#define VX_DEVICE_POOL_H

#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include <utility>
#include <vector>

namespace vx {

template <typename Alloc, typename Free> class DevicePool {
public:
  struct Stats {
    uint64_t hits = 0;
    uint64_t misses = 0;
    size_t pooled_bytes = 0;
    size_t live = 0; /* handed out, not yet released */
  };

  DevicePool(Alloc alloc, Free free, size_t capacity_bytes)
      : alloc_(alloc), free_(free), budget_(capacity_bytes) {}
  ~DevicePool() { drain(); }
  DevicePool(const DevicePool &) = delete;
  DevicePool &operator=(const DevicePool &) = delete;

  void *acquire(size_t bytes) {
    if (bytes == 0)
      return nullptr;
    if (void *kept = pop(bytes))
      return kept;
    /* The allocator runs outside the lock: it may take milliseconds. */
    void *fresh = alloc_(bytes);
    if (!fresh) {
      drain(); /* what the pool holds may be what is in the way */
      fresh = alloc_(bytes);
    }
    if (fresh) {
      std::lock_guard<std::mutex> lock(mu_);
      ++s_.live;
    }
    return fresh;
  }

  void release(void *p, size_t bytes) {
    if (!p)
      return;
    {
      std::lock_guard<std::mutex> lock(mu_);
      if (s_.live)
        --s_.live;
      if (s_.pooled_bytes + bytes <= budget_) {
        kept_[bytes].push_back(p);
        s_.pooled_bytes += bytes;
        return;
      }
    }
    free_(p, bytes);
  }

  /* Give everything kept back to the allocator. */
  void drain() {
    std::unordered_map<size_t, std::vector<void *>> all;
    {
      std::lock_guard<std::mutex> lock(mu_);
      all.swap(kept_);
      s_.pooled_bytes = 0;
    }
    for (auto &bucket : all)
      for (void *p : bucket.second)
        free_(p, bucket.first);
  }

  Stats stats() {
    std::lock_guard<std::mutex> lock(mu_);
    return s_;
  }

private:
  void *pop(size_t bytes) {
    std::lock_guard<std::mutex> lock(mu_);
    auto bucket = kept_.find(bytes);
    if (bucket == kept_.end() || bucket->second.empty()) {
      ++s_.misses;
      return nullptr;
    }
    void *p = bucket->second.back();
    bucket->second.pop_back();
    s_.pooled_bytes -= bytes;
    ++s_.hits;
    ++s_.live;
    return p;
  }

  Alloc alloc_;
  Free free_;
  size_t budget_;
  std::mutex mu_;
  std::unordered_map<size_t, std::vector<void *>> kept_;
  Stats s_;
};

/* VX_CUDA_POOL_MAX_MB, default 2048 MiB; 0 turns pooling off. */
inline size_t vx_pool_capacity_bytes() {
  const size_t mib = (size_t)1 << 20;
  const char *text = getenv("VX_CUDA_POOL_MAX_MB");
  char *stop = nullptr;
  if (!text)
    return 2048 * mib;
  const unsigned long long n = strtoull(text, &stop, 10);
  return stop == text ? 2048 * mib : (size_t)n * mib;
}

} // namespace vx

#endif /* VX_DEVICE_POOL_H */
