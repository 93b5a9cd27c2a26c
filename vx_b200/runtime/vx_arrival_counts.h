/* vx_arrival_counts.h -- the zeroed device counters that a kernel with code
 * after a nest of blocks needs, kept between launches.
 *
 * Each launch leaves its counter at 0 again, so the counter of the last launch
 * of the same `spawn` site on the same topology and stream can serve the next
 * one without a fresh allocation and copy.  One kept counter per
 * (site, topology, stream).  Same behaviour as the reference's
 * runtime/vx_arrival_counts.h:38-81.
 */
#ifndef VX_ARRIVAL_COUNTS_H
#define VX_ARRIVAL_COUNTS_H

#include <cstddef>
#include <cstdint>
#include <map>
#include <mutex>
#include <tuple>

namespace vx {

class ArrivalCounts {
public:
  /* The kept counter if it has at least `bytes`, else nullptr (the kept one,
     if any, stays). */
  void *take(const void *site, uint32_t topology, const void *stream,
             size_t bytes) {
    std::lock_guard<std::mutex> lock(mu_);
    auto at = kept_.find(Where(site, topology, stream));
    if (at == kept_.end() || at->second.second < bytes)
      return nullptr;
    void *counter = at->second.first;
    kept_.erase(at);
    return counter;
  }

  /* Keep `count` for the next launch. Returns the counter the caller must
     free: none, `count` itself when a counter at least as large is kept
     already, or the smaller one that `count` replaced. */
  void *give(const void *site, uint32_t topology, const void *stream,
             void *count, size_t bytes) {
    std::lock_guard<std::mutex> lock(mu_);
    auto put = kept_.emplace(Where(site, topology, stream),
                             std::make_pair(count, bytes));
    if (put.second)
      return nullptr;
    auto &have = put.first->second;
    if (have.second >= bytes)
      return count;
    void *spare = have.first;
    have = std::make_pair(count, bytes);
    return spare;
  }

  size_t size() {
    std::lock_guard<std::mutex> lock(mu_);
    return kept_.size();
  }

private:
  using Where = std::tuple<const void *, uint32_t, const void *>;
  std::mutex mu_;
  std::map<Where, std::pair<void *, size_t>> kept_;
};

} // namespace vx

#endif /* VX_ARRIVAL_COUNTS_H */
