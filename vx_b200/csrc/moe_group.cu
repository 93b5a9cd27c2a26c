/* moe_group.cu -- the (token, slot) pairs of a mixture-of-experts layer grouped
 * by expert: nn_moe_group_count, nn_moe_group_offsets, nn_moe_group_place and
 * nn_moe_group of stdlib/std/nn.vx:1056-1294.
 *
 * The result is a stable counting sort. order[] lists the pairs expert by
 * expert, each group starting at a multiple of `align` and padded to one;
 * a position i that holds no pair holds n + i. starts[e] is where group e
 * begins, starts[experts] where the last one ends with its padding;
 * tile_expert[t] names the expert that owns positions align*t .. align*t +
 * align - 1, or -1 past the last group. counts[b][e] and base[b][e] are the
 * per-block histogram and the per-block write cursor, a row for each 256 pairs:
 * they are outputs of the reference's kernels, so they are written here with
 * the same meaning.
 *
 * Integer work on a few thousand values: three short launches, the middle one a
 * single block. The histogram of a block is built with shared-memory atomics
 * (the reference has each of 1024 lanes scan the 256 keys), the group starts
 * with a two-level shuffle scan over the 1024 experts.
 */
#include "kernels.h"
#include "launch.cuh"

#include <cstdio>

namespace vxb {
namespace {

constexpr int kPairsPerBlock = 256;
constexpr int kMostExperts = 1024;

__device__ int g_group_status; /* 0x6E: an id that names no expert; 0x6F: a
                                  position outside `order` */

__global__ void __launch_bounds__(kPairsPerBlock)
group_count_kernel(int32_t *counts, int64_t pitch, const int32_t *ids, int n,
                   int experts) {
  __shared__ int hist[kMostExperts];
  for (int e = threadIdx.x; e < kMostExperts; e += kPairsPerBlock)
    hist[e] = 0;
  chain_release();
  chain_wait();
  __syncthreads();
  const int p = blockIdx.x * kPairsPerBlock + threadIdx.x;
  if (p < n) {
    const int id = ids[p];
    if (id >= 0 && id < experts)
      atomicAdd(&hist[id], 1);
    else
      atomicCAS(&g_group_status, 0, 0x6E);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += kPairsPerBlock)
    counts[blockIdx.x * pitch + e] = hist[e];
}

/* One block of 1024 threads; thread e owns expert e. */
__global__ void __launch_bounds__(kMostExperts)
group_offsets_kernel(int32_t *base, int64_t base_pitch, int32_t *starts,
                     int32_t *tile_expert, int tiles, int32_t *order, int room,
                     const int32_t *counts, int64_t counts_pitch, int n,
                     int experts, int align) {
  __shared__ int first[kMostExperts]; /* where group e starts */
  __shared__ int size[kMostExperts];  /* its pairs, without padding */
  __shared__ int warp_total[32];
  __shared__ int end_of_groups;
  chain_release();
  chain_wait();
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  const int blocks = (n + kPairsPerBlock - 1) / kPairsPerBlock;

  int mine = 0;
  if (e < experts)
    for (int b = 0; b < blocks; ++b)
      mine += counts[b * counts_pitch + e];
  const int padded = e < experts ? (mine + align - 1) / align * align : 0;

  /* exclusive prefix sum of `padded` over the 1024 threads */
  int scan = padded;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, scan, o);
    if (lane >= o)
      scan += up;
  }
  if (lane == 31)
    warp_total[warp] = scan;
  __syncthreads();
  if (warp == 0) {
    const int total = warp_total[lane];
    int s = total;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o)
        s += up;
    }
    warp_total[lane] = s - total; /* exclusive */
    if (lane == 31)
      end_of_groups = s;
  }
  __syncthreads();
  const int start = warp_total[warp] + scan - padded;
  first[e] = start;
  size[e] = mine;
  if (e < experts) {
    starts[e] = start;
    int cursor = start;
    for (int b = 0; b < blocks; ++b) {
      base[b * base_pitch + e] = cursor;
      cursor += counts[b * counts_pitch + e];
    }
  }
  const int end = end_of_groups;
  if (e == 0)
    starts[experts] = end;
  __syncthreads();

  /* The owner of each tile, and n + i wherever no pair will be placed: the
     padding at the end of a group's last tile, and everything past the last
     group. */
  for (int t = threadIdx.x; t < tiles; t += kMostExperts) {
    const int64_t at = (int64_t)t * align;
    if (at < end) {
      int lo = 0, hi = experts; /* the last expert whose group starts at or before `at` */
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (first[mid] <= at)
          lo = mid;
        else
          hi = mid;
      }
      tile_expert[t] = lo;
      int64_t i = (int64_t)first[lo] + size[lo];
      if (i < at)
        i = at;
      for (; i < at + align; ++i)
        order[i] = (int32_t)(n + i);
    } else {
      tile_expert[t] = -1;
      for (int64_t i = at; i < at + align && i < room; ++i)
        order[i] = (int32_t)(n + i);
    }
  }
}

__global__ void __launch_bounds__(kPairsPerBlock)
group_place_kernel(int32_t *order, int room, const int32_t *ids,
                   const int32_t *base, int64_t pitch, int n, int experts) {
  __shared__ int keys[kPairsPerBlock];
  chain_release();
  chain_wait();
  const int l = threadIdx.x;
  const int p = blockIdx.x * kPairsPerBlock + l;
  const int id = p < n ? ids[p] : -1;
  keys[l] = id;
  __syncthreads();
  if (id < 0 || id >= experts)
    return; /* past the end, or refused by the count kernel already */
  int rank = 0; /* the pairs of this expert before this one in the block */
  for (int j = 0; j < l; ++j)
    rank += keys[j] == id;
  const int at = base[blockIdx.x * pitch + id] + rank;
  if (at >= 0 && at < room)
    order[at] = p;
  else
    atomicCAS(&g_group_status, 0, 0x6F); /* `base` is not of these ids */
}

const char *launched(const char *what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess)
    return nullptr;
  static thread_local char msg[200];
  snprintf(msg, sizeof msg, "%s: %s", what, cudaGetErrorString(e));
  return msg;
}

} // namespace

const char *moe_group_count(int32_t *counts, int64_t pitch, const int32_t *ids, int n,
                            int experts, cudaStream_t stream) {
  if (experts < 1 || experts > kMostExperts || n < 0)
    return "`experts` must be 1 to 1024, and n at least 0";
  const int blocks = (n + kPairsPerBlock - 1) / kPairsPerBlock;
  if (blocks == 0)
    return nullptr;
  launch_chained(group_count_kernel, dim3(blocks), dim3(kPairsPerBlock), 0, stream,
                 counts, pitch, ids, n, experts);
  return launched("the count launch");
}

const char *moe_group_offsets(int32_t *base, int64_t base_pitch, int32_t *starts,
                              int32_t *tile_expert, int tiles, int32_t *order,
                              int room, const int32_t *counts, int64_t counts_pitch,
                              int n, int experts, int align, cudaStream_t stream) {
  if (experts < 1 || experts > kMostExperts || align < 1 || n < 0)
    return "`experts` must be 1 to 1024, and `align` above 0";
  launch_chained(group_offsets_kernel, dim3(1), dim3(kMostExperts), 0, stream, base,
                 base_pitch, starts, tile_expert, tiles, order, room, counts,
                 counts_pitch, n, experts, align);
  return launched("the offsets launch");
}

const char *moe_group_place(int32_t *order, int room, const int32_t *ids,
                            const int32_t *base, int64_t pitch, int n, int experts,
                            cudaStream_t stream) {
  const int blocks = (n + kPairsPerBlock - 1) / kPairsPerBlock;
  if (blocks <= 0)
    return nullptr;
  launch_chained(group_place_kernel, dim3(blocks), dim3(kPairsPerBlock), 0, stream,
                 order, room, ids, base, pitch, n, experts);
  return launched("the place launch");
}

int moe_group_status(cudaStream_t stream) {
  int v = 0, zero = 0;
  if (cudaStreamSynchronize(stream) != cudaSuccess)
    return -1;
  if (cudaMemcpyFromSymbol(&v, g_group_status, sizeof v) != cudaSuccess)
    return -1;
  if (v)
    cudaMemcpyToSymbol(g_group_status, &zero, sizeof zero);
  return v;
}

} // namespace vxb
