/* gemm_umma_pair.cu -- the bf16/f16 GEMM on CTA pairs: C[m,n] = A[m,k] * B[k,n],
 * f32 accumulation in tensor memory, output of the input type (the arithmetic
 * of the reference's cublasGemmEx call, runtime/cuda_dispatch.cpp:1014-1022).
 *
 * Why pairs.  A one-CTA tcgen05.mma of 128x256x16 fetches 128x16 of A and
 * 256x16 of B from that SM's shared memory and issues every 166 cycles where
 * the arithmetic needs 128: the operand fetch is the limit (78 % tensor-pipe
 * activity in gemm_umma.cu).  With tcgen05.mma.cta_group::2 the two SMs of a
 * TPC compute one 256x256 tile: each SM holds 128 rows of A and 128 columns of
 * B, the hardware passes each half of B to the other SM, and each SM fetches
 * half as much B per instruction.
 *
 * A cluster of two CTAs per tile, persistent, 192 threads each:
 *   warp 0      one thread loads THIS CTA's 128x64 of A and 64x128 of B per
 *               K block with plain TMA (no multicast: each CTA fetches its own
 *               halves) into a 6-deep ring; the byte counts of both CTAs are
 *               reported to the LEADER's (CTA 0's) full barrier;
 *   warp 1      allocates the pair's tensor memory; in the leader one thread
 *               issues the M = 256 MMAs and commits each stage back to both
 *               loaders and each finished tile to both epilogues
 *               (tcgen05.commit to the same barrier in both CTAs);
 *   warps 2-5   read this CTA's 128x256 half of the accumulator out of its own
 *               TMEM, round and store; then tell the leader the accumulator is
 *               free (an arrival on the leader's barrier through the cluster
 *               address space).
 * Two accumulators of 256 columns alternate, so a tile's epilogue runs under
 * the next tile's MMAs.  Every wait is bounded; a role that gives up records
 * where in g_pair_status, raises its CTA's stop flag, and every thread of both
 * CTAs still reaches the final cluster barrier and frees the tensor memory.
 */
#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

namespace vxb {

bool make_map_16(CUtensorMap *map, const void *base, int64_t inner, int64_t rows,
                 int64_t ld, int box_inner, int box_rows, bool is_bf16);

namespace {

constexpr int BM = 256, BN = 256, BK = 64, UK = 16; /* the pair's tile */
constexpr int HM = BM / 2, HN = BN / 2;             /* one CTA's halves */
constexpr int STAGES = 6;
constexpr int A_BYTES = HM * BK * 2; /* 16 KiB */
constexpr int B_BYTES = HN * BK * 2; /* 16 KiB */
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* align */ + 256;
constexpr int THREADS = 192;
constexpr int GROUP_M = 8;

enum { ST_LOADER_EMPTY = 0x41, ST_MMA_FULL = 0x51, ST_MMA_TMEM_EMPTY = 0x52,
       ST_EPI_TMEM_FULL = 0x61 };

__device__ int g_pair_status; /* first wait that ran out since the last read */

struct Barriers {
  uint64_t full[STAGES];  /* used in the leader: both CTAs' loads landed */
  uint64_t empty[STAGES]; /* in each CTA: the MMAs that read the stage are done */
  uint64_t tmem_full[2];  /* in each CTA: a tile's accumulator is complete */
  uint64_t tmem_empty[2]; /* in the leader: both epilogues have read it */
  uint32_t tmem_base;
  int stop;
};

__device__ inline void tile_coords(int tile, int m_tiles, int n_tiles, int &tm,
                                   int &tn) {
  const int per_group = GROUP_M * n_tiles;
  const int group = tile / per_group;
  const int first = group * GROUP_M;
  const int rows = min(m_tiles - first, GROUP_M);
  const int in_group = tile - group * per_group;
  tm = first + in_group % rows;
  tn = in_group / rows;
}

template <typename T> __device__ inline uint32_t pack2(float lo, float hi);
template <> __device__ inline uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&v);
}
template <> __device__ inline uint32_t pack2<__half>(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&v);
}

/* kBNMajor: B is used as stored, [k, n] with n contiguous, in [64 k][64 n]
   boxes; otherwise B was transposed beforehand ([n, k]) and a CTA's tile is
   [128 n][64 k]. */
template <typename T, bool kBNMajor>
__global__ void __launch_bounds__(THREADS, 1)
umma_pair_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                      const __grid_constant__ CUtensorMap map_b,
                      T *__restrict__ C, int64_t ldc, int m, int n, int k) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Barriers *bars = reinterpret_cast<Barriers *>(smem + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = ptx::cluster_ctarank(); /* 0: the leader */
  const int pair = blockIdx.x / 2, pairs = gridDim.x / 2;
  const int m_tiles = (m + BM - 1) / BM, n_tiles = (n + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles;
  const int k_blocks = (k + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&bars->full[s], 1);
      ptx::mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&bars->tmem_full[a], 1);
      ptx::mbar_init(&bars->tmem_empty[a], 8); /* four warps of each CTA */
    }
    bars->stop = 0;
    ptx::fence_proxy_async_smem();
    ptx::fence_barrier_init();
  }
  if (warp == 1)
    ptx::tmem_alloc_pair(&bars->tmem_base, 512);
  ptx::tc_fence_before_sync();
  ptx::cluster_sync_all(); /* both CTAs' barriers exist before either is used */
  ptx::tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  volatile int *stop = &bars->stop;

  if (warp == 0) {
    /* ---------------------------------------------------------- loader */
    if (lane == 0) {
      ptx::tma_prefetch_desc(&map_a);
      ptx::tma_prefetch_desc(&map_b);
      int it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < tiles; tile += pairs) {
        int tm, tn;
        tile_coords(tile, m_tiles, n_tiles, tm, tn);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!ptx::mbar_wait(&bars->empty[s], phase ^ 1, stop)) {
            atomicCAS(&g_pair_status, 0, ST_LOADER_EMPTY);
            *stop = 1;
            ok = false;
            break;
          }
          uint8_t *sa = smem + s * STAGE_BYTES, *sb = sa + A_BYTES;
          const uint32_t leader_full =
              ptx::map_to_cta(ptx::smem_addr(&bars->full[s]), 0);
          if (rank == 0)
            ptx::mbar_expect_tx(&bars->full[s], 2 * STAGE_BYTES);
          ptx::tma_load_2d_pair(sa, &map_a, kb * BK, tm * BM + (int)rank * HM,
                                leader_full);
          if (kBNMajor) {
#pragma unroll
            for (int j = 0; j < HN / 64; ++j)
              ptx::tma_load_2d_pair(sb + j * (64 * BK * 2), &map_b,
                                    tn * BN + (int)rank * HN + j * 64, kb * BK,
                                    leader_full);
          } else {
            ptx::tma_load_2d_pair(sb, &map_b, kb * BK, tn * BN + (int)rank * HN,
                                  leader_full);
          }
        }
      }
      /* Do not leave while a copy may still land in this CTA's memory: the
         stages this CTA filled last are released by MMAs that ran after the
         copies landed. The leader can also ask its own full barriers. */
      if (rank == 0)
        for (int back = 0; back < STAGES && back < it; ++back) {
          const int j = it - 1 - back;
          ptx::mbar_wait_alone(&bars->full[j % STAGES], (j / STAGES) & 1);
        }
    }
  } else if (warp == 1) {
    /* ------------------------------------- MMA issuer (the leader's only) */
    if (lane == 0 && rank == 0) {
      const uint32_t idesc =
          ptx::idesc_f16(std::is_same<T, __nv_bfloat16>::value, false, kBNMajor,
                         BM, BN);
      int it = 0, t = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < tiles; tile += pairs, ++t) {
        const int acc = t & 1;
        const uint32_t acc_phase = (t >> 1) & 1;
        if (!ptx::mbar_wait_cluster(&bars->tmem_empty[acc], acc_phase ^ 1, stop)) {
          atomicCAS(&g_pair_status, 0, ST_MMA_TMEM_EMPTY);
          *stop = 1;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!ptx::mbar_wait_cluster(&bars->full[s], (it / STAGES) & 1, stop)) {
            atomicCAS(&g_pair_status, 0, ST_MMA_FULL);
            *stop = 1;
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t sa = ptx::smem_addr(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UK; ++kk) {
            /* Both descriptors name offsets that hold in either CTA's shared
               memory. A: K-major, 128-byte rows, 8-row groups 1 KiB apart.
               B N-major: 64-column blocks 8 KiB apart, 8-row K groups 1 KiB
               apart, a K step is 16 rows; B K-major: as A. */
            const uint64_t da = ptx::smem_desc_sw128(sa + kk * UK * 2, 16, 1024);
            const uint64_t db =
                kBNMajor ? ptx::smem_desc_sw128(sb + kk * UK * 128, 64 * BK * 2,
                                                1024)
                         : ptx::smem_desc_sw128(sb + kk * UK * 2, 16, 1024);
            ptx::umma_f16_ss_pair(d_tmem, da, db, idesc, (kb | kk) != 0);
          }
          ptx::umma_commit_pair(&bars->empty[s]);
        }
        if (ok)
          ptx::umma_commit_pair(&bars->tmem_full[acc]);
      }
    }
  } else {
    /* ---------------------------------------------------------- epilogue */
    const int quarter = warp & 3; /* the TMEM lanes this warp may read */
    int t = 0;
    for (int tile = pair; tile < tiles; tile += pairs, ++t) {
      int tm, tn;
      tile_coords(tile, m_tiles, n_tiles, tm, tn);
      const int acc = t & 1;
      if (!ptx::mbar_wait(&bars->tmem_full[acc], (t >> 1) & 1, stop)) {
        atomicCAS(&g_pair_status, 0, ST_EPI_TMEM_FULL);
        *stop = 1;
        break;
      }
      ptx::tc_fence_after_sync();
      const int row = tm * BM + (int)rank * HM + quarter * 32 + lane;
      const int col0 = tn * BN;
      T *crow = C + (int64_t)row * ldc + col0;
      const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(taddr + c * 32, v);
        ptx::tmem_ld_wait();
        if (row < m) {
          const int col = col0 + c * 32;
          if (col + 32 <= n) {
            uint4 *dst = reinterpret_cast<uint4 *>(crow + c * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = pack2<T>(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
              o.y = pack2<T>(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
              o.z = pack2<T>(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
              o.w = pack2<T>(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
              dst[q] = o;
            }
          } else {
            for (int e = 0; e < 32; ++e)
              if (col + e < n) {
                const uint32_t p = pack2<T>(__uint_as_float(v[e]), 0.0f);
                reinterpret_cast<uint16_t *>(crow)[c * 32 + e] = (uint16_t)p;
              }
          }
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        ptx::mbar_arrive_cluster(
            ptx::map_to_cta(ptx::smem_addr(&bars->tmem_empty[acc]), 0));
    }
  }

  /* Nobody leaves while the other CTA may still read this one's shared memory
     or signal its barriers. */
  ptx::tc_fence_before_sync();
  __syncwarp();
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem, 512);
  }
}

template <typename T, bool kBNMajor>
const char *launch_pair(const CUtensorMap &ma, const CUtensorMap &mb, void *c,
                        int64_t ldc, int m, int n, int k, cudaStream_t stream) {
  auto kernel = umma_pair_gemm_kernel<T, kBNMajor>;
  if (allow_dynamic_smem((const void *)kernel, SMEM_BYTES) != cudaSuccess)
    return "the paired tcgen05 GEMM could not get its shared memory";
  const int tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  /* As many pairs as run at once (one CTA per SM: 74 pairs on 148 SMs), or as
     there are tiles. Asked once per device. */
  static int resident_pairs[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  int pairs = dev >= 0 && dev < 64 ? resident_pairs[dev] : 0;
  if (pairs == 0) {
    cfg.gridDim = dim3(2 * 74);
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess ||
        clusters < 1) {
      cudaGetLastError();
      return "the paired tcgen05 GEMM cannot run a cluster of two on this GPU";
    }
    pairs = clusters;
    if (dev >= 0 && dev < 64)
      resident_pairs[dev] = pairs;
  }
  if (pairs > tiles)
    pairs = tiles;
  cfg.gridDim = dim3(2 * pairs);
  const cudaError_t e =
      cudaLaunchKernelEx(&cfg, kernel, ma, mb, (T *)c, ldc, m, n, k);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

} // namespace

/* route: 4 = B as stored (N-major operand), 5 = B transposed beforehand into
   `b` ([n, k], ldb = k). Same alignment rules as the one-CTA kernel. */
const char *gemm_16_pair(int route, bool is_bf16, const void *a, int64_t lda,
                         const void *b, int64_t ldb, void *c, int64_t ldc,
                         int64_t m, int64_t n, int64_t k, cudaStream_t stream) {
  CUtensorMap ma, mb;
  if (!make_map_16(&ma, a, k, m, lda, BK, HM, is_bf16))
    return "cuTensorMapEncodeTiled refused the A matrix";
  if (route == 5) {
    if (!make_map_16(&mb, b, k, n, ldb, BK, HN, is_bf16))
      return "cuTensorMapEncodeTiled refused the transposed B matrix";
    return is_bf16 ? launch_pair<__nv_bfloat16, false>(ma, mb, c, ldc, (int)m,
                                                       (int)n, (int)k, stream)
                   : launch_pair<__half, false>(ma, mb, c, ldc, (int)m, (int)n,
                                                (int)k, stream);
  }
  if (!make_map_16(&mb, b, n, k, ldb, 64, BK, is_bf16))
    return "cuTensorMapEncodeTiled refused the B matrix";
  return is_bf16 ? launch_pair<__nv_bfloat16, true>(ma, mb, c, ldc, (int)m,
                                                    (int)n, (int)k, stream)
                 : launch_pair<__half, true>(ma, mb, c, ldc, (int)m, (int)n,
                                             (int)k, stream);
}

int gemm_pair_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_pair_status, sizeof v) != cudaSuccess)
    return -1;
  if (v)
    cudaMemcpyToSymbol(g_pair_status, &zero, sizeof zero);
  return v;
}

} // namespace vxb
