/* gemm_umma.cu -- C[m,n] = A[m,k] * B[k,n] for bf16/f16 inputs on the sm_100a
 * tensor cores, f32 accumulation in tensor memory, output of the input type.
 *
 * This is the arithmetic of the reference's cublasGemmEx call for 16-bit
 * tensors (runtime/cuda_dispatch.cpp:1014-1022: CUBLAS_COMPUTE_32F, C of the
 * input type), on row-major operands as the dispatch plan describes them.
 *
 * One persistent CTA per SM, 192 threads, three roles:
 *   warp 0      one thread issues TMA loads of A (128x64) and B (64x256) tiles
 *               into a 4-deep ring of 128-byte-swizzled shared memory stages;
 *   warp 1      allocates the 512 TMEM columns; one thread issues
 *               tcgen05.mma (M=128, N=256, K=16, four per stage) and commits
 *               each stage back to the loader and each finished tile to the
 *               epilogue;
 *   warps 2-5   read a finished 128x256 f32 accumulator out of TMEM (each warp
 *               its own 32 lanes), round to the output type and store.
 * TMEM holds two accumulators, so the epilogue of tile i overlaps the MMAs of
 * tile i+1.  Tiles are visited in groups of 16 row-tiles so that the CTAs that
 * run together share A and B panels in L2.
 *
 * A is K-major as stored.  B, stored [k, n] with n contiguous, is given to the
 * tensor core as an N-major operand: four 64x64 TMA boxes per stage, leading
 * byte offset 8 KiB between 64-column blocks, stride byte offset 1 KiB between
 * 8-row groups.  (Route 2 instead transposes B first and uses a K-major B.)
 *
 * Edges: TMA zero-fills loads past m, n or k, and the epilogue guards its
 * stores, so any m, n, k work as long as the bases are 16-byte aligned and the
 * row strides are multiples of 8 elements.
 */
#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

namespace vxb {

const char *gemm_16_plain(bool is_bf16, const void *a, int64_t lda,
                          const void *b, int64_t ldb, void *c, int64_t ldc,
                          int64_t m, int64_t n, int64_t k, cudaStream_t stream);
/* gemm_umma_pair.cu: the same product on CTA pairs (256x256 tiles). */
const char *gemm_16_pair(int route, bool is_bf16, const void *a, int64_t lda,
                         const void *b, int64_t ldb, void *c, int64_t ldc,
                         int64_t m, int64_t n, int64_t k, cudaStream_t stream);
int gemm_pair_status();

namespace {

constexpr int BM = 128, BN = 256, BK = 64, UK = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;       /* 16 KiB */
constexpr int B_BYTES = BN * BK * 2;       /* 32 KiB */
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* align */ + 256;
constexpr int THREADS = 192;
constexpr int GROUP_M = 16;

/* Where a wait ran out: role * 16 + which barrier. */
enum { ST_OK = 0, ST_LOADER_EMPTY = 0x11, ST_MMA_FULL = 0x21,
       ST_MMA_TMEM_EMPTY = 0x22, ST_EPI_TMEM_FULL = 0x31 };

__device__ int g_status; /* first failure of any CTA since the last read */

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
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

/* kBNMajor: B tiles are [64 k][64 n] boxes (B as stored); otherwise B was
   transposed beforehand and tiles are [256 n][64 k]. */
template <typename T, bool kBNMajor>
__global__ void __launch_bounds__(THREADS, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                 const __grid_constant__ CUtensorMap map_b, T *__restrict__ C,
                 int64_t ldc, int m, int n, int k) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Barriers *bars = reinterpret_cast<Barriers *>(smem + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
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
      ptx::mbar_init(&bars->tmem_empty[a], 4);
    }
    bars->stop = 0;
    ptx::fence_proxy_async_smem();
    ptx::fence_barrier_init();
  }
  if (warp == 1)
    ptx::tmem_alloc(&bars->tmem_base, 512);
  ptx::tc_fence_before_sync();
  __syncthreads();
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
      for (int tile = blockIdx.x; ok && tile < tiles; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, m_tiles, n_tiles, tm, tn);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!ptx::mbar_wait(&bars->empty[s], phase ^ 1, stop)) {
            atomicCAS(&g_status, 0, ST_LOADER_EMPTY);
            *stop = 1;
            ok = false;
            break;
          }
          uint8_t *sa = smem + s * STAGE_BYTES, *sb = sa + A_BYTES;
          ptx::mbar_expect_tx(&bars->full[s], STAGE_BYTES);
          ptx::tma_load_2d(sa, &map_a, kb * BK, tm * BM, &bars->full[s]);
          if (kBNMajor) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              ptx::tma_load_2d(sb + j * (64 * BK * 2), &map_b, tn * BN + j * 64,
                               kb * BK, &bars->full[s]);
          } else {
            ptx::tma_load_2d(sb, &map_b, kb * BK, tn * BN, &bars->full[s]);
          }
        }
      }
      /* Do not leave while a copy may still land in this CTA's memory. */
      for (int back = 0; back < STAGES && back < it; ++back) {
        const int j = it - 1 - back;
        ptx::mbar_wait_alone(&bars->full[j % STAGES], (j / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    /* ------------------------------------------------------ MMA issuer */
    if (lane == 0) {
      const uint32_t idesc =
          ptx::idesc_f16(sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value,
                         false, kBNMajor, BM, BN);
      int it = 0, t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < tiles; tile += gridDim.x, ++t) {
        const int acc = t & 1;
        const uint32_t acc_phase = (t >> 1) & 1;
        if (!ptx::mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1, stop)) {
          atomicCAS(&g_status, 0, ST_MMA_TMEM_EMPTY);
          *stop = 1;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!ptx::mbar_wait(&bars->full[s], (it / STAGES) & 1, stop)) {
            atomicCAS(&g_status, 0, ST_MMA_FULL);
            *stop = 1;
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t sa = ptx::smem_addr(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UK; ++kk) {
            /* A: K-major, rows of 128 bytes, 8-row groups 1 KiB apart; a K
               step of 16 elements is 32 bytes along the row. */
            const uint64_t da = ptx::smem_desc_sw128(sa + kk * UK * 2, 16, 1024);
            /* B N-major: 64-column blocks 8 KiB apart (leading offset), 8-row
               K groups 1 KiB apart (stride offset); a K step is 16 rows.
               B K-major: as A. */
            const uint64_t db =
                kBNMajor ? ptx::smem_desc_sw128(sb + kk * UK * 128, 64 * BK * 2,
                                                1024)
                         : ptx::smem_desc_sw128(sb + kk * UK * 2, 16, 1024);
            ptx::umma_f16_ss(d_tmem, da, db, idesc, (kb | kk) != 0);
          }
          ptx::umma_commit(&bars->empty[s]);
        }
        if (ok)
          ptx::umma_commit(&bars->tmem_full[acc]);
      }
    }
  } else {
    /* ---------------------------------------------------------- epilogue */
    const int quarter = warp & 3; /* the TMEM lanes this warp may read */
    int t = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++t) {
      int tm, tn;
      tile_coords(tile, m_tiles, n_tiles, tm, tn);
      const int acc = t & 1;
      if (!ptx::mbar_wait(&bars->tmem_full[acc], (t >> 1) & 1, stop)) {
        atomicCAS(&g_status, 0, ST_EPI_TMEM_FULL);
        *stop = 1;
        break;
      }
      ptx::tc_fence_after_sync();
      const int row = tm * BM + quarter * 32 + lane;
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
        ptx::mbar_arrive(&bars->tmem_empty[acc]);
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem, 512);
  }
}

/* ---- host side ------------------------------------------------------------- */
typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t,
                                void *, const cuuint64_t *, const cuuint64_t *,
                                const cuuint32_t *, const cuuint32_t *,
                                CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encoder() {
  static EncodeTiled fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault,
                                &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return (EncodeTiled) nullptr;
    }
    return (EncodeTiled)p;
  }();
  return fn;
}

} // namespace

/* A 2-D map over a row-major matrix of 16-bit elements: `inner` contiguous
   elements per row, `rows` rows `ld` elements apart; boxes of box_inner x
   box_rows, 128-byte swizzle (box_inner must be 64). */
bool make_map_16(CUtensorMap *map, const void *base, int64_t inner, int64_t rows,
                 int64_t ld, int box_inner, int box_rows, bool is_bf16) {
  EncodeTiled enc = encoder();
  if (!enc)
    return false;
  const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return enc(map,
             is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                     : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
             2, const_cast<void *>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

namespace {

int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

template <typename T, bool kBNMajor>
const char *launch_umma(const CUtensorMap &ma, const CUtensorMap &mb, void *c,
                        int64_t ldc, int m, int n, int k, cudaStream_t stream) {
  if (allow_dynamic_smem((const void *)umma_gemm_kernel<T, kBNMajor>,
                         SMEM_BYTES) != cudaSuccess)
    return "the tcgen05 GEMM could not get its shared memory";
  const int tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  umma_gemm_kernel<T, kBNMajor>
      <<<grid, THREADS, SMEM_BYTES, stream>>>(ma, mb, (T *)c, ldc, m, n, k);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

bool umma_shape_ok(const void *a, int64_t lda, const void *b, int64_t ldb,
                   const void *c, int64_t ldc, int64_t m, int64_t n, int64_t k) {
  auto al = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
  return al(a) && al(b) && al(c) && lda % 8 == 0 && ldb % 8 == 0 &&
         ldc % 8 == 0 && m < (1 << 30) && n < (1 << 30) && k < (1 << 30) &&
         k >= 1;
}

} // namespace

const char *gemm_16_route(int route, bool is_bf16, const void *a, int64_t lda,
                          const void *b, int64_t ldb, void *c, int64_t ldc,
                          int64_t m, int64_t n, int64_t k, void *scratch,
                          cudaStream_t stream) {
  if (m <= 0 || n <= 0)
    return nullptr;
  if (route == 3)
    return gemm_16_plain(is_bf16, a, lda, b, ldb, c, ldc, m, n, k, stream);
  if (!umma_shape_ok(a, lda, b, ldb, c, ldc, m, n, k))
    return "the tcgen05 GEMM needs 16-byte aligned bases and row strides that "
           "are multiples of 8 elements";
  if (route == 4)
    return gemm_16_pair(4, is_bf16, a, lda, b, ldb, c, ldc, m, n, k, stream);
  if (route == 5) {
    if (!scratch || ((uintptr_t)scratch & 15) || k % 8 != 0)
      return "the transposed-B route needs a 16-byte aligned scratch matrix "
             "and k a multiple of 8";
    if (const char *why = transpose_16(b, ldb, scratch, k, k, n, stream))
      return why;
    return gemm_16_pair(5, is_bf16, a, lda, scratch, k, c, ldc, m, n, k, stream);
  }
  CUtensorMap ma, mb;
  if (!make_map_16(&ma, a, k, m, lda, BK, BM, is_bf16))
    return "cuTensorMapEncodeTiled refused the A matrix";
  if (route == 2) {
    if (!scratch || ((uintptr_t)scratch & 15) || k % 8 != 0)
      return "the transposed-B route needs a 16-byte aligned scratch matrix "
             "and k a multiple of 8";
    if (const char *why = transpose_16(b, ldb, scratch, k, k, n, stream))
      return why;
    if (!make_map_16(&mb, scratch, k, n, k, BK, BN, is_bf16))
      return "cuTensorMapEncodeTiled refused the transposed B matrix";
    return is_bf16 ? launch_umma<__nv_bfloat16, false>(ma, mb, c, ldc, (int)m,
                                                       (int)n, (int)k, stream)
                   : launch_umma<__half, false>(ma, mb, c, ldc, (int)m, (int)n,
                                                (int)k, stream);
  }
  if (!make_map_16(&mb, b, n, k, ldb, 64, BK, is_bf16))
    return "cuTensorMapEncodeTiled refused the B matrix";
  return is_bf16 ? launch_umma<__nv_bfloat16, true>(ma, mb, c, ldc, (int)m,
                                                    (int)n, (int)k, stream)
                 : launch_umma<__half, true>(ma, mb, c, ldc, (int)m, (int)n,
                                             (int)k, stream);
}

const char *gemm_16(bool is_bf16, const void *a, int64_t lda, const void *b,
                    int64_t ldb, void *c, int64_t ldc, int64_t m, int64_t n,
                    int64_t k, cudaStream_t stream) {
  /* The tensor-core kernel moves whole 128x256 tiles; below a few tiles, and
     for strides TMA cannot describe, the plain kernel is the one to use. */
  const bool small = m * n < 128 * 256 || k < 64;
  if (small || !umma_shape_ok(a, lda, b, ldb, c, ldc, m, n, k) || !encoder())
    return gemm_16_plain(is_bf16, a, lda, b, ldb, c, ldc, m, n, k, stream);
  /* One CTA per 128x256 tile, or a CTA pair per 256x256 tile. The single CTA's
     MMA is held to 77 % of the tensor pipe by its operand fetch and the pair's
     runs near the full rate, so a pair finishes its tile (twice the work on
     two SMs) in about 0.82 of the time one CTA needs for its own; but there
     are half as many pair tiles, so for a small product the last wave decides,
     and below two waves of pair tiles the cluster's start-up shows (2048^3:
     823 against 912 TFLOP/s). Cost in units of a one-CTA tile time. */
  const int64_t t1 = ((m + 127) / 128) * ((n + 255) / 256);
  const int64_t t2 = ((m + 255) / 256) * ((n + 255) / 256);
  const int sms = sm_count();
  const double cost1 = (double)((t1 + sms - 1) / sms);
  const double cost2 = (double)((t2 + sms / 2 - 1) / (sms / 2)) * 0.82;
  /* VXB_GEMM_ROUTE=1 or 4 pins the choice (for measurements). */
  const char *force = getenv("VXB_GEMM_ROUTE");
  const int route = force && (force[0] == '1' || force[0] == '4')
                        ? force[0] - '0'
                        : (cost2 < cost1 && t2 >= sms ? 4 : 1);
  return gemm_16_route(route, is_bf16, a, lda, b, ldb, c, ldc, m, n, k, nullptr,
                       stream);
}

int gemm_status(cudaStream_t stream) {
  int v = 0, zero = 0;
  if (cudaStreamSynchronize(stream) != cudaSuccess)
    return -1;
  if (cudaMemcpyFromSymbol(&v, g_status, sizeof v) != cudaSuccess)
    return -1;
  if (v)
    cudaMemcpyToSymbol(g_status, &zero, sizeof zero);
  const int pair = gemm_pair_status();
  return v ? v : pair;
}

} // namespace vxb
