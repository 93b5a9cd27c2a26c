/* gemm_simt.cu -- f32 and f64 matrix products on the FP32/FP64 pipes, the f32
 * matrix-vector product of the flat entry point, and small data movers.
 *
 * The f32 GEMM is the reference's default arithmetic for `a @ b` on f32
 * tensors (runtime/cuda_dispatch.cpp:996-1003 calls cublasSgemm in true FP32;
 * TF32 is opt-in there).  One-pass TF32 cannot meet the 1e-4 bound against the
 * CPU loop, so this kernel keeps every product and sum in f32: each C[i][j] is
 * one thread's chain of FMAs over ascending k.
 *
 * Tiling: a CTA of 256 threads owns a 128x128 tile of C; k advances 16 at a
 * time through two shared-memory stages (A stored k-major so that both
 * operands are read as float4 without bank conflicts); a thread keeps an 8x8
 * block of C in registers as two 4-wide halves 64 columns apart, which makes
 * every shared-memory read of B a conflict-free float4.
 */
#include "kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdio>

namespace vxb {
namespace {

constexpr int TM = 128, TN = 128, TK = 16, NT = 256;

template <bool kVec>
__global__ void __launch_bounds__(NT, 2)
sgemm_kernel(const float *__restrict__ A, int64_t lda,
             const float *__restrict__ B, int64_t ldb, float *__restrict__ C,
             int64_t ldc, int m, int n, int k) {
  __shared__ __align__(16) float As[2][TK][TM + 4];
  __shared__ __align__(16) float Bs[2][TK][TN + 4];

  const int tid = threadIdx.x;
  const int row0 = blockIdx.y * TM, col0 = blockIdx.x * TN;
  const int ty = tid / 16, tx = tid % 16; /* 16 x 16 threads */

  /* global -> register staging: A tile 128x16 = 2048 floats = 2 float4 per
     thread; B tile 16x128 likewise. */
  const int a_r = tid / 4, a_c = (tid % 4) * 4;   /* rows a_r and a_r + 64 */
  const int b_r = tid / 32, b_c = (tid % 32) * 4; /* rows b_r and b_r + 8  */
  float4 ra[2], rb[2];

  auto load_tiles = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = row0 + a_r + h * 64, c = k0 + a_c;
      if (kVec && r < m && c + 3 < k) {
        ra[h] = *reinterpret_cast<const float4 *>(A + (int64_t)r * lda + c);
      } else {
        float t[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          t[e] = (r < m && c + e < k) ? A[(int64_t)r * lda + c + e] : 0.0f;
        ra[h] = make_float4(t[0], t[1], t[2], t[3]);
      }
      const int br = k0 + b_r + h * 8, bc = col0 + b_c;
      if (kVec && br < k && bc + 3 < n) {
        rb[h] = *reinterpret_cast<const float4 *>(B + (int64_t)br * ldb + bc);
      } else {
        float t[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          t[e] = (br < k && bc + e < n) ? B[(int64_t)br * ldb + bc + e] : 0.0f;
        rb[h] = make_float4(t[0], t[1], t[2], t[3]);
      }
    }
  };
  auto store_tiles = [&](int s) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      As[s][a_c + 0][a_r + h * 64] = ra[h].x;
      As[s][a_c + 1][a_r + h * 64] = ra[h].y;
      As[s][a_c + 2][a_r + h * 64] = ra[h].z;
      As[s][a_c + 3][a_r + h * 64] = ra[h].w;
      *reinterpret_cast<float4 *>(&Bs[s][b_r + h * 8][b_c]) = rb[h];
    }
  };

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j)
      acc[i][j] = 0.0f;

  load_tiles(0);
  store_tiles(0);
  __syncthreads();

  int stage = 0;
  for (int k0 = 0; k0 < k; k0 += TK) {
    const bool more = k0 + TK < k;
    if (more)
      load_tiles(k0 + TK);
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4 *>(&As[stage][kk][ty * 4]);
      const float4 a1 =
          *reinterpret_cast<const float4 *>(&As[stage][kk][ty * 4 + 64]);
      const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[stage][kk][tx * 4]);
      const float4 b1 =
          *reinterpret_cast<const float4 *>(&Bs[stage][kk][tx * 4 + 64]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j)
          acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (more) {
      store_tiles(stage ^ 1);
      __syncthreads();
      stage ^= 1;
    }
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = row0 + ty * 4 + (i & 3) + (i >> 2) * 64;
    if (r >= m)
      continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int c = col0 + tx * 4 + h * 64;
      float *dst = C + (int64_t)r * ldc + c;
      if (kVec && c + 3 < n) {
        *reinterpret_cast<float4 *>(dst) = make_float4(
            acc[i][h * 4 + 0], acc[i][h * 4 + 1], acc[i][h * 4 + 2],
            acc[i][h * 4 + 3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (c + e < n)
            dst[e] = acc[i][h * 4 + e];
      }
    }
  }
}

/* f64: 64x64 tile, 4x4 per thread. FP64 is a narrow pipe on this part; the
   kernel only has to be right and reasonable. */
__global__ void __launch_bounds__(256)
dgemm_kernel(const double *__restrict__ A, int64_t lda,
             const double *__restrict__ B, int64_t ldb, double *__restrict__ C,
             int64_t ldc, int m, int n, int k) {
  __shared__ double As[16][64 + 1];
  __shared__ double Bs[16][64];
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const int row0 = blockIdx.y * 64, col0 = blockIdx.x * 64;
  double acc[4][4] = {};
  for (int k0 = 0; k0 < k; k0 += 16) {
    for (int i = tid; i < 64 * 16; i += 256) {
      const int r = i / 16, c = i % 16;
      As[c][r] = (row0 + r < m && k0 + c < k)
                     ? A[(int64_t)(row0 + r) * lda + k0 + c]
                     : 0.0;
      const int br = i / 64, bc = i % 64;
      Bs[br][bc] = (k0 + br < k && col0 + bc < n)
                       ? B[(int64_t)(k0 + br) * ldb + col0 + bc]
                       : 0.0;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      double av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        av[i] = As[kk][ty * 4 + i];
        bv[i] = Bs[kk][tx + 16 * i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc[i][j] = fma(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      const int r = row0 + ty * 4 + i, c = col0 + tx + 16 * j;
      if (r < m && c < n)
        C[(int64_t)r * ldc + c] = acc[i][j];
    }
}

/* Plain 16-bit GEMM for shapes the tcgen05 kernel does not take (unaligned
   strides, tiny sizes): 64x64 tile, f32 accumulate, output of the input type. */
template <typename T> __device__ inline float to_f32(T v);
template <> __device__ inline float to_f32(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <> __device__ inline float to_f32(__half v) { return __half2float(v); }
template <typename T> __device__ inline T from_f32(float v);
template <> __device__ inline __nv_bfloat16 from_f32(float v) {
  return __float2bfloat16_rn(v);
}
template <> __device__ inline __half from_f32(float v) {
  return __float2half_rn(v);
}

template <typename T>
__global__ void __launch_bounds__(256)
gemm16_plain_kernel(const T *__restrict__ A, int64_t lda,
                    const T *__restrict__ B, int64_t ldb, T *__restrict__ C,
                    int64_t ldc, int m, int n, int k) {
  __shared__ float As[16][64 + 1];
  __shared__ float Bs[16][64];
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const int row0 = blockIdx.y * 64, col0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < k; k0 += 16) {
    for (int i = tid; i < 64 * 16; i += 256) {
      const int r = i / 16, c = i % 16;
      As[c][r] = (row0 + r < m && k0 + c < k)
                     ? to_f32(A[(int64_t)(row0 + r) * lda + k0 + c])
                     : 0.0f;
      const int br = i / 64, bc = i % 64;
      Bs[br][bc] = (k0 + br < k && col0 + bc < n)
                       ? to_f32(B[(int64_t)(k0 + br) * ldb + col0 + bc])
                       : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        av[i] = As[kk][ty * 4 + i];
        bv[i] = Bs[kk][tx + 16 * i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      const int r = row0 + ty * 4 + i, c = col0 + tx + 16 * j;
      if (r < m && c < n)
        C[(int64_t)r * ldc + c] = from_f32<T>(acc[i][j]);
    }
}

/* out[c][r] = in[r][c] for 16-bit elements, through a 32x32 (+1) tile. */
__global__ void transpose16_kernel(const uint16_t *__restrict__ in,
                                   int64_t ld_in, uint16_t *__restrict__ out,
                                   int64_t ld_out, int64_t rows, int64_t cols) {
  __shared__ uint16_t tile[32][33];
  const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int64_t r = r0 + j, c = c0 + threadIdx.x;
    tile[j][threadIdx.x] = (r < rows && c < cols) ? in[r * ld_in + c] : 0;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int64_t c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols)
      out[c * ld_out + r] = tile[threadIdx.x][j];
  }
}

/* Counter-based random numbers: one 64-bit mix of (seed, index) per value
   (splitmix64 finaliser), Box-Muller for normals. The same index always gives
   the same value, whatever the launch shape. */
__device__ inline uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <bool kNormal>
__global__ void fill_kernel(void *out, bool as_bf16, int64_t n, uint64_t seed,
                            float p0, float p1) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    const uint64_t bits = mix64(seed * 0xD1342543DE82EF95ull + (uint64_t)i);
    const float u1 = ((float)(uint32_t)(bits >> 40) + 0.5f) * (1.0f / 16777216.0f);
    float v;
    if (kNormal) {
      const float u2 =
          ((float)(uint32_t)((bits >> 16) & 0xFFFFFF) + 0.5f) * (1.0f / 16777216.0f);
      v = p0 * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
    } else {
      v = p0 + (p1 - p0) * ((float)(uint32_t)(bits >> 40) * (1.0f / 16777216.0f));
    }
    if (as_bf16)
      ((__nv_bfloat16 *)out)[i] = __float2bfloat16_rn(v);
    else
      ((float *)out)[i] = v;
  }
}

/* An all-gather of column blocks lands as [ranks][m][n_local]; the row-major
   [m, ranks*n_local] matrix needs rank r's block at column r*n_local. 16 bytes
   per thread when the block width allows it. */
__global__ void interleave_kernel(const uint4 *__restrict__ in,
                                  uint4 *__restrict__ out, int ranks, int64_t m,
                                  int64_t vec_per_row_local) {
  const int64_t total = (int64_t)ranks * m * vec_per_row_local;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const int64_t v = i % vec_per_row_local;
    const int64_t row = (i / vec_per_row_local) % m;
    const int64_t r = i / (vec_per_row_local * m);
    out[(row * ranks + r) * vec_per_row_local + v] = in[i];
  }
}

const char *last_error(const char *what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess)
    return nullptr;
  static thread_local char msg[256];
  snprintf(msg, sizeof msg, "%s: %s", what, cudaGetErrorString(e));
  return msg;
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

} // namespace

const char *gemm_f32(const float *a, int64_t lda, const float *b, int64_t ldb,
                     float *c, int64_t ldc, int64_t m, int64_t n, int64_t k,
                     cudaStream_t stream) {
  if (m <= 0 || n <= 0)
    return nullptr;
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX)
    return "a dimension does not fit in 32 bits";
  const dim3 grid((unsigned)((n + TN - 1) / TN), (unsigned)((m + TM - 1) / TM));
  if (grid.y > 65535)
    return "more than 65535 row tiles";
  const bool vec = aligned16(a) && aligned16(b) && aligned16(c) &&
                   lda % 4 == 0 && ldb % 4 == 0 && ldc % 4 == 0;
  if (vec)
    sgemm_kernel<true><<<grid, NT, 0, stream>>>(a, lda, b, ldb, c, ldc, (int)m,
                                                (int)n, (int)k);
  else
    sgemm_kernel<false><<<grid, NT, 0, stream>>>(a, lda, b, ldb, c, ldc, (int)m,
                                                 (int)n, (int)k);
  return last_error("the f32 GEMM launch");
}

const char *gemm_f64(const double *a, int64_t lda, const double *b, int64_t ldb,
                     double *c, int64_t ldc, int64_t m, int64_t n, int64_t k,
                     cudaStream_t stream) {
  if (m <= 0 || n <= 0)
    return nullptr;
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX)
    return "a dimension does not fit in 32 bits";
  const dim3 grid((unsigned)((n + 63) / 64), (unsigned)((m + 63) / 64));
  if (grid.y > 65535)
    return "more than 65535 row tiles";
  dgemm_kernel<<<grid, 256, 0, stream>>>(a, lda, b, ldb, c, ldc, (int)m, (int)n,
                                         (int)k);
  return last_error("the f64 GEMM launch");
}

const char *gemm_16_plain(bool is_bf16, const void *a, int64_t lda,
                          const void *b, int64_t ldb, void *c, int64_t ldc,
                          int64_t m, int64_t n, int64_t k,
                          cudaStream_t stream) {
  if (m <= 0 || n <= 0)
    return nullptr;
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX)
    return "a dimension does not fit in 32 bits";
  const dim3 grid((unsigned)((n + 63) / 64), (unsigned)((m + 63) / 64));
  if (grid.y > 65535)
    return "more than 65535 row tiles";
  if (is_bf16)
    gemm16_plain_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        (const __nv_bfloat16 *)a, lda, (const __nv_bfloat16 *)b, ldb,
        (__nv_bfloat16 *)c, ldc, (int)m, (int)n, (int)k);
  else
    gemm16_plain_kernel<__half><<<grid, 256, 0, stream>>>(
        (const __half *)a, lda, (const __half *)b, ldb, (__half *)c, ldc,
        (int)m, (int)n, (int)k);
  return last_error("the 16-bit GEMM launch");
}

const char *transpose_16(const void *in, int64_t ld_in, void *out,
                         int64_t ld_out, int64_t rows, int64_t cols,
                         cudaStream_t stream) {
  const dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
  if (grid.y > 65535)
    return "more than 65535 row tiles";
  transpose16_kernel<<<grid, dim3(32, 8), 0, stream>>>(
      (const uint16_t *)in, ld_in, (uint16_t *)out, ld_out, rows, cols);
  return last_error("the transpose launch");
}

const char *fill_normal(void *out, bool as_bf16, int64_t n, uint64_t seed,
                        float sigma, cudaStream_t stream) {
  if (n <= 0)
    return nullptr;
  const int blocks = (int)std::min<int64_t>((n + 255) / 256, 148 * 16);
  fill_kernel<true><<<blocks, 256, 0, stream>>>(out, as_bf16, n, seed, sigma, 0);
  return last_error("the fill launch");
}

const char *fill_uniform(void *out, bool as_bf16, int64_t n, uint64_t seed,
                         float lo, float hi, cudaStream_t stream) {
  if (n <= 0)
    return nullptr;
  const int blocks = (int)std::min<int64_t>((n + 255) / 256, 148 * 16);
  fill_kernel<false><<<blocks, 256, 0, stream>>>(out, as_bf16, n, seed, lo, hi);
  return last_error("the fill launch");
}

const char *interleave_gathered(const void *gathered, void *out, int ranks,
                                int64_t m, int64_t n_local, int elem_bytes,
                                cudaStream_t stream) {
  if ((n_local * elem_bytes) % 16 != 0 || !aligned16(gathered) ||
      !aligned16(out))
    return "a gathered block row is not a multiple of 16 bytes";
  const int64_t vec = n_local * elem_bytes / 16;
  const int64_t total = (int64_t)ranks * m * vec;
  const int blocks = (int)std::min<int64_t>((total + 255) / 256, 148 * 16);
  interleave_kernel<<<blocks, 256, 0, stream>>>((const uint4 *)gathered,
                                                (uint4 *)out, ranks, m, vec);
  return last_error("the interleave launch");
}

} // namespace vxb
