/* gemm_f32_split.cu -- C = A B in f32 on the tensor cores.
 *
 * The reference sends an f32 matmul to cuBLAS Sgemm (cuda_dispatch.cpp:988-1023),
 * which runs on the FP32 pipe. A B200 has twenty times more bf16 tensor
 * throughput than FP32, and an f32 value is the exact sum of three bf16 terms
 * (8 + 8 + 8 mantissa bits, the remainders are exact in f32), so
 *   a b = (a1 + a2 + a3)(b1 + b2 + b3)
 *       = a1 b1 + a1 b2 + a2 b1 + a1 b3 + a2 b2 + a3 b1 + (terms below 2^-24 |a b|)
 * with every product bf16 x bf16 exact in f32 and the sums in f32. Laid out
 * as ONE bf16 GEMM over K' = 6 k:
 *   A' [m, 6k] = a1 | a1 | a1 | a2 | a2 | a3
 *   B' [n, 6k] = b1 | b2 | b3 | b1 | b2 | b1      (B transposed on the way)
 * it runs on the CTA-pair kernel of the prefill (tcgen05.mma.cta_group::2,
 * f32 partial sums per run of K', added in run order).
 */
#include "kernels.h"
#include "launch.cuh"

#include <cuda_bf16.h>

namespace vxb {
namespace {

__device__ __forceinline__ void three_terms(float v, __nv_bfloat16 &t1,
                                            __nv_bfloat16 &t2, __nv_bfloat16 &t3) {
  t1 = __float2bfloat16(v);
  const float r1 = v - __bfloat162float(t1);
  t2 = __float2bfloat16(r1);
  t3 = __float2bfloat16(r1 - __bfloat162float(t2));
}

/* A' from A: one thread per eight consecutive values of a row (k is a
   multiple of 64), six 16-byte stores. */
__global__ void __launch_bounds__(256)
split_a_kernel(__nv_bfloat16 *out, const float *a, int64_t lda, int m, int k) {
  chain_release();
  chain_wait();
  const int per_row = k / 8;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)m * per_row)
    return;
  const int64_t r = idx / per_row;
  const int c = (int)(idx - r * per_row) * 8;
  const float *src = a + r * lda + c;
  uint32_t w1[4], w2[4], w3[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat16 x1, x2, x3, y1, y2, y3;
    three_terms(src[2 * j], x1, x2, x3);
    three_terms(src[2 * j + 1], y1, y2, y3);
    w1[j] = (uint32_t)__bfloat16_as_ushort(x1) | (uint32_t)__bfloat16_as_ushort(y1) << 16;
    w2[j] = (uint32_t)__bfloat16_as_ushort(x2) | (uint32_t)__bfloat16_as_ushort(y2) << 16;
    w3[j] = (uint32_t)__bfloat16_as_ushort(x3) | (uint32_t)__bfloat16_as_ushort(y3) << 16;
  }
  const uint4 t1 = make_uint4(w1[0], w1[1], w1[2], w1[3]);
  const uint4 t2 = make_uint4(w2[0], w2[1], w2[2], w2[3]);
  const uint4 t3 = make_uint4(w3[0], w3[1], w3[2], w3[3]);
  __nv_bfloat16 *row = out + r * 6 * k + c;
  *reinterpret_cast<uint4 *>(row) = t1;
  *reinterpret_cast<uint4 *>(row + k) = t1;
  *reinterpret_cast<uint4 *>(row + 2 * (int64_t)k) = t1;
  *reinterpret_cast<uint4 *>(row + 3 * (int64_t)k) = t2;
  *reinterpret_cast<uint4 *>(row + 4 * (int64_t)k) = t2;
  *reinterpret_cast<uint4 *>(row + 5 * (int64_t)k) = t3;
}

/* B' from B [k, n]: a block transposes a 32 x 32 tile through shared memory,
   so that B is read along n and B' written along k. */
__global__ void __launch_bounds__(256)
split_bt_kernel(__nv_bfloat16 *out, const float *b, int64_t ldb, int k, int n) {
  __shared__ __nv_bfloat16 tile[3][32][34];
  chain_release();
  chain_wait();
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; /* 32 x 8 */
  for (int r = ty; r < 32; r += 8) {
    __nv_bfloat16 t1, t2, t3;
    const float v = (k0 + r < k && n0 + tx < n) ? b[(int64_t)(k0 + r) * ldb + n0 + tx]
                                                 : 0.0f;
    three_terms(v, t1, t2, t3);
    tile[0][r][tx] = t1;
    tile[1][r][tx] = t2;
    tile[2][r][tx] = t3;
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    if (n0 + j >= n || k0 + tx >= k)
      continue;
    __nv_bfloat16 *row = out + (int64_t)(n0 + j) * 6 * k + k0 + tx;
    const __nv_bfloat16 t1 = tile[0][tx][j], t2 = tile[1][tx][j], t3 = tile[2][tx][j];
    row[0] = t1;
    row[k] = t2;
    row[2 * (int64_t)k] = t3;
    row[3 * (int64_t)k] = t1;
    row[4 * (int64_t)k] = t2;
    row[5 * (int64_t)k] = t1;
  }
}

/* C = the runs' partial sums, in run order; four values per thread (n is a
   multiple of 4). vec: C's rows are 16-byte aligned. */
__global__ void __launch_bounds__(256)
sum_runs_kernel(float *c, int64_t ldc, const float *partials, int splits, int m,
                int n, int vec) {
  chain_release();
  chain_wait();
  const int per_row = n / 4;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)m * per_row)
    return;
  const int64_t r = idx / per_row;
  const int j = (int)(idx - r * per_row) * 4;
  const int64_t at = r * n + j;
  float4 s = *reinterpret_cast<const float4 *>(partials + at);
  for (int q = 1; q < splits; ++q) {
    const float4 v =
        *reinterpret_cast<const float4 *>(partials + (int64_t)q * m * n + at);
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  float *dst = c + r * ldc + j;
  if (vec) {
    *reinterpret_cast<float4 *>(dst) = s;
  } else {
    dst[0] = s.x; dst[1] = s.y; dst[2] = s.z; dst[3] = s.w;
  }
}

bool direct(int splits, int64_t n, int64_t ldc) { return splits == 1 && ldc == n; }

} // namespace

size_t gemm_f32_split_scratch_bytes(int64_t m, int64_t n, int64_t k, int64_t ldc) {
  /* n % 4: the GEMM stores its f32 results four at a time */
  if (k % 64 != 0 || n % 4 != 0 || m < 128 || n < 128 || m > (1 << 30) || n > (1 << 30) ||
      6 * k > (1ll << 31) - 1 || m * n * k < (1ll << 24))
    return 0;
  const int splits = rows_gemm_splits_of((int)m, (int)n, 6 * k);
  size_t bytes = (size_t)(m + n) * 6 * k * 2;
  bytes = (bytes + 255) & ~(size_t)255;
  if (!direct(splits, n, ldc))
    bytes += (size_t)splits * m * n * 4;
  return bytes;
}

const char *gemm_f32_split(const float *a, int64_t lda, const float *b, int64_t ldb,
                           float *c, int64_t ldc, int64_t m, int64_t n, int64_t k,
                           void *scratch, cudaStream_t stream) {
  if (!gemm_f32_split_scratch_bytes(m, n, k, ldc) || !scratch)
    return "the shape is not for the tensor-core f32 product";
  __nv_bfloat16 *a6 = (__nv_bfloat16 *)scratch;
  __nv_bfloat16 *b6 = a6 + m * 6 * k;
  const size_t terms_bytes = ((size_t)(m + n) * 6 * k * 2 + 255) & ~(size_t)255;
  float *partials = (float *)((char *)scratch + terms_bytes);
  launch_chained(split_a_kernel, dim3((unsigned)((m * (k / 8) + 255) / 256)), dim3(256),
                 0, stream, a6, a, lda, (int)m, (int)k);
  launch_chained(split_bt_kernel, dim3((unsigned)((n + 31) / 32), (unsigned)((k + 31) / 32)),
                 dim3(256), 0, stream, b6, b, ldb, (int)k, (int)n);
  if (cudaGetLastError() != cudaSuccess)
    return "the term-splitting launches failed";
  int splits = rows_gemm_splits_of((int)m, (int)n, 6 * k);
  float *out = direct(splits, n, ldc) ? c : partials;
  if (const char *why = rows_gemm_of(a6, 6 * k, b6, 6 * k, (int)m, (int)n, out, &splits,
                                     stream))
    return why;
  if (out != c) {
    const int vec = ldc % 4 == 0 && ((uintptr_t)c & 15) == 0;
    launch_chained(sum_runs_kernel, dim3((unsigned)((m * (n / 4) + 255) / 256)),
                   dim3(256), 0, stream, c, ldc, partials, splits, (int)m, (int)n, vec);
    if (cudaGetLastError() != cudaSuccess)
      return "the launch that adds the runs failed";
  }
  return nullptr;
}

} // namespace vxb
