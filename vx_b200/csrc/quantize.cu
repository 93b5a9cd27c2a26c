/* quantize.cu -- bf16 matrices into the two quantised formats of std::nn, on
 * the GPU: what a host needs to make an fp8 or Q4_0 model out of bf16 weights
 * (synthetic ones here; the reference's programs load theirs already
 * quantised).
 *
 * fp8 (stdlib/std/nn.vx:1296-1303): f8e4m3 codes (OCP, bias 7, no infinity)
 * with one f32 scale per block of 128 x 128 weights: scale = the block's
 * largest magnitude / 448 (448 is the largest e4m3 value), code = w / scale
 * rounded to nearest even and saturated, so the NaN codes 0x7f and 0xff never
 * occur.
 * Q4_0 (nn.vx:1645-1663, "as in llama.cpp"): per 32 weights of a row, d = the
 * value of largest magnitude (with its sign) / -8, code = min(15, floor(w / d
 * + 8.5)), weight = (code - 8) * d, d kept as f16.
 */
#include "kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstdio>

namespace vxb {
namespace {

__device__ __forceinline__ float bf_at(const void *p, int64_t i) {
  return __uint_as_float((uint32_t)((const uint16_t *)p)[i] << 16);
}

/* One block of 256 threads per 128 x 128 block of the matrix. */
__global__ void __launch_bounds__(256)
quantize_fp8_kernel(const void *w, int rows, int cols, uint8_t *codes,
                    float *scales) {
  __shared__ float red[8];
  const int bc = blockIdx.x, br = blockIdx.y;
  const int r0 = br * 128, c0 = bc * 128;
  float big = 0.0f;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = r0 + i / 128, c = c0 + i % 128;
    if (r < rows)
      big = fmaxf(big, fabsf(bf_at(w, (int64_t)r * cols + c)));
  }
  for (int o = 16; o > 0; o >>= 1)
    big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, o));
  if ((threadIdx.x & 31) == 0)
    red[threadIdx.x >> 5] = big;
  __syncthreads();
  big = red[0];
  for (int k = 1; k < 8; ++k)
    big = fmaxf(big, red[k]);
  const float scale = big > 0.0f ? big / 448.0f : 1.0f;
  if (threadIdx.x == 0)
    scales[(int64_t)br * (cols / 128) + bc] = scale;
  const float inv = 1.0f / scale;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = r0 + i / 128, c = c0 + i % 128;
    if (r < rows)
      codes[(int64_t)r * cols + c] = (uint8_t)__nv_cvt_float_to_fp8(
          bf_at(w, (int64_t)r * cols + c) * inv, __NV_SATFINITE, __NV_E4M3);
  }
}

/* One thread per group of 32 weights: 16 bytes of codes (nibble t of 32-bit
   word j is weight 8 j + t) and one f16 scale. */
__global__ void __launch_bounds__(256)
quantize_q4_kernel(const void *w, int64_t groups, uint4 *codes, __half *scales) {
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups)
    return;
  float v[32], amax = 0.0f, vmax = 0.0f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    v[i] = bf_at(w, g * 32 + i);
    if (fabsf(v[i]) > amax) {
      amax = fabsf(v[i]);
      vmax = v[i];
    }
  }
  const float d = vmax / -8.0f;
  const float id = d != 0.0f ? 1.0f / d : 0.0f;
  uint32_t words[4] = {0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    /* one rounding for the product, one for the sum (no fused multiply-add):
       the code does not depend on how the compiler contracts the line */
    int code = (int)__fadd_rn(__fmul_rn(v[i], id), 8.5f);
    code = code < 0 ? 0 : (code > 15 ? 15 : code);
    words[i / 8] |= (uint32_t)code << (4 * (i % 8));
  }
  codes[g] = make_uint4(words[0], words[1], words[2], words[3]);
  scales[g] = __float2half(d);
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

const char *quantize_fp8(const void *w_bf16, int rows, int cols, void *codes,
                         float *scales, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || cols % 128 != 0)
    return "an fp8 matrix has a multiple of 128 columns";
  const dim3 grid(cols / 128, (rows + 127) / 128);
  quantize_fp8_kernel<<<grid, 256, 0, stream>>>(w_bf16, rows, cols,
                                                (uint8_t *)codes, scales);
  return launched("the fp8 quantisation");
}

const char *quantize_q4(const void *w_bf16, int rows, int cols, void *codes,
                        void *scales_f16, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || cols % 32 != 0 || ((uintptr_t)codes & 15))
    return "a Q4_0 matrix has a multiple of 32 columns, and its codes start on "
           "a 16-byte boundary";
  const int64_t groups = (int64_t)rows * (cols / 32);
  quantize_q4_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, stream>>>(
      w_bf16, groups, (uint4 *)codes, (__half *)scales_f16);
  return launched("the Q4_0 quantisation");
}

} // namespace vxb
