/* gemm_fp8_rows.cu -- y[n, rows] = x[n, cols] . W^T for an fp8 matrix W and many
 * rows of f32 activations, on the tensor cores.
 *
 * The format is that of nn_matvec_fp8 (stdlib/std/nn.vx:1296-1306): f8e4m3
 * codes, four to a u32 word, and an f32 scale for each block of 128 x 128. The
 * reference has no kernel for n positions in fp8; this one exists so that a
 * decoder with fp8 weights can read a prompt in one pass (vx_decoder_prefill),
 * and as a direct call (vx_b200_gemm_fp8).
 *
 * The plan is the one of moe_grouped.cu: sixteen positions are the N side of two
 * mma.sync.m16n8k16, sixteen weight rows the M side, the activations three bf16
 * terms that sum to the f32 value exactly, a warp carrying two row tiles that
 * share every B fragment, the codes arriving 64 bytes a row through a cp.async
 * buffer of the warp's own. What differs is the unpacking. An e4m3 code is
 * exact in bf16 (3 bits of mantissa, exponents well inside bf16's): its seven
 * low bits shifted left by four are a bf16 with the same mantissa and an
 * exponent field 120 too small, sign moved to bit 15; one bf16 multiply by
 * 2^120 puts the value right, subnormal codes included (they become bf16
 * subnormals before the multiply). A lane's word holds the codes of columns
 * 4t .. 4t + 3 of a 16-column step; codes 0 and 2 go to the MMA's k slots 2t and
 * 2t + 1, codes 1 and 3 to 2t + 8 and 2t + 9, and the staged terms sit in that
 * order (0 2 1 3) so that no lane shuffles anything. The block's scale is
 * applied to the f32 sum of 64 columns.
 */
#include "kernels.h"
#include "launch.cuh"

#include <cstdio>

namespace vxb {
namespace {

constexpr int kWarps = 8;
constexpr int kRowTiles = 2;       /* 16-row tiles a warp carries */
constexpr int kPositions = 16;     /* of a block: two MMA columns of eight */
constexpr int kChunk = 512;        /* columns staged at a time */
constexpr int kStepCols = 64;      /* columns of one trip through the buffer */
/* a position's terms of a chunk; the pad keeps the four positions a half-warp
   reads together (8 bytes a lane) in different banks */
constexpr int kTermStride = kChunk * 2 + 32;
/* 64 bytes a row, rows 80 bytes apart: the eight rows a 4-byte load touches
   fall in different banks */
constexpr int kRowStride = 80;
constexpr int kStepBytes = 2 * kRowTiles * 8 * kRowStride;
constexpr int kWarpBytes = 2 * kStepBytes;
constexpr int kSmemBytes = 3 * kPositions * kTermStride + kWarps * kWarpBytes;

struct Fp8RowsArgs {
  const uint32_t *w;       /* [rows, cols / 4] */
  const float *scales;     /* [ceil(rows / 128), cols / 128] */
  const float *x;          /* [n, cols] f32, or */
  const uint16_t *x_terms; /* [n, 3 cols] bf16: x1 | x2 | x3 of a row */
  float *out;              /* [n, rows] */
  int n, rows, cols;
};

__device__ __forceinline__ void mma_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1,
                                            uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
               "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

/* The codes in bits 0-7 and 16-23 of `two` as two bf16 values. */
__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2(uint32_t two) {
  const uint32_t small = ((two & 0x007f007fu) << 4) | ((two & 0x00800080u) << 8);
  uint32_t d;
  const uint32_t up = 0x7b807b80u, zero = 0x80008000u; /* 2^120 twice; -0 twice */
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(small), "r"(up), "r"(zero));
  return d;
}

__device__ __forceinline__ uint32_t bf16x2_of(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
/* two values as three words of two bf16 each, term by term: v = t[0] + t[1] +
   t[2] exactly */
__device__ __forceinline__ void three_bf16x2(float lo, float hi, uint32_t (&t)[3]) {
  t[0] = bf16x2_of(lo, hi);
  lo -= __uint_as_float(t[0] << 16);
  hi -= __uint_as_float(t[0] & 0xffff0000u);
  t[1] = bf16x2_of(lo, hi);
  lo -= __uint_as_float(t[1] << 16);
  hi -= __uint_as_float(t[1] & 0xffff0000u);
  t[2] = bf16x2_of(lo, hi);
}

__device__ __forceinline__ void copy16_async(void *smem_dst, const void *src) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src)
               : "memory");
}
__device__ __forceinline__ void copies_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int LEFT> __device__ __forceinline__ void copies_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(LEFT) : "memory");
}

__global__ void __launch_bounds__(kWarps * 32, 2)
gemm_fp8_rows_kernel(const Fp8RowsArgs a) {
  constexpr int M = kRowTiles, NT = kPositions / 8;
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char *terms = smem;
  chain_release();
  chain_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  unsigned char *mine = smem + 3 * kPositions * kTermStride + warp * kWarpBytes;
  const int first_position = blockIdx.x * kPositions;

  const int words = a.cols / 4, scale_cols = a.cols / 128;
  /* The rows behind A rows g (h = 0) and g + 8 (h = 1) of each tile of this
     warp; a row past the end reads row 0 and is not written. */
  const int row_tiles = (a.rows + 15) / 16;
  bool valid[M][2];
  int row[M][2];
  const uint32_t *wrow[M][2];
  const float *srow[M][2];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const int rt = (blockIdx.y * kWarps + warp) * M + m;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = rt * 16 + g + 8 * h;
      valid[m][h] = rt < row_tiles && r < a.rows;
      row[m][h] = valid[m][h] ? r : 0;
      wrow[m][h] = a.w + (int64_t)row[m][h] * words;
      srow[m][h] = a.scales + (int64_t)(row[m][h] >> 7) * scale_cols;
    }
  }
  const bool any = (blockIdx.y * kWarps + warp) * M < row_tiles;
  float acc[M][NT][4];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int n = 0; n < NT; ++n)
      acc[m][n][0] = acc[m][n][1] = acc[m][n][2] = acc[m][n][3] = 0.0f;

  /* step s of the chunk at column c0: 64 columns of this lane's four rows */
  auto fetch_step = [&](int c0, int s) {
    unsigned char *dst = mine + (s & 1) * kStepBytes + g * kRowStride + t * 16;
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        copy16_async(dst + (m * 2 + h) * 8 * kRowStride,
                     wrow[m][h] + (c0 + kStepCols * s) / 4 + 4 * t);
    copies_commit();
  };

  for (int c0 = 0; c0 < a.cols; c0 += kChunk) {
    const int ncols = a.cols - c0 < kChunk ? a.cols - c0 : kChunk;
    const int steps = any ? ncols / kStepCols : 0;
    __syncthreads(); /* the last chunk has been read */
    if (steps > 0)
      fetch_step(c0, 0); /* under the staging below */
    /* eight columns of one position per item: three words of terms, each four
       columns in the order 0 2 1 3 */
    for (int item = threadIdx.x; item < kPositions * (ncols / 8); item += kWarps * 32) {
      const int j = item / (ncols / 8), word = item - j * (ncols / 8);
      const int p = first_position + j;
      unsigned char *dst = terms + j * kTermStride + word * 16;
      if (a.x_terms) {
        const uint16_t *src = a.x_terms + (int64_t)(p < a.n ? p : 0) * 3 * a.cols + c0 +
                              word * 8;
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          uint4 q = make_uint4(0, 0, 0, 0);
          if (p < a.n) {
            const uint4 v = *reinterpret_cast<const uint4 *>(src + (int64_t)k * a.cols);
            q = make_uint4(__byte_perm(v.x, v.y, 0x5410), __byte_perm(v.x, v.y, 0x7632),
                           __byte_perm(v.z, v.w, 0x5410), __byte_perm(v.z, v.w, 0x7632));
          }
          *reinterpret_cast<uint4 *>(dst + k * kPositions * kTermStride) = q;
        }
        continue;
      }
      float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (p < a.n) {
        const float4 *src =
            reinterpret_cast<const float4 *>(a.x + (int64_t)p * a.cols + c0 + word * 8);
        const float4 lo = src[0], hi = src[1];
        v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
        v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
      }
      uint32_t tm[4][3];
      three_bf16x2(v[0], v[2], tm[0]);
      three_bf16x2(v[1], v[3], tm[1]);
      three_bf16x2(v[4], v[6], tm[2]);
      three_bf16x2(v[5], v[7], tm[3]);
#pragma unroll
      for (int k = 0; k < 3; ++k)
        *reinterpret_cast<uint4 *>(dst + k * kPositions * kTermStride) =
            make_uint4(tm[0][k], tm[1][k], tm[2][k], tm[3][k]);
    }
    __syncthreads();
    if (!any)
      continue;

    for (int s = 0; s < steps; ++s) {
      if (s + 1 < steps) {
        fetch_step(c0, s + 1);
        copies_wait<1>();
      } else {
        copies_wait<0>();
      }
      __syncwarp(); /* every lane's part of step s has landed */
      float scale[M][2];
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          scale[m][h] = __ldg(srow[m][h] + ((c0 + kStepCols * s) >> 7));
      const unsigned char *src = mine + (s & 1) * kStepBytes + g * kRowStride + t * 4;
      float c[M][NT][4];
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n)
          c[m][n][0] = c[m][n][1] = c[m][n][2] = c[m][n][3] = 0.0f;
#pragma unroll
      for (int u = 0; u < 4; ++u) { /* sixteen columns each */
        uint32_t even[M][2], odd[M][2];
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t wd = *reinterpret_cast<const uint32_t *>(
                src + (m * 2 + h) * 8 * kRowStride + u * 16);
            even[m][h] = e4m3x2_to_bf16x2(wd & 0x00ff00ffu);        /* codes 0, 2 */
            odd[m][h] = e4m3x2_to_bf16x2((wd >> 8) & 0x00ff00ffu);  /* codes 1, 3 */
          }
        const int at = (kStepCols * s + 16 * u + 4 * t) * 2;
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int k = 0; k < 3; ++k) {
            const uint2 b = *reinterpret_cast<const uint2 *>(
                terms + (k * kPositions + n * 8 + g) * kTermStride + at);
#pragma unroll
            for (int m = 0; m < M; ++m)
              mma_16x8x16(c[m][n], even[m][0], even[m][1], odd[m][0], odd[m][1], b.x,
                          b.y);
          }
      }
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          acc[m][n][0] = fmaf(scale[m][0], c[m][n][0], acc[m][n][0]);
          acc[m][n][1] = fmaf(scale[m][0], c[m][n][1], acc[m][n][1]);
          acc[m][n][2] = fmaf(scale[m][1], c[m][n][2], acc[m][n][2]);
          acc[m][n][3] = fmaf(scale[m][1], c[m][n][3], acc[m][n][3]);
        }
      __syncwarp(); /* stage s & 1 may be filled again */
    }
  }

  /* acc[m][n][0..1]: A row g, positions 8 n + 2t and 8 n + 2t + 1; [2..3]: row g + 8 */
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const int p0 = first_position + n * 8 + 2 * t, p1 = p0 + 1;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (!valid[m][h])
          continue;
        if (p0 < a.n)
          a.out[(int64_t)p0 * a.rows + row[m][h]] = acc[m][n][2 * h];
        if (p1 < a.n)
          a.out[(int64_t)p1 * a.rows + row[m][h]] = acc[m][n][2 * h + 1];
      }
    }
}

const char *launch(const Fp8RowsArgs &a, cudaStream_t stream) {
  if (a.n <= 0 || a.rows <= 0 || a.cols <= 0 || a.cols % 128 != 0)
    return "an fp8 product needs columns in multiples of 128";
  if (((uintptr_t)a.w | (uintptr_t)a.x | (uintptr_t)a.x_terms | (uintptr_t)a.out) & 15)
    return "the codes, the activations and the output must be 16-byte aligned";
  if (allow_dynamic_smem((const void *)gemm_fp8_rows_kernel, kSmemBytes) != cudaSuccess)
    return "the fp8 product could not get its shared memory on this GPU";
  const int row_tiles = (a.rows + 15) / 16, per_block = kWarps * kRowTiles;
  const dim3 grid((a.n + kPositions - 1) / kPositions,
                  (row_tiles + per_block - 1) / per_block);
  if (grid.y > 65535)
    return "too many rows";
  launch_chained(gemm_fp8_rows_kernel, grid, dim3(kWarps * 32), kSmemBytes, stream, a);
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess)
    return nullptr;
  static thread_local char msg[200];
  snprintf(msg, sizeof msg, "the fp8 product: %s", cudaGetErrorString(e));
  return msg;
}

} // namespace

const char *gemm_fp8(float *y, const void *w, const void *scales, const float *x, int n,
                     int rows, int cols, cudaStream_t stream) {
  Fp8RowsArgs a{};
  a.w = (const uint32_t *)w;
  a.scales = (const float *)scales;
  a.x = x;
  a.out = y;
  a.n = n;
  a.rows = rows;
  a.cols = cols;
  return launch(a, stream);
}

const char *rows_gemm_fp8(const void *terms, const void *w, const void *scales, int t,
                          int n, int cols, float *partials, cudaStream_t stream) {
  Fp8RowsArgs a{};
  a.w = (const uint32_t *)w;
  a.scales = (const float *)scales;
  a.x_terms = (const uint16_t *)terms;
  a.out = partials;
  a.n = t;
  a.rows = n;
  a.cols = cols;
  return launch(a, stream);
}

} // namespace vxb
