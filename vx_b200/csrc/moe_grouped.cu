/* moe_grouped.cu -- the Q4_0 expert projections of many positions on the tensor
 * cores, fed by the grouping of moe_group.cu.
 *
 * nn_moe_swiglu_q4_rows and nn_moe_down_q4_add_rows (stdlib/std/nn.vx:2952-3155)
 * give every (position, slot) pair a block of its own and count on the cache to
 * keep an expert's rows near while the pairs that share it pass by. Here the
 * pairs arrive sorted by expert in tiles of eight or sixteen (nn_moe_group with
 * align 8 or 16), and a tile is the N side of one or two mma.sync.m16n8k16:
 * sixteen weight rows are unpacked once and multiply all pairs of the tile.
 *
 *   A (16 x 16, bf16)  weights. A lane holds one 32-bit word (eight 4-bit codes)
 *                      of row g and one of row g + 8, g = lane / 4; the four
 *                      lanes of a row hold the four words of one 32-column
 *                      group, which is also one scale. code - 8 is exact in
 *                      bf16 (0x4300 | code is 128 + code; minus 136).
 *   B (16 x 8, bf16)   activations, pair j of the tile in column j, as three
 *                      bf16 terms whose sum is the f32 value exactly; one MMA
 *                      per term into the same accumulator. The terms of a tile
 *                      are made once per block, in shared memory, in the order
 *                      of the codes inside a word (0 4 1 5 2 6 3 7) so that one
 *                      mask yields two A elements.
 *   C (16 x 8, f32)    the 32 columns of a group; times the group's two scales
 *                      it is added to the lane's running sums.
 *
 * A warp carries two 16-row tiles, so a B fragment read from shared memory
 * feeds both. Its codes come 128 columns at a time through a small buffer of
 * its own (cp.async, 16 bytes a lane, the next step in flight under the
 * current one) and are read back a word a lane: asked for straight from global
 * memory, a word a lane is sixteen rows of 16 bytes per load, and the load
 * pipe, not the tensor pipe, set the pace (81 % against 38 % busy).
 *
 * SwiGLU takes rows 0-7 of A from the gate matrix and rows 8-15 from the up
 * matrix, so a lane ends with the gate and the up value of the same (row,
 * pair) and finishes in registers. The down projection writes weight * dot for
 * every pair to a scratch the caller gives, and a second kernel adds a
 * position's k rows to y in slot order: no atomics, the same sum every run.
 *
 * Not the one-position kernels' order of sums: these are additive entry points
 * (vx_b200_moe_*_grouped), checked against f64 loops by the criterion of the
 * reference's Q4_0 tests, and the vx_nn_*_rows exports keep the bit-for-bit
 * property.
 *
 * One matrix and the positions as they come (no order, no tile_expert) is a
 * Q4_0 GEMM: vx_b200_gemm_q4 on f32 activations, and rows_gemm_q4 on the terms
 * that the prompt pass of a decoder keeps between its GEMMs (prefill.cu).
 */
#include "kernels.h"
#include "launch.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>

namespace vxb {
namespace {

constexpr int kWarps = 8;
constexpr int kRowTiles = 2;       /* 16-row tiles a warp carries: they share B */
constexpr int kChunk = 512;        /* columns staged at a time: 16 groups */
/* a pair's terms of a chunk, padded so that the two pairs a quarter-warp reads
   together fall in different banks */
constexpr int kTermStride = kChunk * 2 + 64;
/* A warp's weights of one step (128 columns of its 32 rows) pass through shared
   memory: 64 bytes a row, rows 80 bytes apart so that the eight rows a load
   touches fall in different banks; two steps in flight. */
constexpr int kRowStride = 80;
constexpr int kStepBytes = 2 * kRowTiles * 8 * kRowStride;
static_assert(kChunk == 4 * 128, "lane t of a row keeps the scales of step t: four steps a chunk");
constexpr int kWarpBytes = 2 * kStepBytes;
constexpr int smem_bytes(int pairs) {
  return 3 * pairs * kTermStride + kWarps * kWarpBytes;
}

struct GroupedArgs {
  const uint32_t *w;          /* all experts, [experts * expert_rows, cols / 8] */
  const __half *scales;       /* [experts * expert_rows, cols / 32] */
  const int32_t *order;       /* from nn_moe_group, align 8 or 16; null: position
                                 i of tile t is pair t * align + i */
  const int32_t *tile_expert; /* null: one matrix, every tile its own */
  const float *x;             /* input of pair p: row p / x_div, x_pitch apart */
  int64_t x_pitch;
  int x_div;
  const uint16_t *x_terms;    /* or the input as three bf16 terms, [rows, 3 cols]
                                 (x1 | x2 | x3 of a row, as prefill.cu leaves them) */
  float *out;                 /* output of pair p: row p, out_pitch apart */
  int64_t out_pitch;
  const float *pair_scale;    /* down: the router's weight of pair p */
  int pairs, rows, cols, experts;
  int64_t expert_rows;        /* 2 * rows (gate then up) or rows */
  int four_groups;            /* cols % 128 == 0, codes 16-byte and scales 8-byte
                                 aligned: 128 columns a step through shared memory */
};

__device__ __forceinline__ void mma_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1,
                                            uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
               "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

/* the same with C = 0: the first product of a group needs no cleared registers */
__device__ __forceinline__ void mma_16x8x16_first(float (&c)[4], uint32_t a0,
                                                  uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
               "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
               : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

/* two codes (bits 0-3 and 16-19 of `two`) as two bf16 values code - 8 */
__device__ __forceinline__ uint32_t codes_to_bf16x2(uint32_t two) {
  uint32_t d;
  const uint32_t biased = two | 0x43004300u, off = 0x43084308u;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(biased), "r"(off));
  return d;
}

/* an f16 as f32 by a mixed-precision add, which runs on the FMA pipe (a cvt
   goes to the quarter-rate pipe) */
__device__ __forceinline__ float half_value(uint32_t b) {
  float d;
  asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"((unsigned short)b), "f"(-0.0f));
  return d;
}
/* d[0..1] += s * c[0..1] in one instruction */
__device__ __forceinline__ void scale_add2(float &d0, float &d1, float s, float c0,
                                           float c1) {
  unsigned long long d, cc, ss;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(d0), "f"(d1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(cc) : "f"(c0), "f"(c1));
  asm("mov.b64 %0, {%1, %1};" : "=l"(ss) : "f"(s));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(ss), "l"(cc));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}

/* Two values as three words of two bf16 each (lo in the low half), term by
   term: v = t[0] + t[1] + t[2] exactly, 24 bits of mantissa in three times 8.
   One conversion rounds both values. */
__device__ __forceinline__ uint32_t bf16x2_of(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
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

/* NT: the tile's pairs in MMA columns of eight (1: align 8, 2: align 16). */
template <bool SWIGLU, int NT>
__global__ void __launch_bounds__(kWarps * 32, 2)
moe_grouped_kernel(const GroupedArgs a) {
  constexpr int PAIRS = 8 * NT;
  constexpr int M = kRowTiles;
  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char *terms = smem;
  __shared__ int pair_of[PAIRS];
  chain_release();
  chain_wait();
  const int tile = blockIdx.x;
  const int expert = a.tile_expert ? a.tile_expert[tile] : 0;
  if (expert < 0 || expert >= a.experts)
    return; /* past the last group: the whole block leaves together */
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  unsigned char *mine = smem + 3 * PAIRS * kTermStride + warp * kWarpBytes;
  if (threadIdx.x < PAIRS) {
    const int at = tile * PAIRS + threadIdx.x;
    const int p = a.order ? a.order[at] : at;
    pair_of[threadIdx.x] = p >= 0 && p < a.pairs ? p : -1;
  }

  const int words = a.cols / 8, groups = a.cols / 32;
  /* The rows behind A rows g (h = 0) and g + 8 (h = 1) of each 16-row tile of
     this warp. A tile past the end reads row 0 and is not written. */
  const int row_tiles = SWIGLU ? a.rows / 8 : (a.rows + 15) / 16;
  bool live[M];
  int64_t row[M][2];
  const uint32_t *wrow[M][2];
  const unsigned short *srow[M][2];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const int rt = (blockIdx.y * kWarps + warp) * M + m;
    live[m] = rt < row_tiles;
    if (SWIGLU) {
      row[m][0] = live[m] ? rt * 8 + g : 0;
      row[m][1] = row[m][0] + a.rows;
    } else {
      row[m][0] = live[m] ? rt * 16 + g : 0;
      row[m][1] = row[m][0] + 8 < a.rows ? row[m][0] + 8 : row[m][0]; /* a last tile of 8 rows */
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t r = (int64_t)expert * a.expert_rows + row[m][h];
      wrow[m][h] = a.w + r * words;
      srow[m][h] = reinterpret_cast<const unsigned short *>(a.scales) + r * groups;
    }
  }
  const bool any = live[0]; /* tiles are handed out in order: the first is the test */
  float acc[M][NT][4];
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int n = 0; n < NT; ++n)
      acc[m][n][0] = acc[m][n][1] = acc[m][n][2] = acc[m][n][3] = 0.0f;

  /* One group of 32 columns, group `q` of the staged chunk: this lane's word of
     each of its four rows and the rows' scales. B is read once for both tiles. */
  auto group = [&](int q, const uint32_t (&wd)[M][2], const float (&sc)[M][2]) {
    constexpr uint32_t MASK = 0x000f000fu;
    uint32_t ac[M][2][4];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < 4; ++i)
          ac[m][h][i] = codes_to_bf16x2((wd[m][h] >> (4 * i)) & MASK);
    float c[M][NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
      for (int k = 0; k < 3; ++k) {
        const uint4 b = *reinterpret_cast<const uint4 *>(
            terms + (k * PAIRS + n * 8 + g) * kTermStride + q * 64 + t * 16);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          if (k == 0)
            mma_16x8x16_first(c[m][n], ac[m][0][0], ac[m][1][0], ac[m][0][1],
                              ac[m][1][1], b.x, b.y);
          else
            mma_16x8x16(c[m][n], ac[m][0][0], ac[m][1][0], ac[m][0][1], ac[m][1][1],
                        b.x, b.y);
          mma_16x8x16(c[m][n], ac[m][0][2], ac[m][1][2], ac[m][0][3], ac[m][1][3], b.z,
                      b.w);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        scale_add2(acc[m][n][0], acc[m][n][1], sc[m][0], c[m][n][0], c[m][n][1]);
        scale_add2(acc[m][n][2], acc[m][n][3], sc[m][1], c[m][n][2], c[m][n][3]);
      }
  };

  /* The codes of step `s` of the chunk at group g0 (128 columns of the four
     rows of this lane's g) on their way to stage s & 1 of the warp's buffer. */
  auto fetch_step = [&](int g0, int s) {
    unsigned char *dst = mine + (s & 1) * kStepBytes + g * kRowStride + t * 16;
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        copy16_async(dst + (m * 2 + h) * 8 * kRowStride,
                     wrow[m][h] + (g0 + 4 * s) * 4 + 4 * t);
    copies_commit();
  };

  for (int c0 = 0; c0 < a.cols; c0 += kChunk) {
    const int ncols = a.cols - c0 < kChunk ? a.cols - c0 : kChunk;
    const int g0 = c0 / 32, nq = ncols / 32;
    const int steps = a.four_groups && any ? nq / 4 : 0;
    __syncthreads(); /* pair_of is written; the last chunk has been read */
    if (steps > 0)
      fetch_step(g0, 0); /* under the staging below */
    /* eight columns of one pair per step: three words of permuted terms */
    for (int item = threadIdx.x; item < PAIRS * (ncols / 8); item += kWarps * 32) {
      const int j = item / (ncols / 8), word = item - j * (ncols / 8);
      const int p = pair_of[j];
      unsigned char *dst = terms + j * kTermStride + word * 16;
      if (a.x_terms) {
        /* made by an earlier kernel: only the order inside the word changes */
        const uint16_t *src =
            a.x_terms + (int64_t)(p < 0 ? 0 : p / a.x_div) * 3 * a.cols + c0 + word * 8;
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          uint4 q = make_uint4(0, 0, 0, 0);
          if (p >= 0) {
            const uint4 v = *reinterpret_cast<const uint4 *>(src + (int64_t)k * a.cols);
            q = make_uint4(__byte_perm(v.x, v.z, 0x5410), __byte_perm(v.x, v.z, 0x7632),
                           __byte_perm(v.y, v.w, 0x5410), __byte_perm(v.y, v.w, 0x7632));
          }
          *reinterpret_cast<uint4 *>(dst + k * PAIRS * kTermStride) = q;
        }
        continue;
      }
      float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (p >= 0) {
        const float4 *src = reinterpret_cast<const float4 *>(
            a.x + (int64_t)(p / a.x_div) * a.x_pitch + c0 + word * 8);
        const float4 lo = src[0], hi = src[1];
        v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
        v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
      }
      uint32_t tm[4][3]; /* columns (i, i + 4) of the word, as the codes pair up */
#pragma unroll
      for (int i = 0; i < 4; ++i)
        three_bf16x2(v[i], v[i + 4], tm[i]);
#pragma unroll
      for (int k = 0; k < 3; ++k)
        *reinterpret_cast<uint4 *>(dst + k * PAIRS * kTermStride) =
            make_uint4(tm[0][k], tm[1][k], tm[2][k], tm[3][k]);
    }
    /* Lane t keeps the four scales of step t of each of its rows: one 8-byte
       load a row and chunk, handed round by shuffles. */
    uint2 my_scales[M][2];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        my_scales[m][h] = t < steps
                              ? __ldg(reinterpret_cast<const uint2 *>(srow[m][h] + g0 + 4 * t))
                              : make_uint2(0, 0);
    __syncthreads();
    if (!any)
      continue;

    for (int s = 0; s < steps; ++s) {
      if (s + 1 < steps) {
        fetch_step(g0, s + 1);
        copies_wait<1>();
      } else {
        copies_wait<0>();
      }
      __syncwarp(); /* every lane's part of step s has landed */
      uint2 four[M][2];
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          four[m][h].x = __shfl_sync(0xffffffffu, my_scales[m][h].x, (lane & ~3) | s);
          four[m][h].y = __shfl_sync(0xffffffffu, my_scales[m][h].y, (lane & ~3) | s);
        }
      const unsigned char *src = mine + (s & 1) * kStepBytes + g * kRowStride + t * 4;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint32_t wd[M][2];
        float sc[M][2];
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            wd[m][h] = *reinterpret_cast<const uint32_t *>(
                src + (m * 2 + h) * 8 * kRowStride + u * 16);
            const uint32_t two = u < 2 ? four[m][h].x : four[m][h].y;
            sc[m][h] = half_value((u & 1) ? two >> 16 : two & 0xffffu);
          }
        group(4 * s + u, wd, sc);
      }
      __syncwarp(); /* stage s & 1 may be filled again */
    }
    /* what the steps did not take: a chunk that is not a multiple of 128
       columns, or operands not aligned for them */
    for (int q = 4 * steps; q < nq; ++q) {
      uint32_t wd[M][2];
      float sc[M][2];
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          wd[m][h] = __ldg(wrow[m][h] + (g0 + q) * 4 + t);
          sc[m][h] = half_value(__ldg(srow[m][h] + g0 + q));
        }
      group(q, wd, sc);
    }
  }

  /* acc[m][n][0..1]: A row g, pairs 8 n + 2t and 8 n + 2t + 1; [2..3]: row g + 8 */
#pragma unroll
  for (int m = 0; m < M; ++m) {
    if (!live[m])
      continue;
    const int64_t r0 = row[m][0], r1 = row[m][1];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const int p0 = pair_of[n * 8 + 2 * t], p1 = pair_of[n * 8 + 2 * t + 1];
      if (SWIGLU) {
        const float g0v = acc[m][n][0], g1v = acc[m][n][1];
        if (p0 >= 0)
          a.out[p0 * a.out_pitch + r0] = g0v / (1.0f + expf(0.0f - g0v)) * acc[m][n][2];
        if (p1 >= 0)
          a.out[p1 * a.out_pitch + r0] = g1v / (1.0f + expf(0.0f - g1v)) * acc[m][n][3];
      } else {
        const bool second = r1 != r0;
        if (p0 >= 0) {
          const float s = a.pair_scale ? a.pair_scale[p0] : 1.0f;
          a.out[p0 * a.out_pitch + r0] = s * acc[m][n][0];
          if (second)
            a.out[p0 * a.out_pitch + r1] = s * acc[m][n][2];
        }
        if (p1 >= 0) {
          const float s = a.pair_scale ? a.pair_scale[p1] : 1.0f;
          a.out[p1 * a.out_pitch + r0] = s * acc[m][n][1];
          if (second)
            a.out[p1 * a.out_pitch + r1] = s * acc[m][n][3];
        }
      }
    }
  }
}

/* y[t][r] += d[t * k][r] + ... + d[t * k + k - 1][r], one after another */
__global__ void __launch_bounds__(256)
moe_combine_kernel(float *y, int64_t y_pitch, const float *d, int64_t d_pitch, int n,
                   int k, int rows) {
  chain_release();
  chain_wait();
  const int per_row = rows / 4;
  const int64_t total = (int64_t)n * per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / per_row), r = (int)(i - (int64_t)t * per_row) * 4;
    float4 v = *reinterpret_cast<const float4 *>(y + t * y_pitch + r);
    for (int e = 0; e < k; ++e) {
      const float4 add =
          *reinterpret_cast<const float4 *>(d + ((int64_t)t * k + e) * d_pitch + r);
      v.x += add.x; v.y += add.y; v.z += add.z; v.w += add.w;
    }
    *reinterpret_cast<float4 *>(y + t * y_pitch + r) = v;
  }
}

const char *launched(const char *what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess)
    return nullptr;
  static thread_local char msg[200];
  snprintf(msg, sizeof msg, "%s: %s", what, cudaGetErrorString(e));
  return msg;
}

const char *check_common(const MoeGroupedArgs &m) {
  if (m.n <= 0 || m.k <= 0 || m.experts <= 0 || m.rows <= 0 || m.cols <= 0)
    return "n, k, rows, cols and experts must be positive";
  if (m.cols % 32 != 0 || m.rows % 8 != 0)
    return "cols must be a multiple of 32, and rows of 8";
  if ((int64_t)m.n * m.k > (1 << 30))
    return "too many pairs";
  if (m.align != 8 && m.align != 16)
    return "the pairs must be grouped with align 8 or 16";
  const int64_t room = (int64_t)m.n * m.k + (int64_t)m.experts * (m.align - 1);
  if (m.tiles <= 0 || (int64_t)m.tiles * m.align < room)
    return "`order` and `tile_expert` must come from nn_moe_group with this align: "
           "tiles * align >= n * k + experts * (align - 1)";
  if (((uintptr_t)m.x | (uintptr_t)m.out) & 15 || m.x_pitch % 4 != 0 ||
      m.out_pitch % 4 != 0)
    return "the activations must be 16-byte aligned, with pitches that are "
           "multiples of 4 values";
  return nullptr;
}

template <bool SWIGLU, int NT>
const char *launch_grouped_nt(GroupedArgs &g, int tiles, cudaStream_t stream) {
  constexpr int bytes = smem_bytes(8 * NT);
  if (allow_dynamic_smem((const void *)moe_grouped_kernel<SWIGLU, NT>, bytes) !=
      cudaSuccess)
    return "the grouped expert projection could not get its shared memory on this GPU";
  g.four_groups = g.cols % 128 == 0 && ((uintptr_t)g.scales & 7) == 0 &&
                  ((uintptr_t)g.w & 15) == 0;
  const int row_tiles = SWIGLU ? g.rows / 8 : (g.rows + 15) / 16;
  const int per_block = kWarps * kRowTiles;
  const dim3 grid(tiles, (row_tiles + per_block - 1) / per_block);
  if (grid.y > 65535)
    return "too many rows";
  launch_chained(moe_grouped_kernel<SWIGLU, NT>, grid, dim3(kWarps * 32), bytes, stream,
                 g);
  return launched("the grouped expert projection");
}

template <bool SWIGLU>
const char *launch_grouped(GroupedArgs &g, int tiles, int align, cudaStream_t stream) {
  return align == 16 ? launch_grouped_nt<SWIGLU, 2>(g, tiles, stream)
                     : launch_grouped_nt<SWIGLU, 1>(g, tiles, stream);
}

} // namespace

/* partials[t][r] = (row r of the Q4_0 matrix) . x[t], x given as terms: the
   prompt's GEMM for a decoder with Q4_0 weights. One "expert", the positions
   in tiles of sixteen as they come. */
const char *rows_gemm_q4(const void *terms, const void *w, const void *scales, int t,
                         int n, int cols, float *partials, cudaStream_t stream) {
  if (t <= 0 || n <= 0 || n % 8 != 0 || cols <= 0 || cols % 32 != 0)
    return "a Q4_0 product over a prompt needs rows in multiples of 8 and columns "
           "in multiples of 32";
  if (((uintptr_t)terms | (uintptr_t)partials) & 15)
    return "the terms and the sums must be 16-byte aligned";
  GroupedArgs g{};
  g.w = (const uint32_t *)w;
  g.scales = (const __half *)scales;
  g.x_terms = (const uint16_t *)terms;
  g.x_div = 1;
  g.out = partials;
  g.out_pitch = n;
  g.pairs = t;
  g.rows = n;
  g.cols = cols;
  g.experts = 1;
  g.expert_rows = n;
  return launch_grouped<false>(g, (t + 15) / 16, 16, stream);
}

/* y[t][r] = (row r of the Q4_0 matrix) . x[t] for n rows of f32 activations:
   the same kernel as one matrix, fed f32 values instead of terms. */
const char *gemm_q4(float *y, const void *w, const void *scales, const float *x, int n,
                    int rows, int cols, cudaStream_t stream) {
  if (n <= 0 || rows <= 0 || rows % 8 != 0 || cols <= 0 || cols % 32 != 0)
    return "a Q4_0 product needs rows in multiples of 8 and columns in multiples of 32";
  if (((uintptr_t)x | (uintptr_t)y) & 15)
    return "the activations and the output must be 16-byte aligned";
  GroupedArgs g{};
  g.w = (const uint32_t *)w;
  g.scales = (const __half *)scales;
  g.x = x;
  g.x_pitch = cols;
  g.x_div = 1;
  g.out = y;
  g.out_pitch = rows;
  g.pairs = n;
  g.rows = rows;
  g.cols = cols;
  g.experts = 1;
  g.expert_rows = rows;
  return n > 8 ? launch_grouped<false>(g, (n + 15) / 16, 16, stream)
               : launch_grouped<false>(g, 1, 8, stream);
}

const char *moe_swiglu_q4_grouped(const MoeGroupedArgs &m, cudaStream_t stream) {
  if (const char *why = check_common(m))
    return why;
  GroupedArgs g{};
  g.w = (const uint32_t *)m.w;
  g.scales = (const __half *)m.scales;
  g.order = m.order;
  g.tile_expert = m.tile_expert;
  g.x = m.x;
  g.x_pitch = m.x_pitch;
  g.x_div = m.k; /* x has a row for each position */
  g.out = m.out;
  g.out_pitch = m.out_pitch;
  g.pair_scale = nullptr;
  g.pairs = m.n * m.k;
  g.rows = m.rows;
  g.cols = m.cols;
  g.experts = m.experts;
  g.expert_rows = 2 * (int64_t)m.rows;
  return launch_grouped<true>(g, m.tiles, m.align, stream);
}

const char *moe_down_q4_add_grouped(const MoeGroupedArgs &m, cudaStream_t stream) {
  if (const char *why = check_common(m))
    return why;
  if (!m.pair_weights || !m.scratch || !m.y)
    return "the down projection needs the router's weights, a scratch and y";
  if (((uintptr_t)m.y | (uintptr_t)m.scratch) & 15 || m.y_pitch % 4 != 0)
    return "y and the scratch must be 16-byte aligned";
  GroupedArgs g{};
  g.w = (const uint32_t *)m.w;
  g.scales = (const __half *)m.scales;
  g.order = m.order;
  g.tile_expert = m.tile_expert;
  g.x = m.x;
  g.x_pitch = m.x_pitch;
  g.x_div = 1; /* the input has a row for each pair */
  g.out = m.scratch;
  g.out_pitch = m.rows;
  g.pair_scale = m.pair_weights;
  g.pairs = m.n * m.k;
  g.rows = m.rows;
  g.cols = m.cols;
  g.experts = m.experts;
  g.expert_rows = m.rows;
  if (const char *why = launch_grouped<false>(g, m.tiles, m.align, stream))
    return why;
  const int64_t quads = (int64_t)m.n * (m.rows / 4);
  int blocks = (int)((quads + 255) / 256);
  if (blocks > 148 * 8)
    blocks = 148 * 8;
  launch_chained(moe_combine_kernel, dim3(blocks), dim3(256), 0, stream, m.y, m.y_pitch,
                 (const float *)m.scratch, (int64_t)m.rows, m.n, m.k, m.rows);
  return launched("the sum over a position's experts");
}

} // namespace vxb
