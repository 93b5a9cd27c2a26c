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
 */
#include "kernels.h"
#include "launch.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>

namespace vxb {
namespace {

constexpr int kWarps = 8;          /* a warp carries one tile of 16 rows */
constexpr int kChunk = 1024;       /* columns staged at a time */
/* a pair's terms of a chunk, padded so that the two pairs a quarter-warp reads
   together fall in different banks */
constexpr int kTermStride = kChunk * 2 + 64;
constexpr int smem_bytes(int pairs) { return 3 * pairs * kTermStride; }

struct GroupedArgs {
  const uint32_t *w;          /* all experts, [experts * expert_rows, cols / 8] */
  const __half *scales;       /* [experts * expert_rows, cols / 32] */
  const int32_t *order;       /* from nn_moe_group, align 8 or 16 */
  const int32_t *tile_expert;
  const float *x;             /* input of pair p: row p / x_div, x_pitch apart */
  int64_t x_pitch;
  int x_div;
  float *out;                 /* output of pair p: row p, out_pitch apart */
  int64_t out_pitch;
  const float *pair_scale;    /* down: the router's weight of pair p */
  int pairs, rows, cols, experts;
  int64_t expert_rows;        /* 2 * rows (gate then up) or rows */
  int four_groups;            /* cols % 128 == 0 and the scales 8-byte aligned */
};

__device__ __forceinline__ void mma_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1,
                                            uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
               "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

/* two codes (bits 0-3 and 16-19 of `two`) as two bf16 values code - 8 */
__device__ __forceinline__ uint32_t codes_to_bf16x2(uint32_t two) {
  uint32_t d;
  const uint32_t biased = two | 0x43004300u, off = 0x43084308u;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(biased), "r"(off));
  return d;
}

__device__ __forceinline__ unsigned short bf16_bits(float v) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
__device__ __forceinline__ float bf16_value(unsigned short b) {
  return __uint_as_float((uint32_t)b << 16);
}
__device__ __forceinline__ float half_value(unsigned short b) {
  return __half2float(__ushort_as_half(b));
}

/* v = t[0] + t[1] + t[2] exactly (24 bits of mantissa in three times 8) */
__device__ __forceinline__ void three_bf16(float v, unsigned short (&t)[3]) {
  t[0] = bf16_bits(v);
  const float r1 = v - bf16_value(t[0]);
  t[1] = bf16_bits(r1);
  const float r2 = r1 - bf16_value(t[1]);
  t[2] = bf16_bits(r2);
}

/* NT: the tile's pairs in MMA columns of eight (1: align 8, 2: align 16). */
template <bool SWIGLU, int NT>
__global__ void __launch_bounds__(kWarps * 32, 2)
moe_grouped_kernel(const GroupedArgs a) {
  constexpr int PAIRS = 8 * NT;
  extern __shared__ __align__(16) unsigned char terms[];
  __shared__ int pair_of[PAIRS];
  chain_release();
  chain_wait();
  const int tile = blockIdx.x;
  const int expert = a.tile_expert[tile];
  if (expert < 0 || expert >= a.experts)
    return; /* past the last group: the whole block leaves together */
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  if (threadIdx.x < PAIRS) {
    const int p = a.order[tile * PAIRS + threadIdx.x];
    pair_of[threadIdx.x] = p >= 0 && p < a.pairs ? p : -1;
  }

  const int words = a.cols / 8, groups = a.cols / 32;
  /* the rows behind A rows g and g + 8 of this warp's 16-row tile */
  const int row_tiles = SWIGLU ? a.rows / 8 : (a.rows + 15) / 16;
  const int rt = blockIdx.y * kWarps + warp;
  const bool live = rt < row_tiles;
  int64_t r0, r1;
  if (SWIGLU) {
    r0 = live ? rt * 8 + g : 0;
    r1 = r0 + a.rows;
  } else {
    r0 = live ? rt * 16 + g : 0;
    r1 = r0 + 8 < a.rows ? r0 + 8 : r0; /* a last tile of 8 rows */
  }
  const uint32_t *wa_row =
      a.w + ((int64_t)expert * a.expert_rows + r0) * words + t;
  const uint32_t *wb_row =
      a.w + ((int64_t)expert * a.expert_rows + r1) * words + t;
  const unsigned short *sa_row = reinterpret_cast<const unsigned short *>(a.scales) +
                                 ((int64_t)expert * a.expert_rows + r0) * groups;
  const unsigned short *sb_row = reinterpret_cast<const unsigned short *>(a.scales) +
                                 ((int64_t)expert * a.expert_rows + r1) * groups;
  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
    acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;

  /* One group of 32 columns: the two words of this lane, the group's two
     scales, group `q` of the staged chunk. */
  auto group = [&](int q, uint32_t wa, uint32_t wb, float sa, float sb) {
    constexpr uint32_t M = 0x000f000fu;
    const uint32_t a00 = codes_to_bf16x2(wa & M), a80 = codes_to_bf16x2(wb & M);
    const uint32_t a01 = codes_to_bf16x2((wa >> 4) & M),
                   a81 = codes_to_bf16x2((wb >> 4) & M);
    const uint32_t a02 = codes_to_bf16x2((wa >> 8) & M),
                   a82 = codes_to_bf16x2((wb >> 8) & M);
    const uint32_t a03 = codes_to_bf16x2((wa >> 12) & M),
                   a83 = codes_to_bf16x2((wb >> 12) & M);
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int k = 0; k < 3; ++k) {
        const uint4 b = *reinterpret_cast<const uint4 *>(
            terms + (k * PAIRS + n * 8 + g) * kTermStride + q * 64 + t * 16);
        mma_16x8x16(c, a00, a80, a01, a81, b.x, b.y);
        mma_16x8x16(c, a02, a82, a03, a83, b.z, b.w);
      }
      acc[n][0] = fmaf(sa, c[0], acc[n][0]);
      acc[n][1] = fmaf(sa, c[1], acc[n][1]);
      acc[n][2] = fmaf(sb, c[2], acc[n][2]);
      acc[n][3] = fmaf(sb, c[3], acc[n][3]);
    }
  };

  for (int c0 = 0; c0 < a.cols; c0 += kChunk) {
    const int ncols = a.cols - c0 < kChunk ? a.cols - c0 : kChunk;
    __syncthreads(); /* pair_of is written; the last chunk has been read */
    /* eight columns of one pair per step: three words of permuted terms */
    for (int item = threadIdx.x; item < PAIRS * (ncols / 8); item += kWarps * 32) {
      const int j = item / (ncols / 8), word = item - j * (ncols / 8);
      const int p = pair_of[j];
      float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (p >= 0) {
        const float4 *src = reinterpret_cast<const float4 *>(
            a.x + (int64_t)(p / a.x_div) * a.x_pitch + c0 + word * 8);
        const float4 lo = src[0], hi = src[1];
        v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
        v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
      }
      unsigned short tm[8][3];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        three_bf16(v[i], tm[i]);
#pragma unroll
      for (int k = 0; k < 3; ++k) {
        uint4 q;
        q.x = tm[0][k] | ((uint32_t)tm[4][k] << 16);
        q.y = tm[1][k] | ((uint32_t)tm[5][k] << 16);
        q.z = tm[2][k] | ((uint32_t)tm[6][k] << 16);
        q.w = tm[3][k] | ((uint32_t)tm[7][k] << 16);
        *reinterpret_cast<uint4 *>(terms + (k * PAIRS + j) * kTermStride + word * 16) = q;
      }
    }
    __syncthreads();
    if (!live)
      continue;

    const int g0 = c0 / 32, nq = ncols / 32;
    int q = 0;
    if (a.four_groups) {
      /* Four groups a step: the sixteen loads leave together, so a trip to L2
         is paid once for 128 columns of both rows, and the four scales of a
         row come as one 8-byte word. */
      for (; q + 4 <= nq; q += 4) {
        uint32_t wa[4], wb[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          wa[u] = __ldg(wa_row + (g0 + q + u) * 4);
          wb[u] = __ldg(wb_row + (g0 + q + u) * 4);
        }
        const uint2 sa = __ldg(reinterpret_cast<const uint2 *>(sa_row + g0 + q));
        const uint2 sb = __ldg(reinterpret_cast<const uint2 *>(sb_row + g0 + q));
        group(q, wa[0], wb[0], half_value(sa.x & 0xffffu), half_value(sb.x & 0xffffu));
        group(q + 1, wa[1], wb[1], half_value(sa.x >> 16), half_value(sb.x >> 16));
        group(q + 2, wa[2], wb[2], half_value(sa.y & 0xffffu), half_value(sb.y & 0xffffu));
        group(q + 3, wa[3], wb[3], half_value(sa.y >> 16), half_value(sb.y >> 16));
      }
    }
    for (; q < nq; ++q)
      group(q, __ldg(wa_row + (g0 + q) * 4), __ldg(wb_row + (g0 + q) * 4),
            half_value(__ldg(sa_row + g0 + q)), half_value(__ldg(sb_row + g0 + q)));
  }
  if (!live)
    return;

  /* acc[n][0..1]: A row g, pairs 8 n + 2t and 8 n + 2t + 1; acc[n][2..3]: row g + 8 */
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int p0 = pair_of[n * 8 + 2 * t], p1 = pair_of[n * 8 + 2 * t + 1];
    if (SWIGLU) {
      const float g0v = acc[n][0], g1v = acc[n][1];
      if (p0 >= 0)
        a.out[p0 * a.out_pitch + r0] = g0v / (1.0f + expf(0.0f - g0v)) * acc[n][2];
      if (p1 >= 0)
        a.out[p1 * a.out_pitch + r0] = g1v / (1.0f + expf(0.0f - g1v)) * acc[n][3];
    } else {
      const bool second = r1 != r0;
      if (p0 >= 0) {
        const float s = a.pair_scale[p0];
        a.out[p0 * a.out_pitch + r0] = s * acc[n][0];
        if (second)
          a.out[p0 * a.out_pitch + r1] = s * acc[n][2];
      }
      if (p1 >= 0) {
        const float s = a.pair_scale[p1];
        a.out[p1 * a.out_pitch + r0] = s * acc[n][1];
        if (second)
          a.out[p1 * a.out_pitch + r1] = s * acc[n][3];
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
  g.four_groups = g.cols % 128 == 0 && ((uintptr_t)g.scales & 7) == 0;
  const int row_tiles = SWIGLU ? g.rows / 8 : (g.rows + 15) / 16;
  const dim3 grid(tiles, (row_tiles + kWarps - 1) / kWarps);
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
