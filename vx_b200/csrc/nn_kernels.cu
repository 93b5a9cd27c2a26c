/* nn_kernels.cu -- the decode operators of one transformer token: bandwidth
 * bound, so every kernel is organised around streaming its weights (or its KV
 * cache) once, with 16-byte loads that a warp issues over consecutive
 * addresses, several in flight per lane, and warp-shuffle reductions.
 *
 * The arithmetic is the one the reference states in stdlib/std/nn.vx (bf16
 * weights, f32 activations, f32 sums; half-split RoPE with tables) and in
 * tests/backend/pass/llama2.vx:218-429 (f32 weights, interleaved RoPE computed
 * from pos, eps added after the mean); each kernel names the functions it
 * covers.  Where the reference launches one kernel per operator, these fuse
 * what follows a projection into it: RMSNorm in front of the q/k/v and the
 * gate/up projections, bias + RoPE + KV-cache store behind q/k/v, SwiGLU
 * behind gate/up, the residual add behind the output and down projections, and
 * the merge of the attention parts into the attention kernel itself (inside a
 * thread-block cluster, through distributed shared memory).
 *
 * No float atomics and a fixed order in every reduction: the same inputs give
 * the same bits on every run.
 */
#include "kernels.h"
#include "launch.cuh"
#include "nn_device.cuh"
#include "ptx.cuh"

#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace vxb {
namespace {

constexpr int WARPS = 16;            /* per block, projection kernels */
constexpr int MAX_SMEM_X = 96 * 1024; /* x (all batch rows) staged per block */

/* Sum over the block; every thread gets the result. `red` holds 32 floats. */
__device__ float block_sum(float v, float *red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0)
    red[warp] = v;
  __syncthreads();
  float t = 0.0f;
  for (int w = 0; w < nwarps; ++w) /* fixed order */
    t += red[w];
  return t;
}

/* The 16 weights of an fp8 word as f32: two codes to two f16 with the
   conversion instruction, and an f16 to f32 by adding it to -0.0f in a
   mixed-precision add, which issues with the other additions (a conversion to
   f32 for every weight made the kernel wait for the conversion unit, and
   building bf16 bit patterns with integer operations took more instructions:
   3 560, 3 380 and 2 850 GB/s on the 7B gate/up projection). */
__device__ __forceinline__ float widen_f16(unsigned short h) {
  float d;
  asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"(h), "f"(-0.0f));
  return d;
}
__device__ __forceinline__ void unpack_fp8(const uint4 &wv, float (&wf)[16]) {
  const uint32_t u[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    unsigned short lo, hi;
    asm("mov.b32 {%0, %1}, %2;" : "=h"(lo), "=h"(hi) : "r"(u[j]));
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t two;
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(two) : "h"(h == 0 ? lo : hi));
      unsigned short a, b;
      asm("mov.b32 {%0, %1}, %2;" : "=h"(a), "=h"(b) : "r"(two));
      wf[4 * j + 2 * h] = widen_f16(a);
      wf[4 * j + 2 * h + 1] = widen_f16(b);
    }
  }
}
/* d += a * b on two values at once (one instruction on sm_100) */
__device__ __forceinline__ void fma_pair(float2 &d, const float2 a, const float2 b) {
  unsigned long long dd = *reinterpret_cast<unsigned long long *>(&d);
  asm("fma.rn.f32x2 %0, %1, %2, %0;"
      : "+l"(dd)
      : "l"(*reinterpret_cast<const unsigned long long *>(&a)),
        "l"(*reinterpret_cast<const unsigned long long *>(&b)));
  d = *reinterpret_cast<float2 *>(&dd);
}
__device__ __forceinline__ float2 add_pair(const float2 a, const float2 b) {
  unsigned long long dd;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(dd)
      : "l"(*reinterpret_cast<const unsigned long long *>(&a)),
        "l"(*reinterpret_cast<const unsigned long long *>(&b)));
  return *reinterpret_cast<float2 *>(&dd);
}
__device__ __forceinline__ void unpack_q4(const uint4 &wv, float (&wf)[32]) {
  /* 0x4B000000 | c is the float 2^23 + c for c below 2^23, so a nibble left
     in place t (t below 4) gives 2^23 + 16^t c, and subtracting
     2^23 + 8 * 16^t leaves 16^t (c - 8), exactly: wf[8j + 4h + t] is the
     weight times 16^t, and fma16 takes the factor off the sums (the
     reference takes it off x, nn.vx:1659-1661). The upper four nibbles of a
     32-bit word are shifted down first. Places t and t + 1 go through the
     subtraction as a pair. */
  const uint32_t u[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t lo = u[j], hi = u[j] >> 16;
#pragma unroll
    for (int t = 0; t < 4; t += 2) {
      const uint32_t m0 = 15u << (4 * t), m1 = 15u << (4 * t + 4);
      const float2 off = make_float2(-(8388608.0f + 8.0f * (float)(1 << (4 * t))),
                                     -(8388608.0f + 8.0f * (float)(1 << (4 * t + 4))));
      const float2 a = add_pair(make_float2(__uint_as_float((lo & m0) | 0x4B000000u),
                                            __uint_as_float((lo & m1) | 0x4B000000u)),
                                off);
      const float2 b = add_pair(make_float2(__uint_as_float((hi & m0) | 0x4B000000u),
                                            __uint_as_float((hi & m1) | 0x4B000000u)),
                                off);
      wf[8 * j + t] = a.x;
      wf[8 * j + t + 1] = a.y;
      wf[8 * j + 4 + t] = b.x;
      wf[8 * j + 4 + t + 1] = b.y;
    }
  }
}

/* acc[b] += sum over the E weights of one 16-byte word of w * x[b]; for the
   scaled formats the word's sum is taken first and enters acc[b] times the
   word's scale. */
template <typename W, int B>
__device__ __forceinline__ void
fma16(const uint4 &wv, const float (&xv)[B][PerWord<W>::n], float (&acc)[B],
      float scale) {
  constexpr int E = PerWord<W>::n;
  float wf[E];
  if constexpr (E == 16) {
    unpack_fp8(wv, wf);
  } else if constexpr (E == 32) {
    unpack_q4(wv, wf);
  } else if constexpr (E == 8) {
    wf[0] = bf_lo(wv.x); wf[1] = bf_hi(wv.x);
    wf[2] = bf_lo(wv.y); wf[3] = bf_hi(wv.y);
    wf[E - 4] = bf_lo(wv.z); wf[E - 3] = bf_hi(wv.z);
    wf[E - 2] = bf_lo(wv.w); wf[E - 1] = bf_hi(wv.w);
  } else {
    wf[0] = __uint_as_float(wv.x); wf[1] = __uint_as_float(wv.y);
    wf[2] = __uint_as_float(wv.z); wf[3] = __uint_as_float(wv.w);
  }
  if constexpr (E == 32) {
#pragma unroll
    for (int b = 0; b < B; ++b) {
      float2 p01 = make_float2(0.0f, 0.0f), p23 = p01; /* by nibble place */
#pragma unroll
      for (int e = 0; e < E; e += 4) {
        fma_pair(p01, make_float2(wf[e], wf[e + 1]),
                 make_float2(xv[b][e], xv[b][e + 1]));
        fma_pair(p23, make_float2(wf[e + 2], wf[e + 3]),
                 make_float2(xv[b][e + 2], xv[b][e + 3]));
      }
      const float dot = fmaf(p23.y, 1.0f / 4096.0f,
                             fmaf(p23.x, 1.0f / 256.0f,
                                  fmaf(p01.y, 1.0f / 16.0f, p01.x)));
      acc[b] = fmaf(dot, scale, acc[b]);
    }
  } else if constexpr (Scaled<W>::yes) {
#pragma unroll
    for (int b = 0; b < B; ++b) {
      float2 d2 = make_float2(0.0f, 0.0f); /* even and odd weights apart */
#pragma unroll
      for (int e = 0; e < E; e += 2)
        fma_pair(d2, make_float2(wf[e], wf[e + 1]),
                 make_float2(xv[b][e], xv[b][e + 1]));
      const float dot = d2.x + d2.y;
      acc[b] = fmaf(dot, scale, acc[b]);
    }
  } else {
#pragma unroll
    for (int b = 0; b < B; ++b)
#pragma unroll
      for (int e = 0; e < E; ++e)
        acc[b] = fmaf(wf[e], xv[b][e], acc[b]);
  }
}

/* Weights reach the SM through a per-warp ring in shared memory that bulk
   copies (cp.async.bulk, completion counted on an mbarrier) fill: a warp keeps
   RING_STAGES chunks of both rows of its item in flight, across item
   boundaries, whatever its lanes are doing -- 128 KiB in flight per SM. */
constexpr int RING_STAGES = 4;
constexpr int CHUNK_BYTES = 1024; /* of one row */
/* Q4_0: the f16 scales of a chunk (one per 16 bytes of codes) travel with it,
   behind the two rows' codes in the same stage, when a row's scales are a
   multiple of 16 bytes: read from global memory at their first use they were
   a miss in L1 for every word, and the kernel waited for them. */
template <typename W> struct ChunkScales { static constexpr int bytes = 0; };
template <> struct ChunkScales<Q4W> { static constexpr int bytes = CHUNK_BYTES / 16 * 2; };
template <typename W> __host__ __device__ constexpr int stage_bytes() {
  return 2 * CHUNK_BYTES + 2 * ChunkScales<W>::bytes;
}
template <typename W> __host__ __device__ constexpr int ring_bytes() {
  return WARPS * RING_STAGES * stage_bytes<W>();
}
/* x (all sequences) staged per block: what the ring leaves of 227 KiB */
template <typename W> __host__ __device__ constexpr int max_smem_x() {
  return MAX_SMEM_X < 226 * 1024 - ring_bytes<W>() ? MAX_SMEM_X
                                                   : 226 * 1024 - ring_bytes<W>();
}

__device__ int g_rowdot_status; /* non-zero: a ring wait gave up */
__device__ int g_tp_status;     /* non-zero: a peer's flag never arrived */

/* 96 registers for one sequence: 512 threads then leave a quarter of the
   register file, so that the blocks of the attention kernel that follows
   q/k/v can start (and fetch their old cache rows) beside these. */
template <typename W, int B, int EPI, bool EARLY>
__global__ void __maxnreg__(B == 1 && !Scaled<W>::yes ? 96 : 128)
rowdot_kernel(const RowDotParams p) {
  extern __shared__ __align__(128) unsigned char smem_dyn[];
  unsigned char *ring = smem_dyn;                    /* [warp][stage][2][chunk] */
  float *xs = (float *)(smem_dyn + ring_bytes<W>()); /* [B][cols] when x_in_smem */
  constexpr int STAGE = stage_bytes<W>();
  constexpr int SC = ChunkScales<W>::bytes;
  const bool ring_scales = SC > 0 && p.scales_in_ring;
  __shared__ float ssq[B][WARPS]; /* per-warp sums of squares of x */
  __shared__ __align__(8) uint64_t bars[WARPS][RING_STAGES];
  constexpr int E = PerWord<W>::n;                   /* weights per 16 bytes */
  constexpr int CHUNK_COLS = CHUNK_BYTES / 16 * E;
  constexpr int GROUP = 32 * E; /* the weights of one word of each lane */
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cols = p.cols;
  /* x in shared memory: a lane needs the E consecutive values of its word as
     E / 4 float4s. Within each group of 32 E values they are stored quarter by
     quarter, 128 floats apart (value i of the group: which float4 of its lane,
     then the lane, then the place in the float4), so that the 32 lanes of a
     warp read consecutive float4s. */
  const int xs_stride = (cols + GROUP - 1) / GROUP * GROUP;
  auto xs_at = [](int i) {
    return E > 4 ? (i & ~(GROUP - 1)) | (((i % E) >> 2) << 7) |
                       (((i / E) & 31) << 2) | (i & 3)
                 : i;
  };

  /* ---- this warp's items, as a stream of (item, chunk) units ---- */
  const int64_t total_warps = (int64_t)gridDim.x * WARPS;
  const int64_t gw = (int64_t)blockIdx.x * WARPS + warp;
  const int first = (int)(gw * p.items / total_warps);
  const int last = (int)((gw + 1) * p.items / total_warps);
  const int row_bytes = cols / E * 16;
  const int nch = (row_bytes + CHUNK_BYTES - 1) / CHUNK_BYTES;
  const int units = (last - first) * nch;
  unsigned char *my_ring = ring + warp * (RING_STAGES * STAGE);

  if (lane == 0) {
    for (int s = 0; s < RING_STAGES; ++s)
      ptx::mbar_init(&bars[warp][s], 1);
    ptx::fence_proxy_async_smem();
    ptx::fence_barrier_init();
  }
  __syncwarp();
  /* The loading side walks the same units RING_STAGES ahead, with its own
     counters (no divisions on the way). Lane 0 issues the copies. */
  const int last_bytes = row_bytes - (nch - 1) * CHUNK_BYTES;
  /* An expert's matrix is named by the router's output, which the kernel before
     this one may have written: such a launch waits before it fetches weights. */
  int64_t w_off = 0, s_off = 0;
  bool expert_ok = true;
  if (p.expert_ids) {
    chain_release();
    chain_wait();
    const int id = p.expert_ids[p.expert_slot];
    expert_ok = id >= 0 && id < p.experts;
    w_off = expert_ok ? id * p.expert_bytes : 0;
    s_off = expert_ok ? id * p.scale_bytes : 0;
    if (!expert_ok && threadIdx.x == 0)
      atomicCAS(&g_rowdot_status, 0, 0x5E); /* not the number of an expert */
  }
  int ld_u = 0, ld_item = first, ld_ch = 0, ld_stage = 0;
  const char *ld_r0 = nullptr, *ld_r1 = nullptr, *ld_s0 = nullptr, *ld_s1 = nullptr;
  if (units > 0) {
    const ItemRows it = item_rows<W, EPI>(p, first, w_off, s_off);
    ld_r0 = it.r0;
    ld_r1 = it.r1 ? it.r1 : it.r0;
    ld_s0 = it.sc0;
    ld_s1 = it.r1 ? it.sc1 : it.sc0;
  }
  auto issue_next = [&]() {
    if (ld_u >= units)
      return;
    if (lane == 0) {
      const int bytes = ld_ch == nch - 1 ? last_bytes : CHUNK_BYTES;
      unsigned char *dst = my_ring + ld_stage * STAGE;
      uint64_t *bar = &bars[warp][ld_stage];
      const int sbytes = ring_scales ? bytes / 8 : 0;
      ptx::mbar_expect_tx(bar, 2 * bytes + 2 * sbytes);
      ptx::bulk_load(dst, ld_r0 + ld_ch * CHUNK_BYTES, bytes, bar);
      ptx::bulk_load(dst + CHUNK_BYTES, ld_r1 + ld_ch * CHUNK_BYTES, bytes, bar);
      if (ring_scales) {
        ptx::bulk_load(dst + 2 * CHUNK_BYTES, ld_s0 + ld_ch * SC, sbytes, bar);
        ptx::bulk_load(dst + 2 * CHUNK_BYTES + SC, ld_s1 + ld_ch * SC, sbytes, bar);
      }
    }
    ++ld_u;
    ld_stage = ld_stage + 1 == RING_STAGES ? 0 : ld_stage + 1;
    if (++ld_ch == nch) {
      ld_ch = 0;
      ++ld_item;
      if (ld_u < units) {
        const ItemRows it = item_rows<W, EPI>(p, ld_item, w_off, s_off);
        ld_r0 = it.r0;
        ld_r1 = it.r1 ? it.r1 : it.r0;
        ld_s0 = it.sc0;
        ld_s1 = it.r1 ? it.sc1 : it.sc0;
      }
    }
  };
  /* The weights do not depend on the kernel before this one: start them. */
  for (int u = 0; u < RING_STAGES; ++u)
    issue_next();
  chain_release();
  chain_wait(); /* from here on: x, y, positions of the kernels before */
  const int push_call = EPI == EPI_PUSH ? *p.tp.epoch + 1 : 0;
  const int64_t push_set = push_call & 1;

  /* ---- prologue: x (normalised if asked) into shared memory ---- */
  float inv[B];
#pragma unroll
  for (int b = 0; b < B; ++b)
    inv[b] = 1.0f;
  if (p.norm_w) {
    /* RMSNorm (nn_rms_norm, nn.vx:212-239; rmsnorm, llama2.vx:476-498) is
       y_i = x_i * inv * w_i with inv = 1/sqrt(mean(x^2) + eps). The factor inv
       is common to a whole row product, so the ring is fed x_i * w_i and inv
       multiplies the finished dot product: the weights start to be consumed
       after one pass over x and one barrier, while the sum of squares is only
       needed by the first epilogue. */
    for (int b = 0; b < B; ++b) {
      float ss = 0.0f;
      const float *px = p.x + b * p.x_stride;
      /* Several loads in flight per thread, four values per load: x was
         written by the kernel before and comes from L2, a microsecond away;
         one load at a time made this loop the longest part of a short
         projection. */
      const float4 *px4 = reinterpret_cast<const float4 *>(px);
      const int quads = cols / 4;
      for (int q0 = threadIdx.x; q0 < quads; q0 += 4 * blockDim.x) {
        float4 v[4], wn[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int q = q0 + k * blockDim.x;
          v[k] = wn[k] = make_float4(0, 0, 0, 0);
          if (q < quads) {
            v[k] = px4[q];
            if (p.norm_bf16) {
              const uint2 w = reinterpret_cast<const uint2 *>(p.norm_w)[q];
              wn[k] = make_float4(bf_lo(w.x), bf_hi(w.x), bf_lo(w.y), bf_hi(w.y));
            } else {
              wn[k] = reinterpret_cast<const float4 *>(p.norm_w)[q];
            }
          }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int q = q0 + k * blockDim.x;
          if (q < quads) {
            *reinterpret_cast<float4 *>(&xs[b * xs_stride + xs_at(4 * q)]) =
                make_float4(v[k].x * wn[k].x, v[k].y * wn[k].y, v[k].z * wn[k].z,
                            v[k].w * wn[k].w);
            ss = fmaf(v[k].x, v[k].x, ss);
            ss = fmaf(v[k].y, v[k].y, ss);
            ss = fmaf(v[k].z, v[k].z, ss);
            ss = fmaf(v[k].w, v[k].w, ss);
          }
        }
      }
      ss = warp_sum(ss);
      if (lane == 0)
        ssq[b][warp] = ss;
    }
    __syncthreads();
#pragma unroll
    for (int b = 0; b < B; ++b) {
      float ss = 0.0f;
      for (int w = 0; w < WARPS; ++w) /* fixed order */
        ss += ssq[b][w];
      inv[b] = 1.0f / sqrtf(ss / (float)cols + p.eps);
    }
  } else if (p.x_in_smem) {
    /* four values per load, eight loads in flight: the 11008 inputs of a down
       projection arrive in one trip to L2 instead of three (the permuted
       layout keeps four consecutive values together) */
    for (int b = 0; b < B; ++b) {
      const float4 *px = reinterpret_cast<const float4 *>(p.x + b * p.x_stride);
      const int quads = cols / 4;
      for (int q0 = threadIdx.x; q0 < quads; q0 += 8 * blockDim.x) {
        float4 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int q = q0 + k * blockDim.x;
          v[k] = q < quads ? px[q] : make_float4(0, 0, 0, 0);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int q = q0 + k * blockDim.x;
          if (q < quads)
            *reinterpret_cast<float4 *>(&xs[b * xs_stride + xs_at(4 * q)]) = v[k];
        }
      }
    }
    __syncthreads();
  }
  const float *xbase = p.x_in_smem ? xs : p.x;
  const int64_t xstr = p.x_in_smem ? xs_stride : p.x_stride;
  /* where a lane finds the x of its 16-byte word, and its further quarters */
  const bool x_perm = E > 4 && p.x_in_smem;
  const int lane_x = x_perm ? lane * 4 : lane * E;
  const int hi_off = x_perm ? 128 : 4;

  float s0[B], s1[B];
#pragma unroll
  for (int b = 0; b < B; ++b)
    s0[b] = s1[b] = 0.0f;

  /* One 16-byte word of both rows at byte `off` of the stage, times x. `col`:
     the column of the word's first weight; sc0, sc1: the rows' scales. */
  auto word = [&](const unsigned char *src, const float *xcol, int off, int col,
                  const char *sc0, const char *sc1) {
    const uint4 wa = *reinterpret_cast<const uint4 *>(src + off);
    const uint4 wb = *reinterpret_cast<const uint4 *>(src + CHUNK_BYTES + off);
    float scale_a = 1.0f, scale_b = 1.0f;
    if (E == 16) {
      scale_a = __ldg(reinterpret_cast<const float *>(sc0) + col / 128);
      scale_b = __ldg(reinterpret_cast<const float *>(sc1) + col / 128);
    } else if (E == 32) {
      if (ring_scales) {
        /* the stage's scales sit behind its codes: one per word of each row */
        const __half *sa = reinterpret_cast<const __half *>(
            src - lane * 16 + 2 * CHUNK_BYTES) + off / 16 + lane;
        scale_a = __half2float(sa[0]);
        scale_b = __half2float(sa[SC / 2]);
      } else {
        scale_a = __half2float(__ldg(reinterpret_cast<const __half *>(sc0) + col / 32));
        scale_b = __half2float(__ldg(reinterpret_cast<const __half *>(sc1) + col / 32));
      }
    }
    const float *xw = xcol + off / 16 * E;
    float xv[B][E];
#pragma unroll
    for (int b = 0; b < B; ++b) {
#pragma unroll
      for (int q = 0; q < (E + 3) / 4; ++q) {
        const float4 v =
            *reinterpret_cast<const float4 *>(xw + b * xstr + q * hi_off);
        xv[b][(4 * q) % E] = v.x; xv[b][(4 * q + 1) % E] = v.y;
        xv[b][(4 * q + 2) % E] = v.z; xv[b][(4 * q + 3) % E] = v.w;
      }
    }
    fma16<W, B>(wa, xv, s0, scale_a);
    fma16<W, B>(wb, xv, s1, scale_b);
  };

  /* One sequence and no more items than warps (a rank's slice of a sharded
     model: the launch is a matter of latency): what lane 0's epilogue reads
     from global memory -- the residual an item is added to, or the cosine and
     sine of its pair -- is asked for when the item begins, so that the trip
     to L2 runs under the item's weights instead of after them (27.4 -> 24.2
     us per layer on an eighth of the 7B shape). With several items per warp
     the same loads cost the stream 2 % (82.4 -> 83.9 us per layer on the whole
     shape), so there the epilogue fetches them itself. */
  constexpr bool early = EARLY; /* a kernel of its own: as a run-time choice
                                   it slowed the long launches by 3 % */
  float pre0 = 0.0f, pre1 = 0.0f;
  const int pos_first = (early && EPI == EPI_QKV) ? p.positions[0] : 0;
  int next_item = first, next_ch = 0, next_stage = 0;
  uint32_t next_phase = 0;
  for (int u = 0; u < units; ++u) {
    const int item = next_item, ch = next_ch, s = next_stage;
    const uint32_t phase = next_phase;
    if (early && ch == 0 && lane == 0) {
      if (EPI == EPI_ADD || EPI == EPI_PUSH) {
        pre0 = p.y[2 * item];
        pre1 = 2 * item + 1 < p.rows ? p.y[2 * item + 1] : 0.0f;
      } else if (EPI == EPI_QKV && p.rope_mode == 0) {
        const int half = p.head_dim / 2;
        const int h = item / half;
        if (h < p.q_heads + p.kv_heads) {
          pre0 = p.cos_t[(int64_t)pos_first * p.cs_cols + item - h * half];
          pre1 = p.sin_t[(int64_t)pos_first * p.cs_cols + item - h * half];
        }
      }
    }
    if (++next_ch == nch) {
      next_ch = 0;
      ++next_item;
    }
    if (++next_stage == RING_STAGES) {
      next_stage = 0;
      next_phase ^= 1;
    }
    if (!ptx::mbar_try_wait(&bars[warp][s], phase) &&
        !ptx::mbar_wait_alone(&bars[warp][s], phase)) {
      atomicCAS(&g_rowdot_status, 0, 1);
      break;
    }
    const unsigned char *src = my_ring + s * STAGE + lane * 16;
    const float *xcol = xbase + ch * CHUNK_COLS + lane_x;
    const char *sc0 = nullptr, *sc1 = nullptr;
    if (Scaled<W>::yes) {
      const ItemRows here = item_rows<W, EPI>(p, item, w_off, s_off);
      sc0 = here.sc0;
      sc1 = here.r1 ? here.sc1 : here.sc0;
    }
    const int col0 = ch * CHUNK_COLS + lane * E;
    if (ch != nch - 1 || last_bytes == CHUNK_BYTES) {
#pragma unroll
      for (int i = 0; i < CHUNK_BYTES / 512; ++i)
        word(src, xcol, i * 512, col0 + i * GROUP, sc0, sc1);
    } else {
      for (int off = 0; off + lane * 16 < last_bytes; off += 512)
        word(src, xcol, off, col0 + off / 512 * GROUP, sc0, sc1);
    }
    /* Every lane has read the stage: it may be filled again. */
    __syncwarp();
    issue_next();
    if (ch != nch - 1)
      continue;

    /* ---- the item is complete: reduce, then the epilogue on lane 0 ---- */
    const ItemRows it = item_rows<W, EPI>(p, item, w_off, s_off);
    const char *r1 = it.r1;
    const int head = it.head, idx = it.idx, kind = it.kind;
    float t0[B], t1[B];
#pragma unroll
    for (int b = 0; b < B; ++b) {
      t0[b] = warp_sum(s0[b]) * inv[b];
      t1[b] = warp_sum(s1[b]) * inv[b];
      s0[b] = s1[b] = 0.0f;
    }
    if (EPI == EPI_PUSH) {
      /* This rank's partial of a row-split product. Lane r sends both values
         of the item to rank r (slot `rank` of r's receive buffer, peer memory
         over NVLink, one 16-byte store), then waits for rank r's partial of
         the same two rows in this rank's own buffer (a bounded wait on
         exactly that pair of pairs: every rank runs the same rows at about
         the same time). The partials are added to the residual in rank
         order, the same order on every rank, so y stays identical on all of
         them. The exchange has no kernel of its own, no fence, no counter. */
      const int ra = 2 * item;
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const int64_t in_set = b * p.y_stride + ra;
        float v0 = t0[b], v1 = t1[b]; /* every lane holds the warp's sums */
        if (lane < p.tp.ranks && lane != p.tp.rank) {
          TpPair *to = p.tp.slots[lane] +
                       (push_set * p.tp.ranks + p.tp.rank) * p.tp.count + in_set;
          if (r1)
            pair2_store(to, v0, v1, push_call);
          else
            pair_store(to, v0, push_call);
          const TpPair *from = p.tp.slots[p.tp.rank] +
                               (push_set * p.tp.ranks + lane) * p.tp.count + in_set;
          const long long began = clock64();
          for (int polls = 1;; ++polls) {
            const bool here = r1 ? pair2_load(from, push_call, v0, v1)
                                 : pair_load(from, push_call, v0);
            if (here)
              break;
            /* a wait that ran out anywhere ends every later wait at once; the
               status word is a trip to L2 of its own, so it is looked at on
               every eighth poll only */
            if ((polls & 7) == 0 && (*(volatile int *)&g_tp_status != 0 ||
                                     clock64() - began > ptx::kWaitCycles)) {
              atomicCAS(&g_tp_status, 0, 0x53);
              break;
            }
          }
        }
        float *y = p.y + b * p.y_stride;
        float s0v = lane == 0 ? (early ? pre0 : y[ra]) : 0.0f;
        float s1v = (lane == 0 && r1) ? (early ? pre1 : y[ra + 1]) : 0.0f;
        for (int r = 0; r < p.tp.ranks; ++r) {
          s0v += __shfl_sync(0xffffffffu, v0, r);
          s1v += __shfl_sync(0xffffffffu, v1, r);
        }
        if (lane == 0) {
          y[ra] = s0v;
          if (r1)
            y[ra + 1] = s1v;
        }
      }
      continue;
    }
    if (lane != 0)
      continue;

    /* ---- epilogue, lane 0 ---- */
#pragma unroll
    for (int b = 0; b < B; ++b) {
      if (EPI == EPI_STORE || EPI == EPI_ADD || EPI == EPI_BIAS) {
        float *y = p.y + b * p.y_stride;
        const int ra = 2 * item, rb = 2 * item + 1;
        float v0 = t0[b], v1 = t1[b];
        if (EPI == EPI_ADD) {
          const float scale = p.add_scale ? (expert_ok ? p.add_scale[0] : 0.0f) : 1.0f;
          const float ya = early ? pre0 : y[ra];
          v0 = p.add_scale ? fmaf(scale, v0, ya) : ya + v0;
          if (r1) {
            const float yb = early ? pre1 : y[rb];
            v1 = p.add_scale ? fmaf(scale, v1, yb) : yb + v1;
          }
        } else if (EPI == EPI_BIAS) {
          v0 += bf16_at(p.bias, ra);
          if (r1)
            v1 += bf16_at(p.bias, rb);
        }
        y[ra] = v0;
        if (r1)
          y[rb] = v1;
      } else if (EPI == EPI_SWIGLU) {
        /* nn_swiglu (nn.vx:169-209): g / (1 + e^-g) * u. */
        const float g = t0[b], u = t1[b];
        p.y[b * p.y_stride + item] = g / (1.0f + expf(0.0f - g)) * u;
      } else { /* EPI_QKV */
        const int hd = p.head_dim, half = hd / 2;
        const int ia = p.rope_mode == 0 ? idx : 2 * idx;
        const int ib = p.rope_mode == 0 ? idx + half : 2 * idx + 1;
        float va = t0[b], vb = t1[b];
        if (p.bias) {
          va += bf16_at(p.bias, (int64_t)head * hd + ia);
          vb += bf16_at(p.bias, (int64_t)head * hd + ib);
        }
        const int pos = p.positions[b];
        const int local = kind == 0 ? head
                          : kind == 1 ? head - p.q_heads
                                      : head - p.q_heads - p.kv_heads;
        if (kind == 2) {
          float *vrow = p.v_cache + b * p.cache_batch_stride +
                        ((int64_t)pos * p.kv_heads + local) * hd;
          vrow[ia] = va;
          vrow[ib] = vb;
          continue;
        }
        float c, s;
        if (p.rope_mode == 0) {
          /* nn_rope_and_store (nn.vx:245-280) */
          c = early ? pre0 : p.cos_t[(int64_t)pos * p.cs_cols + idx];
          s = early ? pre1 : p.sin_t[(int64_t)pos * p.cs_cols + idx];
        } else {
          /* llama2.vx:264-293 with rope_freq (llama_rt.vx:82-85): the CPU
             functions are correctly rounded, so go through double. */
          const float e = -((float)(2 * idx)) / (float)hd;
          const float f = (float)pow(10000.0, (double)e);
          const float angle = __fmul_rn((float)pos, f);
          c = (float)cos((double)angle);
          s = (float)sin((double)angle);
        }
        const float oa = __fsub_rn(__fmul_rn(va, c), __fmul_rn(vb, s));
        const float ob = p.rope_mode == 0
                             ? __fadd_rn(__fmul_rn(vb, c), __fmul_rn(va, s))
                             : __fadd_rn(__fmul_rn(va, s), __fmul_rn(vb, c));
        float *dst = kind == 0
                         ? p.y + b * p.y_stride + (int64_t)local * hd
                         : p.k_cache + b * p.cache_batch_stride +
                               ((int64_t)pos * p.kv_heads + local) * hd;
        dst[ia] = oa;
        dst[ib] = ob;
      }
    }
  }

  if (EPI == EPI_PUSH) {
    /* The block that finishes last advances the call count: every block read
       it when it began. */
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(p.tp.done, 1) == (int)gridDim.x - 1) {
        *p.tp.done = 0;
        *p.tp.epoch = push_call;
      }
    }
  }
}

int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

const char *check_launch(const char *what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess)
    return nullptr;
  static thread_local char msg[256];
  snprintf(msg, sizeof msg, "%s: %s", what, cudaGetErrorString(e));
  return msg;
}

template <typename W, int B, int EPI>
const char *launch_rowdot_b(RowDotParams &p, cudaStream_t stream) {
  constexpr int GROUP = 32 * PerWord<W>::n;
  const size_t xbytes =
      (size_t)B * ((p.cols + GROUP - 1) / GROUP * GROUP) * sizeof(float);
  p.x_in_smem = xbytes <= (size_t)max_smem_x<W>();
  if (p.norm_w && !p.x_in_smem)
    return "a fused RMSNorm needs the activations of all sequences to fit in "
           "shared memory beside the ring (96 KiB; 80 KiB with Q4_0 weights)";
  /* Q4_0 scales ride the ring when every row's scales start and end on a
     16-byte boundary */
  p.scales_in_ring = ChunkScales<W>::bytes > 0 && p.cols % 256 == 0 &&
                     !(((uintptr_t)p.s0 | (uintptr_t)p.s1 | (uintptr_t)p.s2) & 15);
  const size_t smem = ring_bytes<W>() + (p.x_in_smem ? xbytes : 0);
  if (allow_dynamic_smem((const void *)rowdot_kernel<W, B, EPI, false>,
                         ring_bytes<W>() + max_smem_x<W>()) != cudaSuccess)
    return "a projection could not get its shared memory on this GPU";
  /* One block of 16 warps per SM with a 128 KiB ring (measured faster than
     two blocks of 8 warps with 64 KiB each: 31.7 vs 34.3 us on the 7B gate/up
     projection). With fewer items than warps (a rank's slice of a
     tensor-parallel model) the items are spread over all SMs, some warps of
     each block idle, rather than packed sixteen to a block on a few SMs: a
     short projection is a matter of latency, and every SM's path to memory
     helps. VXB_ROWDOT_PACK=1 packs (for measurements). */
  static const bool pack = [] {
    const char *e = getenv("VXB_ROWDOT_PACK");
    return e && e[0] == '1';
  }();
  int blocks = sm_count();
  const int wanted = pack ? (p.items + WARPS - 1) / WARPS : p.items;
  if (blocks > wanted)
    blocks = wanted < 1 ? 1 : wanted;
  if (B == 1 && (int64_t)p.items <= (int64_t)blocks * WARPS) {
    if (allow_dynamic_smem((const void *)rowdot_kernel<W, B, EPI, B == 1>,
                           ring_bytes<W>() + max_smem_x<W>()) != cudaSuccess)
      return "a projection could not get its shared memory on this GPU";
    launch_chained(rowdot_kernel<W, B, EPI, B == 1>, dim3(blocks), dim3(WARPS * 32),
                   smem, stream, p);
  } else {
    launch_chained(rowdot_kernel<W, B, EPI, false>, dim3(blocks), dim3(WARPS * 32),
                   smem, stream, p);
  }
  return check_launch("a projection launch");
}

template <typename W, int EPI>
const char *launch_rowdot_w(RowDotParams &p, cudaStream_t stream) {
  switch (p.batch) {
  case 1: return launch_rowdot_b<W, 1, EPI>(p, stream);
  case 2: return launch_rowdot_b<W, 2, EPI>(p, stream);
  case 4: return launch_rowdot_b<W, 4, EPI>(p, stream);
  case 8: return launch_rowdot_b<W, 8, EPI>(p, stream);
  case 16: return launch_rowdot_b<W, 16, EPI>(p, stream);
  default: return "the batch must be 1, 2, 4, 8 or 16";
  }
}

#include "rowdot_quant_mma.cuh"

/* fmt: a kFmt* code of kernels.h. */
template <int EPI>
const char *launch_rowdot(RowDotParams &p, int fmt, cudaStream_t stream) {
  const int per_word = fmt == kFmtF32 ? 4 : fmt == kFmtBf16 ? 8 : fmt == kFmtFp8 ? 16 : 32;
  if (p.cols % 8 != 0 || p.cols % per_word != 0)
    return "the number of columns must be a multiple of 8 (f32, bf16), of 128 "
           "(fp8) or of 32 (Q4_0)";
  if (((uintptr_t)p.w0 | (uintptr_t)p.w1 | (uintptr_t)p.w2 | (uintptr_t)p.x) & 15)
    return "weights and activations must be 16-byte aligned";
  if (p.x_stride % 4 != 0 && p.batch > 1)
    return "the stride between sequences must be a multiple of 4 values";
  if (fmt == kFmtFp8 || fmt == kFmtQ4) {
    if (fmt == kFmtFp8 && p.cols % 128 != 0)
      return "an fp8 matrix has a multiple of 128 columns";
    if (!p.s0 || (p.w1 && !p.s1) || (p.w2 && !p.s2))
      return "a quantised matrix needs its scales";
    if (p.batch != 1)
      return "the quantised projections take one sequence";
    if (EPI == EPI_PUSH)
      return "the quantised projections are not sharded";
    /* the switch is on a constant: only the instantiations below exist */
    if (EPI != EPI_PUSH) {
      constexpr int E = EPI == EPI_PUSH ? EPI_STORE : EPI;
      /* on the tensor cores where the shape allows, else on the FMA pipe */
      const char *r = fmt == kFmtFp8 ? launch_quant_mma<Fp8W, E>(p, stream)
                                     : launch_quant_mma<Q4W, E>(p, stream);
      if (!r || r[0])
        return r;
      return fmt == kFmtFp8 ? launch_rowdot_b<Fp8W, 1, E>(p, stream)
                            : launch_rowdot_b<Q4W, 1, E>(p, stream);
    }
  }
  return fmt == kFmtBf16 ? launch_rowdot_w<__nv_bfloat16, EPI>(p, stream)
                         : launch_rowdot_w<float, EPI>(p, stream);
}

/* ------------------------------------------------------------- rms_norm
 * nn_rms_norm (nn.vx:212-239); one block per sequence. */
__global__ void __launch_bounds__(1024)
rms_norm_kernel(float *y, const float *x, const void *w, int wbf16, int n,
                float eps, int64_t stride) {
  __shared__ float red[32];
  chain_release();
  chain_wait();

  const float *xr = x + blockIdx.x * stride;
  float *yr = y + blockIdx.x * stride;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    ss = fmaf(xr[i], xr[i], ss);
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float wn = wbf16 ? bf16_at(w, i) : ((const float *)w)[i];
    yr[i] = xr[i] * inv * wn;
  }
}

/* ------------------------------------------------------- rope_and_store
 * nn_rope_and_store (nn.vx:245-280), unfused. */
__global__ void rope_store_kernel(float *q_out, float *k_cache, float *v_cache,
                                  const float *q, const float *k,
                                  const float *v, const float *cos_t,
                                  const float *sin_t, int cs_cols, int pos,
                                  int q_heads, int kv_heads, int hd) {
  chain_release();
  chain_wait();
  const int h = blockIdx.x, i = threadIdx.x;
  if (i >= hd)
    return;
  const int half = hd / 2;
  const int j = i < half ? i : i - half;
  const int partner = i < half ? i + half : i - half;
  const float sign = i < half ? -1.0f : 1.0f;
  const float c = cos_t[(int64_t)pos * cs_cols + j];
  const float s = sin_t[(int64_t)pos * cs_cols + j];
  if (h < q_heads) {
    const float *qh = q + h * hd;
    q_out[h * hd + i] =
        __fadd_rn(__fmul_rn(qh[i], c), __fmul_rn(__fmul_rn(sign, qh[partner]), s));
  } else {
    const int g = h - q_heads;
    const float *kh = k + g * hd;
    const int64_t at = ((int64_t)pos * kv_heads + g) * hd + i;
    k_cache[at] =
        __fadd_rn(__fmul_rn(kh[i], c), __fmul_rn(__fmul_rn(sign, kh[partner]), s));
    v_cache[at] = v[g * hd + i];
  }
}

/* The same arithmetic with the parts of a head merged inside a cluster of
   ATT_CLUSTER blocks (distributed shared memory) instead of through global
   memory, a fence, an atomic and a last block: three round trips shorter.
   This is what kAttnAuto runs unless the process chose otherwise. */
constexpr int ATT_CLUSTER = 8;
template <int GH, int ATT_WARPS>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_cluster_kernel(const AttnArgs a) {
  __shared__ AttnShared<GH, ATT_WARPS> sh;
  chain_release();
  attention_unit<GH, true, ATT_CLUSTER, ATT_WARPS>(
      a, blockIdx.x, blockIdx.y, blockIdx.z, threadIdx.x >> 5, threadIdx.x & 31,
      sh, 0);
}

template <int GH>
__global__ void __launch_bounds__(4 * 32)
attention_decode_kernel(const AttnArgs a) {
  __shared__ AttnShared<GH, 4> sh;
  chain_release();
  attention_unit<GH, true, 0, 4>(a, blockIdx.x, blockIdx.y, blockIdx.z,
                                 threadIdx.x >> 5, threadIdx.x & 31, sh, 0);
}

/* ----------------------------------------------------------------- top_k
 * nn_top_k (nn.vx:904-938): the router of a mixture-of-experts layer. The
 * reference sorts 64-bit keys -- the value's bits in an order that keeps the
 * order of the values, then 255 - index, so that of equal values the lower
 * index comes first -- and takes the first k; here each of the n <= 256
 * values counts the keys above its own, which is its place. Then the softmax
 * over the k values, summed in the order of their places. One block. */
__global__ void __launch_bounds__(256)
top_k_kernel(int32_t *ids, float *weights, const float *logits, int n, int k,
             int64_t ids_pitch, int64_t weights_pitch, int64_t logits_pitch) {
  __shared__ long long keys[256];
  __shared__ int order[256];
  chain_release();
  chain_wait();
  /* nn_top_k_rows (nn.vx:2897-2929): a block per position, the same arithmetic */
  ids += blockIdx.x * ids_pitch;
  weights += blockIdx.x * weights_pitch;
  logits += blockIdx.x * logits_pitch;
  const int i = threadIdx.x;
  if (i < n) {
    const int bits = __float_as_int(logits[i]);
    const int ordered = bits < 0 ? bits ^ 0x7fffffff : bits;
    keys[i] = (long long)ordered * 4294967296ll + (255 - i);
  }
  __syncthreads();
  if (i < n) {
    const long long mine = keys[i];
    int place = 0;
    for (int j = 0; j < n; ++j)
      place += keys[j] > mine;
    order[place] = i; /* keys are distinct: every place is taken once */
  }
  __syncthreads();
  if (i < k) {
    const float top = logits[order[0]];
    float total = 0.0f;
    for (int t = 0; t < k; ++t)
      total = total + expf(logits[order[t]] - top);
    const int id = order[i];
    ids[i] = id;
    weights[i] = expf(logits[id] - top) / total;
  }
}

/* ---------------------------------------------------------------- argmax
 * nn_argmax (nn.vx:870-897) and sample_argmax (llama2.vx:460-474): the lowest
 * index of the largest value. One block per sequence. */
__global__ void __launch_bounds__(1024)
argmax_kernel(int32_t *out, const float *logits, int n, int64_t stride) {
  chain_release();
  chain_wait();
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  const float *row = logits + blockIdx.x * stride;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = row[i];
    if (v > bv || (v == bv && i < bi) || bi == 0x7fffffff) {
      bv = v;
      bi = i;
    }
  }
  auto better = [](float v, int i, float ov, int oi) {
    return oi != 0x7fffffff && (i == 0x7fffffff || ov > v || (ov == v && oi < i));
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(bv, bi, ov, oi)) {
      bv = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    best_v[warp] = bv;
    best_i[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    bv = lane < nw ? best_v[lane] : -INFINITY;
    bi = lane < nw ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(bv, bi, ov, oi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0)
      out[blockIdx.x] = bi;
  }
}

/* ----------------------------------------------------------------- embed
 * nn_embed (nn.vx:942-958); a token outside the table gives a row of NaN
 * instead of a read outside it. */
__global__ void embed_kernel(float *x, const void *table, int tbf16,
                             const int32_t *token, int dim, int rows,
                             int64_t x_stride) {
  chain_release();
  chain_wait();
  const int b = blockIdx.y;
  const int t = token[b];
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < dim;
       i += gridDim.x * blockDim.x) {
    float v = __int_as_float(0x7fc00000);
    if (t >= 0 && t < rows)
      v = tbf16 ? bf16_at(table, (int64_t)t * dim + i)
                : ((const float *)table)[(int64_t)t * dim + i];
    x[b * x_stride + i] = v;
  }
}

} // namespace


const char *matvec(const MatvecArgs &a, cudaStream_t stream) {
  if (a.rows <= 0 || a.batch <= 0)
    return nullptr;
  RowDotParams p{};
  p.w0 = a.w;
  p.rows = a.rows;
  p.cols = a.cols;
  p.items = (a.rows + 1) / 2;
  p.x = a.x;
  p.x_stride = a.x_stride;
  p.batch = a.batch;
  p.norm_w = a.norm_w;
  p.norm_bf16 = a.norm_bf16;
  p.eps = a.eps;
  p.y = a.y;
  p.y_stride = a.y_stride;
  p.bias = a.bias;
  p.s0 = a.scales;
  p.row_base = a.row_base;
  const int fmt = a.wfmt ? a.wfmt : (a.wbf16 ? kFmtBf16 : kFmtF32);
  const int per_word = fmt == kFmtF32 ? 4 : fmt == kFmtBf16 ? 8 : fmt == kFmtFp8 ? 16 : 32;
  if (a.expert_ids) {
    if (fmt == kFmtFp8)
      return "the expert projections take bf16 or Q4_0 weights";
    p.expert_ids = a.expert_ids;
    p.expert_slot = a.expert_slot;
    p.experts = a.experts;
    p.expert_bytes = (int64_t)a.rows * (a.cols / per_word * 16);
    p.scale_bytes = fmt == kFmtQ4 ? (int64_t)a.rows * (a.cols / 32) * 2 : 0;
  }
  p.add_scale = a.add_scale;
  switch (a.mode) {
  case 0: return launch_rowdot<EPI_STORE>(p, fmt, stream);
  case 1: return launch_rowdot<EPI_ADD>(p, fmt, stream);
  case 2: return launch_rowdot<EPI_BIAS>(p, fmt, stream);
  case 3:
    if (!a.push || a.push->ranks < 1 || a.push->ranks > kMaxTpRanks)
      return "a pushed projection needs the receive buffers of 1 to 8 ranks";
    if (a.push->count % 2 != 0 || a.y_stride % 2 != 0)
      return "a pushed projection needs an even number of rows";
    p.tp = *a.push;
    return launch_rowdot<EPI_PUSH>(p, fmt, stream);
  default: return "unknown matvec mode";
  }
}

const char *matvec_f32(float *y, const float *x, const float *w, int n, int d,
                       cudaStream_t stream) {
  if (n % 8 != 0 || (((uintptr_t)w | (uintptr_t)x) & 15)) {
    /* Any n: the f32 GEMM with a one-column B. */
    return gemm_f32(w, n, x, 1, y, 1, d, 1, n, stream);
  }
  MatvecArgs a{};
  a.w = w;
  a.wbf16 = false;
  a.rows = d;
  a.cols = n;
  a.x = x;
  a.x_stride = n;
  a.y = y;
  a.y_stride = d;
  a.batch = 1;
  return matvec(a, stream);
}

const char *swiglu(const SwigluArgs &a, cudaStream_t stream) {
  if (a.rows <= 0 || a.batch <= 0)
    return nullptr;
  RowDotParams p{};
  p.w0 = a.w;
  p.w1 = a.w_up;
  p.rows = a.rows;
  p.cols = a.cols;
  p.items = a.rows;
  p.x = a.x;
  p.x_stride = a.x_stride;
  p.batch = a.batch;
  p.norm_w = a.norm_w;
  p.norm_bf16 = a.norm_bf16;
  p.eps = a.eps;
  p.y = a.out;
  p.y_stride = a.out_stride;
  p.s0 = a.scales;
  p.s1 = a.scales_up;
  p.row_base = a.row_base;
  if (a.expert_ids) {
    const int fmt = a.wfmt ? a.wfmt : (a.wbf16 ? kFmtBf16 : kFmtF32);
    const int per_word = fmt == kFmtF32 ? 4 : fmt == kFmtBf16 ? 8 : fmt == kFmtFp8 ? 16 : 32;
    if (fmt == kFmtFp8 || a.w_up)
      return "the expert projections take bf16 or Q4_0 weights, gate and up rows "
             "in one matrix";
    p.expert_ids = a.expert_ids;
    p.expert_slot = a.expert_slot;
    p.experts = a.experts;
    p.expert_bytes = (int64_t)2 * a.rows * (a.cols / per_word * 16);
    p.scale_bytes = fmt == kFmtQ4 ? (int64_t)2 * a.rows * (a.cols / 32) * 2 : 0;
  }
  return launch_rowdot<EPI_SWIGLU>(p, a.wfmt ? a.wfmt : (a.wbf16 ? kFmtBf16 : kFmtF32),
                                   stream);
}

const char *qkv_rope_store(const QkvArgs &a, cudaStream_t stream) {
  if (a.head_dim % 2 != 0)
    return "head_dim must be even";
  RowDotParams p{};
  p.w0 = a.wq;
  p.w1 = a.wk;
  p.w2 = a.wv;
  p.rows = (a.q_heads + 2 * a.kv_heads) * a.head_dim;
  p.cols = a.cols;
  p.items = p.rows / 2;
  p.x = a.x;
  p.x_stride = a.x_stride;
  p.batch = a.batch;
  p.norm_w = a.norm_w;
  p.norm_bf16 = a.norm_bf16;
  p.eps = a.eps;
  p.y = a.q_out;
  p.y_stride = (int64_t)a.q_heads * a.head_dim;
  p.bias = a.bias;
  p.q_heads = a.q_heads;
  p.kv_heads = a.kv_heads;
  p.head_dim = a.head_dim;
  p.rope_mode = a.rope_mode;
  p.cos_t = a.cos_t;
  p.sin_t = a.sin_t;
  p.cs_cols = a.cs_cols;
  p.theta = a.theta;
  p.positions = a.positions;
  p.k_cache = a.k_cache;
  p.v_cache = a.v_cache;
  p.cache_batch_stride = a.cache_batch_stride;
  p.max_seq = a.max_seq;
  p.s0 = a.sq;
  p.s1 = a.sk;
  p.s2 = a.sv;
  return launch_rowdot<EPI_QKV>(p, a.wfmt ? a.wfmt : (a.wbf16 ? kFmtBf16 : kFmtF32),
                                stream);
}

int tp_status(cudaStream_t stream) {
  int v = 0, zero = 0;
  if (cudaStreamSynchronize(stream) != cudaSuccess)
    return -1;
  if (cudaMemcpyFromSymbol(&v, g_tp_status, sizeof v) != cudaSuccess)
    return -1;
  if (v)
    cudaMemcpyToSymbol(g_tp_status, &zero, sizeof zero);
  int r = 0;
  if (cudaMemcpyFromSymbol(&r, g_rowdot_status, sizeof r) == cudaSuccess && r) {
    cudaMemcpyToSymbol(g_rowdot_status, &zero, sizeof zero);
    if (!v)
      v = 0x52;
  }
  return v;
}

const char *rms_norm(float *y, const float *x, const void *w, bool wbf16, int n,
                     float eps, int batch, int64_t stride, cudaStream_t stream) {
  if (n <= 0 || batch <= 0)
    return nullptr;
  launch_chained(rms_norm_kernel, dim3(batch), dim3(1024), 0, stream, y, x, w,
                 (int)wbf16, n, eps, stride);
  return check_launch("the RMSNorm launch");
}

const char *rope_and_store(float *q_out, float *k_cache, float *v_cache,
                           const float *q, const float *k, const float *v,
                           const float *cos_t, const float *sin_t, int cs_cols,
                           int pos, int q_heads, int kv_heads, int head_dim,
                           cudaStream_t stream) {
  if (head_dim > 1024)
    return "head_dim is larger than a block";
  launch_chained(rope_store_kernel, dim3(q_heads + kv_heads),
                 dim3(((head_dim + 31) / 32) * 32), 0, stream, q_out, k_cache,
                 v_cache, q, k, v, cos_t, sin_t, cs_cols, pos, q_heads,
                 kv_heads, head_dim);
  return check_launch("the RoPE launch");
}

size_t attn_scratch_floats(int batch, int q_heads, int head_dim, int max_seq,
                           int split) {
  return (size_t)batch * q_heads * ((size_t)max_seq / split + 1) *
         (head_dim + 2);
}

const char *attention_decode(const AttnArgs &a, cudaStream_t stream) {
  if (a.head_dim % 4 != 0 || a.head_dim > 128)
    return "head_dim must be a multiple of 4, and at most 128";
  if (a.q_heads % a.kv_heads != 0)
    return "q_heads must be a multiple of kv_heads";
  if (a.split < 1)
    return "the split must be at least one position";
  if (((uintptr_t)a.scratch & 7) || ((uintptr_t)a.q & 15) ||
      ((uintptr_t)a.k_cache & 15) || ((uintptr_t)a.v_cache & 15) ||
      ((uintptr_t)a.out & 15))
    return "q, the caches and out must be 16-byte aligned, the scratch 8-byte";
  const int group = a.q_heads / a.kv_heads;
  const int gh = group >= 4 ? 4 : (group >= 2 ? 2 : 1);
  const int tiles = (group + gh - 1) / gh;
  int which = a.kernel == kAttnAuto ? attention_kernel_choice(-1) : a.kernel;
  if (which == kAttnAuto)
    which = kAttnCluster;
  if (which == kAttnSplit && (!a.scratch || !a.counters))
    return "the split attention kernel needs scratch memory and counters";
  if (which != kAttnCluster && which != kAttnSplit)
    return "unknown attention kernel";
  if (which == kAttnCluster) {
    const dim3 cgrid(ATT_CLUSTER, a.kv_heads * tiles, a.batch);
    /* Warps per block by how many blocks there are: with few heads (a rank of
       a tensor-parallel job holds 4 or 8 of 32) sixteen warps per block put
       the positions of a head on 128 warps, one round trip to memory each;
       with every SM already holding several blocks, four. Measured at
       position 520 on one rank's share of the 7B shape, microseconds per
       layer for 4 / 8 / 16 warps: 1/2 of the heads 53.4 / 51.8 / 54.3, 1/4
       37.7 / 37.3 / 36.0, 1/8 28.6 / 27.3 / 26.5; all heads 387 / 389 / 361
       tokens/s. */
    const int64_t blocks = (int64_t)cgrid.x * cgrid.y * cgrid.z;
    int warps = 2 * blocks <= sm_count() ? 16 : (blocks <= 2 * sm_count() ? 8 : 4);
    /* VXB_ATTN_WARPS=4, 8 or 16 pins it (for measurements) */
    if (const char *pin = getenv("VXB_ATTN_WARPS")) {
      const int v = atoi(pin);
      if (v == 4 || v == 8 || v == 16)
        warps = v;
    }
    auto go = [&](auto kernel) {
      launch_chained_cluster(kernel, cgrid, dim3(warps * 32), ATT_CLUSTER, stream, a);
    };
    if (gh == 4) {
      if (warps == 16) go(attention_cluster_kernel<4, 16>);
      else if (warps == 8) go(attention_cluster_kernel<4, 8>);
      else go(attention_cluster_kernel<4, 4>);
    } else if (gh == 2) {
      if (warps == 16) go(attention_cluster_kernel<2, 16>);
      else if (warps == 8) go(attention_cluster_kernel<2, 8>);
      else go(attention_cluster_kernel<2, 4>);
    } else {
      if (warps == 16) go(attention_cluster_kernel<1, 16>);
      else if (warps == 8) go(attention_cluster_kernel<1, 8>);
      else go(attention_cluster_kernel<1, 4>);
    }
    return check_launch("the attention launch");
  }
  const dim3 grid(a.max_pos / a.split + 1, a.kv_heads * tiles, a.batch);
  if (gh == 4)
    launch_chained(attention_decode_kernel<4>, grid, dim3(4 * 32), 0, stream, a);
  else if (gh == 2)
    launch_chained(attention_decode_kernel<2>, grid, dim3(4 * 32), 0, stream, a);
  else
    launch_chained(attention_decode_kernel<1>, grid, dim3(4 * 32), 0, stream, a);
  return check_launch("the attention launch");
}

int attention_kernel_choice(int which) {
  static std::mutex mu;
  static int choice = kAttnAuto;
  std::lock_guard<std::mutex> lock(mu);
  const int before = choice;
  if (which == kAttnAuto || which == kAttnCluster || which == kAttnSplit)
    choice = which;
  return before;
}

const char *attention_decode_clustered(const AttnArgs &a, cudaStream_t stream) {
  AttnArgs b = a;
  b.scratch = nullptr;
  b.counters = nullptr;
  b.kernel = kAttnCluster;
  return attention_decode(b, stream);
}

const char *top_k(int32_t *ids, float *weights, const float *logits, int n, int k,
                  cudaStream_t stream) {
  return top_k_rows(ids, weights, logits, 1, n, k, 0, 0, 0, stream);
}

const char *top_k_rows(int32_t *ids, float *weights, const float *logits,
                       int positions, int n, int k, int64_t ids_pitch,
                       int64_t weights_pitch, int64_t logits_pitch,
                       cudaStream_t stream) {
  if (n < 1 || n > 256 || k < 1 || k > n)
    return "n must be 1 to 256, and k must be 1 to n";
  if (positions < 1)
    return nullptr;
  launch_chained(top_k_kernel, dim3(positions), dim3(256), 0, stream, ids, weights,
                 logits, n, k, ids_pitch, weights_pitch, logits_pitch);
  return check_launch("the router launch");
}

const char *argmax(int32_t *out, const float *logits, int n, int batch,
                   int64_t stride, cudaStream_t stream) {
  if (n <= 0 || batch <= 0)
    return nullptr;
  launch_chained(argmax_kernel, dim3(batch), dim3(1024), 0, stream, out, logits,
                 n, stride);
  return check_launch("the argmax launch");
}

const char *embed(float *x, const void *table, bool tbf16, const int32_t *token,
                  int dim, int rows, int batch, int64_t x_stride,
                  cudaStream_t stream) {
  const dim3 grid((dim + 255) / 256, batch);
  launch_chained(embed_kernel, grid, dim3(256), 0, stream, x, table, (int)tbf16,
                 token, dim, rows, x_stride);
  return check_launch("the embed launch");
}

} // namespace vxb
