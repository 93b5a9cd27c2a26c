/* nn_device.cuh -- device functions that more than one file of the decode
 * path uses: bf16 unpacking, warp reductions, the (value, call) pairs of the
 * tensor-parallel exchange, and one unit of decode attention.
 */
#ifndef VXB_NN_DEVICE_CUH
#define VXB_NN_DEVICE_CUH

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

#include <cooperative_groups.h>

#include <cstdint>

namespace vxb {
namespace {

__device__ __forceinline__ float bf_lo(uint32_t u) {
  return __uint_as_float(u << 16);
}
__device__ __forceinline__ float bf_hi(uint32_t u) {
  return __uint_as_float(u & 0xffff0000u);
}
__device__ __forceinline__ float bf16_at(const void *p, int64_t i) {
  return __uint_as_float((uint32_t)((const uint16_t *)p)[i] << 16);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

/* The pushed exchange moves (value, call) pairs: an aligned 8-byte store
   arrives whole, so a pair that carries the expected call number is complete
   and is its own arrival flag. An item's two rows travel as two pairs in one
   16-byte store; each half is still checked by its own call number. Stores
   and loads bypass L1 (volatile): a pair is seen when it arrives. */
__device__ __forceinline__ void pair_store(TpPair *at, float v, int call) {
  asm volatile("st.volatile.global.v2.b32 [%0], {%1, %2};" ::"l"(at),
               "r"(__float_as_uint(v)), "r"(call)
               : "memory");
}
__device__ __forceinline__ void pair2_store(TpPair *at, float v0, float v1,
                                            int call) {
  asm volatile("st.volatile.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(at),
               "r"(__float_as_uint(v0)), "r"(call), "r"(__float_as_uint(v1)),
               "r"(call)
               : "memory");
}
__device__ __forceinline__ bool pair_load(const TpPair *at, int call, float &v) {
  uint32_t bits;
  int seen;
  asm volatile("ld.volatile.global.v2.b32 {%0, %1}, [%2];"
               : "=r"(bits), "=r"(seen)
               : "l"(at)
               : "memory");
  v = __uint_as_float(bits);
  return seen == call;
}
__device__ __forceinline__ bool pair2_load(const TpPair *at, int call, float &v0,
                                           float &v1) {
  uint32_t b0, b1;
  int c0, c1;
  asm volatile("ld.volatile.global.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(b0), "=r"(c0), "=r"(b1), "=r"(c1)
               : "l"(at)
               : "memory");
  v0 = __uint_as_float(b0);
  v1 = __uint_as_float(b1);
  return c0 == call && c1 == call;
}

/* ------------------------------------------------------ decode attention
 * nn_attention with its parts and merge (nn.vx:349-866), and the attention
 * loops of llama2.vx:295-358.  A block owns one KV head, one run of `split`
 * positions and up to GH query heads that share the KV head; each warp takes
 * every fourth position, its lanes hold four values of head_dim each, keeps a
 * running (max, sum, weighted V) per query head, and the four warps are merged
 * in warp order.  The block that finishes last for a (sequence, head tile)
 * merges the parts of all splits in split order. */
/* What the ATT_WARPS warps of one unit share. */
template <int GH, int ATT_WARPS> struct AttnShared {
  float m[ATT_WARPS][GH], l[ATT_WARPS][GH];
  __align__(16) float acc[ATT_WARPS][GH][128];
  int is_last;
};
template <int ATT_WARPS> __device__ __forceinline__ void sync_unit_warps(int bar_id) {
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(ATT_WARPS * 32) : "memory");
}

/* One unit of work: (split, KV head and head tile `y`, sequence b), done by the
   ATT_WARPS warps (4, 8 or 16: as many as fill the GPU for the number of heads
   there are) that meet at named barrier `bar_id`. CHAINED: the caller is a
   kernel of its own in a chain of dependent launches. */
template <int GH, bool CHAINED, int CL, int ATT_WARPS, int NB = 8>
__device__ __forceinline__ void
attention_unit(const AttnArgs &a, int split_idx, int y, int b, int warp,
               int lane, AttnShared<GH, ATT_WARPS> &sh, int bar_id) {
  /* The position was written by the step before this one, and every cache row
     below it by earlier steps: those may be read before the kernels of this
     step have finished. Row `pos` and q come from the kernel just before. */
  const int hd = a.head_dim, hd4 = hd / 4;
  const int group = a.q_heads / a.kv_heads;
  const int tiles = (group + GH - 1) / GH;
  const int g = y / tiles, tile = y - g * tiles;
  const int h0 = g * group + tile * GH;
  const int nh = min(GH, group - tile * GH);
  const int pos = a.positions[b];
  /* CL > 0: the unit is one block of a cluster of CL that covers the whole
     head; block r takes the r-th run of ceil((pos + 1) / CL) positions (maybe
     none), and the runs are merged through distributed shared memory. */
  const int run = CL > 0 ? (pos + CL) / CL : a.split;
  const int t_begin = split_idx * run;
  if (CL == 0 && t_begin > pos)
    return;
  const int t_end = max(t_begin, min(t_begin + run, pos + 1));
  const int splits = pos / a.split + 1;
  const float scale = 1.0f / sqrtf((float)hd);
  const bool active = lane < hd4;

  const float *kc = a.k_cache + b * a.cache_batch_stride;
  const float *vc = a.v_cache + b * a.cache_batch_stride;
  const float *qb = a.q + (int64_t)b * a.q_heads * hd;

  /* Cache rows below `settled` were written by earlier steps and may be read
     before the kernels of this step have finished; the rest only after. */
  const int settled = !a.rows_settled ? 0
                      : a.fresh_from  ? min(pos, a.fresh_from[0])
                                      : pos;
  /* A warp takes every ATT_WARPS-th position, NB of them at a time so that
     their loads are in flight together: with 32 positions per block of four
     warps that is one round trip to memory per warp. */
  float4 kv[NB], vv[NB];
  auto load_batch = [&](int t0, bool old_rows_only) {
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const int t = t0 + j * ATT_WARPS;
      const bool take = active && t < t_end &&
                        (old_rows_only ? t < settled
                                       : t >= settled || t0 != t_begin + warp || !CHAINED);
      if (take) {
        const int64_t row = ((int64_t)t * a.kv_heads + g) * hd + lane * 4;
        kv[j] = *reinterpret_cast<const float4 *>(kc + row);
        vv[j] = *reinterpret_cast<const float4 *>(vc + row);
      } else if (!old_rows_only && !(active && t < t_end)) {
        kv[j] = vv[j] = make_float4(0, 0, 0, 0);
      }
    }
  };
#pragma unroll
  for (int j = 0; j < NB; ++j)
    kv[j] = vv[j] = make_float4(0, 0, 0, 0);
  if (CHAINED) {
    load_batch(t_begin + warp, true);
    chain_wait();
  }
  load_batch(t_begin + warp, false); /* CHAINED: only row `pos`, if it is here */

  float4 qv[GH];
  float m[GH], l[GH];
  float4 acc[GH];
#pragma unroll
  for (int h = 0; h < GH; ++h) {
    /* q is rewritten for every layer: read it past L1, which may still hold
       the layer before when the layers share a kernel */
    qv[h] = (active && h < nh)
                ? __ldcg(reinterpret_cast<const float4 *>(qb + (h0 + h) * hd +
                                                          lane * 4))
                : make_float4(0, 0, 0, 0);
    m[h] = -3.0e38f;
    l[h] = 0.0f;
    acc[h] = make_float4(0, 0, 0, 0);
  }

  for (int t0 = t_begin + warp; t0 < t_end; t0 += NB * ATT_WARPS) {
    if (t0 != t_begin + warp)
      load_batch(t0, false);
#pragma unroll
    for (int h = 0; h < GH; ++h) {
      float d[NB];
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        d[j] = qv[h].x * kv[j].x;
        d[j] = fmaf(qv[h].y, kv[j].y, d[j]);
        d[j] = fmaf(qv[h].z, kv[j].z, d[j]);
        d[j] = fmaf(qv[h].w, kv[j].w, d[j]);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int j = 0; j < NB; ++j)
          d[j] += __shfl_xor_sync(0xffffffffu, d[j], o);
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        if (t0 + j * ATT_WARPS >= t_end)
          continue;
        const float s = d[j] * scale;
        const float mn = fmaxf(m[h], s);
        const float fix = expf(m[h] - mn);
        const float pw = expf(s - mn);
        l[h] = l[h] * fix + pw;
        acc[h].x = acc[h].x * fix + pw * vv[j].x;
        acc[h].y = acc[h].y * fix + pw * vv[j].y;
        acc[h].z = acc[h].z * fix + pw * vv[j].z;
        acc[h].w = acc[h].w * fix + pw * vv[j].w;
        m[h] = mn;
      }
    }
  }

  /* ---- merge the warps, in warp order ---- */
  float (&sm_m)[ATT_WARPS][GH] = sh.m;
  float (&sm_l)[ATT_WARPS][GH] = sh.l;
  float (&sm_acc)[ATT_WARPS][GH][128] = sh.acc;
  int &is_last = sh.is_last;
#pragma unroll
  for (int h = 0; h < GH; ++h) {
    if (lane == 0) {
      sm_m[warp][h] = m[h];
      sm_l[warp][h] = l[h];
    }
    if (active)
      *reinterpret_cast<float4 *>(&sm_acc[warp][h][lane * 4]) = acc[h];
  }
  sync_unit_warps<ATT_WARPS>(bar_id);
  const int row_floats = hd + 2;
  float *part = a.scratch;
  auto part_at = [&](int head, int sp) {
    return part + (((int64_t)b * a.q_heads + head) * (a.max_pos / a.split + 1) +
                   sp) * row_floats;
  };
  if (CL > 0) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    if (warp == 0) {
      /* the block's part, left in row 0 of its own shared arrays */
      for (int h = 0; h < nh; ++h) {
        float big = -3.0e38f;
        for (int w = 0; w < ATT_WARPS; ++w)
          big = fmaxf(big, sm_m[w][h]);
        float total = 0.0f;
        float4 o = make_float4(0, 0, 0, 0);
        for (int w = 0; w < ATT_WARPS; ++w) {
          const float f = expf(sm_m[w][h] - big);
          total += f * sm_l[w][h];
          if (active) {
            const float4 v =
                *reinterpret_cast<const float4 *>(&sm_acc[w][h][lane * 4]);
            o.x += f * v.x; o.y += f * v.y; o.z += f * v.z; o.w += f * v.w;
          }
        }
        __syncwarp();
        if (active)
          *reinterpret_cast<float4 *>(&sm_acc[0][h][lane * 4]) = o;
        if (lane == 0) {
          sm_m[0][h] = big;
          sm_l[0][h] = total;
        }
      }
    }
    cluster.sync();
    if (cluster.block_rank() == 0) {
      /* block 0 merges the runs in order: warp h takes head h */
      for (int h = warp; h < nh; h += ATT_WARPS) {
        constexpr int NP = CL > 0 ? CL : 1; /* CL == 0 never gets here */
        float pm[NP], pl[NP];
        float4 pa[NP];
#pragma unroll
        for (int r = 0; r < CL; ++r) {
          const AttnShared<GH, ATT_WARPS> *peer = cluster.map_shared_rank(&sh, r);
          pm[r] = peer->m[0][h];
          pl[r] = peer->l[0][h];
          pa[r] = active
                      ? *reinterpret_cast<const float4 *>(&peer->acc[0][h][lane * 4])
                      : make_float4(0, 0, 0, 0);
        }
        float big = -3.0e38f;
#pragma unroll
        for (int r = 0; r < CL; ++r)
          big = fmaxf(big, pm[r]);
        float total = 0.0f;
        float4 o = make_float4(0, 0, 0, 0);
#pragma unroll
        for (int r = 0; r < CL; ++r) {
          const float f = expf(pm[r] - big);
          total += f * pl[r];
          o.x += f * pa[r].x; o.y += f * pa[r].y;
          o.z += f * pa[r].z; o.w += f * pa[r].w;
        }
        if (active) {
          float *dst = a.out + ((int64_t)b * a.q_heads + h0 + h) * hd + lane * 4;
          *reinterpret_cast<float4 *>(dst) =
              make_float4(o.x / total, o.y / total, o.z / total, o.w / total);
        }
      }
    }
    cluster.sync(); /* nobody leaves while block 0 may still read its part */
    return;
  }
  if (warp == 0) {
    for (int h = 0; h < nh; ++h) {
      float big = -3.0e38f;
      for (int w = 0; w < ATT_WARPS; ++w)
        big = fmaxf(big, sm_m[w][h]);
      float total = 0.0f;
      float4 o = make_float4(0, 0, 0, 0);
      for (int w = 0; w < ATT_WARPS; ++w) {
        const float f = expf(sm_m[w][h] - big);
        total += f * sm_l[w][h];
        if (active) {
          const float4 v = *reinterpret_cast<const float4 *>(&sm_acc[w][h][lane * 4]);
          o.x += f * v.x; o.y += f * v.y; o.z += f * v.z; o.w += f * v.w;
        }
      }
      /* A part row has head_dim + 2 floats, so rows are 8-byte aligned only. */
      float *dst = part_at(h0 + h, split_idx);
      if (active) {
        *reinterpret_cast<float2 *>(dst + lane * 4) = make_float2(o.x, o.y);
        *reinterpret_cast<float2 *>(dst + lane * 4 + 2) = make_float2(o.z, o.w);
      }
      if (lane == 0) {
        dst[hd] = big;
        dst[hd + 1] = total;
      }
    }
    __threadfence();
    __syncwarp();
    if (lane == 0) {
      int32_t *counter = a.counters + (int64_t)b * a.kv_heads * tiles + y;
      const int seen = atomicAdd(counter, 1);
      is_last = seen == splits - 1;
      if (is_last)
        *counter = 0; /* ready for the next launch */
    }
  }
  sync_unit_warps<ATT_WARPS>(bar_id);
  if (!is_last)
    return;
  __threadfence();

  /* ---- the last block of this head tile merges the splits, in order ---- */
  for (int h = warp; h < nh; h += ATT_WARPS) {
    float big = -3.0e38f;
    for (int sp = lane; sp < splits; sp += 32)
      big = fmaxf(big, __ldcg(part_at(h0 + h, sp) + hd));
    big = warp_max(big);
    float total = 0.0f;
    float4 o = make_float4(0, 0, 0, 0);
#pragma unroll 8
    for (int sp = 0; sp < splits; ++sp) {
      const float *src = part_at(h0 + h, sp);
      const float f = expf(__ldcg(src + hd) - big);
      total += f * __ldcg(src + hd + 1);
      if (active) {
        const float2 va = __ldcg(reinterpret_cast<const float2 *>(src + lane * 4));
        const float2 vb =
            __ldcg(reinterpret_cast<const float2 *>(src + lane * 4 + 2));
        o.x += f * va.x; o.y += f * va.y; o.z += f * vb.x; o.w += f * vb.y;
      }
    }
    if (active) {
      float *dst = a.out + ((int64_t)b * a.q_heads + h0 + h) * hd + lane * 4;
      *reinterpret_cast<float4 *>(dst) =
          make_float4(o.x / total, o.y / total, o.z / total, o.w / total);
    }
  }
}

/* ---------------------------------------------------------------- row dots
 * One kernel for every projection of the decoder.  An ITEM is a pair of weight
 * rows whose results the epilogue needs together; a warp owns a contiguous,
 * balanced range of items and streams both rows of an item at once. */
enum { EPI_STORE = 0, EPI_ADD = 1, EPI_BIAS = 2, EPI_SWIGLU = 3, EPI_QKV = 4,
       EPI_PUSH = 5 };

struct RowDotParams {
  /* weights */
  const void *w0, *w1, *w2; /* matvec: w0; swiglu: gate w0, up w1; qkv: q,k,v */
  /* the scales of w0, w1, w2 (fp8: f32 [ceil(rows/128), cols/128]; Q4_0: f16
     [rows, cols/32]); row_base: the row of the whole matrix that row 0 of w0
     is, when w0 is a run of rows inside a matrix with one table of scales */
  const void *s0, *s1, *s2;
  int row_base;
  int rows, cols;
  int items;
  /* activations */
  const float *x;
  int64_t x_stride;
  int batch;
  int x_in_smem;
  const void *norm_w;
  int norm_bf16;
  float eps;
  /* outputs */
  float *y;
  int64_t y_stride;
  const void *bias;
  /* qkv */
  int q_heads, kv_heads, head_dim, rope_mode;
  const float *cos_t, *sin_t;
  int cs_cols;
  float theta;
  const int32_t *positions;
  float *k_cache, *v_cache;
  int64_t cache_batch_stride;
  int max_seq;
  /* EPI_PUSH */
  TpPush tp;
  /* a mixture-of-experts layer: w0 (and s0) hold `experts` matrices one after
     another, expert_bytes (scale_bytes) apart, and this launch takes matrix
     expert_ids[expert_slot] (device memory: the router wrote it). add_scale
     (EPI_ADD): y += add_scale[0] * s. */
  const int32_t *expert_ids;
  int expert_slot, experts;
  int64_t expert_bytes, scale_bytes;
  const float *add_scale;
  int scales_in_ring; /* Q4_0: set by the launcher */
};

/* Weight formats. A row is a run of 16-byte words; a word holds E weights:
   4 f32, 8 bf16, 16 fp8 (f8e4m3 codes with an f32 scale per block of 128 x 128
   weights, nn.vx:1296-1303) or 32 Q4_0 codes (4 bits, weight = (code - 8) *
   an f16 scale per 32 weights of a row, nn.vx:1645-1663). */
struct Fp8W {};
struct Q4W {};
template <typename W> struct PerWord { static constexpr int n = 16 / (int)sizeof(W); };
template <> struct PerWord<Fp8W> { static constexpr int n = 16; };
template <> struct PerWord<Q4W> { static constexpr int n = 32; };
template <typename W> struct Scaled { static constexpr bool yes = false; };
template <> struct Scaled<Fp8W> { static constexpr bool yes = true; };
template <> struct Scaled<Q4W> { static constexpr bool yes = true; };

/* The two weight rows of an item (byte addresses), where their scales are,
   and for q/k/v which head and pair it is. */
struct ItemRows {
  const char *r0, *r1; /* r1 == nullptr: an odd last row */
  const char *sc0, *sc1; /* scaled formats: the scales of the rows' first column */
  int head, idx, kind; /* qkv: kind 0 q, 1 k, 2 v */
};
template <typename W>
__device__ __forceinline__ const char *scale_row(const void *scales, int row,
                                                 int cols) {
  if (PerWord<W>::n == 16) /* fp8: one row of scales per 128 rows */
    return (const char *)scales + (int64_t)(row / 128) * (cols / 128) * 4;
  return (const char *)scales + (int64_t)row * (cols / 32) * 2; /* Q4_0 */
}
template <typename W, int EPI>
__device__ __forceinline__ ItemRows item_rows(const RowDotParams &p, int item,
                                              int64_t w_off = 0, int64_t s_off = 0) {
  ItemRows it;
  const int cols = p.cols;
  const int64_t row_bytes = (int64_t)cols * 16 / PerWord<W>::n;
  it.head = it.idx = it.kind = 0;
  it.sc0 = it.sc1 = nullptr;
  if (EPI == EPI_SWIGLU) {
    it.r0 = (const char *)p.w0 + w_off + item * row_bytes;
    it.r1 = p.w1 ? (const char *)p.w1 + item * row_bytes
                 : (const char *)p.w0 + w_off + (p.rows + item) * row_bytes;
    if (Scaled<W>::yes) {
      it.sc0 = scale_row<W>(p.s0, p.row_base + item, cols) + s_off;
      it.sc1 = p.w1 ? scale_row<W>(p.s1, item, cols)
                    : scale_row<W>(p.s0, p.row_base + p.rows + item, cols) + s_off;
    }
  } else if (EPI == EPI_QKV) {
    const int half = p.head_dim / 2;
    it.head = item / half;
    it.idx = item - it.head * half;
    const int a = p.rope_mode == 0 ? it.idx : 2 * it.idx;
    const int b = p.rope_mode == 0 ? it.idx + half : 2 * it.idx + 1;
    const char *base;
    const void *sbase = p.s0;
    int local = it.head, srow = p.row_base;
    if (it.head < p.q_heads) {
      base = (const char *)p.w0;
    } else if (it.head < p.q_heads + p.kv_heads) {
      it.kind = 1;
      local = it.head - p.q_heads;
      if (p.w1) {
        base = (const char *)p.w1;
        sbase = p.s1;
        srow = 0;
      } else {
        base = (const char *)p.w0 + p.q_heads * p.head_dim * row_bytes;
        srow += p.q_heads * p.head_dim;
      }
    } else {
      it.kind = 2;
      local = it.head - p.q_heads - p.kv_heads;
      if (p.w2) {
        base = (const char *)p.w2;
        sbase = p.s2;
        srow = 0;
      } else {
        base = (const char *)p.w0 +
               (p.q_heads + p.kv_heads) * p.head_dim * row_bytes;
        srow += (p.q_heads + p.kv_heads) * p.head_dim;
      }
    }
    it.r0 = base + ((int64_t)local * p.head_dim + a) * row_bytes;
    it.r1 = base + ((int64_t)local * p.head_dim + b) * row_bytes;
    if (Scaled<W>::yes) {
      it.sc0 = scale_row<W>(sbase, srow + local * p.head_dim + a, cols);
      it.sc1 = scale_row<W>(sbase, srow + local * p.head_dim + b, cols);
    }
  } else {
    it.r0 = (const char *)p.w0 + w_off + (int64_t)(2 * item) * row_bytes;
    it.r1 = 2 * item + 1 < p.rows ? it.r0 + row_bytes : nullptr;
    if (Scaled<W>::yes) {
      it.sc0 = scale_row<W>(p.s0, p.row_base + 2 * item, cols) + s_off;
      it.sc1 = scale_row<W>(p.s0, p.row_base + 2 * item + 1, cols) + s_off;
    }
  }
  return it;
}

} // namespace
} // namespace vxb

#endif /* VXB_NN_DEVICE_CUH */
