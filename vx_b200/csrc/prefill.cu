/* prefill.cu -- a whole prompt through the layers at once: the kernels behind
 * vx_decoder_prefill for the std::nn flavour (bf16 weights, f32 activations).
 *
 * The reference has multi-row kernels for this (stdlib/std/nn.vx:2317-3066:
 * nn_matvec_rows :2802, nn_rms_norm_rows :2835, nn_qkv_*_rows :2614,
 * nn_embed_rows :2933), each "the kernel of the same name without _rows ...
 * for each position", and its llama programs feed a prompt one decode step at
 * a time.  Here the T positions of a prompt are the rows of GEMMs on the
 * tensor cores:
 *
 *   y[t, r] = sum_c W[r, c] x[t, c]      for all t at once.
 *
 * To keep f32 activations (the decode path's arithmetic, and with it the
 * tokens), every x is split into three bf16 terms x = x1 + x2 + x3 (the
 * remainders are exact in f32), laid side by side as a [T, 3 cols] bf16 matrix;
 * the GEMM then runs over K' = 3 cols with the weight tile of K block kb taken
 * from column block kb mod (cols / 64): three exact bf16 x bf16 products per
 * weight, summed in f32 in tensor memory.
 *
 * rows_gemm_kernel: CTA pairs (tcgen05.mma.cta_group::2) as in
 * gemm_umma_pair.cu, 256 positions x 256 weight rows per tile.  A work item is
 * (tile, one of S runs of the K' dimension), S chosen so that the items fill
 * whole waves of the 74 pairs; an item's f32 sums go to partials[s][t][r], and
 * the small kernel that follows each GEMM adds the runs in run order (the
 * result does not depend on timing) and applies the projection's epilogue:
 * bias + RoPE + KV-cache store, residual add, SwiGLU, and leaves its output as
 * the three terms the next GEMM reads.  Attention over the prompt is a tiled
 * f32 kernel on the FMA pipe (the work is 2 % of the projections'), so the
 * cache and the scores keep the decode path's precision.
 */
#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>

#include <cstdio>

namespace vxb {

bool make_map_16(CUtensorMap *map, const void *base, int64_t inner, int64_t rows,
                 int64_t ld, int box_inner, int box_rows, bool is_bf16);

namespace {

constexpr int BM = 256, BN = 256, BK = 64, UK = 16;
constexpr int HM = BM / 2, HN = BN / 2;
constexpr int STAGES = 6;
constexpr int A_BYTES = HM * BK * 2, B_BYTES = HN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int THREADS = 192;

enum { ST_LOADER_EMPTY = 0x71, ST_MMA_FULL = 0x72, ST_MMA_TMEM_EMPTY = 0x73,
       ST_EPI_TMEM_FULL = 0x74 };
__device__ int g_rows_status;

struct Barriers {
  uint64_t full[STAGES], empty[STAGES];
  uint64_t tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  int stop;
};

struct RowsGemm {
  int t, n;        /* positions, weight rows */
  int k_blocks;    /* of the term matrix: 3 * cols / 64 */
  int w_blocks;    /* of the weights: cols / 64 */
  int splits;
  float *partials; /* [splits][t][n] */
};

/* Item -> (tile of positions, tile of weight rows, run). The runs and position
   tiles of one weight tile are neighbours, so that the pairs that run together
   read the same weights and find them in L2. */
__device__ inline void item_coords(int item, int m_tiles, int splits, int &tm,
                                   int &tn, int &run) {
  const int per_n = m_tiles * splits;
  tn = item / per_n;
  const int rest = item - tn * per_n;
  tm = rest / splits;
  run = rest - tm * splits;
}

__global__ void __launch_bounds__(THREADS, 1)
rows_gemm_kernel(const __grid_constant__ CUtensorMap map_x,
                 const __grid_constant__ CUtensorMap map_w, const RowsGemm g) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Barriers *bars = reinterpret_cast<Barriers *>(smem + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = ptx::cluster_ctarank();
  const int pair = blockIdx.x / 2, pairs = gridDim.x / 2;
  const int m_tiles = (g.t + BM - 1) / BM, n_tiles = (g.n + BN - 1) / BN;
  const int items = m_tiles * n_tiles * g.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&bars->full[s], 1);
      ptx::mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&bars->tmem_full[a], 1);
      ptx::mbar_init(&bars->tmem_empty[a], 8);
    }
    bars->stop = 0;
    ptx::fence_proxy_async_smem();
    ptx::fence_barrier_init();
  }
  if (warp == 1)
    ptx::tmem_alloc_pair(&bars->tmem_base, 512);
  ptx::tc_fence_before_sync();
  ptx::cluster_sync_all();
  ptx::tc_fence_after_sync();
  /* Set up under the tail of the kernel before; its output (the terms) is read,
     and the partial sums it may still read are overwritten, only from here. */
  chain_release();
  chain_wait();
  const uint32_t tmem = bars->tmem_base;
  volatile int *stop = &bars->stop;
  /* the K' blocks of run r: a balanced cut of 0 .. k_blocks */
  auto run_first = [&](int r) { return (int)((int64_t)r * g.k_blocks / g.splits); };

  if (warp == 0) {
    if (lane == 0) {
      ptx::tma_prefetch_desc(&map_x);
      ptx::tma_prefetch_desc(&map_w);
      int it = 0;
      bool ok = true;
      for (int item = pair; ok && item < items; item += pairs) {
        int tm, tn, run;
        item_coords(item, m_tiles, g.splits, tm, tn, run);
        const int kb1 = run_first(run + 1);
        for (int kb = run_first(run); kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1;
          if (!ptx::mbar_wait(&bars->empty[s], phase ^ 1, stop)) {
            atomicCAS(&g_rows_status, 0, ST_LOADER_EMPTY);
            *stop = 1;
            ok = false;
            break;
          }
          uint8_t *sa = smem + s * STAGE_BYTES, *sb = sa + A_BYTES;
          const uint32_t leader_full =
              ptx::map_to_cta(ptx::smem_addr(&bars->full[s]), 0);
          if (rank == 0)
            ptx::mbar_expect_tx(&bars->full[s], 2 * STAGE_BYTES);
          ptx::tma_load_2d_pair(sa, &map_x, kb * BK, tm * BM + (int)rank * HM,
                                leader_full);
          ptx::tma_load_2d_pair(sb, &map_w, (kb % g.w_blocks) * BK,
                                tn * BN + (int)rank * HN, leader_full);
        }
      }
      if (rank == 0)
        for (int back = 0; back < STAGES && back < it; ++back) {
          const int j = it - 1 - back;
          ptx::mbar_wait_alone(&bars->full[j % STAGES], (j / STAGES) & 1);
        }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = ptx::idesc_f16(true, false, false, BM, BN);
      int it = 0, t = 0;
      bool ok = true;
      for (int item = pair; ok && item < items; item += pairs, ++t) {
        int tm, tn, run;
        item_coords(item, m_tiles, g.splits, tm, tn, run);
        const int acc = t & 1;
        if (!ptx::mbar_wait_cluster(&bars->tmem_empty[acc], ((t >> 1) & 1) ^ 1,
                                    stop)) {
          atomicCAS(&g_rows_status, 0, ST_MMA_TMEM_EMPTY);
          *stop = 1;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem + acc * BN;
        const int kb0 = run_first(run), kb1 = run_first(run + 1);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!ptx::mbar_wait_cluster(&bars->full[s], (it / STAGES) & 1, stop)) {
            atomicCAS(&g_rows_status, 0, ST_MMA_FULL);
            *stop = 1;
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t sa = ptx::smem_addr(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UK; ++kk) {
            const uint64_t da = ptx::smem_desc_sw128(sa + kk * UK * 2, 16, 1024);
            const uint64_t db = ptx::smem_desc_sw128(sb + kk * UK * 2, 16, 1024);
            ptx::umma_f16_ss_pair(d_tmem, da, db, idesc, (kb != kb0) | (kk != 0));
          }
          ptx::umma_commit_pair(&bars->empty[s]);
        }
        if (ok)
          ptx::umma_commit_pair(&bars->tmem_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    int t = 0;
    for (int item = pair; item < items; item += pairs, ++t) {
      int tm, tn, run;
      item_coords(item, m_tiles, g.splits, tm, tn, run);
      const int acc = t & 1;
      if (!ptx::mbar_wait(&bars->tmem_full[acc], (t >> 1) & 1, stop)) {
        atomicCAS(&g_rows_status, 0, ST_EPI_TMEM_FULL);
        *stop = 1;
        break;
      }
      ptx::tc_fence_after_sync();
      const int row = tm * BM + (int)rank * HM + quarter * 32 + lane; /* position */
      const int col0 = tn * BN;
      float *out = g.partials + ((int64_t)run * g.t + row) * g.n + col0;
      const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(taddr + c * 32, v);
        ptx::tmem_ld_wait();
        if (row < g.t) {
          const int col = col0 + c * 32;
          if (col + 32 <= g.n) {
            float4 *dst = reinterpret_cast<float4 *>(out + c * 32);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              dst[q] = make_float4(__uint_as_float(v[4 * q]),
                                   __uint_as_float(v[4 * q + 1]),
                                   __uint_as_float(v[4 * q + 2]),
                                   __uint_as_float(v[4 * q + 3]));
          } else {
            for (int e = 0; e < 32; ++e)
              if (col + e < g.n)
                out[c * 32 + e] = __uint_as_float(v[e]);
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

  ptx::tc_fence_before_sync();
  __syncwarp();
  ptx::cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem, 512);
  }
}

/* ---- what sits between the GEMMs ------------------------------------------- */
__device__ __forceinline__ float bf16_val(const void *p, int64_t i) {
  return __uint_as_float((uint32_t)((const uint16_t *)p)[i] << 16);
}
/* v as three bf16 terms at column i of row t of a [T, 3 cols] matrix. */
__device__ __forceinline__ void store_terms(__nv_bfloat16 *terms, int cols,
                                            int64_t t, int i, float v) {
  const __nv_bfloat16 t1 = __float2bfloat16(v);
  const float r1 = v - __bfloat162float(t1);
  const __nv_bfloat16 t2 = __float2bfloat16(r1);
  const float r2 = r1 - __bfloat162float(t2);
  __nv_bfloat16 *row = terms + t * 3 * cols;
  row[i] = t1;
  row[cols + i] = t2;
  row[2 * cols + i] = __float2bfloat16(r2);
}
/* The sum of the runs' partials of (t, r), in run order. */
__device__ __forceinline__ float sum_runs(const float *partials, int splits,
                                          int64_t t_count, int64_t n, int64_t t,
                                          int64_t r) {
  float s = partials[t * n + r];
  for (int k = 1; k < splits; ++k)
    s += partials[((int64_t)k * t_count + t) * n + r];
  return s;
}

/* The same for four consecutive values (r a multiple of 4). */
__device__ __forceinline__ float4 sum_runs4(const float *partials, int splits,
                                            int64_t t_count, int64_t n, int64_t t,
                                            int64_t r) {
  float4 s = *reinterpret_cast<const float4 *>(partials + t * n + r);
  for (int k = 1; k < splits; ++k) {
    const float4 v = *reinterpret_cast<const float4 *>(
        partials + ((int64_t)k * t_count + t) * n + r);
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  return s;
}
/* Eight consecutive values (i a multiple of 8) as their three terms: one
   16-byte store per term. */
__device__ __forceinline__ void store_terms8(__nv_bfloat16 *terms, int cols,
                                             int64_t t, int i, const float (&v)[8]) {
  uint32_t w1[4], w2[4], w3[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t parts[3] = {0, 0, 0};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float x = v[2 * j + h];
      const __nv_bfloat16 t1 = __float2bfloat16(x);
      const float r1 = x - __bfloat162float(t1);
      const __nv_bfloat16 t2 = __float2bfloat16(r1);
      const float r2 = r1 - __bfloat162float(t2);
      const __nv_bfloat16 t3 = __float2bfloat16(r2);
      parts[0] |= (uint32_t)__bfloat16_as_ushort(t1) << (16 * h);
      parts[1] |= (uint32_t)__bfloat16_as_ushort(t2) << (16 * h);
      parts[2] |= (uint32_t)__bfloat16_as_ushort(t3) << (16 * h);
    }
    w1[j] = parts[0];
    w2[j] = parts[1];
    w3[j] = parts[2];
  }
  __nv_bfloat16 *row = terms + t * 3 * cols;
  *reinterpret_cast<uint4 *>(row + i) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
  *reinterpret_cast<uint4 *>(row + cols + i) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
  *reinterpret_cast<uint4 *>(row + 2 * cols + i) = make_uint4(w3[0], w3[1], w3[2], w3[3]);
}

/* nn_rms_norm_rows (nn.vx:2835): terms of x[t] / sqrt(mean(x[t]^2) + eps) * w;
   one block per position. */
__global__ void __launch_bounds__(256)
norm_terms_kernel(__nv_bfloat16 *terms, const float *x, const void *w, int dim,
                  float eps) {
  __shared__ float red[8];
  chain_release();
  chain_wait();
  const int64_t t = blockIdx.x;
  const float *xr = x + t * dim;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x)
    ss = fmaf(xr[i], xr[i], ss);
  for (int o = 16; o > 0; o >>= 1)
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0)
    red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.0f;
  for (int k = 0; k < 8; ++k) /* fixed order */
    total += red[k];
  const float inv = 1.0f / sqrtf(total / (float)dim + eps);
  for (int i = threadIdx.x; i < dim; i += blockDim.x)
    store_terms(terms, dim, t, i, xr[i] * bf16_val(w, i) * inv);
}

/* After the output or the down projection, when an RMSNorm follows: x[t] += the
   product, and the terms of the normalised x[t] for the next GEMM, in one pass
   over the row (the sums in the order of residual_finish_kernel and
   norm_terms_kernel). One block per position; dim <= 256 * 32. */
__global__ void __launch_bounds__(256)
residual_norm_kernel(__nv_bfloat16 *terms, float *x, const float *partials,
                     int splits, int t_count, const void *w, int dim, float eps) {
  __shared__ float red[8];
  chain_release();
  chain_wait();
  const int64_t t = blockIdx.x;
  float *xr = x + t * dim;
  constexpr int PER = 32;
  float v[PER];
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int i = threadIdx.x + k * 256;
    v[k] = 0.0f;
    if (i < dim) {
      v[k] = xr[i] + sum_runs(partials, splits, t_count, dim, t, i);
      xr[i] = v[k];
      ss = fmaf(v[k], v[k], ss);
    }
  }
  for (int o = 16; o > 0; o >>= 1)
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0)
    red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.0f;
  for (int k = 0; k < 8; ++k) /* fixed order */
    total += red[k];
  const float inv = 1.0f / sqrtf(total / (float)dim + eps);
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < dim)
      store_terms(terms, dim, t, i, v[k] * bf16_val(w, i) * inv);
  }
}

/* After the q/k/v GEMM: bias, half-split RoPE (nn_rope_and_store,
   nn.vx:245-280), q to q_out[t], k and v to row first_pos + t of the cache.
   One thread per (position, head, pair i / i + hd/2). */
__global__ void __launch_bounds__(256)
qkv_finish_kernel(const float *partials, int splits, int t_count, int q_heads,
                  int kv_heads, int hd, const void *bias, const float *cos_t,
                  const float *sin_t, const int32_t *first_pos, float *q_out,
                  float *k_cache, float *v_cache) {
  chain_release();
  chain_wait();
  /* one thread per (position, head, four pairs i..i+3 / i + hd/2 ..) */
  const int half = hd / 2, quads = half / 4, heads = q_heads + 2 * kv_heads;
  const int64_t n = (int64_t)heads * hd;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)t_count * heads * quads)
    return;
  const int i = (int)(idx % quads) * 4;
  const int head = (int)((idx / quads) % heads);
  const int64_t t = idx / ((int64_t)quads * heads);
  const int64_t ra = (int64_t)head * hd + i, rb = ra + half;
  float4 va = sum_runs4(partials, splits, t_count, n, t, ra);
  float4 vb = sum_runs4(partials, splits, t_count, n, t, rb);
  if (bias) {
    va.x += bf16_val(bias, ra); va.y += bf16_val(bias, ra + 1);
    va.z += bf16_val(bias, ra + 2); va.w += bf16_val(bias, ra + 3);
    vb.x += bf16_val(bias, rb); vb.y += bf16_val(bias, rb + 1);
    vb.z += bf16_val(bias, rb + 2); vb.w += bf16_val(bias, rb + 3);
  }
  const int pos = first_pos[0] + (int)t;
  if (head >= q_heads + kv_heads) {
    float *row = v_cache + ((int64_t)pos * kv_heads + (head - q_heads - kv_heads)) * hd;
    *reinterpret_cast<float4 *>(row + i) = va;
    *reinterpret_cast<float4 *>(row + i + half) = vb;
    return;
  }
  const float4 c = *reinterpret_cast<const float4 *>(cos_t + (int64_t)pos * half + i);
  const float4 s = *reinterpret_cast<const float4 *>(sin_t + (int64_t)pos * half + i);
  float4 oa, ob;
  oa.x = __fsub_rn(__fmul_rn(va.x, c.x), __fmul_rn(vb.x, s.x));
  oa.y = __fsub_rn(__fmul_rn(va.y, c.y), __fmul_rn(vb.y, s.y));
  oa.z = __fsub_rn(__fmul_rn(va.z, c.z), __fmul_rn(vb.z, s.z));
  oa.w = __fsub_rn(__fmul_rn(va.w, c.w), __fmul_rn(vb.w, s.w));
  ob.x = __fadd_rn(__fmul_rn(vb.x, c.x), __fmul_rn(va.x, s.x));
  ob.y = __fadd_rn(__fmul_rn(vb.y, c.y), __fmul_rn(va.y, s.y));
  ob.z = __fadd_rn(__fmul_rn(vb.z, c.z), __fmul_rn(va.z, s.z));
  ob.w = __fadd_rn(__fmul_rn(vb.w, c.w), __fmul_rn(va.w, s.w));
  float *dst = head < q_heads
                   ? q_out + (t * q_heads + head) * hd
                   : k_cache + ((int64_t)pos * kv_heads + (head - q_heads)) * hd;
  *reinterpret_cast<float4 *>(dst + i) = oa;
  *reinterpret_cast<float4 *>(dst + i + half) = ob;
}

/* After the output or the down projection: x[t, r] += the product. */
__global__ void __launch_bounds__(256)
residual_finish_kernel(float *x, const float *partials, int splits, int t_count,
                       int n) {
  chain_release();
  chain_wait();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)t_count * n)
    return;
  const int64_t t = idx / n, r = idx - t * n;
  x[idx] = x[idx] + sum_runs(partials, splits, t_count, n, t, r);
}

/* After the gate/up GEMM: silu(g) * u (nn_swiglu, nn.vx:169-209) as the terms
   the down projection reads. Rows 0..hidden are gate, hidden..2 hidden up. */
__global__ void __launch_bounds__(256)
swiglu_finish_kernel(__nv_bfloat16 *terms, const float *partials, int splits,
                     int t_count, int hidden) {
  chain_release();
  chain_wait();
  /* one thread per (position, eight consecutive rows): hidden % 8 == 0 */
  const int per_row = hidden / 8;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)t_count * per_row)
    return;
  const int64_t t = idx / per_row;
  const int r = (int)(idx - t * per_row) * 8;
  const int64_t n = 2 * (int64_t)hidden;
  const float4 g0 = sum_runs4(partials, splits, t_count, n, t, r);
  const float4 g1 = sum_runs4(partials, splits, t_count, n, t, r + 4);
  const float4 u0 = sum_runs4(partials, splits, t_count, n, t, hidden + r);
  const float4 u1 = sum_runs4(partials, splits, t_count, n, t, hidden + r + 4);
  const float gate[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
  const float up[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
  float out[8];
#pragma unroll
  for (int e = 0; e < 8; ++e)
    out[e] = gate[e] / (1.0f + expf(0.0f - gate[e])) * up[e];
  store_terms8(terms, hidden, t, r, out);
}

/* ---- attention over the prompt, f32 on the FMA pipe -------------------------
 * One block per (64 positions, query head): scores of the 64 queries against
 * 32 cache rows at a time, an online softmax (running maximum and sum per
 * query), and the weighted sum of V; rows 0 .. first_pos + t of the cache for
 * the query at prompt position t (nn_attention, nn.vx:349-866, for every
 * position). head_dim 128. The output goes out as the three bf16 terms of the
 * output projection's input. */
constexpr int AQ = 64, AK = 32, AD = 128;
constexpr int ATT_THREADS = 256;
/* 76 KiB: two blocks share an SM, so one block's loads and barriers run under
   the other's arithmetic */
constexpr int ATT_SMEM = (AQ * (AD + 4) + 2 * AK * (AD + 4) + AQ * (AK + 4)) * 4;

__global__ void __launch_bounds__(ATT_THREADS, 2)
rows_attention_kernel(__nv_bfloat16 *terms, const float *q, const float *k_cache,
                      const float *v_cache, const int32_t *first_pos, int t_count,
                      int q_heads, int kv_heads) {
  extern __shared__ __align__(16) float att_smem[];
  float (*sq)[AD + 4] = reinterpret_cast<float (*)[AD + 4]>(att_smem);
  float (*sk)[AD + 4] = reinterpret_cast<float (*)[AD + 4]>(att_smem + AQ * (AD + 4));
  float (*sv)[AD + 4] =
      reinterpret_cast<float (*)[AD + 4]>(att_smem + (AQ + AK) * (AD + 4));
  float (*sp)[AK + 4] =
      reinterpret_cast<float (*)[AK + 4]>(att_smem + (AQ + 2 * AK) * (AD + 4));

  chain_release();
  chain_wait();
  const int head = blockIdx.y, g = head / (q_heads / kv_heads);
  const int t0 = blockIdx.x * AQ;
  const int base = first_pos[0];
  const int tid = threadIdx.x;
  const float scale = 1.0f / sqrtf((float)AD);

  /* the 64 queries of this block */
  for (int i = tid; i < AQ * (AD / 4); i += ATT_THREADS) {
    const int r = i / (AD / 4), c4 = i % (AD / 4);
    float4 v = make_float4(0, 0, 0, 0);
    if (t0 + r < t_count)
      v = *reinterpret_cast<const float4 *>(
          q + ((int64_t)(t0 + r) * q_heads + head) * AD + c4 * 4);
    *reinterpret_cast<float4 *>(&sq[r][c4 * 4]) = v;
  }
  /* scores: thread (ty, tx) of 16 x 16 owns queries ty*4.. and keys tx and
     tx + 16; output: queries ty*4.., values tx*8.. */
  constexpr int KB = AK / 16; /* keys per thread */
  const int ty = tid / 16, tx = tid % 16;
  float m[4], l[4], o[4][8];
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    m[a] = -3.0e38f;
    l[a] = 0.0f;
#pragma unroll
    for (int b = 0; b < 8; ++b)
      o[a][b] = 0.0f;
  }
  const int last_key = base + min(t0 + AQ, t_count) - 1; /* of the block's last query */
  for (int k0 = 0; k0 <= last_key; k0 += AK) {
    __syncthreads(); /* the tiles of the step before are done with */
    for (int i = tid; i < AK * (AD / 4); i += ATT_THREADS) {
      const int r = i / (AD / 4), c4 = i % (AD / 4);
      float4 kv = make_float4(0, 0, 0, 0), vv = kv;
      if (k0 + r <= last_key) {
        const int64_t at = ((int64_t)(k0 + r) * kv_heads + g) * AD + c4 * 4;
        kv = *reinterpret_cast<const float4 *>(k_cache + at);
        vv = *reinterpret_cast<const float4 *>(v_cache + at);
      }
      *reinterpret_cast<float4 *>(&sk[r][c4 * 4]) = kv;
      *reinterpret_cast<float4 *>(&sv[r][c4 * 4]) = vv;
    }
    __syncthreads();
    float s[4][KB];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < KB; ++b)
        s[a][b] = 0.0f;
    for (int d = 0; d < AD; d += 4) {
      float4 qa[4], kb[KB];
#pragma unroll
      for (int a = 0; a < 4; ++a)
        qa[a] = *reinterpret_cast<const float4 *>(&sq[ty * 4 + a][d]);
#pragma unroll
      for (int b = 0; b < KB; ++b)
        kb[b] = *reinterpret_cast<const float4 *>(&sk[tx + 16 * b][d]);
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < KB; ++b) {
          s[a][b] = fmaf(qa[a].x, kb[b].x, s[a][b]);
          s[a][b] = fmaf(qa[a].y, kb[b].y, s[a][b]);
          s[a][b] = fmaf(qa[a].z, kb[b].z, s[a][b]);
          s[a][b] = fmaf(qa[a].w, kb[b].w, s[a][b]);
        }
    }
    /* mask, the step's maximum per query over the 16 threads of its row,
       probabilities into shared memory, rescale of what was summed so far */
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int qpos = base + t0 + ty * 4 + a;
      float big = -3.0e38f;
#pragma unroll
      for (int b = 0; b < KB; ++b) {
        const int key = k0 + tx + 16 * b;
        s[a][b] = key <= qpos ? s[a][b] * scale : -3.0e38f;
        big = fmaxf(big, s[a][b]);
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1)
        big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, off));
      const float mn = fmaxf(m[a], big);
      const float fix = expf(m[a] - mn);
      float sum = 0.0f;
#pragma unroll
      for (int b = 0; b < KB; ++b) {
        const int key = k0 + tx + 16 * b;
        const float pw = key <= qpos ? expf(s[a][b] - mn) : 0.0f;
        sp[ty * 4 + a][tx + 16 * b] = pw;
        sum += pw;
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1)
        sum += __shfl_xor_sync(0xffffffffu, sum, off);
      l[a] = l[a] * fix + sum;
      m[a] = mn;
#pragma unroll
      for (int b = 0; b < 8; ++b)
        o[a][b] *= fix;
    }
    __syncthreads();
    for (int key = 0; key < AK; ++key) {
      const float4 v0 = *reinterpret_cast<const float4 *>(&sv[key][tx * 8]);
      const float4 v1 = *reinterpret_cast<const float4 *>(&sv[key][tx * 8 + 4]);
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float pw = sp[ty * 4 + a][key];
        o[a][0] = fmaf(pw, v0.x, o[a][0]); o[a][1] = fmaf(pw, v0.y, o[a][1]);
        o[a][2] = fmaf(pw, v0.z, o[a][2]); o[a][3] = fmaf(pw, v0.w, o[a][3]);
        o[a][4] = fmaf(pw, v1.x, o[a][4]); o[a][5] = fmaf(pw, v1.y, o[a][5]);
        o[a][6] = fmaf(pw, v1.z, o[a][6]); o[a][7] = fmaf(pw, v1.w, o[a][7]);
      }
    }
  }
  const int cols = q_heads * AD;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int t = t0 + ty * 4 + a;
    if (t >= t_count)
      continue;
#pragma unroll
    for (int b = 0; b < 8; ++b)
      store_terms(terms, cols, t, head * AD + tx * 8 + b, o[a][b] / l[a]);
  }
}

/* ---- Q4_0 weights for the CTA-pair GEMM --------------------------------------
 * A Q4_0 weight is (code - 8) * scale with an f16 scale: 4 + 11 significant
 * bits, so two bf16 terms hold it exactly. A matrix goes to a scratch as
 * [n, 2 cols] = w1 | w2; the activations' terms are laid out as
 * x1 | x1 | x2 | x2 | x3 | x3, and the GEMM, which lets K block kb of the first
 * operand meet K block kb mod (2 cols / 64) of the second, multiplies every x
 * term with every w term. */
__global__ void __launch_bounds__(256)
q4_two_terms_kernel(__nv_bfloat16 *out, const uint32_t *codes, const __half *scales,
                    int64_t words_total, int cols) {
  chain_release();
  chain_wait();
  const int words = cols / 8;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < words_total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / words;
    const int wd = (int)(i - r * words);
    const uint32_t code = codes[i];
    const float scale = __half2float(scales[r * (cols / 32) + wd / 4]);
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t h2 = 0, l2 = 0;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float v = (float)((int)((code >> (8 * j + 4 * h)) & 15u) - 8) * scale;
        const __nv_bfloat16 t1 = __float2bfloat16(v);
        const __nv_bfloat16 t2 = __float2bfloat16(v - __bfloat162float(t1));
        h2 |= (uint32_t)__bfloat16_as_ushort(t1) << (16 * h);
        l2 |= (uint32_t)__bfloat16_as_ushort(t2) << (16 * h);
      }
      hi[j] = h2;
      lo[j] = l2;
    }
    __nv_bfloat16 *row = out + r * 2 * cols + wd * 8;
    *reinterpret_cast<uint4 *>(row) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    *reinterpret_cast<uint4 *>(row + cols) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  }
}

/* An fp8 weight is the value of its e4m3 code times the f32 scale of its block
 * of 128 x 128, rounded to f32 as a plain multiplication rounds it; that f32 is
 * three bf16 terms exactly. A matrix goes to a scratch as [n, 3 cols] =
 * w1 | w2 | w3, the activations' terms are laid out as
 * x1 | x1 | x1 | x2 | x2 | x2 | x3, and the seven segments meet w1 w2 w3 w1 w2 w3
 * w1: the six products an f32 product needs, and x2 w3 besides. */
__global__ void __launch_bounds__(256)
fp8_three_terms_kernel(__nv_bfloat16 *out, const uint2 *codes, const float *scales,
                       int64_t eights_total, int cols) {
  chain_release();
  chain_wait();
  const int eights = cols / 8;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < eights_total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / eights;
    const int e8 = (int)(i - r * eights);
    const uint2 eight = codes[i];
    const float scale = scales[(r >> 7) * (cols / 128) + e8 / 16];
    const uint32_t word[2] = {eight.x, eight.y};
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const unsigned short two = (unsigned short)(word[j >> 1] >> (16 * (j & 1)));
      uint32_t halves;
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(halves) : "h"(two));
      v[2 * j] = __half2float(__ushort_as_half((unsigned short)(halves & 0xffffu))) * scale;
      v[2 * j + 1] = __half2float(__ushort_as_half((unsigned short)(halves >> 16))) * scale;
    }
    store_terms8(out, cols, r, e8 * 8, v);
  }
}

/* [t, 3 cols] = x1 | x2 | x3  ->  [t, segments cols], segment s a copy of term
   from[s] */
struct SpreadPlan {
  int segments;
  int from[8];
};
__global__ void __launch_bounds__(256)
spread_terms_kernel(uint4 *out, const uint4 *in, int64_t quads_total, int cols,
                    const SpreadPlan plan) {
  chain_release();
  chain_wait();
  const int per_term = cols / 8;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < quads_total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / (plan.segments * per_term);
    const int rest = (int)(i - row * plan.segments * per_term);
    const int seg = rest / per_term, c = rest - seg * per_term;
    out[i] = in[row * 3 * per_term + plan.from[seg] * per_term + c];
  }
}

const char *last_launch(const char *what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess)
    return nullptr;
  static thread_local char msg[200];
  snprintf(msg, sizeof msg, "%s: %s", what, cudaGetErrorString(e));
  return msg;
}

int resident_pairs() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && cached[dev])
    return cached[dev];
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS);
  cfg.gridDim = dim3(2 * 74);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, rows_gemm_kernel, &cfg) !=
          cudaSuccess ||
      clusters < 1) {
    cudaGetLastError();
    return 0;
  }
  if (dev >= 0 && dev < 64)
    cached[dev] = clusters;
  return clusters;
}

} // namespace

int rows_gemm_splits(int t, int n, int cols) {
  return rows_gemm_splits_of(t, n, 3 * (int64_t)cols);
}

int rows_gemm_splits_of(int t, int n, int64_t term_cols) {
  const int tiles = ((t + BM - 1) / BM) * ((n + BN - 1) / BN);
  const int k_blocks = (int)(term_cols / BK);
  const int pairs = 74;
  /* the number of runs, up to 12, that leaves the last wave fullest */
  int best = 1;
  double best_fill = 0.0;
  for (int s = 1; s <= 12 && s <= k_blocks; ++s) {
    const int items = tiles * s;
    const double fill = (double)items / (((items + pairs - 1) / pairs) * pairs);
    if (fill > best_fill + 0.02) {
      best_fill = fill;
      best = s;
    }
  }
  return best;
}

size_t rows_gemm_partial_floats(int t, int n, int cols) {
  return (size_t)rows_gemm_splits(t, n, cols) * t * n;
}

const char *rows_gemm(const void *terms, const void *w, int t, int n, int cols,
                      float *partials, int *splits_out, cudaStream_t stream) {
  return rows_gemm_of(terms, 3 * (int64_t)cols, w, cols, t, n, partials, splits_out,
                      stream);
}

const char *rows_gemm_of(const void *terms, int64_t term_cols, const void *w,
                         int64_t w_cols, int t, int n, float *partials,
                         int *splits_out, cudaStream_t stream) {
  if (term_cols % BK != 0 || w_cols % BK != 0)
    return "the multi-position projections need columns in multiples of 64";
  if (allow_dynamic_smem((const void *)rows_gemm_kernel, SMEM_BYTES) != cudaSuccess)
    return "the multi-position GEMM could not get its shared memory";
  CUtensorMap mx, mw;
  if (!make_map_16(&mx, terms, term_cols, t, term_cols, BK, HM, true))
    return "cuTensorMapEncodeTiled refused the activations";
  if (!make_map_16(&mw, w, w_cols, n, w_cols, BK, HN, true))
    return "cuTensorMapEncodeTiled refused the weights";
  RowsGemm g;
  g.t = t;
  g.n = n;
  g.k_blocks = (int)(term_cols / BK);
  g.w_blocks = (int)(w_cols / BK);
  g.splits = rows_gemm_splits_of(t, n, term_cols);
  g.partials = partials;
  *splits_out = g.splits;
  int pairs = resident_pairs();
  if (pairs < 1)
    return "the multi-position GEMM cannot run a cluster of two on this GPU";
  const int items = ((t + BM - 1) / BM) * ((n + BN - 1) / BN) * g.splits;
  if (pairs > items)
    pairs = items;
  const cudaError_t e =
      launch_chained_cluster_smem(rows_gemm_kernel, dim3(2 * pairs), dim3(THREADS), 2,
                                  SMEM_BYTES, stream, mx, mw, g);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char *rows_q4_two_terms(void *out, const void *codes, const void *scales, int n,
                              int cols, cudaStream_t stream) {
  if (cols % 32 != 0 || ((uintptr_t)out & 15))
    return "a Q4_0 matrix has columns in multiples of 32";
  const int64_t words = (int64_t)n * (cols / 8);
  int blocks = (int)((words + 255) / 256);
  if (blocks > 148 * 16)
    blocks = 148 * 16;
  launch_chained(q4_two_terms_kernel, dim3(blocks), dim3(256), 0, stream,
                 (__nv_bfloat16 *)out, (const uint32_t *)codes, (const __half *)scales,
                 words, cols);
  return last_launch("the Q4_0 weights as two bf16 terms");
}

const char *rows_fp8_three_terms(void *out, const void *codes, const void *scales,
                                 int n, int cols, cudaStream_t stream) {
  if (cols % 128 != 0 || (((uintptr_t)out | (uintptr_t)codes) & 15))
    return "an fp8 matrix has columns in multiples of 128";
  const int64_t eights = (int64_t)n * (cols / 8);
  int blocks = (int)((eights + 255) / 256);
  if (blocks > 148 * 16)
    blocks = 148 * 16;
  launch_chained(fp8_three_terms_kernel, dim3(blocks), dim3(256), 0, stream,
                 (__nv_bfloat16 *)out, (const uint2 *)codes, (const float *)scales,
                 eights, cols);
  return last_launch("the fp8 weights as three bf16 terms");
}

const char *rows_spread_terms(void *out, const void *terms, int t, int cols,
                              int segments, const int *from, cudaStream_t stream) {
  if (cols % 8 != 0 || (((uintptr_t)out | (uintptr_t)terms) & 15) || segments < 1 ||
      segments > 8)
    return "terms come in multiples of 8 columns, spread over at most 8 segments";
  SpreadPlan plan{};
  plan.segments = segments;
  for (int s = 0; s < segments; ++s) {
    if (from[s] < 0 || from[s] > 2)
      return "a segment is a copy of term 0, 1 or 2";
    plan.from[s] = from[s];
  }
  const int64_t quads = (int64_t)t * segments * (cols / 8);
  int blocks = (int)((quads + 255) / 256);
  if (blocks > 148 * 16)
    blocks = 148 * 16;
  launch_chained(spread_terms_kernel, dim3(blocks), dim3(256), 0, stream, (uint4 *)out,
                 (const uint4 *)terms, quads, cols, plan);
  return last_launch("the spread terms");
}

const char *rows_norm_terms(void *terms, const float *x, const void *w, int t,
                            int dim, float eps, cudaStream_t stream) {
  launch_chained(norm_terms_kernel, dim3(t), dim3(256), 0, stream,
                 (__nv_bfloat16 *)terms, x, w, dim, eps);
  return last_launch("the multi-position RMSNorm");
}

const char *rows_qkv_finish(const float *partials, int splits, int t, int q_heads,
                            int kv_heads, int hd, const void *bias,
                            const float *cos_t, const float *sin_t,
                            const int32_t *first_pos, float *q_out, float *k_cache,
                            float *v_cache, cudaStream_t stream) {
  if (hd % 8 != 0)
    return "the multi-position RoPE takes head_dim in multiples of 8";
  const int64_t n = (int64_t)t * (q_heads + 2 * kv_heads) * (hd / 8);
  launch_chained(qkv_finish_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                 stream, partials, splits, t, q_heads, kv_heads, hd, bias, cos_t,
                 sin_t, first_pos, q_out, k_cache, v_cache);
  return last_launch("the multi-position RoPE and cache store");
}

const char *rows_residual_finish(float *x, const float *partials, int splits, int t,
                                 int n, cudaStream_t stream) {
  const int64_t count = (int64_t)t * n;
  launch_chained(residual_finish_kernel, dim3((unsigned)((count + 255) / 256)),
                 dim3(256), 0, stream, x, partials, splits, t, n);
  return last_launch("the multi-position residual add");
}

const char *rows_residual_norm(void *terms, float *x, const float *partials,
                               int splits, int t, const void *w, int dim, float eps,
                               cudaStream_t stream) {
  if (dim > 256 * 32)
    return "the fused residual and RMSNorm take rows of at most 8192 values";
  launch_chained(residual_norm_kernel, dim3(t), dim3(256), 0, stream,
                 (__nv_bfloat16 *)terms, x, partials, splits, t, w, dim, eps);
  return last_launch("the multi-position residual add and RMSNorm");
}

const char *rows_swiglu_finish(void *terms, const float *partials, int splits, int t,
                               int hidden, cudaStream_t stream) {
  if (hidden % 8 != 0)
    return "the multi-position SwiGLU takes a hidden size in multiples of 8";
  const int64_t count = (int64_t)t * (hidden / 8);
  launch_chained(swiglu_finish_kernel, dim3((unsigned)((count + 255) / 256)),
                 dim3(256), 0, stream, (__nv_bfloat16 *)terms, partials, splits, t,
                 hidden);
  return last_launch("the multi-position SwiGLU");
}

const char *rows_attention(void *terms, const float *q, const float *k_cache,
                           const float *v_cache, const int32_t *first_pos, int t,
                           int q_heads, int kv_heads, int hd, cudaStream_t stream) {
  if (hd != AD)
    return "the multi-position attention takes head_dim 128";
  if (allow_dynamic_smem((const void *)rows_attention_kernel, ATT_SMEM) !=
      cudaSuccess)
    return "the multi-position attention could not get its shared memory";
  const dim3 grid((t + AQ - 1) / AQ, q_heads);
  launch_chained(rows_attention_kernel, grid, dim3(ATT_THREADS), ATT_SMEM, stream,
                 (__nv_bfloat16 *)terms, q, k_cache, v_cache, first_pos, t, q_heads,
                 kv_heads);
  return last_launch("the multi-position attention");
}

int rows_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_rows_status, sizeof v) != cudaSuccess)
    return -1;
  if (v)
    cudaMemcpyToSymbol(g_rows_status, &zero, sizeof zero);
  return v;
}

} // namespace vxb
