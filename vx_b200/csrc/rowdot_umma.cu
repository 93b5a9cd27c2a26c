/* rowdot_umma.cu -- the decode projections for 8 to 16 sequences per step, on
 * the tensor cores.
 *
 * y[b, r] = sum_c W[r, c] * x[b, c] with bf16 weights and f32 activations is a
 * weight stream for one sequence (rowdot_kernel, nn_kernels.cu), but sixteen
 * sequences need sixteen FMAs per weight and the FP32 pipe cannot follow HBM.
 * The tensor core can: tcgen05.mma with M = 128 weight rows, K = 16, and the
 * sequences on N.  To keep f32 activations, each x is split into three bf16
 * terms x = x1 + x2 + x3 (8 + 8 + 8 mantissa bits, the remainders are exact in
 * f32), so N = 3 * batch columns, every product bf16 x bf16 is exact in f32,
 * and the three partial results are added in the epilogue.  What differs from
 * the FMA kernel is the order of the additions only.
 *
 * Work item = (tile of 128 weight rows, one of S runs of the K dimension); S
 * is chosen per projection so that the items fill whole waves of the 148
 * persistent CTAs.  Roles as in gemm_umma.cu: warp 0 one thread of TMA loads
 * (W: two boxes of 64 rows, so that a tile can take its two halves from
 * different places: gate and up rows, or q/k/v matrices; x terms: one box of
 * N rows) into an 8-stage ring; warp 1 one thread of MMAs into one of four
 * 64-column TMEM accumulators; warps 2-5 the epilogue, which adds the three
 * terms and stores the item's partial sums.  A second, small kernel adds the
 * runs of a tile in run order (so the result does not depend on timing) and
 * applies the projection's epilogue: store, residual add, SwiGLU, or bias +
 * RoPE + KV-cache store (head_dim 128: a tile is one head, and the rotation
 * partners i and i + 64 sit in the two halves of the tile).  (Doing that in
 * the main kernel, by whichever CTA finished a tile last, cost a fence and an
 * atomic round trip per item and made the epilogue warps the bottleneck:
 * 42.8 us per projection on average against 23.1 + 5.7 us this way.)
 */
#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace vxb {

bool make_map_16(CUtensorMap *map, const void *base, int64_t inner, int64_t rows,
                 int64_t ld, int box_inner, int box_rows, bool is_bf16);

namespace {

constexpr int TM = 128, BK = 64, UK = 16;
constexpr int STAGES = 8;
constexpr int A_BYTES = TM * BK * 2; /* 16 KiB */
constexpr int MAX_N = 64;            /* TMEM columns per accumulator */
constexpr int ACCS = 4;
constexpr int THREADS = 192;

enum { RM_LOADER = 0x81, RM_MMA_FULL, RM_MMA_TMEM, RM_EPI_TMEM };

__device__ int g_rowmma_status;

struct Bars {
  uint64_t full[STAGES], empty[STAGES];
  uint64_t tmem_full[ACCS], tmem_empty[ACCS];
  uint32_t tmem_base;
  int stop;
};

/* Device-side view of one projection. */
struct MmaParams {
  int mode;            /* EPI_* of kernels.h's modes: 0 store, 1 add, 3 swiglu, 4 qkv */
  int tiles, splits, k_blocks;
  int rows, cols, batch, n; /* n = columns of the MMA: 3 * batch rounded up to 16 */
  /* where the two 64-row halves of tile t come from: map index and first row */
  int half_rows;       /* rows of w0 before the second source (swiglu with one
                          matrix: hidden; qkv fused: unused) */
  int q_heads, kv_heads;
  int fused;           /* swiglu/qkv: all rows in matrix 0 */
  float *y;
  int64_t y_stride;
  const void *bias;    /* qkv, bf16 */
  const float *cos_t, *sin_t;
  const int32_t *positions;
  float *k_cache, *v_cache;
  int64_t cache_batch_stride;
  float *partials;     /* [splits][batch][tiles * 128] */
  /* the finishing kernel may also leave its output as the three bf16 terms
     that the next projection reads (NULL: no) */
  __nv_bfloat16 *terms;
  int terms_n; /* rows of the term matrix (48 or 32) */
};

/* v as three bf16 terms into rows b, batch + b, 2 batch + b of xs, column i. */
__device__ __forceinline__ void store_terms(__nv_bfloat16 *xs, int cols, int batch,
                                            int b, int i, float v) {
  const __nv_bfloat16 t1 = __float2bfloat16(v);
  const float r1 = v - __bfloat162float(t1);
  const __nv_bfloat16 t2 = __float2bfloat16(r1);
  const float r2 = r1 - __bfloat162float(t2);
  xs[(int64_t)(0 * batch + b) * cols + i] = t1;
  xs[(int64_t)(1 * batch + b) * cols + i] = t2;
  xs[(int64_t)(2 * batch + b) * cols + i] = __float2bfloat16(r2);
}

__device__ __forceinline__ void half_source(const MmaParams &p, int tile, int half,
                                            int &which, int &row0) {
  which = 0;
  if (p.mode == 3) { /* SwiGLU: 64 gate rows, then the 64 up rows of the same units */
    row0 = tile * 64;
    if (half == 1) {
      if (p.fused)
        row0 += p.half_rows;
      else
        which = 1;
    }
  } else if (p.mode == 4 && !p.fused) { /* q, k, v matrices; a tile is a head */
    int head = tile;
    if (head >= p.q_heads + p.kv_heads) {
      which = 2;
      head -= p.q_heads + p.kv_heads;
    } else if (head >= p.q_heads) {
      which = 1;
      head -= p.q_heads;
    }
    row0 = head * 128 + half * 64;
  } else {
    row0 = tile * 128 + half * 64;
  }
}

__device__ __forceinline__ float bf16_val(const void *p, int64_t i) {
  return __uint_as_float((uint32_t)((const uint16_t *)p)[i] << 16);
}

__global__ void __launch_bounds__(THREADS, 1)
rowdot_mma_kernel(const __grid_constant__ CUtensorMap map_w0,
                  const __grid_constant__ CUtensorMap map_w1,
                  const __grid_constant__ CUtensorMap map_w2,
                  const __grid_constant__ CUtensorMap map_x, const MmaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int b_bytes = p.n * BK * 2;
  const int stage_bytes = A_BYTES + ((b_bytes + 1023) & ~1023);
  Bars *bars = reinterpret_cast<Bars *>(smem + STAGES * stage_bytes);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  chain_release();
  const int items = p.tiles * p.splits;
  /* item -> (tile, run of K blocks): runs of a tile are consecutive items */
  auto item_range = [&](int item, int &tile, int &split, int &kb0, int &kb1) {
    tile = item / p.splits;
    split = item - tile * p.splits;
    kb0 = (int)((int64_t)split * p.k_blocks / p.splits);
    kb1 = (int)((int64_t)(split + 1) * p.k_blocks / p.splits);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&bars->full[s], 1);
      ptx::mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < ACCS; ++a) {
      ptx::mbar_init(&bars->tmem_full[a], 1);
      ptx::mbar_init(&bars->tmem_empty[a], 4);
    }
    bars->stop = 0;
    ptx::fence_proxy_async_smem();
    ptx::fence_barrier_init();
  }
  if (warp == 1)
    ptx::tmem_alloc(&bars->tmem_base, ACCS * MAX_N);
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  volatile int *stop = &bars->stop;

  if (warp == 0) {
    /* ---------------------------------------------------------- loader */
    if (lane == 0) {
      ptx::tma_prefetch_desc(&map_w0);
      ptx::tma_prefetch_desc(&map_x);
      int it = 0;
      bool ok = true;
      /* This block's (item, K block) pairs in order. */
      int cur_item = blockIdx.x, cur_kb = 0, cur_kb1 = 0;
      bool opened = false;
      int which[2] = {0, 0}, row0[2] = {0, 0};
      auto next_block = [&](int &kb_out) -> bool {
        for (;;) {
          if (!opened) {
            if (cur_item >= items)
              return false;
            int tile, split, kb0;
            item_range(cur_item, tile, split, kb0, cur_kb1);
            half_source(p, tile, 0, which[0], row0[0]);
            half_source(p, tile, 1, which[1], row0[1]);
            cur_kb = kb0;
            opened = true;
          }
          if (cur_kb < cur_kb1) {
            kb_out = cur_kb++;
            return true;
          }
          opened = false;
          cur_item += gridDim.x;
        }
      };
      auto load_weights = [&](int s, int kb) {
        uint8_t *sa = smem + s * stage_bytes;
        ptx::mbar_expect_tx(&bars->full[s], A_BYTES + b_bytes);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const CUtensorMap *m = which[h] == 0 ? &map_w0
                                 : which[h] == 1 ? &map_w1 : &map_w2;
          ptx::tma_load_2d(sa + h * (A_BYTES / 2), m, kb * BK, row0[h],
                           &bars->full[s]);
        }
      };
      /* The weights do not depend on the kernel before; the x terms do: the
         whole ring of weights is asked for first, then the wait, then the
         terms of those stages. */
      int kbs[STAGES];
      int kb = 0;
      while (it < STAGES && next_block(kb)) {
        load_weights(it, kb);
        kbs[it++] = kb;
      }
      chain_wait();
      for (int s = 0; s < it; ++s)
        ptx::tma_load_2d(smem + s * stage_bytes + A_BYTES, &map_x, kbs[s] * BK, 0,
                         &bars->full[s]);
      while (ok && next_block(kb)) {
        const int s = it % STAGES;
        if (!ptx::mbar_wait(&bars->empty[s], ((it / STAGES) & 1) ^ 1, stop)) {
          atomicCAS(&g_rowmma_status, 0, RM_LOADER);
          *stop = 1;
          ok = false;
          break;
        }
        load_weights(s, kb);
        ptx::tma_load_2d(smem + s * stage_bytes + A_BYTES, &map_x, kb * BK, 0,
                         &bars->full[s]);
        ++it;
      }
      for (int back = 0; back < STAGES && back < it; ++back) {
        const int j = it - 1 - back;
        ptx::mbar_wait_alone(&bars->full[j % STAGES], (j / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    /* ------------------------------------------------------ MMA issuer */
    if (lane == 0) {
      const uint32_t idesc = ptx::idesc_f16(true, false, false, TM, p.n);
      int it = 0, t = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < items; item += gridDim.x, ++t) {
        int tile, split, kb0, kb1;
        item_range(item, tile, split, kb0, kb1);
        const int acc = t % ACCS;
        if (!ptx::mbar_wait(&bars->tmem_empty[acc], ((t / ACCS) & 1) ^ 1, stop)) {
          atomicCAS(&g_rowmma_status, 0, RM_MMA_TMEM);
          *stop = 1;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem + acc * MAX_N;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          if (!ptx::mbar_wait(&bars->full[s], (it / STAGES) & 1, stop)) {
            atomicCAS(&g_rowmma_status, 0, RM_MMA_FULL);
            *stop = 1;
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t sa = ptx::smem_addr(smem + s * stage_bytes);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UK; ++kk)
            ptx::umma_f16_ss(d_tmem, ptx::smem_desc_sw128(sa + kk * UK * 2, 16, 1024),
                             ptx::smem_desc_sw128(sb + kk * UK * 2, 16, 1024), idesc,
                             (kb != kb0) || kk != 0);
          ptx::umma_commit(&bars->empty[s]);
        }
        if (ok)
          ptx::umma_commit(&bars->tmem_full[acc]);
      }
    }
  } else {
    /* ---------------------------------------------------------- epilogue
       Four warps, a weight row per thread. */
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane; /* row within the tile */
    const int B = p.batch;
    int t = 0;
    for (int item = blockIdx.x; item < items; item += gridDim.x, ++t) {
      int tile, split, kb0, kb1;
      item_range(item, tile, split, kb0, kb1);
      const int acc = t % ACCS;
      if (!ptx::mbar_wait(&bars->tmem_full[acc], (t / ACCS) & 1, stop)) {
        atomicCAS(&g_rowmma_status, 0, RM_EPI_TMEM);
        *stop = 1;
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + acc * MAX_N;
      float sum[16]; /* per sequence: the three terms added, high to low */
      {
        uint32_t v[MAX_N];
        ptx::tmem_ld_32x32b_x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
        ptx::tmem_ld_32x32b_x32(taddr + 32,
                                *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
        ptx::tmem_ld_wait();
#pragma unroll
        for (int b = 0; b < 16; ++b)
          sum[b] = 0.0f;
        if (B == 16) {
#pragma unroll
          for (int b = 0; b < 16; ++b)
            sum[b] = (__uint_as_float(v[b]) + __uint_as_float(v[16 + b])) +
                     __uint_as_float(v[32 + b]);
        } else { /* 8 */
#pragma unroll
          for (int b = 0; b < 8; ++b)
            sum[b] = (__uint_as_float(v[b]) + __uint_as_float(v[8 + b])) +
                     __uint_as_float(v[16 + b]);
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        ptx::mbar_arrive(&bars->tmem_empty[acc]);

      /* this run's part of the tile; proj_finish_kernel adds the runs */
      const int64_t padded_rows = (int64_t)p.tiles * TM;
      float *mine = p.partials + ((int64_t)split * B) * padded_rows + tile * TM + r;
#pragma unroll
      for (int b = 0; b < 16; ++b)
        if (b < B)
          mine[b * padded_rows] = sum[b];
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem, ACCS * MAX_N);
  }
}

/* The runs of K added in run order (so the result does not depend on
   timing), then the projection's own epilogue. One thread per sequence and
   per output row (modes 0, 1), SwiGLU unit (mode 3) or rotation pair (mode 4). */
__global__ void __launch_bounds__(256)
proj_finish_kernel(const MmaParams p) {
  chain_release();
  chain_wait();
  const int B = p.batch;
  const int64_t padded_rows = (int64_t)p.tiles * TM;
  const int per_seq = p.mode == 0 || p.mode == 1 ? p.rows : p.tiles * 64;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)per_seq * B)
    return;
  const int b = (int)(idx / per_seq), e = (int)(idx - (int64_t)b * per_seq);
  /* the value of padded row `row`, all runs */
  auto total = [&](int64_t row) {
    const float *at = p.partials + (int64_t)b * padded_rows + row;
    float v[16];
#pragma unroll
    for (int s = 0; s < 16; ++s)
      v[s] = s < p.splits ? __ldcg(at + (int64_t)s * B * padded_rows) : 0.0f;
    float t = 0.0f;
#pragma unroll
    for (int s = 0; s < 16; ++s)
      if (s < p.splits)
        t += v[s];
    return t;
  };
  if (p.mode == 0 || p.mode == 1) {
    float *y = p.y + b * p.y_stride + e;
    const float t = total(e);
    *y = p.mode == 1 ? *y + t : t;
    return;
  }
  const int tile = e / 64, r = e - tile * 64;
  const float lo = total((int64_t)tile * TM + r), hi = total((int64_t)tile * TM + r + 64);
  if (p.mode == 3) {
    if (e < p.rows) { /* nn_swiglu (nn.vx:169-209): g / (1 + e^-g) * u */
      const float h = lo / (1.0f + expf(0.0f - lo)) * hi;
      p.y[b * p.y_stride + e] = h;
      if (p.terms) {
        store_terms(p.terms, p.rows, B, b, e, h);
        if (b == 0)
          for (int row = 3 * B; row < p.terms_n; ++row)
            p.terms[(int64_t)row * p.rows + e] = __float2bfloat16(0.0f);
      }
    }
    return;
  }
  /* q/k/v: tile = head; pairs (r, r + 64), nn_rope_and_store (nn.vx:245-280) */
  const int head = tile;
  const int kind = head < p.q_heads ? 0 : (head < p.q_heads + p.kv_heads ? 1 : 2);
  const int local = kind == 0 ? head
                    : kind == 1 ? head - p.q_heads
                                : head - p.q_heads - p.kv_heads;
  float va = lo, vb = hi;
  if (p.bias) {
    va += bf16_val(p.bias, (int64_t)head * 128 + r);
    vb += bf16_val(p.bias, (int64_t)head * 128 + r + 64);
  }
  const int pos = p.positions[b];
  if (kind == 2) {
    float *vrow = p.v_cache + b * p.cache_batch_stride +
                  ((int64_t)pos * p.kv_heads + local) * 128;
    vrow[r] = va;
    vrow[r + 64] = vb;
    return;
  }
  const float c = p.cos_t[(int64_t)pos * 64 + r];
  const float sn = p.sin_t[(int64_t)pos * 64 + r];
  float *dst = kind == 0 ? p.y + b * p.y_stride + (int64_t)local * 128
                         : p.k_cache + b * p.cache_batch_stride +
                               ((int64_t)pos * p.kv_heads + local) * 128;
  dst[r] = __fsub_rn(__fmul_rn(va, c), __fmul_rn(vb, sn));
  dst[r + 64] = __fadd_rn(__fmul_rn(vb, c), __fmul_rn(va, sn));
}

/* x (f32, optionally RMS-normalised first: nn_rms_norm, nn.vx:212-239) as three
   bf16 terms: row p * batch + b of xs holds term p of sequence b; rows from
   3 * batch up to n are zero. Block (b, chunk) writes 1024 columns of sequence
   b (blockIdx.x >= batch: of the zero rows); each block of a normalised row
   takes the row's sum of squares itself, in the same order. */
__global__ void __launch_bounds__(1024)
split3_kernel(__nv_bfloat16 *xs, const float *x, int64_t x_stride, int cols,
              int batch, int n, const void *norm_w, float eps) {
  __shared__ float red[32];
  chain_release();
  chain_wait();
  const int b = blockIdx.x;
  const int i = blockIdx.y * 1024 + threadIdx.x;
  if (b >= batch) { /* padding rows */
    if (i < cols)
      for (int row = 3 * batch; row < n; ++row)
        xs[(int64_t)row * cols + i] = __float2bfloat16(0.0f);
    return;
  }
  const float *xr = x + b * x_stride;
  float inv = 1.0f;
  if (norm_w) {
    float ss = 0.0f;
    for (int j = threadIdx.x; j < cols; j += blockDim.x)
      ss = fmaf(xr[j], xr[j], ss);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0)
      red[warp] = ss;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) /* fixed order */
      t += red[w];
    inv = 1.0f / sqrtf(t / (float)cols + eps);
  }
  if (i < cols) {
    float v = xr[i];
    if (norm_w)
      v = v * inv * bf16_val(norm_w, i);
    const __nv_bfloat16 t1 = __float2bfloat16(v);
    const float r1 = v - __bfloat162float(t1);
    const __nv_bfloat16 t2 = __float2bfloat16(r1);
    const float r2 = r1 - __bfloat162float(t2);
    const __nv_bfloat16 t3 = __float2bfloat16(r2);
    xs[(int64_t)(0 * batch + b) * cols + i] = t1;
    xs[(int64_t)(1 * batch + b) * cols + i] = t2;
    xs[(int64_t)(2 * batch + b) * cols + i] = t3;
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

/* The smallest number of K runs that fills the CTAs' waves to 95 %, else the
   best there is; a run keeps at least four K blocks. */
int pick_splits(int tiles, int k_blocks, int ctas) {
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= 16 && k_blocks / s >= 4; ++s) {
    const int items = tiles * s;
    const double eff = (double)items / (((items + ctas - 1) / ctas) * (double)ctas);
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best = s;
    }
    if (eff >= 0.95)
      return s;
  }
  return best;
}

} // namespace

const char *batched_proj_refusal(const BatchedProj &a) {
  if (a.batch != 8 && a.batch != 16)
    return "the tensor-core projections take 8 or 16 sequences";
  if (a.cols % 64 != 0)
    return "the number of columns must be a multiple of 64";
  if (a.mode == 4 && a.head_dim != 128)
    return "q/k/v on the tensor cores needs head_dim 128";
  if (a.mode == 3 && a.rows % 64 != 0)
    return "SwiGLU on the tensor cores needs a multiple of 64 units";
  if (a.mode != 0 && a.mode != 1 && a.mode != 3 && a.mode != 4)
    return "unknown mode";
  return nullptr;
}

size_t batched_proj_scratch_floats(int rows_max, int batch) {
  /* up to 16 runs of [batch][rows rounded up to 128] */
  return (size_t)16 * batch * ((rows_max + 127) / 128 * 128);
}

const char *batched_proj(const BatchedProj &a, cudaStream_t stream) {
  if (const char *why = batched_proj_refusal(a))
    return why;
  const int n = (3 * a.batch + 15) / 16 * 16;
  /* the activations' three terms, unless the projection before left them */
  if (!a.x_terms_ready)
    launch_chained(split3_kernel,
                 dim3(a.batch + (n > 3 * a.batch ? 1 : 0), (a.cols + 1023) / 1024),
                 dim3(1024), 0, stream, (__nv_bfloat16 *)a.xs, a.x, a.x_stride, a.cols, a.batch,
                 n, a.norm_w, a.eps);
  MmaParams p{};
  p.mode = a.mode;
  p.rows = a.rows;
  p.cols = a.cols;
  p.batch = a.batch;
  p.n = n;
  p.k_blocks = a.cols / BK;
  p.q_heads = a.q_heads;
  p.kv_heads = a.kv_heads;
  p.y = a.y;
  p.y_stride = a.y_stride;
  p.bias = a.bias;
  p.cos_t = a.cos_t;
  p.sin_t = a.sin_t;
  p.positions = a.positions;
  p.k_cache = a.k_cache;
  p.v_cache = a.v_cache;
  p.cache_batch_stride = a.cache_batch_stride;
  p.partials = a.scratch;
  p.terms = a.next_terms ? (__nv_bfloat16 *)a.xs : nullptr;
  p.terms_n = a.next_terms ? (3 * a.batch + 15) / 16 * 16 : 0;
  if (a.next_terms && a.mode != 3)
    return "only the SwiGLU projection can leave terms";
  int64_t rows0 = a.rows, rows1 = 0, rows2 = 0; /* rows of the three matrices */
  if (a.mode == 3) {
    p.tiles = a.rows / 64;
    p.fused = a.w1 == nullptr;
    p.half_rows = a.rows;
    rows0 = p.fused ? 2 * (int64_t)a.rows : a.rows;
    rows1 = a.rows;
  } else if (a.mode == 4) {
    p.tiles = a.q_heads + 2 * a.kv_heads;
    p.fused = a.w1 == nullptr;
    rows0 = p.fused ? (int64_t)p.tiles * 128 : (int64_t)a.q_heads * 128;
    rows1 = rows2 = (int64_t)a.kv_heads * 128;
  } else {
    p.tiles = (a.rows + TM - 1) / TM;
  }
  p.splits = pick_splits(p.tiles, p.k_blocks, sm_count());
  CUtensorMap m0, m1, m2, mx;
  if (!make_map_16(&m0, a.w0, a.cols, rows0, a.cols, 64, 64, true))
    return "cuTensorMapEncodeTiled refused the weights";
  m1 = m2 = m0;
  if (a.w1 && !make_map_16(&m1, a.w1, a.cols, rows1, a.cols, 64, 64, true))
    return "cuTensorMapEncodeTiled refused the second weight matrix";
  if (a.w2 && !make_map_16(&m2, a.w2, a.cols, rows2, a.cols, 64, 64, true))
    return "cuTensorMapEncodeTiled refused the third weight matrix";
  if (!make_map_16(&mx, a.xs, a.cols, n, a.cols, 64, n, true))
    return "cuTensorMapEncodeTiled refused the activations";
  const int b_bytes = n * BK * 2;
  const int stage_bytes = A_BYTES + ((b_bytes + 1023) & ~1023);
  const size_t smem = (size_t)STAGES * stage_bytes + 1024 + sizeof(Bars) + 64;
  if (allow_dynamic_smem((const void *)rowdot_mma_kernel,
                         STAGES * (A_BYTES + 8192) + 1024 + (int)sizeof(Bars) +
                             64) != cudaSuccess)
    return "the batched projection could not get its shared memory";
  const int items = p.tiles * p.splits;
  const int ctas = items < sm_count() ? items : sm_count();
  launch_chained(rowdot_mma_kernel, dim3(ctas), dim3(THREADS), smem, stream, m0, m1,
                 m2, mx, p);
  const int64_t outputs =
      (int64_t)a.batch * (p.mode == 0 || p.mode == 1 ? p.rows : p.tiles * 64);
  launch_chained(proj_finish_kernel, dim3((unsigned)((outputs + 255) / 256)),
                 dim3(256), 0, stream, p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    static thread_local char msg[160];
    snprintf(msg, sizeof msg, "the batched projection launch: %s",
             cudaGetErrorString(e));
    return msg;
  }
  return nullptr;
}

int batched_proj_status(cudaStream_t stream) {
  int v = 0, zero = 0;
  if (cudaStreamSynchronize(stream) != cudaSuccess)
    return -1;
  if (cudaMemcpyFromSymbol(&v, g_rowmma_status, sizeof v) != cudaSuccess)
    return -1;
  if (v)
    cudaMemcpyToSymbol(g_rowmma_status, &zero, sizeof zero);
  return v;
}

} // namespace vxb
