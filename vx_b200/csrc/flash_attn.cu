/* flash_attn.cu -- attention forward over whole sequences, bf16 in and out,
 * on the sm_100a tensor cores: out = softmax(q k^T * scale [causal]) v with
 * an f32 online softmax, never materialising the S x S scores.
 *
 * The arithmetic is the reference's attention (scores * scale, subtract the
 * running maximum, exponentiate, weighted sum of V over the sum of weights:
 * tests/optimizations/pass/std_nn_kernels_match_loops_on_the_cpu.vx:347-390)
 * applied to every query row, with the probabilities rounded to bf16 before
 * they multiply V, as every tensor-core flash attention does.
 *
 * One CTA owns NQ (1 or 2) tiles of 128 query rows of one (batch, head) and
 * walks the KV sequence in tiles of 64 rows:
 *   warp 0        TMA: the Q tiles once, then K and V tiles into a 3-deep ring;
 *   warp 1        one thread issues tcgen05.mma: S = Q K^T (128x64, K = 128)
 *                 into one of two TMEM score buffers per Q tile, and
 *                 O += P V (128x128, K = 64) into the Q tile's TMEM accumulator;
 *                 S of tile j is issued before P V of tile j-1, so the tensor
 *                 core has work while the softmax of tile j-1 runs;
 *   warps 2..     one warpgroup per Q tile, one thread per query row: read S
 *                 from TMEM, running max / sum in the exp2 domain, write P as
 *                 bf16 into 128-byte-swizzled shared memory for the P V
 *                 product.  O is rescaled (TMEM load, multiply, store) only
 *                 when a row's maximum has grown by more than 2^8 since the
 *                 value in use, which is rare after the first tile; the final
 *                 division by the row sum makes the result independent of the
 *                 maximum in use.
 * With NQ = 2 the two warpgroups alternate on the tensor core, which hides
 * most of the softmax time, and K/V tiles are read once for 256 query rows.
 */
#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>

#include <cstdlib>
#include <mutex>

namespace vxb {

bool make_map_16(CUtensorMap *map, const void *base, int64_t inner, int64_t rows,
                 int64_t ld, int box_inner, int box_rows, bool is_bf16);
const char *flash_attention_fwd_v2(const void *q, const void *k, const void *v,
                                   void *out, int B, int H, int S, float scale,
                                   bool causal, cudaStream_t stream);
int flash2_status();

namespace {

constexpr int HD = 128;       /* head_dim */
constexpr int BQ = 128;       /* query rows per tile */
constexpr int BKV = 64;       /* KV rows per tile */
constexpr int KV_STAGES = 3;
constexpr int Q_BYTES = BQ * HD * 2;        /* 32 KiB, two 16 KiB boxes */
constexpr int K_BYTES = BKV * HD * 2;       /* 16 KiB, two 8 KiB boxes  */
constexpr int KV_STAGE_BYTES = 2 * K_BYTES; /* K then V */
constexpr int P_BYTES = BQ * BKV * 2;       /* 16 KiB */

enum { FS_Q = 0x41, FS_KV_FREE = 0x42, FS_KV_FULL = 0x43, FS_S_FREE = 0x44,
       FS_P_FULL = 0x45, FS_S_FULL = 0x46, FS_PV_DONE = 0x47 };

__device__ int g_flash_status;

template <int NQ> struct FlashBars {
  uint64_t q_full;
  uint64_t kv_full[KV_STAGES];
  uint64_t kv_free[KV_STAGES];
  uint64_t s_full[NQ][2];
  uint64_t s_free[NQ][2];
  uint64_t p_full[NQ];
  uint64_t pv_done[NQ];
  uint32_t tmem_base;
  int stop;
  float xmax[NQ][2][2][BQ]; /* [tile][parity][half][row]: a half's row max */
  float xsum[NQ][2][BQ];    /* [tile][half][row]: a half's row sum */
};

template <int NQ> constexpr int flash_smem_bytes() {
  return NQ * Q_BYTES + KV_STAGES * KV_STAGE_BYTES + NQ * P_BYTES + 1024 +
         (int)sizeof(FlashBars<NQ>) + 256;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#define FLASH_GIVE_UP(code)                                                    \
  do {                                                                         \
    atomicCAS(&g_flash_status, 0, (code));                                     \
    *stop = 1;                                                                 \
  } while (0)

template <int NQ>
__global__ void __launch_bounds__(64 + NQ * 256, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap map_q,
                 const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v,
                 __nv_bfloat16 *__restrict__ out, int S, float scale_log2,
                 int causal) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *sm_q = smem;
  uint8_t *sm_kv = sm_q + NQ * Q_BYTES;
  uint8_t *sm_p = sm_kv + KV_STAGES * KV_STAGE_BYTES;
  FlashBars<NQ> *bars = reinterpret_cast<FlashBars<NQ> *>(sm_p + NQ * P_BYTES);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  /* Heavy (late) query tiles first: under a causal mask they have the most KV
     tiles, and the tail of the grid should be the cheap ones. */
  const int q_block = gridDim.x - 1 - blockIdx.x;
  const int q_base = q_block * BQ * NQ;           /* first query row of CTA */
  const int64_t head_row = (int64_t)blockIdx.y * S; /* row of this head in the
                                                       [B*H*S, D] view */
  int n_tiles[NQ], n_max = 0;
#pragma unroll
  for (int w = 0; w < NQ; ++w) {
    n_tiles[w] = causal ? (q_base + w * BQ + BQ) / BKV : S / BKV;
    n_max = max(n_max, n_tiles[w]);
  }

  if (threadIdx.x == 0) {
    ptx::mbar_init(&bars->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      ptx::mbar_init(&bars->kv_full[s], 1);
      ptx::mbar_init(&bars->kv_free[s], 1);
    }
    for (int w = 0; w < NQ; ++w) {
      for (int b = 0; b < 2; ++b) {
        ptx::mbar_init(&bars->s_full[w][b], 1);
        ptx::mbar_init(&bars->s_free[w][b], 8);
      }
      ptx::mbar_init(&bars->p_full[w], 8);
      ptx::mbar_init(&bars->pv_done[w], 1);
    }
    bars->stop = 0;
    ptx::fence_proxy_async_smem();
    ptx::fence_barrier_init();
  }
  if (warp == 1)
    ptx::tmem_alloc(&bars->tmem_base, 512);
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  volatile int *stop = &bars->stop;

  if (warp == 0) {
    /* ------------------------------------------------------------ loader */
    if (lane == 0) {
      ptx::tma_prefetch_desc(&map_q);
      ptx::tma_prefetch_desc(&map_k);
      ptx::tma_prefetch_desc(&map_v);
      ptx::mbar_expect_tx(&bars->q_full, NQ * Q_BYTES);
      for (int w = 0; w < NQ; ++w)
        for (int h = 0; h < 2; ++h)
          ptx::tma_load_2d(sm_q + w * Q_BYTES + h * (Q_BYTES / 2), &map_q,
                           h * 64, (int)(head_row + q_base + w * BQ),
                           &bars->q_full);
      int issued = 0;
      for (int j = 0; j < n_max; ++j, ++issued) {
        const int s = j % KV_STAGES;
        if (!ptx::mbar_wait(&bars->kv_free[s], ((j / KV_STAGES) & 1) ^ 1, stop)) {
          FLASH_GIVE_UP(FS_KV_FREE);
          break;
        }
        uint8_t *dst = sm_kv + s * KV_STAGE_BYTES;
        ptx::mbar_expect_tx(&bars->kv_full[s], KV_STAGE_BYTES);
        const int row = (int)(head_row + j * BKV);
        for (int h = 0; h < 2; ++h) {
          ptx::tma_load_2d(dst + h * (K_BYTES / 2), &map_k, h * 64, row,
                           &bars->kv_full[s]);
          ptx::tma_load_2d(dst + K_BYTES + h * (K_BYTES / 2), &map_v, h * 64,
                           row, &bars->kv_full[s]);
        }
      }
      /* Stay until every copy this thread started has landed. */
      ptx::mbar_wait_alone(&bars->q_full, 0);
      for (int back = 0; back < KV_STAGES && back < issued; ++back) {
        const int j = issued - 1 - back;
        ptx::mbar_wait_alone(&bars->kv_full[j % KV_STAGES],
                             (j / KV_STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    /* -------------------------------------------------------- MMA issuer */
    if (lane == 0) {
      const uint32_t idesc_s = ptx::idesc_f16(true, false, false, BQ, BKV);
      const uint32_t idesc_o = ptx::idesc_f16(true, false, true, BQ, HD);
      bool ok = ptx::mbar_wait(&bars->q_full, 0, stop);
      if (!ok)
        FLASH_GIVE_UP(FS_Q);
      ptx::tc_fence_after_sync();
      for (int j = 0; ok && j <= n_max; ++j) {
        if (j < n_max) {
          const int s = j % KV_STAGES;
          if (!ptx::mbar_wait(&bars->kv_full[s], (j / KV_STAGES) & 1, stop)) {
            FLASH_GIVE_UP(FS_KV_FULL);
            break;
          }
          const uint32_t k_addr = ptx::smem_addr(sm_kv + s * KV_STAGE_BYTES);
          for (int w = 0; w < NQ && ok; ++w) {
            if (j >= n_tiles[w])
              continue;
            const int buf = j & 1;
            if (!ptx::mbar_wait(&bars->s_free[w][buf], ((j >> 1) & 1) ^ 1,
                                stop)) {
              FLASH_GIVE_UP(FS_S_FREE);
              ok = false;
              break;
            }
            ptx::tc_fence_after_sync();
            const uint32_t q_addr = ptx::smem_addr(sm_q + w * Q_BYTES);
            const uint32_t d_tmem = tmem + w * 256 + buf * BKV;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
              const uint64_t da = ptx::smem_desc_sw128(
                  q_addr + (kk / 4) * (Q_BYTES / 2) + (kk % 4) * 32, 16, 1024);
              const uint64_t db = ptx::smem_desc_sw128(
                  k_addr + (kk / 4) * (K_BYTES / 2) + (kk % 4) * 32, 16, 1024);
              ptx::umma_f16_ss(d_tmem, da, db, idesc_s, kk != 0);
            }
            ptx::umma_commit(&bars->s_full[w][buf]);
          }
        }
        if (ok && j >= 1) {
          const int jj = j - 1, s = jj % KV_STAGES;
          const uint32_t v_addr =
              ptx::smem_addr(sm_kv + s * KV_STAGE_BYTES + K_BYTES);
          for (int w = 0; w < NQ && ok; ++w) {
            if (jj >= n_tiles[w])
              continue;
            if (!ptx::mbar_wait(&bars->p_full[w], jj & 1, stop)) {
              FLASH_GIVE_UP(FS_P_FULL);
              ok = false;
              break;
            }
            ptx::tc_fence_after_sync();
            const uint32_t p_addr = ptx::smem_addr(sm_p + w * P_BYTES);
            const uint32_t o_tmem = tmem + w * 256 + 128;
#pragma unroll
            for (int kk = 0; kk < BKV / 16; ++kk) {
              /* P: K-major, one 128-byte row per query row. V: N-major, two
                 64-column blocks 8 KiB apart, 8-row groups 1 KiB apart; a K
                 step is 16 KV rows. */
              const uint64_t da =
                  ptx::smem_desc_sw128(p_addr + kk * 32, 16, 1024);
              const uint64_t db = ptx::smem_desc_sw128(v_addr + kk * 16 * 128,
                                                       K_BYTES / 2, 1024);
              ptx::umma_f16_ss(o_tmem, da, db, idesc_o, (jj | kk) != 0);
            }
            ptx::umma_commit(&bars->pv_done[w]);
          }
          if (ok)
            ptx::umma_commit(&bars->kv_free[s]);
        }
      }
    }
  } else {
    /* ------------------------------------------------ softmax warpgroups
       Eight warps per Q tile: two threads share a query row, each with 32 of
       the tile's 64 KV columns (and 64 of the 128 output columns). They agree
       on the row maximum through shared memory once per tile; their partial
       row sums meet only at the end. */
    const int w = (warp - 2) / 8;          /* which Q tile */
    const int half = ((warp - 2) & 7) / 4; /* which 32 KV columns */
    const int quarter = warp & 3;          /* TMEM lanes this warp may touch */
    const int row = quarter * 32 + lane;   /* row within the Q tile */
    const int q_row = q_base + w * BQ + row;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_tmem = tmem + lane_base + w * 256 + half * 32;
    const uint32_t o_tmem = tmem + lane_base + w * 256 + 128 + half * 64;
    uint8_t *p_row = sm_p + w * P_BYTES + row * 128;
    const int n_mine = n_tiles[w];
    float m_used = -INFINITY, l_sum = 0.0f;
    bool ok = true;

    for (int j = 0; j < n_mine; ++j) {
      const int buf = j & 1;
      if (ok && !ptx::mbar_wait(&bars->s_full[w][buf], (j >> 1) & 1, stop)) {
        FLASH_GIVE_UP(FS_S_FULL);
        ok = false;
      }
      if (!ok) {
        /* Gave up: keep meeting the partner at the tile's barrier. */
        asm volatile("bar.sync %0, %1;" ::"r"(1 + w), "r"(256) : "memory");
        continue;
      }
      ptx::tc_fence_after_sync();
      uint32_t raw[32];
      ptx::tmem_ld_32x32b_x32(s_tmem + buf * BKV, raw);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        ptx::mbar_arrive(&bars->s_free[w][buf]);

      const int k0 = j * BKV + half * 32;
      const bool diagonal = causal && j * BKV + BKV - 1 > q_base + w * BQ;
      /* Raw scores; the scale (positive) is folded into the exponent's FMA.
         Four running maxima keep the chain short. */
      float sv[32];
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float v = __uint_as_float(raw[c]);
        if (diagonal && k0 + c > q_row)
          v = -INFINITY;
        sv[c] = v;
        mx4[c & 3] = fmaxf(mx4[c & 3], v);
      }
      const float mine = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      bars->xmax[w][buf][half][row] = mine;
      asm volatile("bar.sync %0, %1;" ::"r"(1 + w), "r"(256) : "memory");
      const float mx = fmaxf(mine, bars->xmax[w][buf][half ^ 1][row]) * scale_log2;
      /* Keep the maximum in use unless the new one is more than 2^8 above it. */
      const bool grow = mx > m_used + 8.0f;
      const float m_new = grow ? mx : m_used;
      const float fix = grow ? ex2(m_used - m_new) : 1.0f;

      if (j > 0) {
        if (!ptx::mbar_wait(&bars->pv_done[w], (j - 1) & 1, stop)) {
          FLASH_GIVE_UP(FS_PV_DONE);
          ok = false;
          continue;
        }
        ptx::tc_fence_after_sync();
        if (__any_sync(0xffffffffu, grow)) {
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t o[32];
            ptx::tmem_ld_32x32b_x32(o_tmem + c * 32, o);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e)
              o[e] = __float_as_uint(__uint_as_float(o[e]) * fix);
            uint32_t lo[16], hi[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              lo[e] = o[e];
              hi[e] = o[16 + e];
            }
            ptx::tmem_st_32x32b_x16(o_tmem + c * 32, lo);
            ptx::tmem_st_32x32b_x16(o_tmem + c * 32 + 16, hi);
          }
          ptx::tmem_st_wait();
        }
      }
      m_used = m_new;

      /* p = 2^(s * scale - m); the row sum adds the f32 weights in four
         independent chains, the bf16 copies go to the P V product. */
      float part4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      uint32_t packed[16];
      const float neg_m = -m_used;
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const float p0 = ex2(fmaf(sv[c], scale_log2, neg_m));
        const float p1 = ex2(fmaf(sv[c + 1], scale_log2, neg_m));
        part4[(c >> 1) & 3] += p0 + p1;
        const __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
        packed[c >> 1] = *reinterpret_cast<const uint32_t *>(&pr);
      }
      const float part = (part4[0] + part4[1]) + (part4[2] + part4[3]);
      l_sum = l_sum * fix + part;
      /* Row r of P is one 128-byte swizzle row: 16-byte chunk c sits at chunk
         position c ^ (r % 8). This thread has chunks 4*half .. 4*half + 3. */
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 v = make_uint4(packed[c * 4], packed[c * 4 + 1],
                                   packed[c * 4 + 2], packed[c * 4 + 3]);
        *reinterpret_cast<uint4 *>(p_row + (((half * 4 + c) ^ (row & 7)) << 4)) = v;
      }
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        ptx::mbar_arrive(&bars->p_full[w]);
    }

    /* The two halves of a row add their sums; a warpgroup that gave up still
       comes to the barrier so that its partner does not wait for it. */
    bars->xsum[w][half][row] = l_sum;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + w), "r"(256) : "memory");
    l_sum += bars->xsum[w][half ^ 1][row];
    if (ok && n_mine > 0) {
      if (!ptx::mbar_wait(&bars->pv_done[w], (n_mine - 1) & 1, stop)) {
        FLASH_GIVE_UP(FS_PV_DONE);
      } else {
        ptx::tc_fence_after_sync();
        const float inv = 1.0f / l_sum;
        __nv_bfloat16 *dst =
            out + ((int64_t)head_row + q_row) * HD + half * 64;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t o[32];
          ptx::tmem_ld_32x32b_x32(o_tmem + c * 32, o);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __nv_bfloat162 pr = __floats2bfloat162_rn(
                  __uint_as_float(o[q4 * 8 + 2 * e]) * inv,
                  __uint_as_float(o[q4 * 8 + 2 * e + 1]) * inv);
              pk[e] = *reinterpret_cast<const uint32_t *>(&pr);
            }
            *reinterpret_cast<uint4 *>(dst + c * 32 + q4 * 8) =
                make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem, 512);
  }
}

template <int NQ>
const char *launch_flash(const CUtensorMap &mq, const CUtensorMap &mk,
                         const CUtensorMap &mv, void *out, int B, int H, int S,
                         float scale, bool causal, cudaStream_t stream) {
  if (allow_dynamic_smem((const void *)flash_fwd_kernel<NQ>,
                         flash_smem_bytes<NQ>()) != cudaSuccess)
    return "flash attention could not get its shared memory";
  const dim3 grid(S / (BQ * NQ), B * H);
  flash_fwd_kernel<NQ><<<grid, 64 + NQ * 256, flash_smem_bytes<NQ>(), stream>>>(
      mq, mk, mv, (__nv_bfloat16 *)out, S, scale * 1.4426950408889634f,
      causal ? 1 : 0);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

} // namespace

const char *flash_attention_fwd(const void *q, const void *k, const void *v,
                                void *out, int B, int H, int S, int D,
                                float scale, bool causal, cudaStream_t stream) {
  if (D != HD)
    return "flash attention is built for head_dim 128";
  if (B <= 0 || H <= 0 || S <= 0)
    return nullptr;
  if (S % BQ != 0)
    return "the sequence length must be a multiple of 128";
  if ((int64_t)B * H > 65535)
    return "more than 65535 (batch, head) pairs";
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15)
    return "q, k, v and out must be 16-byte aligned";
  const int64_t rows = (int64_t)B * H * S;
  CUtensorMap mq, mk, mv;
  if (!make_map_16(&mq, q, HD, rows, HD, 64, BQ, true) ||
      !make_map_16(&mk, k, HD, rows, HD, 64, BKV, true) ||
      !make_map_16(&mv, v, HD, rows, HD, 64, BKV, true))
    return "cuTensorMapEncodeTiled refused q, k or v";
  if (S % (2 * BQ) == 0) {
    /* Sequences that are whole pairs of Q tiles take the second kernel
       (flash_attn_v2.cu); VXB_FLASH_V1=1 keeps the first. */
    static const bool v1 = [] {
      const char *e = getenv("VXB_FLASH_V1");
      return e && *e && *e != '0';
    }();
    if (!v1)
      return flash_attention_fwd_v2(q, k, v, out, B, H, S, scale, causal, stream);
    return launch_flash<2>(mq, mk, mv, out, B, H, S, scale, causal, stream);
  }
  return launch_flash<1>(mq, mk, mv, out, B, H, S, scale, causal, stream);
}

int flash_status(cudaStream_t stream) {
  int v = 0, zero = 0;
  if (cudaStreamSynchronize(stream) != cudaSuccess)
    return -1;
  if (cudaMemcpyFromSymbol(&v, g_flash_status, sizeof v) != cudaSuccess)
    return -1;
  if (v)
    cudaMemcpyToSymbol(g_flash_status, &zero, sizeof zero);
  const int v2 = flash2_status();
  return v ? v : v2;
}

} // namespace vxb
