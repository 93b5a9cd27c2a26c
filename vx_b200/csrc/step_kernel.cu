/* step_kernel.cu -- every layer of one decode step of one sequence in ONE
 * kernel launch.
 *
 * A decode step of a Llama-shaped model is a chain of short operators, each
 * needing the whole output of the one before: RMSNorm + q/k/v + RoPE + cache
 * store, attention, output projection + residual, RMSNorm + gate/up + SwiGLU,
 * down projection + residual (nn.vx:169-280, 349-866; the layer loop of
 * llama2_100.vx).  As separate launches each of them pays for the start and
 * the drain of a grid, and the stream of weights from HBM stops at every
 * boundary.  Here one block per SM stays resident for the whole step:
 *
 *  - every warp owns a ring in shared memory that bulk copies fill with the
 *    weight rows of ITS items, and the loading side walks the list of
 *    projections of the whole step ahead of the arithmetic: while the blocks
 *    meet at a barrier or do a layer's attention, the rings fill with the next
 *    projection's weights, so HBM keeps streaming;
 *  - between two operators the blocks meet at a barrier in global memory (one
 *    arrival per block, one polling thread per block);
 *  - attention is cut into units of (KV head, run of positions) that groups of
 *    four warps take; the group that finishes a head last merges its parts;
 *  - with several tensor-parallel ranks, the row-split projections exchange
 *    their partial sums from inside their epilogue, as the projection kernel
 *    of nn_kernels.cu does (see TpPush).
 *
 * The arithmetic of every operator -- the order of every sum -- is the one of
 * the separate kernels, so a step gives the same activations either way.
 *
 * Every wait is bounded (about a second); one that runs out sets the status
 * word, which ends every later wait at once, and the kernel leaves after its
 * copies in flight have landed.  The launch is cooperative: the blocks are
 * resident together or the launch fails.
 */
#include "kernels.h"
#include "launch.cuh"
#include "nn_device.cuh"
#include "ptx.cuh"

#include <cstdio>
#include <cstdlib>

namespace vxb {
namespace {

int sm_count() {
  int dev = 0, v = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
  return v > 0 ? v : 148;
}
const char *check_launch(const char *what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess)
    return nullptr;
  static thread_local char msg[256];
  snprintf(msg, sizeof msg, "%s: %s", what, cudaGetErrorString(e));
  return msg;
}

constexpr int S_WARPS = 16;
constexpr int S_THREADS = S_WARPS * 32;
constexpr int S_STAGES = 5;            /* chunks of both rows in flight per warp */
constexpr int S_CHUNK = 1024;          /* bytes of one row */
constexpr int S_WARP_RING = S_STAGES * 2 * S_CHUNK;
constexpr int S_RING_BYTES = S_WARPS * S_WARP_RING;
constexpr int S_XS_FLOATS = kStepMaxCols; /* the widest input of a projection */
constexpr int S_SMEM = S_RING_BYTES + S_XS_FLOATS * 4;
constexpr int S_GROUPS = S_WARPS / 4;  /* attention: groups of four warps */

__device__ int g_step_status; /* non-zero: a wait gave up (which: see below) */
enum { GAVE_UP_RING = 0x71, GAVE_UP_BARRIER = 0x72, GAVE_UP_PEER = 0x73 };

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool step_failed() {
  return *(volatile int *)&g_step_status != 0;
}

/* All blocks have passed `target / gridDim.x` barriers. One thread per block
   arrives and polls; the writes of the whole block before the barrier are
   visible to every block after it (fence, then the arrival; acquire on the
   polling side). */
__device__ __forceinline__ void grid_barrier(int32_t *arrivals, int target) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(arrivals, 1);
    const long long began = clock64();
    int spins = 0;
    for (;;) {
      int seen;
      asm volatile("ld.acquire.gpu.global.s32 %0, [%1];"
                   : "=r"(seen)
                   : "l"(arrivals)
                   : "memory");
      if (seen >= target)
        break;
      if ((++spins & 63) == 0 &&
          (step_failed() || clock64() - began > ptx::kWaitCycles)) {
        atomicCAS(&g_step_status, 0, GAVE_UP_BARRIER);
        break;
      }
    }
  }
  __syncthreads();
}

/* The two weight rows of item `item` of a projection. */
struct StepRows {
  const char *r0, *r1;
  bool two;
};
__device__ __forceinline__ StepRows step_rows(const StepOp &op, int item,
                                              int q_heads, int kv_heads, int hd) {
  StepRows r;
  const int64_t rb = (int64_t)op.cols * 2;
  r.two = true;
  if (op.kind == kStepSwiglu) {
    r.r0 = (const char *)op.w0 + item * rb;
    r.r1 = (const char *)op.w1 + item * rb;
  } else if (op.kind == kStepQkv) {
    const int half = hd / 2;
    const int head = item / half, idx = item - head * half;
    const char *base =
        head < q_heads ? (const char *)op.w0 + (int64_t)head * hd * rb
        : head < q_heads + kv_heads
            ? (const char *)op.w1 + (int64_t)(head - q_heads) * hd * rb
            : (const char *)op.w2 + (int64_t)(head - q_heads - kv_heads) * hd * rb;
    r.r0 = base + idx * rb;
    r.r1 = base + (idx + half) * rb;
  } else {
    r.r0 = (const char *)op.w0 + (int64_t)(2 * item) * rb;
    r.two = 2 * item + 1 < op.rows;
    r.r1 = r.two ? r.r0 + rb : r.r0;
  }
  return r;
}

/* Where a value of x sits in shared memory: within each group of 256 values
   the two quarters of a lane's eight are stored 128 floats apart, so that the
   32 lanes of a warp read consecutive float4s (as in the projection kernel). */
__device__ __forceinline__ int xs_at(int i) {
  return (i & ~255) | (((i & 7) >> 2) << 7) | (((i >> 3) & 31) << 2) | (i & 3);
}

template <int GH>
__global__ void __launch_bounds__(S_THREADS, 1) decode_step_kernel(const StepArgs a) {
  extern __shared__ __align__(128) unsigned char smem_dyn[];
  unsigned char *ring = smem_dyn;
  float *xs = (float *)(smem_dyn + S_RING_BYTES);
  __shared__ float ssq[S_WARPS];
  __shared__ __align__(8) uint64_t bars[S_WARPS][S_STAGES];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t total_warps = (int64_t)gridDim.x * S_WARPS;
  const int64_t gw = (int64_t)blockIdx.x * S_WARPS + warp;
  unsigned char *my_ring = ring + warp * S_WARP_RING;
  const int hd = a.head_dim;

  if (lane == 0) {
    for (int s = 0; s < S_STAGES; ++s)
      ptx::mbar_init(&bars[warp][s], 1);
    ptx::fence_proxy_async_smem();
    ptx::fence_barrier_init();
  }
  __syncwarp();

  /* ---- the loading side: this warp's items of every projection, in order ---- */
  int ld_op = -1, ld_item = 0, ld_end = 0, ld_ch = 0, ld_nch = 1, ld_last = 0;
  int ld_stage = 0, issued = 0;
  const char *ld_r0 = nullptr, *ld_r1 = nullptr;
  auto ld_open_item = [&]() {
    /* moves to the next projection that has items for this warp, if needed */
    while (ld_op < a.n_ops && ld_item >= ld_end) {
      if (++ld_op >= a.n_ops)
        return;
      const StepOp &op = a.ops[ld_op];
      ld_item = (int)(gw * op.items / total_warps);
      ld_end = (int)((gw + 1) * op.items / total_warps);
      const int row_bytes = op.cols * 2;
      ld_nch = (row_bytes + S_CHUNK - 1) / S_CHUNK;
      ld_last = row_bytes - (ld_nch - 1) * S_CHUNK;
    }
    const StepRows r = step_rows(a.ops[ld_op], ld_item, a.q_heads, a.kv_heads, hd);
    ld_r0 = r.r0;
    ld_r1 = r.r1;
  };
  auto issue_next = [&]() {
    if (ld_op >= a.n_ops)
      return;
    if (lane == 0) {
      const int bytes = ld_ch == ld_nch - 1 ? ld_last : S_CHUNK;
      unsigned char *dst = my_ring + ld_stage * (2 * S_CHUNK);
      uint64_t *bar = &bars[warp][ld_stage];
      ptx::mbar_expect_tx(bar, 2 * bytes);
      ptx::bulk_load(dst, ld_r0 + ld_ch * S_CHUNK, bytes, bar);
      ptx::bulk_load(dst + S_CHUNK, ld_r1 + ld_ch * S_CHUNK, bytes, bar);
    }
    ++issued;
    ld_stage = ld_stage + 1 == S_STAGES ? 0 : ld_stage + 1;
    if (++ld_ch == ld_nch) {
      ld_ch = 0;
      ++ld_item;
      ld_open_item();
    }
  };
  ld_open_item();
  for (int u = 0; u < S_STAGES; ++u)
    issue_next();

  const int ranks = a.tp.ranks;
  const int epoch0 = ranks > 1 ? *(volatile int32_t *)a.tp.epoch : 0;
  int pushes = 0, barriers = 0;
  int c_stage = 0, consumed = 0;
  uint32_t c_phase = 0;
  bool dead = false; /* this warp gave up on its ring */
  const int pos = a.positions[0];

  for (int o = 0; o < a.n_ops; ++o) {
    const StepOp op = a.ops[o];
    const int kind = op.kind, cols = op.cols;
    const bool tracing = a.trace && blockIdx.x == 0 && threadIdx.x == 0;
    unsigned long long *tr = a.trace + (int64_t)o * kStepTraceSlots;
    if (tracing)
      tr[0] = now_ns();
    if (o > 0)
      grid_barrier(a.arrivals, ++barriers * (int)gridDim.x);
    if (tracing)
      tr[1] = now_ns();

    /* ---- prologue: x (times the norm weights, if any) into shared memory ---- */
    float inv = 1.0f;
    {
      const float4 *px4 = reinterpret_cast<const float4 *>(op.x);
      const int quads = cols / 4;
      if (op.norm_w) {
        /* RMSNorm (nn_rms_norm, nn.vx:212-239): y_i = x_i * inv * w_i. The ring
           is fed x_i * w_i and inv multiplies the finished dot products. */
        float ss = 0.0f;
        for (int q0 = threadIdx.x; q0 < quads; q0 += 4 * S_THREADS) {
          float4 v[4], wn[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int q = q0 + k * S_THREADS;
            v[k] = wn[k] = make_float4(0, 0, 0, 0);
            if (q < quads) {
              v[k] = __ldcg(px4 + q);
              const uint2 w = __ldg(reinterpret_cast<const uint2 *>(op.norm_w) + q);
              wn[k] = make_float4(bf_lo(w.x), bf_hi(w.x), bf_lo(w.y), bf_hi(w.y));
            }
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int q = q0 + k * S_THREADS;
            if (q < quads) {
              *reinterpret_cast<float4 *>(&xs[xs_at(4 * q)]) =
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
          ssq[warp] = ss;
        __syncthreads();
        float total = 0.0f;
        for (int w = 0; w < S_WARPS; ++w) /* fixed order */
          total += ssq[w];
        inv = 1.0f / sqrtf(total / (float)cols + a.eps);
      } else {
        for (int q0 = threadIdx.x; q0 < quads; q0 += 8 * S_THREADS) {
          float4 v[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int q = q0 + k * S_THREADS;
            v[k] = q < quads ? __ldcg(px4 + q) : make_float4(0, 0, 0, 0);
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int q = q0 + k * S_THREADS;
            if (q < quads)
              *reinterpret_cast<float4 *>(&xs[xs_at(4 * q)]) = v[k];
          }
        }
        __syncthreads();
      }
    }

    if (tracing)
      tr[2] = now_ns();
    /* ---- this warp's items ---- */
    const int first = (int)(gw * op.items / total_warps);
    const int last = (int)((gw + 1) * op.items / total_warps);
    const int row_bytes = cols * 2;
    const int nch = (row_bytes + S_CHUNK - 1) / S_CHUNK;
    const int last_bytes = row_bytes - (nch - 1) * S_CHUNK;
    const int push_call = (kind == kStepAdd && ranks > 1) ? epoch0 + ++pushes : 0;
    const int64_t push_set = push_call & 1;

    for (int item = first; item < last && !dead; ++item) {
      float s0 = 0.0f, s1 = 0.0f;
      for (int ch = 0; ch < nch; ++ch) {
        const int s = c_stage;
        const uint32_t phase = c_phase;
        const bool landed = ptx::mbar_try_wait(&bars[warp][s], phase) ||
                            ptx::mbar_wait(&bars[warp][s], phase, &g_step_status);
        if (!__all_sync(0xffffffffu, landed)) { /* the same answer on every lane */
          atomicCAS(&g_step_status, 0, GAVE_UP_RING);
          dead = true;
          break;
        }
        ++consumed;
        if (++c_stage == S_STAGES) {
          c_stage = 0;
          c_phase ^= 1;
        }
        const unsigned char *src = my_ring + s * (2 * S_CHUNK) + lane * 16;
        const float *xcol = xs + ch * (S_CHUNK / 2) + lane * 4;
        auto word = [&](int off) {
          const uint4 wa = *reinterpret_cast<const uint4 *>(src + off);
          const uint4 wb = *reinterpret_cast<const uint4 *>(src + S_CHUNK + off);
          const float *xw = xcol + off / 2;
          const float4 xa = *reinterpret_cast<const float4 *>(xw);
          const float4 xb = *reinterpret_cast<const float4 *>(xw + 128);
          s0 = fmaf(bf_lo(wa.x), xa.x, s0); s0 = fmaf(bf_hi(wa.x), xa.y, s0);
          s0 = fmaf(bf_lo(wa.y), xa.z, s0); s0 = fmaf(bf_hi(wa.y), xa.w, s0);
          s0 = fmaf(bf_lo(wa.z), xb.x, s0); s0 = fmaf(bf_hi(wa.z), xb.y, s0);
          s0 = fmaf(bf_lo(wa.w), xb.z, s0); s0 = fmaf(bf_hi(wa.w), xb.w, s0);
          s1 = fmaf(bf_lo(wb.x), xa.x, s1); s1 = fmaf(bf_hi(wb.x), xa.y, s1);
          s1 = fmaf(bf_lo(wb.y), xa.z, s1); s1 = fmaf(bf_hi(wb.y), xa.w, s1);
          s1 = fmaf(bf_lo(wb.z), xb.x, s1); s1 = fmaf(bf_hi(wb.z), xb.y, s1);
          s1 = fmaf(bf_lo(wb.w), xb.z, s1); s1 = fmaf(bf_hi(wb.w), xb.w, s1);
        };
        if (ch != nch - 1 || last_bytes == S_CHUNK) {
          word(0);
          word(512);
        } else {
          for (int off = 0; off + lane * 16 < last_bytes; off += 512)
            word(off);
        }
        __syncwarp(); /* every lane has read the stage: it may be filled again */
        issue_next();
      }
      if (dead)
        break;

      /* ---- the item is complete ---- */
      const float t0 = warp_sum(s0) * inv, t1 = warp_sum(s1) * inv;
      if (kind == kStepAdd) {
        const int ra = 2 * item;
        const bool two = ra + 1 < op.rows;
        float v0 = t0, v1 = t1;
        if (ranks > 1) {
          /* lane r sends both values to rank r and waits for rank r's values
             of the same rows; the partials are added in rank order */
          if (lane < ranks && lane != a.tp.rank) {
            TpPair *to = a.tp.slots[lane] +
                         (push_set * ranks + a.tp.rank) * a.tp.count + ra;
            if (two)
              pair2_store(to, v0, v1, push_call);
            else
              pair_store(to, v0, push_call);
            const TpPair *from = a.tp.slots[a.tp.rank] +
                                 (push_set * ranks + lane) * a.tp.count + ra;
            const long long began = clock64();
            int spins = 0;
            for (;;) {
              const bool here = two ? pair2_load(from, push_call, v0, v1)
                                    : pair_load(from, push_call, v0);
              if (here)
                break;
              if ((++spins & 15) == 0 &&
                  (step_failed() || clock64() - began > ptx::kWaitCycles)) {
                atomicCAS(&g_step_status, 0, GAVE_UP_PEER);
                break;
              }
            }
          }
          float a0 = lane == 0 ? __ldcg(op.y + ra) : 0.0f;
          float a1 = (lane == 0 && two) ? __ldcg(op.y + ra + 1) : 0.0f;
          for (int r = 0; r < ranks; ++r) {
            a0 += __shfl_sync(0xffffffffu, v0, r);
            a1 += __shfl_sync(0xffffffffu, v1, r);
          }
          v0 = a0;
          v1 = a1;
        } else if (lane == 0) {
          v0 = __ldcg(op.y + ra) + v0;
          if (two)
            v1 = __ldcg(op.y + ra + 1) + v1;
        }
        if (lane == 0) {
          op.y[ra] = v0;
          if (two)
            op.y[ra + 1] = v1;
        }
        continue;
      }
      if (lane != 0)
        continue;
      if (kind == kStepStore) {
        op.y[2 * item] = t0;
        if (2 * item + 1 < op.rows)
          op.y[2 * item + 1] = t1;
      } else if (kind == kStepSwiglu) {
        /* nn_swiglu (nn.vx:169-209): g / (1 + e^-g) * u */
        op.y[item] = t0 / (1.0f + expf(0.0f - t0)) * t1;
      } else { /* kStepQkv: bias, RoPE with tables, q out, k and v into the cache
                  (nn_rope_and_store, nn.vx:245-280) */
        const int half = hd / 2;
        const int head = item / half, idx = item - head * half;
        const int ia = idx, ib = idx + half;
        float va = t0, vb = t1;
        if (op.bias) {
          va += bf16_at(op.bias, (int64_t)head * hd + ia);
          vb += bf16_at(op.bias, (int64_t)head * hd + ib);
        }
        if (head >= a.q_heads + a.kv_heads) {
          float *vrow = op.v_cache +
                        ((int64_t)pos * a.kv_heads + head - a.q_heads - a.kv_heads) * hd;
          vrow[ia] = va;
          vrow[ib] = vb;
        } else {
          const float c = a.cos_t[(int64_t)pos * half + idx];
          const float s = a.sin_t[(int64_t)pos * half + idx];
          const float oa = __fsub_rn(__fmul_rn(va, c), __fmul_rn(vb, s));
          const float ob = __fadd_rn(__fmul_rn(vb, c), __fmul_rn(va, s));
          float *dst = head < a.q_heads
                           ? a.q + (int64_t)head * hd
                           : op.k_cache +
                                 ((int64_t)pos * a.kv_heads + head - a.q_heads) * hd;
          dst[ia] = oa;
          dst[ib] = ob;
        }
      }
    }

    if (tracing)
      tr[3] = now_ns();
    if (kind != kStepQkv)
      continue;
    /* ---- the layer's attention (nn_attention, nn.vx:349-866) ---- */
    grid_barrier(a.arrivals, ++barriers * (int)gridDim.x);
    if (tracing)
      tr[4] = now_ns();
    {
      AttnArgs at = {};
      at.q = a.q;
      at.k_cache = op.k_cache;
      at.v_cache = op.v_cache;
      at.cache_batch_stride = 0;
      at.out = a.att;
      at.q_heads = a.q_heads;
      at.kv_heads = a.kv_heads;
      at.head_dim = hd;
      at.batch = 1;
      at.positions = a.positions;
      at.max_pos = pos;
      at.scratch = a.scratch;
      at.counters = a.counters;
      at.rows_settled = 0;
      at.fresh_from = nullptr;
      at.kernel = kAttnSplit;
      const int group = a.q_heads / a.kv_heads;
      const int tiles = (group + GH - 1) / GH;
      const int ys = a.kv_heads * tiles;
      const int groups = (int)gridDim.x * S_GROUPS;
      /* as many runs per head as there are groups of warps for it; a run is a
         multiple of four positions (one per warp), at least 32 */
      const int want = groups / ys > 0 ? groups / ys : 1;
      int run = (pos + want) / want;
      run = (run + 3) & ~3;
      if (run < 32)
        run = 32;
      at.split = run;
      const int runs = pos / run + 1;
      typedef AttnShared<GH, 4> Shared;
      Shared *sh = reinterpret_cast<Shared *>(xs) + (warp >> 2);
      for (int unit = blockIdx.x * S_GROUPS + (warp >> 2); unit < ys * runs;
           unit += groups)
        attention_unit<GH, false, 0, 4, (GH > 1 ? 4 : 8)>(
            at, unit / ys, unit % ys, 0, warp & 3, lane, *sh, 1 + (warp >> 2));
    }
    if (tracing)
      tr[5] = now_ns();
  }

  /* ---- leaving ---- */
  if (dead) {
    /* copies still in flight write this block's shared memory: let them land */
    while (consumed < issued) {
      ptx::mbar_wait_alone(&bars[warp][c_stage], c_phase);
      ++consumed;
      if (++c_stage == S_STAGES) {
        c_stage = 0;
        c_phase ^= 1;
      }
    }
  }
  if (ranks > 1 && pushes > 0) {
    /* every block read the count of finished calls before its first barrier */
    if (blockIdx.x == 0 && threadIdx.x == 0)
      *a.tp.epoch = epoch0 + pushes;
  }
}

template <int GH> const char *launch_step(const StepArgs &a, cudaStream_t stream) {
  auto kernel = decode_step_kernel<GH>;
  if (allow_dynamic_smem((const void *)kernel, S_SMEM) != cudaSuccess)
    return "the step kernel could not get its shared memory on this GPU";
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, S_THREADS,
                                                    S_SMEM) != cudaSuccess ||
      per_sm < 1)
    return "the step kernel does not fit an SM of this GPU";
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sm_count());
  cfg.blockDim = dim3(S_THREADS);
  cfg.dynamicSmemBytes = S_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, a);
  return check_launch("the step launch");
}

} // namespace

const char *decode_step(const StepArgs &a, cudaStream_t stream) {
  if (a.head_dim != 128)
    return "the step kernel takes heads of 128 values";
  if (a.q_heads % a.kv_heads != 0)
    return "q_heads must be a multiple of kv_heads";
  if (a.n_ops < 1 || !a.ops || !a.arrivals)
    return "the step kernel needs its list of projections and its barrier word";
  if (a.tp.ranks > kMaxTpRanks)
    return "too many tensor-parallel ranks";
  const int group = a.q_heads / a.kv_heads;
  if (group >= 4)
    return launch_step<4>(a, stream);
  if (group >= 2)
    return launch_step<2>(a, stream);
  return launch_step<1>(a, stream);
}

/* parts of (at most) one run per group of four warps and head, and one more */
size_t step_scratch_floats(int q_heads) {
  return (size_t)q_heads * (148 * 2 * S_GROUPS + 2) * (128 + 2);
}

int step_status(cudaStream_t stream) {
  int v = 0;
  cudaMemcpyFromSymbolAsync(&v, g_step_status, sizeof v, 0, cudaMemcpyDeviceToHost,
                            stream);
  cudaStreamSynchronize(stream);
  return v;
}

} // namespace vxb
