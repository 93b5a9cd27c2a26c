/* rowdot_quant_mma.cuh -- the fp8 and Q4_0 projections of ONE sequence on the
 * tensor cores (nn_matvec_fp8 / nn_swiglu_fp8 / nn_qkv_fp8, nn.vx:1306-1577;
 * the Q4_0 forms, nn.vx:1666-2190). Part of nn_kernels.cu (included there).
 *
 * With one-byte and half-byte weights the projection kernel is bound by
 * instruction issue, not by HBM: every weight costs a conversion to f32, a
 * multiply-add and its share of the loads (six instructions per weight and
 * lane).  Here a warp takes 16 weight rows at a time as the A operand of
 * mma.sync.m16n8k16, and the f32 activations enter as the B operand split into
 * three 16-bit terms whose sum is x exactly (bf16 terms beside Q4_0 codes,
 * which become small bf16 integers; f16 terms, the second and third scaled by
 * 2^11 and 2^22, beside fp8 codes, which the conversion instruction turns into
 * f16 two at a time).  The products are exact in f32 and the tensor core
 * accumulates them in f32, so a weight costs a fraction of an instruction.
 *
 * The 16 rows of a warp's tile are the two rows of eight ITEMS of the
 * projection kernel (rows g and g + 8 of the A operand are rows r0 and r1 of
 * item 8 tile + g), so every epilogue -- residual add, bias, SwiGLU, RoPE and
 * cache store -- finds its pair of results in one lane.  The order of the
 * columns inside a k-step is permuted, the same way for A and B, so that each
 * lane reads its codes and its activations with wide loads.
 *
 * Weights arrive through a per-warp ring filled by TMA: two tiled copies per
 * k-step, each eight rows of 128 bytes (the eight r0 rows, the eight r1 rows;
 * for Q4_0 two more bring the rows' f16 scales of the step), 128-byte swizzled
 * so that the lanes' loads do not meet in a bank.  (One bulk copy per row was
 * correct and slower than the FMA-pipe kernel: 700 000 copies of 128 bytes per
 * projection kept the copy unit, not HBM, busy.)  With fewer tiles
 * than warps the k-steps of a tile are divided among 2, 4, 8 or 16
 * neighbouring warps, whose partial sums meet in shared memory in a fixed
 * order.  Every wait is bounded.
 */
#ifndef VXB_ROWDOT_QUANT_MMA_CUH
#define VXB_ROWDOT_QUANT_MMA_CUH

constexpr int QTHREADS = WARPS * 32;
constexpr int STEP_ROW_BYTES = 128; /* of one row per k-step */

__device__ int g_quant_status; /* non-zero: a ring wait gave up */

template <typename W> struct QFmt;
template <> struct QFmt<Fp8W> {
  static constexpr int codes = 128;       /* per row and k-step: one block of scales */
  static constexpr int scale_bytes = 0;   /* scales are read from global memory */
  static constexpr int x_pad = 16;        /* bytes between the terms' rows, mod 128 */
};
template <> struct QFmt<Q4W> {
  static constexpr int codes = 256;
  static constexpr int scale_bytes = 256; /* 16 rows x eight f16 per k-step */
  static constexpr int x_pad = 64;
};
constexpr int STAGE_CODES_BYTES = 2048; /* two boxes of 8 rows x 128 bytes */
constexpr int MAX_STAGES = 8;

/* A map over `rows` rows of `inner` bytes, `pitch` bytes apart, for boxes of 8
   rows x box_inner bytes. */
inline bool make_byte_map(CUtensorMap *map, const void *base, uint64_t inner,
                          uint64_t rows, uint64_t pitch, uint32_t box_inner,
                          bool swizzle) {
  typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t,
                                  void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiled enc = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return (EncodeTiled) nullptr;
    }
    return (EncodeTiled)p;
  }();
  if (!enc || rows == 0)
    return false;
  const cuuint64_t dims[2] = {inner, rows};
  const cuuint64_t strides[1] = {pitch};
  const cuuint32_t box[2] = {box_inner, 8};
  const cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims,
             strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

__host__ __device__ inline int x_term_stride(int cols, int pad) {
  return (cols * 2 + 127) / 128 * 128 + pad; /* bytes */
}

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4],
                                        uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
               "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4],
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
               "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
/* the two fp8 (e4m3) codes in the low (HI = false) or high 16 bits of `four`,
   as two f16: the lower byte in the lower half */
template <bool HI> __device__ __forceinline__ uint32_t fp8x2_to_f16x2(uint32_t four) {
  uint32_t out;
  if (HI)
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, hi;\n\t}"
        : "=r"(out)
        : "r"(four));
  else
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t}"
        : "=r"(out)
        : "r"(four));
  return out;
}
__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

/* What lane 0 of the projection kernel does with the two results of an item,
   for one sequence (the epilogues of rowdot_kernel). */
template <int EPI>
__device__ __forceinline__ void finish_item(const RowDotParams &p, int item, float t0,
                                            float t1) {
  if (EPI == EPI_STORE || EPI == EPI_ADD || EPI == EPI_BIAS) {
    const int ra = 2 * item, rb = 2 * item + 1;
    const bool two = rb < p.rows;
    float v0 = t0, v1 = t1;
    if (EPI == EPI_ADD) {
      v0 = p.y[ra] + v0;
      if (two)
        v1 = p.y[rb] + v1;
    } else if (EPI == EPI_BIAS) {
      v0 += bf16_at(p.bias, ra);
      if (two)
        v1 += bf16_at(p.bias, rb);
    }
    p.y[ra] = v0;
    if (two)
      p.y[rb] = v1;
  } else if (EPI == EPI_SWIGLU) {
    /* nn_swiglu (nn.vx:169-209): g / (1 + e^-g) * u */
    p.y[item] = t0 / (1.0f + expf(0.0f - t0)) * t1;
  } else { /* EPI_QKV with tables: nn_rope_and_store (nn.vx:245-280) */
    const int hd = p.head_dim, half = hd / 2;
    const int head = item / half, idx = item - head * half;
    const int ia = idx, ib = idx + half;
    float va = t0, vb = t1;
    if (p.bias) {
      va += bf16_at(p.bias, (int64_t)head * hd + ia);
      vb += bf16_at(p.bias, (int64_t)head * hd + ib);
    }
    const int pos = p.positions[0];
    if (head >= p.q_heads + p.kv_heads) {
      float *vrow = p.v_cache +
                    ((int64_t)pos * p.kv_heads + head - p.q_heads - p.kv_heads) * hd;
      vrow[ia] = va;
      vrow[ib] = vb;
      return;
    }
    const float c = p.cos_t[(int64_t)pos * p.cs_cols + idx];
    const float s = p.sin_t[(int64_t)pos * p.cs_cols + idx];
    const float oa = __fsub_rn(__fmul_rn(va, c), __fmul_rn(vb, s));
    const float ob = __fadd_rn(__fmul_rn(vb, c), __fmul_rn(va, s));
    float *dst = head < p.q_heads
                     ? p.y + (int64_t)head * hd
                     : p.k_cache + ((int64_t)pos * p.kv_heads + head - p.q_heads) * hd;
    dst[ia] = oa;
    dst[ib] = ob;
  }
}

struct QuantPlan {
  int tiles;  /* of eight items */
  int split;  /* warps that share a tile's k-steps: 1, 2, 4, 8 or 16 */
  int ksteps; /* per row */
  /* Just enough warps per block for one unit each (a multiple of split), and
     the shared memory the others would have had goes into deeper rings: what
     is in flight per SM, not the number of warps, feeds HBM. */
  int warps, stages;
};

template <typename W, int EPI>
__global__ void __launch_bounds__(QTHREADS, 1)
quant_mma_kernel(const RowDotParams p, const QuantPlan plan,
                 const __grid_constant__ CUtensorMap map_a,
                 const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_sa,
                 const __grid_constant__ CUtensorMap map_sb) {
  typedef QFmt<W> F;
  constexpr bool FP8 = F::codes == 128;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  /* swizzled boxes want 1 KiB alignment */
  unsigned char *smem_dyn =
      smem_raw + ((1024 - (ptx::smem_addr(smem_raw) & 1023)) & 1023);
  const int stages = plan.stages, nwarps = plan.warps;
  const int nthreads = nwarps * 32;
  /* a warp's ring: its stages of codes, then its stages of scales, rounded up
     to the 1 KiB the swizzled boxes of the next warp want */
  const int warp_ring = (stages * (STAGE_CODES_BYTES + F::scale_bytes) + 1023) & ~1023;
  unsigned char *ring = smem_dyn;
  unsigned char *xterms = smem_dyn + nwarps * warp_ring;
  __shared__ float ssq[WARPS];
  __shared__ float2 parts[WARPS][8];
  __shared__ __align__(8) uint64_t bars[WARPS][MAX_STAGES];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int cols = p.cols;
  const int xstride = x_term_stride(cols, F::x_pad);
  unsigned char *my_ring = ring + warp * warp_ring;
  unsigned char *my_scales = my_ring + stages * STAGE_CODES_BYTES;

  if (lane == 0) {
    for (int s = 0; s < stages; ++s)
      ptx::mbar_init(&bars[warp][s], 1);
    ptx::fence_proxy_async_smem();
    ptx::fence_barrier_init();
  }
  __syncwarp();

  const int64_t total_warps = (int64_t)gridDim.x * nwarps;
  const int64_t gw = (int64_t)blockIdx.x * nwarps + warp;
  const int64_t units = (int64_t)plan.tiles * plan.split;
  const int rounds = (int)((units + total_warps - 1) / total_warps);

  /* ---- the loading side: one unit (a tile's share of the k-steps) at a time;
     lane 0 issues two (Q4_0: four) tiled copies per k-step. ya, yb: the rows
     of the two maps where the tile's r0 and r1 rows begin. ---- */
  int ld_stage = 0, ld_ks = 0, ld_end = 0, issued = 0, ld_ya = 0, ld_yb = 0;
  auto open_unit = [&](int64_t u) {
    const int tile = (int)(u / plan.split), part = (int)(u % plan.split);
    ld_ks = (int)((int64_t)part * plan.ksteps / plan.split);
    ld_end = (int)((int64_t)(part + 1) * plan.ksteps / plan.split);
    if (EPI == EPI_QKV) {
      const int half = p.head_dim / 2;
      const int head = tile * 8 / half;
      ld_ya = head * p.head_dim + (tile * 8 - head * half);
      ld_yb = ld_ya + half;
    } else {
      ld_ya = ld_yb = tile * 8;
    }
  };
  auto issue_next = [&]() {
    if (ld_ks >= ld_end)
      return;
    if (lane == 0) {
      unsigned char *dst = my_ring + ld_stage * STAGE_CODES_BYTES;
      uint64_t *bar = &bars[warp][ld_stage];
      ptx::mbar_expect_tx(bar, STAGE_CODES_BYTES + F::scale_bytes);
      ptx::tma_load_2d(dst, &map_a, ld_ks * STEP_ROW_BYTES, ld_ya, bar);
      ptx::tma_load_2d(dst + 1024, &map_b, ld_ks * STEP_ROW_BYTES, ld_yb, bar);
      if (!FP8) {
        unsigned char *sd = my_scales + ld_stage * F::scale_bytes;
        ptx::tma_load_2d(sd, &map_sa, ld_ks * 16, ld_ya, bar);
        ptx::tma_load_2d(sd + 128, &map_sb, ld_ks * 16, ld_yb, bar);
      }
    }
    ++issued;
    ++ld_ks;
    ld_stage = ld_stage + 1 == stages ? 0 : ld_stage + 1;
  };
  /* The weights do not depend on the kernel before this one: start them. */
  if (gw < units) {
    open_unit(gw);
    for (int s = 0; s < stages; ++s)
      issue_next();
  }
  chain_release();
  chain_wait();

  /* ---- x (times the norm weights, if any) as three 16-bit terms ---- */
  float inv = 1.0f;
  {
    float ss = 0.0f;
    const float4 *px4 = reinterpret_cast<const float4 *>(p.x);
    const int quads = cols / 4;
    for (int q = threadIdx.x; q < quads; q += nthreads) {
      float4 v = px4[q];
      if (p.norm_w) {
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss);
        ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        float4 wn;
        if (p.norm_bf16) {
          const uint2 w = reinterpret_cast<const uint2 *>(p.norm_w)[q];
          wn = make_float4(bf_lo(w.x), bf_hi(w.x), bf_lo(w.y), bf_hi(w.y));
        } else {
          wn = reinterpret_cast<const float4 *>(p.norm_w)[q];
        }
        v = make_float4(v.x * wn.x, v.y * wn.y, v.z * wn.z, v.w * wn.w);
      }
      const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = 4 * q + j;
        unsigned short t1, t2, t3;
        int at = i;
        if (FP8) {
          const __half h1 = __float2half_rn(e[j]);
          const float r1 = (e[j] - __half2float(h1)) * 2048.0f;
          const __half h2 = __float2half_rn(r1);
          const float r2 = (r1 - __half2float(h2)) * 2048.0f;
          t1 = __half_as_ushort(h1);
          t2 = __half_as_ushort(h2);
          t3 = __half_as_ushort(__float2half_rn(r2));
        } else {
          const __nv_bfloat16 b1 = __float2bfloat16_rn(e[j]);
          const float r1 = e[j] - __bfloat162float(b1);
          const __nv_bfloat16 b2 = __float2bfloat16_rn(r1);
          const float r2 = r1 - __bfloat162float(b2);
          t1 = __bfloat16_as_ushort(b1);
          t2 = __bfloat16_as_ushort(b2);
          t3 = __bfloat16_as_ushort(__float2bfloat16_rn(r2));
          /* inside a run of 8 the order is 0 4 1 5 2 6 3 7: the codes of a
             32-bit word pair up as (0, 4), (1, 5), (2, 6), (3, 7) */
          at = (i & ~7) | ((i & 3) * 2 + ((i >> 2) & 1));
        }
        *reinterpret_cast<unsigned short *>(xterms + at * 2) = t1;
        *reinterpret_cast<unsigned short *>(xterms + xstride + at * 2) = t2;
        *reinterpret_cast<unsigned short *>(xterms + 2 * xstride + at * 2) = t3;
      }
    }
    if (p.norm_w) {
      ss = warp_sum(ss);
      if (lane == 0)
        ssq[warp] = ss;
    }
    __syncthreads();
    if (p.norm_w) {
      float total = 0.0f;
      for (int w = 0; w < nwarps; ++w) /* fixed order */
        total += ssq[w];
      inv = 1.0f / sqrtf(total / (float)cols + p.eps);
    }
  }
  /* how the three columns of results add up to the product with x */
  const float m0 = t == 0 ? 1.0f : (t == 1 ? (FP8 ? 1.0f / 4194304.0f : 1.0f) : 0.0f);
  const float m1 = t == 0 ? (FP8 ? 1.0f / 2048.0f : 1.0f) : 0.0f;
  const unsigned char *xb = xterms + (g < 3 ? g : 0) * xstride;

  int c_stage = 0, consumed = 0;
  uint32_t c_phase = 0;
  bool gave_up = false;
  for (int r = 0; r < rounds; ++r) {
    const int64_t u = (int64_t)r * total_warps + gw;
    const bool has = u < units;
    const int tile = has ? (int)(u / plan.split) : 0;
    const int part = has ? (int)(u % plan.split) : 0;
    float lo0 = 0.0f, lo1 = 0.0f, hi0 = 0.0f, hi1 = 0.0f;
    if (has) {
      if (r > 0) {
        open_unit(u);
        for (int s = 0; s < stages; ++s)
          issue_next();
      }
      const int ks0 = (int)((int64_t)part * plan.ksteps / plan.split);
      const int ks1 = (int)((int64_t)(part + 1) * plan.ksteps / plan.split);
      int item = tile * 8 + g;
      if (item >= p.items)
        item = p.items - 1;
      const ItemRows mine = item_rows<W, EPI>(p, item);
      const float *sc_lo = reinterpret_cast<const float *>(mine.sc0);
      const float *sc_hi = reinterpret_cast<const float *>(mine.r1 ? mine.sc1 : mine.sc0);
      for (int ks = ks0; ks < ks1; ++ks) {
        /* a wait that runs out is reported, and the warp goes on without
           waiting again: its results are wrong, but it meets the block at
           every barrier */
        if (!gave_up && !ptx::mbar_try_wait(&bars[warp][c_stage], c_phase) &&
            !ptx::mbar_wait_alone(&bars[warp][c_stage], c_phase)) {
          atomicCAS(&g_quant_status, 0, 0x51);
          gave_up = true;
        }
        const unsigned char *st = my_ring + c_stage * STAGE_CODES_BYTES;
        const unsigned char *ssc = my_scales + c_stage * F::scale_bytes;
        (void)ssc;
        ++consumed;
        if (++c_stage == stages) {
          c_stage = 0;
          c_phase ^= 1;
        }
        if (FP8) {
          float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
          for (int grp = 0; grp < 2; ++grp) {
            /* 16-byte chunk c of box row g sits at chunk c ^ g (128-byte swizzle) */
            const int at = g * 128 + (((grp * 4 + t) ^ g) << 4);
            const uint4 al = *reinterpret_cast<const uint4 *>(st + at);
            const uint4 ah = *reinterpret_cast<const uint4 *>(st + 1024 + at);
            uint4 b01 = make_uint4(0, 0, 0, 0), b23 = b01;
            if (g < 3) {
              const uint4 *bp = reinterpret_cast<const uint4 *>(
                  xb + ((int64_t)ks * 128 + grp * 64 + t * 16) * 2);
              b01 = bp[0];
              b23 = bp[1];
            }
            const uint32_t wl[4] = {al.x, al.y, al.z, al.w};
            const uint32_t wh[4] = {ah.x, ah.y, ah.z, ah.w};
            const uint32_t bw[8] = {b01.x, b01.y, b01.z, b01.w,
                                    b23.x, b23.y, b23.z, b23.w};
#pragma unroll
            for (int m = 0; m < 4; ++m) {
              const uint32_t a[4] = {fp8x2_to_f16x2<false>(wl[m]),
                                     fp8x2_to_f16x2<false>(wh[m]),
                                     fp8x2_to_f16x2<true>(wl[m]),
                                     fp8x2_to_f16x2<true>(wh[m])};
              mma_f16(c, a, bw[2 * m], bw[2 * m + 1]);
            }
          }
          const float s_lo = __ldg(sc_lo + ks), s_hi = __ldg(sc_hi + ks);
          lo0 = fmaf(s_lo, c[0], lo0);
          lo1 = fmaf(s_lo, c[1], lo1);
          hi0 = fmaf(s_hi, c[2], hi0);
          hi1 = fmaf(s_hi, c[3], hi1);
        } else {
          const uint4 sl = *reinterpret_cast<const uint4 *>(ssc + g * 16);
          const uint4 sh = *reinterpret_cast<const uint4 *>(ssc + 128 + g * 16);
          const uint32_t slw[4] = {sl.x, sl.y, sl.z, sl.w};
          const uint32_t shw[4] = {sh.x, sh.y, sh.z, sh.w};
#pragma unroll
          for (int b = 0; b < 8; ++b) {
            const int at = g * 128 + ((b ^ g) << 4) + 4 * t;
            const uint32_t wl = *reinterpret_cast<const uint32_t *>(st + at);
            const uint32_t wh = *reinterpret_cast<const uint32_t *>(st + 1024 + at);
            uint4 bx = make_uint4(0, 0, 0, 0);
            if (g < 3)
              bx = *reinterpret_cast<const uint4 *>(
                  xb + ((int64_t)ks * 256 + 32 * b + 8 * t) * 2);
            /* a nibble OR-ed into 0x4300 is the bf16 128 + code; less 136 it
               is code - 8, exactly */
            constexpr uint32_t MAGIC = 0x43004300u, OFF = 0x43084308u, M = 0x000F000Fu;
            const uint32_t l0 = sub_bf16x2((wl & M) | MAGIC, OFF);
            const uint32_t l1 = sub_bf16x2(((wl >> 4) & M) | MAGIC, OFF);
            const uint32_t l2 = sub_bf16x2(((wl >> 8) & M) | MAGIC, OFF);
            const uint32_t l3 = sub_bf16x2(((wl >> 12) & M) | MAGIC, OFF);
            const uint32_t h0 = sub_bf16x2((wh & M) | MAGIC, OFF);
            const uint32_t h1 = sub_bf16x2(((wh >> 4) & M) | MAGIC, OFF);
            const uint32_t h2 = sub_bf16x2(((wh >> 8) & M) | MAGIC, OFF);
            const uint32_t h3 = sub_bf16x2(((wh >> 12) & M) | MAGIC, OFF);
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const uint32_t a0[4] = {l0, h0, l1, h1};
            mma_bf16(c, a0, bx.x, bx.y);
            const uint32_t a1[4] = {l2, h2, l3, h3};
            mma_bf16(c, a1, bx.z, bx.w);
            const uint32_t pl = slw[b >> 1], ph = shw[b >> 1];
            const float s_lo = __half2float(
                __ushort_as_half((unsigned short)((b & 1) ? pl >> 16 : pl & 0xffffu)));
            const float s_hi = __half2float(
                __ushort_as_half((unsigned short)((b & 1) ? ph >> 16 : ph & 0xffffu)));
            lo0 = fmaf(s_lo, c[0], lo0);
            lo1 = fmaf(s_lo, c[1], lo1);
            hi0 = fmaf(s_hi, c[2], hi0);
            hi1 = fmaf(s_hi, c[3], hi1);
          }
        }
        __syncwarp(); /* every lane has read the stage: it may be filled again */
        issue_next();
      }
    }
    /* the three columns, then the four lanes of a row */
    float lo = fmaf(m1, lo1, m0 * lo0), hi = fmaf(m1, hi1, m0 * hi0);
    lo += __shfl_xor_sync(0xffffffffu, lo, 1);
    hi += __shfl_xor_sync(0xffffffffu, hi, 1);
    lo += __shfl_xor_sync(0xffffffffu, lo, 2);
    hi += __shfl_xor_sync(0xffffffffu, hi, 2);
    if (t == 0)
      parts[warp][g] = make_float2(lo, hi);
    __syncthreads();
    if (has && part == 0 && t == 0) {
      float2 total = parts[warp][g];
      for (int q = 1; q < plan.split; ++q) { /* the warps of the tile, in order */
        total.x += parts[warp + q][g].x;
        total.y += parts[warp + q][g].y;
      }
      const int item = tile * 8 + g;
      if (item < p.items)
        finish_item<EPI>(p, item, total.x * inv, total.y * inv);
    }
    __syncthreads();
  }
  if (gave_up) {
    /* copies still in flight write this block's shared memory: let them land */
    while (consumed < issued) {
      ptx::mbar_wait_alone(&bars[warp][c_stage], c_phase);
      ++consumed;
      if (++c_stage == stages) {
        c_stage = 0;
        c_phase ^= 1;
      }
    }
  }
}

/* nullptr: launched; "": this projection is not for this kernel (the caller
   takes the other one); anything else: an error. */
template <typename W, int EPI>
const char *launch_quant_mma(RowDotParams &p, cudaStream_t stream) {
  typedef QFmt<W> F;
  static const bool wanted = [] {
    const char *e = getenv("VXB_QUANT_MMA");
    return !(e && e[0] == '0');
  }();
  constexpr bool FP8 = F::codes == 128;
  if (!wanted || p.batch != 1 || p.expert_ids || p.items < 1 || p.cols % F::codes != 0 ||
      p.cols % 4 != 0)
    return "";
  if (EPI == EPI_QKV &&
      (p.rope_mode != 0 || p.w1 || p.w2 || (p.head_dim / 2) % 8 != 0))
    return "";
  QuantPlan plan;
  plan.tiles = (p.items + 7) / 8;
  plan.ksteps = p.cols / F::codes;
  const int blocks = sm_count();
  plan.split = 1;
  while (plan.split < 16 && 2 * plan.split <= plan.ksteps &&
         (int64_t)plan.tiles * plan.split * 2 <= (int64_t)blocks * WARPS)
    plan.split *= 2;
  const int64_t units = (int64_t)plan.tiles * plan.split;
  int warps = (int)((units + blocks - 1) / blocks);
  warps = (warps + plan.split - 1) / plan.split * plan.split;
  if (warps > WARPS)
    warps = WARPS;
  if (warps < 4)
    warps = 4 > plan.split ? 4 : plan.split; /* enough threads to stage x */
  const size_t xbytes = 3 * (size_t)x_term_stride(p.cols, F::x_pad);
  const size_t budget = 223 * 1024;
  auto ring_of = [](int stages) { /* as the kernel lays it out */
    return (size_t)((stages * (STAGE_CODES_BYTES + F::scale_bytes) + 1023) & ~1023);
  };
  int stages = MAX_STAGES;
  while (stages > 2 && xbytes + warps * ring_of(stages) > budget)
    --stages;
  if (xbytes + warps * ring_of(stages) > budget)
    return "";
  plan.warps = warps;
  plan.stages = stages;
  const size_t smem = 1024 + warps * ring_of(stages) + xbytes;
  /* the rows of the tiles' r0 and r1 halves as two maps (see item_rows) */
  const uint64_t rb = (uint64_t)p.cols / PerWord<W>::n * 16; /* bytes of a row */
  const uint64_t sb = (uint64_t)p.cols / 16;                 /* Q4_0: of its scales */
  const char *w0 = (const char *)p.w0, *s0 = (const char *)p.s0 + p.row_base * sb;
  CUtensorMap ma, mb, msa, msb;
  bool ok;
  if (EPI == EPI_SWIGLU) {
    ok = make_byte_map(&ma, w0, rb, p.rows, rb, 128, true) &&
         make_byte_map(&mb, p.w1 ? (const char *)p.w1 : w0 + p.rows * rb, rb, p.rows, rb,
                       128, true);
    if (ok && !FP8)
      ok = make_byte_map(&msa, s0, sb, p.rows, sb, 16, false) &&
           make_byte_map(&msb, p.w1 ? (const char *)p.s1 : s0 + p.rows * sb, sb, p.rows,
                         sb, 16, false);
  } else if (EPI == EPI_QKV) {
    const uint64_t all = (uint64_t)(p.q_heads + 2 * p.kv_heads) * p.head_dim;
    ok = make_byte_map(&ma, w0, rb, all, rb, 128, true);
    mb = ma;
    if (ok && !FP8) {
      ok = make_byte_map(&msa, s0, sb, all, sb, 16, false);
      msb = msa;
    }
  } else {
    if (p.rows < 2)
      return "";
    ok = make_byte_map(&ma, w0, rb, (p.rows + 1) / 2, 2 * rb, 128, true) &&
         make_byte_map(&mb, w0 + rb, rb, p.rows / 2, 2 * rb, 128, true);
    if (ok && !FP8)
      ok = make_byte_map(&msa, s0, sb, (p.rows + 1) / 2, 2 * sb, 16, false) &&
           make_byte_map(&msb, s0 + sb, sb, p.rows / 2, 2 * sb, 16, false);
  }
  if (!ok)
    return "";
  if (FP8)
    msa = msb = ma;
  auto kernel = quant_mma_kernel<W, EPI>;
  if (allow_dynamic_smem((const void *)kernel, 224 * 1024) != cudaSuccess)
    return "a quantised projection could not get its shared memory on this GPU";
  launch_chained(kernel, dim3(blocks), dim3(plan.warps * 32), smem, stream, p, plan, ma, mb,
                 msa, msb);
  return check_launch("a quantised projection launch");
}

#endif /* VXB_ROWDOT_QUANT_MMA_CUH */
