/* kernels.h -- what the host side of the dispatch library asks of the sm_100a
 * kernels.  Every launcher queues work on `stream` and returns; none waits,
 * allocates or frees, so each can be recorded into a CUDA graph.  A launcher
 * that can refuse returns NULL for "queued" or a sentence saying why not.
 */
#ifndef VXB_KERNELS_H
#define VXB_KERNELS_H

#include <cuda_runtime.h>
#include <stdint.h>

namespace vxb {

/* ---- C[m,n] = A[m,k] * B[k,n], all row-major, strides in elements --------- */
const char *gemm_f32(const float *a, int64_t lda, const float *b, int64_t ldb,
                     float *c, int64_t ldc, int64_t m, int64_t n, int64_t k,
                     cudaStream_t stream);
/* The f32 product on the tensor cores (gemm_f32_split.cu): A and B as three
   bf16 terms each, the six largest of the nine term products summed in f32
   (what is left out is below 2^-24 of |a||b|). scratch_bytes: 0 when the shape
   is not for it (k must be a multiple of 64; small products stay on the FMA
   pipe), else the size of the scratch the call needs. */
size_t gemm_f32_split_scratch_bytes(int64_t m, int64_t n, int64_t k, int64_t ldc);
const char *gemm_f32_split(const float *a, int64_t lda, const float *b, int64_t ldb,
                           float *c, int64_t ldc, int64_t m, int64_t n, int64_t k,
                           void *scratch, cudaStream_t stream);
const char *gemm_f64(const double *a, int64_t lda, const double *b, int64_t ldb,
                     double *c, int64_t ldc, int64_t m, int64_t n, int64_t k,
                     cudaStream_t stream);
/* 16-bit inputs (is_bf16: bf16, else f16), f32 accumulation, output of the
   input type.  The tcgen05 path needs 16-byte aligned bases and row strides;
   anything else takes the warp-tiled kernel below it. */
const char *gemm_16(bool is_bf16, const void *a, int64_t lda, const void *b,
                    int64_t ldb, void *c, int64_t ldc, int64_t m, int64_t n,
                    int64_t k, cudaStream_t stream);
/* Forced routes, for tests and benchmarks. route: 0 = pick, 1 = tcgen05 with
   B read as stored (N-major operand), 2 = tcgen05 after transposing B into
   `scratch` ([n,k], caller-owned), 3 = the plain tiled kernel, 4 and 5 = 1
   and 2 on CTA pairs (tcgen05.mma.cta_group::2, 256x256 tiles). */
const char *gemm_16_route(int route, bool is_bf16, const void *a, int64_t lda,
                          const void *b, int64_t ldb, void *c, int64_t ldc,
                          int64_t m, int64_t n, int64_t k, void *scratch,
                          cudaStream_t stream);
/* Status words of the tcgen05 kernels (device memory, one per device): 0 = ok;
   otherwise the first wait that ran out. Read with gemm_status(). */
int gemm_status(cudaStream_t stream);

/* y[d] = W[d,n] . x[n], f32 (the flat entry point). */
const char *matvec_f32(float *y, const float *x, const float *w, int n, int d,
                       cudaStream_t stream);

/* ---- decode operators ------------------------------------------------------
 * W is row-major [rows, cols] in one of four formats; x and y are f32 with
 * `batch` vectors, row b of x at x + b*x_stride. wfmt 0: bf16 (wbf16) or f32.
 * kFmtFp8: f8e4m3 codes, one byte each, with f32 scales [ceil(rows/128),
 * cols/128] (stdlib/std/nn.vx:1296-1303); kFmtQ4: Q4_0, two codes a byte,
 * weight = (code - 8) * an f16 scale per 32 weights of a row
 * (nn.vx:1645-1663). The quantised formats take one sequence.               */
enum { kFmtF32 = 1, kFmtBf16 = 2, kFmtFp8 = 3, kFmtQ4 = 4 };
struct MatvecArgs {
  const void *w;
  bool wbf16;
  int wfmt;            /* 0: as wbf16 says */
  const void *scales;  /* kFmtFp8, kFmtQ4 */
  int row_base;        /* w is rows row_base.. of the matrix `scales` is for */
  int rows, cols;
  const float *x;
  int64_t x_stride;
  float *y;
  int64_t y_stride;
  int batch;
  /* prologue: x is RMS-normalised with this weight first (NULL: x as is) */
  const void *norm_w;
  bool norm_bf16;
  float eps;
  /* epilogue */
  /* a mixture-of-experts layer (nn.vx:960-1066): w (and scales) hold `experts`
     matrices of rows x cols one after another and this call takes matrix
     expert_ids[expert_slot], an index in device memory; NULL: w is the matrix.
     add_scale (mode 1): y += add_scale[0] * s, a device scalar. */
  const int32_t *expert_ids;
  int expert_slot, experts;
  const float *add_scale;
  int mode;            /* 0 y = s, 1 y += s, 2 y = s + bias,
                          3 y += the sum of all ranks' s (see TpPush) */
  const void *bias;    /* mode 2, bf16 */
  const struct TpPush *push; /* mode 3 */
};

/* Mode 3: the projection is one rank's partial of a row-split product, and
   y += the sum over ranks of the partials, in one kernel. A warp that finishes
   two rows stores its two values straight into slot `rank` of every OTHER
   rank's receive buffer (stores over NVLink into peer memory) as (value, call
   number) pairs -- an aligned 8-byte store arrives whole, so a pair is its own
   arrival flag and the exchange needs no fence, no counter and no separate
   signal -- then waits (bounded) for the other ranks' pairs of the same two
   rows in its own buffer and adds all partials to y in rank order: every rank
   adds the same values in the same order, so y stays identical on all ranks.
   Receive buffers: pairs [2 sets][ranks][count]; call c (1, 2, ...) uses set
   c & 1: a rank cannot be two calls ahead of another, because it needs that
   rank's values of the call between. `epoch` (device int32) holds the number
   of calls completed so far; the block that finishes last (counted in `done`,
   zero between launches) advances it. */
constexpr int kMaxTpRanks = 8;
struct TpPair {
  float value;
  int32_t call;
};
struct TpPush {
  TpPair *slots[kMaxTpRanks]; /* per rank: its receive slots */
  int ranks, rank;
  int64_t count;              /* values per slot: batch * rows (even) */
  int32_t *epoch;             /* this rank's, device memory */
  int32_t *done;
};
int tp_status(cudaStream_t stream);
const char *matvec(const MatvecArgs &a, cudaStream_t stream);

/* out[r] = silu(g_r) * u_r, g from row r and u from row rows + r of w. */
struct SwigluArgs {
  const void *w;
  bool wbf16;
  int wfmt;
  const void *scales, *scales_up; /* of w, and of w_up when that is given */
  int row_base;
  /* as in MatvecArgs: w holds `experts` matrices of 2 rows x cols */
  const int32_t *expert_ids;
  int expert_slot, experts;
  int rows, cols;
  const void *w_up; /* NULL: up rows follow the gate rows in w */
  const float *x;
  int64_t x_stride;
  float *out;
  int64_t out_stride;
  int batch;
  const void *norm_w;
  bool norm_bf16;
  float eps;
};
const char *swiglu(const SwigluArgs &a, cudaStream_t stream);

const char *rms_norm(float *y, const float *x, const void *w, bool wbf16, int n,
                     float eps, int batch, int64_t stride, cudaStream_t stream);

/* q/k/v projection + bias + RoPE + KV-cache store in one kernel.
   rope_mode 0: half-split pairs (i, i+hd/2) with cos/sin tables [*, hd/2];
   rope_mode 1: interleaved pairs (i, i+1), angle pos * theta^(-(i%hd)/hd).
   w rows: q heads, k heads, v heads (wk/wv NULL) or three matrices.
   positions: device int32[batch] (the position of each sequence).
   caches: [batch][max_seq, kv_heads, hd] f32. */
struct QkvArgs {
  const void *wq, *wk, *wv; /* wk == NULL: fused rows in wq */
  bool wbf16;
  int wfmt;
  const void *sq, *sk, *sv; /* the scales of wq, wk, wv */
  const void *bias; /* bf16 or NULL */
  int q_heads, kv_heads, head_dim, cols;
  const float *x;
  int64_t x_stride;
  int batch;
  const void *norm_w;
  bool norm_bf16;
  float eps;
  int rope_mode;
  const float *cos_t, *sin_t;
  int cs_cols;
  float theta;
  const int32_t *positions;
  float *q_out; /* [batch][q_heads*hd] */
  float *k_cache, *v_cache;
  int64_t cache_batch_stride;
  int max_seq;
};
const char *qkv_rope_store(const QkvArgs &a, cudaStream_t stream);

/* The unfused pieces, for the operator surface. */
const char *rope_and_store(float *q_out, float *k_cache, float *v_cache,
                           const float *q, const float *k, const float *v,
                           const float *cos_t, const float *sin_t, int cs_cols,
                           int pos, int q_heads, int kv_heads, int head_dim,
                           cudaStream_t stream);

/* Attention of one new token per sequence over rows 0..pos of its KV cache
   (nn_attention with its parts and merge, stdlib/std/nn.vx:343-368, 823-866).
   The positions are cut into runs, each run gives a partial (max, sum,
   weighted V) per head, and the partials are merged in run order. Two kernels
   do the same arithmetic and differ in where the partials meet:
     kAttnCluster  a cluster of 8 blocks per head tile, merged through
                   distributed shared memory; needs no scratch, and sequences
                   may share one cache (cache_batch_stride 0);
     kAttnSplit    one block per `split` positions (the reference's 32 below
                   position 640 and 64 from there on, or what the caller
                   says), partials in `scratch`, merged by whichever block of
                   a head tile finishes last, counted in `counters`.
   scratch: f32 [batch][q_heads][max_pos / split + 1][head_dim + 2];
   counters: int32 [batch][head tiles], zero before the launch, zero after. */
enum { kAttnAuto = 0, kAttnCluster = 1, kAttnSplit = 2 };
struct AttnArgs {
  const float *q; /* [batch][q_heads*hd] */
  const float *k_cache, *v_cache;
  int64_t cache_batch_stride;
  float *out; /* [batch][q_heads*hd] */
  int q_heads, kv_heads, head_dim, batch;
  const int32_t *positions; /* device, [batch] */
  int max_pos;              /* host bound on positions: sizes the grid */
  float *scratch;
  int32_t *counters;
  int split; /* positions per block (kAttnSplit) */
  /* device, or NULL: rows from fresh_from[0] on were written by the kernel
     just before (a run of prompt positions sharing one cache); NULL: only row
     `position` of each sequence was */
  const int32_t *fresh_from;
  int kernel; /* kAttnAuto: the process-wide choice, which starts as cluster */
  /* 1: the caller vouches that every cache row below the position was written
     before the chain of dependent launches this kernel is part of began (a
     decoder: earlier tokens are earlier graph launches), so those rows may be
     fetched before the wait for the kernel in front. 0: everything is read
     after that wait (the stand-alone operator: the rows may come from a run
     of short kernels launched just before, each of which lets its successor
     start early). */
  int rows_settled;
};
size_t attn_scratch_floats(int batch, int q_heads, int head_dim, int max_seq,
                           int split);
const char *attention_decode(const AttnArgs &a, cudaStream_t stream);
/* One decode step of one sequence (bf16 weights, heads of 128 values, RoPE
   from tables) as ONE cooperative launch: the list of its projections in the
   order they run, with the layer's attention after each q/k/v projection. */
enum { kStepQkv = 1, kStepAdd = 2, kStepSwiglu = 3, kStepStore = 4 };
constexpr int kStepMaxCols = 11264; /* the widest input a projection may have */
struct StepOp {
  /* bf16 rows of `cols` values. kStepQkv: the rows of the q, k and v heads;
     kStepSwiglu: gate rows, up rows; otherwise w0 */
  const void *w0, *w1, *w2;
  const void *norm_w; /* bf16 RMSNorm weights applied to x first, or NULL */
  const void *bias;   /* kStepQkv: bf16, or NULL */
  const float *x;     /* cols values */
  /* kStepAdd: y[r] += row r . x (summed over the ranks); kStepStore: y[r] =;
     kStepSwiglu: y[r] = silu(gate_r . x) * (up_r . x); kStepQkv: unused (q
     goes to StepArgs::q) */
  float *y;
  float *k_cache, *v_cache; /* kStepQkv: this layer's, [position][kv_heads][128] */
  int kind;
  int items; /* pairs of rows: kStepSwiglu rows; kStepQkv heads * 64; else ceil(rows / 2) */
  int rows, cols;
};
struct StepArgs {
  const StepOp *ops; /* device memory */
  int n_ops;
  int q_heads, kv_heads, head_dim; /* of this rank */
  float eps;
  const float *cos_t, *sin_t; /* [position][64] */
  const int32_t *positions;   /* device: the position of this step */
  float *q, *att;             /* q_heads * 128 values each */
  float *scratch;             /* attention parts: step_scratch_floats() */
  int32_t *counters;          /* attention: one per KV head tile, zero */
  int32_t *arrivals;          /* the barrier word: zero when the kernel starts */
  TpPush tp;                  /* ranks <= 1: no exchange; done is unused */
  /* NULL, or kStepTraceSlots nanosecond clock readings per projection that
     thread 0 of block 0 leaves: at the top of the loop, after the barrier,
     after the prologue, after its warp's items, and (q/k/v) after the barrier
     in front of attention and after attention */
  unsigned long long *trace;
};
constexpr int kStepTraceSlots = 6;
size_t step_scratch_floats(int q_heads);
const char *decode_step(const StepArgs &a, cudaStream_t stream);
int step_status(cudaStream_t stream);

/* The process-wide choice that kAttnAuto stands for; returns the one before. */
int attention_kernel_choice(int which);
/* Shorthand for kernel = kAttnCluster with no scratch. */
const char *attention_decode_clustered(const AttnArgs &a, cudaStream_t stream);

/* ---- the projections for 8 or 16 sequences, on the tensor cores -------------
 * y = W x with bf16 W [rows, cols] and f32 x [batch][cols] taken as three bf16
 * terms (rowdot_umma.cu). mode: 0 y = s, 1 y += s, 3 SwiGLU (rows = units; w0
 * gate rows, w1 up rows or NULL: up rows follow in w0), 4 q/k/v + bias + RoPE +
 * KV store (head_dim 128; w1/w2 k and v matrices or NULL: rows follow in w0).
 * xs: bf16 [48 or 32][cols] work space for the terms; scratch:
 * batched_proj_scratch_floats() floats for the partial sums of the K runs. */
struct BatchedProj {
  int mode;
  const void *w0, *w1, *w2;
  int rows, cols, batch;
  const float *x;
  int64_t x_stride;
  const void *norm_w; /* bf16, or NULL */
  float eps;
  float *y;
  int64_t y_stride;
  const void *bias;
  int q_heads, kv_heads, head_dim;
  const float *cos_t, *sin_t;
  const int32_t *positions;
  float *k_cache, *v_cache;
  int64_t cache_batch_stride;
  void *xs;
  float *scratch;
  /* chaining: x's terms are in xs already (left by the projection before);
     leave this projection's output there as terms for the next one (mode 3:
     SwiGLU's output is the down projection's input). A residual projection
     followed by an RMSNorm cannot: the norm needs the whole row, and one block
     per sequence doing both was no faster than the two kernels. */
  int x_terms_ready, next_terms;
};
const char *batched_proj_refusal(const BatchedProj &a);
size_t batched_proj_scratch_floats(int rows_max, int batch);
const char *batched_proj(const BatchedProj &a, cudaStream_t stream);
int batched_proj_status(cudaStream_t stream);

/* ---- a whole prompt at once (prefill.cu) ---------------------------------------
 * T positions as the rows of GEMMs on CTA pairs. Activations travel between
 * the GEMMs as "terms": a bf16 matrix [T, 3 cols] holding x as x1 | x2 | x3
 * with x = x1 + x2 + x3 exactly. rows_gemm leaves partials[run][t][r], the sums
 * of `*splits_out` runs of the K dimension; the *_finish calls add the runs in
 * run order and apply the projection's epilogue. */
int rows_gemm_splits(int t, int n, int cols);
size_t rows_gemm_partial_floats(int t, int n, int cols);
/* partials[run][t][r] = sum over the run's part of c of W[r, c] x[t, c];
   w bf16 [n, cols], cols a multiple of 64. */
const char *rows_gemm(const void *terms, const void *w, int t, int n, int cols,
                      float *partials, int *splits_out, cudaStream_t stream);
/* The same GEMM for any two bf16 matrices: terms [t, term_cols], w [n, w_cols];
   K block kb of the terms meets K block kb mod (w_cols / 64) of w (term_cols
   need not be a multiple of w_cols). */
int rows_gemm_splits_of(int t, int n, int64_t term_cols);
const char *rows_gemm_of(const void *terms, int64_t term_cols, const void *w,
                         int64_t w_cols, int t, int n, float *partials,
                         int *splits_out, cudaStream_t stream);
/* For quantised weights on that GEMM. Q4_0: a matrix [n, cols] as [n, 2 cols]
   bf16 = w1 | w2 with w1 + w2 = (code - 8) * scale exactly, against terms spread
   to x1 | x1 | x2 | x2 | x3 | x3 (segments 6, from {0,0,1,1,2,2}). fp8: the f32
   value code * scale as [n, 3 cols] = w1 | w2 | w3, against x1 | x1 | x1 | x2 |
   x2 | x2 | x3. rows_gemm_of(spread, segments * cols, unpacked, 2 or 3 cols,
   ...) then sums the products: the second operand's K blocks wrap round. */
const char *rows_q4_two_terms(void *out, const void *codes, const void *scales, int n,
                              int cols, cudaStream_t stream);
const char *rows_fp8_three_terms(void *out, const void *codes, const void *scales,
                                 int n, int cols, cudaStream_t stream);
const char *rows_spread_terms(void *out, const void *terms, int t, int cols,
                              int segments, const int *from, cudaStream_t stream);
/* terms of RMSNorm(x[t]) * w for every position (nn_rms_norm_rows). */
const char *rows_norm_terms(void *terms, const float *x, const void *w, int t,
                            int dim, float eps, cudaStream_t stream);
/* bias + half-split RoPE; q to q_out [t][q_heads*hd], k and v to cache rows
   first_pos[0] + t. */
const char *rows_qkv_finish(const float *partials, int splits, int t, int q_heads,
                            int kv_heads, int hd, const void *bias,
                            const float *cos_t, const float *sin_t,
                            const int32_t *first_pos, float *q_out, float *k_cache,
                            float *v_cache, cudaStream_t stream);
/* x[t][r] += the product, r below n. */
const char *rows_residual_finish(float *x, const float *partials, int splits, int t,
                                 int n, cudaStream_t stream);
/* terms of silu(gate) * up; partials have 2 hidden rows: gate, then up. */
/* x[t] += the product, then the terms of RMSNorm(x[t]) * w: the residual add
   and the normalisation that follows it, in one pass (dim <= 8192). */
const char *rows_residual_norm(void *terms, float *x, const float *partials,
                               int splits, int t, const void *w, int dim, float eps,
                               cudaStream_t stream);
const char *rows_swiglu_finish(void *terms, const float *partials, int splits, int t,
                               int hidden, cudaStream_t stream);
/* Causal attention of the T prompt positions over cache rows 0 ..
   first_pos[0] + t, f32; the output as terms [T, 3 q_heads hd]. head_dim 128. */
const char *rows_attention(void *terms, const float *q, const float *k_cache,
                           const float *v_cache, const int32_t *first_pos, int t,
                           int q_heads, int kv_heads, int hd, cudaStream_t stream);
int rows_status();

/* nn_top_k (nn.vx:904-938): ids[j] = the index of the j-th largest of the
   first n logits (n <= 256; of equal values the lower index first), weights[j]
   = the softmax over those k values. */
const char *top_k(int32_t *ids, float *weights, const float *logits, int n, int k,
                  cudaStream_t stream);
/* nn_top_k_rows (nn.vx:2897-2929): the same for `positions` rows of logits,
   one block each; row t of a tensor starts t * its pitch values in. */
const char *top_k_rows(int32_t *ids, float *weights, const float *logits,
                       int positions, int n, int k, int64_t ids_pitch,
                       int64_t weights_pitch, int64_t logits_pitch,
                       cudaStream_t stream);

/* ---- the pairs of a mixture-of-experts layer grouped by expert (moe_group.cu;
   nn.vx:1056-1294). counts and base: a row of `pitch` values for each 256
   pairs. order: `room` positions; tile_expert: `tiles` values. */
const char *moe_group_count(int32_t *counts, int64_t pitch, const int32_t *ids, int n,
                            int experts, cudaStream_t stream);
const char *moe_group_offsets(int32_t *base, int64_t base_pitch, int32_t *starts,
                              int32_t *tile_expert, int tiles, int32_t *order,
                              int room, const int32_t *counts, int64_t counts_pitch,
                              int n, int experts, int align, cudaStream_t stream);
const char *moe_group_place(int32_t *order, int room, const int32_t *ids,
                            const int32_t *base, int64_t pitch, int n, int experts,
                            cudaStream_t stream);
/* The Q4_0 experts of n positions on the tensor cores (moe_grouped.cu), an
   expert's rows unpacked once for each tile of `align` (8 or 16) pairs. order
   and tile_expert: nn_moe_group's, with that align, of the n * k ids. */
struct MoeGroupedArgs {
  const void *w, *scales;       /* all experts, one matrix after another */
  const int32_t *order, *tile_expert;
  int tiles, align;
  const float *x;               /* swiglu: [n, cols]; down: [n * k, cols] */
  int64_t x_pitch;
  float *out;                   /* swiglu: [n * k, rows] */
  int64_t out_pitch;
  float *y;                     /* down: [n, rows], added to */
  int64_t y_pitch;
  const float *pair_weights;    /* down: [n * k], the router's weights */
  float *scratch;               /* down: n * k * rows values */
  int n, k, rows, cols, experts;
};
const char *moe_swiglu_q4_grouped(const MoeGroupedArgs &m, cudaStream_t stream);
/* The same two for an fp8 matrix (gemm_fp8_rows.cu): e4m3 codes 4 to a word, an
   f32 scale per block of 128 x 128; cols a multiple of 128. */
const char *gemm_fp8(float *y, const void *w, const void *scales, const float *x, int n,
                     int rows, int cols, cudaStream_t stream);
const char *rows_gemm_fp8(const void *terms, const void *w, const void *scales, int t,
                          int n, int cols, float *partials, cudaStream_t stream);
/* y[n, rows] = x[n, cols] times the transpose of a Q4_0 matrix [rows, cols], on
   the same kernel. */
const char *gemm_q4(float *y, const void *w, const void *scales, const float *x, int n,
                    int rows, int cols, cudaStream_t stream);
/* The prompt's GEMM for Q4_0 weights on the same kernel: partials[t][r] = (row r
   of w) . x[t], x as the terms of prefill.cu ([t, 3 cols] bf16), one run. */
const char *rows_gemm_q4(const void *terms, const void *w, const void *scales, int t,
                         int n, int cols, float *partials, cudaStream_t stream);
const char *moe_down_q4_add_grouped(const MoeGroupedArgs &m, cudaStream_t stream);
/* 0, or once 0x6E after an id that named no expert (0x6F: a `base` that sent a
   pair outside `order`); waits for the stream. */
int moe_group_status(cudaStream_t stream);
const char *argmax(int32_t *out, const float *logits, int n, int batch,
                   int64_t stride, cudaStream_t stream);
const char *embed(float *x, const void *table, bool tbf16, const int32_t *token,
                  int dim, int rows, int batch, int64_t x_stride,
                  cudaStream_t stream);

/* ---- flash attention forward, bf16, [B,H,S,D] ------------------------------ */
const char *flash_attention_fwd(const void *q, const void *k, const void *v,
                                void *out, int B, int H, int S, int D,
                                float scale, bool causal, cudaStream_t stream);
int flash_status(cudaStream_t stream);

/* ---- small utilities --------------------------------------------------------*/
const char *transpose_16(const void *in, int64_t ld_in, void *out,
                         int64_t ld_out, int64_t rows, int64_t cols,
                         cudaStream_t stream);
/* out[i] = N(0, sigma^2) (or U[lo,hi)) from a counter-based generator, as f32
   or rounded to bf16. Used to make synthetic weights on the device. */
const char *fill_normal(void *out, bool as_bf16, int64_t n, uint64_t seed,
                        float sigma, cudaStream_t stream);
const char *fill_uniform(void *out, bool as_bf16, int64_t n, uint64_t seed,
                         float lo, float hi, cudaStream_t stream);
/* A bf16 matrix [rows, cols] into fp8 codes (one byte each) with f32 scales
   [ceil(rows/128), cols/128], or into Q4_0 codes (two a byte) with f16 scales
   [rows, cols/32]: quantize.cu. */
const char *quantize_fp8(const void *w_bf16, int rows, int cols, void *codes,
                         float *scales, cudaStream_t stream);
const char *quantize_q4(const void *w_bf16, int rows, int cols, void *codes,
                        void *scales_f16, cudaStream_t stream);
const char *interleave_gathered(const void *gathered, void *out, int ranks,
                                int64_t m, int64_t n_local, int elem_bytes,
                                cudaStream_t stream);

} // namespace vxb

#endif /* VXB_KERNELS_H */
