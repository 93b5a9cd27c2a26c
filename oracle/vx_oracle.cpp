/* vx_oracle.cpp -- TEST INFRASTRUCTURE, NOT PRODUCT.
 *
 * A CPU restatement of the arithmetic that the reference's own CPU path does
 * for the operators this repository runs on the GPU.  Only the tests, the
 * smoke check and the cpu_baseline / reference legs of the benchmark load it;
 * no product code path may.  Each function names the reference file:line whose
 * loop it restates.  Build with -ffp-contract=off: the reference's loops carry
 * no contraction or reassociation flags, so a product and the add after it are
 * two roundings.
 *
 * Threads only ever split INDEPENDENT outputs (rows, heads); the order of the
 * additions inside one output is the reference's.
 *
 * Parity pins: the known answers of the reference's backend tests
 * (tests/backend/pass/gpu_matmul_roles.vx, gpu_matmul_dtypes.vx,
 * matmul_into_buffer.vx, benchmarks/matmul_execution.vx) and the argmax answer
 * of tests/optimizations/pass/std_nn_kernels_match_loops_on_the_cpu.vx are
 * checked in tests/test_oracle_golden.py.  The Llama decode has NO golden
 * tokens in the reference tree (its programs need a checkpoint that is not in
 * it): parity unpinned for that function, pinned by construction only.
 */
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

#if defined(_OPENMP)
#include <omp.h>
#endif

extern "C" {

/* ---- threads --------------------------------------------------------------*/
static int g_threads = 1;
void oracle_set_threads(int n) {
  g_threads = n < 1 ? 1 : n;
#if defined(_OPENMP)
  omp_set_num_threads(g_threads);
#endif
}
int oracle_get_threads(void) { return g_threads; }

/* ---- bf16 <-> f32, round to nearest even, NaN kept quiet -------------------
 * (reference: `as bf16` lowers through arith.truncf with
 * arith-expand{include-bf16}, src/driver.rs:2224-2233: exact RNE).           */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u)
    return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
void oracle_f32_to_bf16(const float *in, uint16_t *out, int64_t n) {
  for (int64_t i = 0; i < n; ++i)
    out[i] = f32_to_bf16(in[i]);
}
void oracle_bf16_to_f32(const uint16_t *in, float *out, int64_t n) {
  for (int64_t i = 0; i < n; ++i)
    out[i] = bf16_to_f32(in[i]);
}

/* ---- correctly rounded f32 math --------------------------------------------
 * The reference's CPU exp/sin/cos/powf are correctly rounded
 * (stdlib/core/num.vx:2404-2479, stdlib/core/libm.vx:8-20).  Computing in
 * double and rounding once differs from that only in double-rounding cases
 * that need ~29 zero/one bits in a row.                                      */
static inline float cr_expf(float x) { return (float)exp((double)x); }
static inline float cr_sinf(float x) { return (float)sin((double)x); }
static inline float cr_cosf(float x) { return (float)cos((double)x); }
static inline float cr_powf(float x, float y) {
  return (float)pow((double)x, (double)y);
}
static inline float cr_sqrtf(float x) { return sqrtf(x); }

/* ---- GEMM -------------------------------------------------------------------
 * runtime/host_dispatch_common.h:65-79 (vx_host_gemm_typed): i, j, k loops, a
 * T accumulator, k ascending.  The same nest as benchmarks/
 * matmul_execution.vx:20-28 and as linalg.matmul lowered to loops.           */
void oracle_gemm_f32(const float *a, int64_t lda, const float *b, int64_t ldb,
                     float *c, int64_t ldc, int64_t m, int64_t n, int64_t k) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; ++i)
    for (int64_t j = 0; j < n; ++j) {
      float acc = 0.0f;
      for (int64_t q = 0; q < k; ++q)
        acc += a[i * lda + q] * b[q * ldb + j];
      c[i * ldc + j] = acc;
    }
}

/* The same sums with the j loop innermost so that the compiler can keep a row
   of accumulators in vector registers: every C[i][j] still adds its k terms in
   ascending order, one rounding per multiply and per add, so the bits are those
   of oracle_gemm_f32.  Used where the plain nest would take minutes. */
void oracle_gemm_f32_rows(const float *a, int64_t lda, const float *b,
                          int64_t ldb, float *c, int64_t ldc, int64_t m,
                          int64_t n, int64_t k) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    float *row = c + i * ldc;
    for (int64_t j = 0; j < n; ++j)
      row[j] = 0.0f;
    for (int64_t q = 0; q < k; ++q) {
      const float av = a[i * lda + q];
      const float *brow = b + q * ldb;
      for (int64_t j = 0; j < n; ++j)
        row[j] += av * brow[j];
    }
  }
}

void oracle_gemm_f64(const double *a, int64_t lda, const double *b, int64_t ldb,
                     double *c, int64_t ldc, int64_t m, int64_t n, int64_t k) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; ++i)
    for (int64_t j = 0; j < n; ++j) {
      double acc = 0.0;
      for (int64_t q = 0; q < k; ++q)
        acc += a[i * lda + q] * b[q * ldb + j];
      c[i * ldc + j] = acc;
    }
}

/* bf16 in, f32 accumulate, bf16 out: the semantics of the reference's GPU
   route (runtime/cuda_dispatch.cpp:1014-1022, cublasGemmEx with
   CUBLAS_COMPUTE_32F and a bf16 C).  Rows [row0,row1) only, so that a large
   product can be checked on a sample of rows. */
void oracle_gemm_bf16_rows(const uint16_t *a, int64_t lda, const uint16_t *b,
                           int64_t ldb, uint16_t *c, int64_t ldc, int64_t n,
                           int64_t k, const int64_t *rows, int64_t nrows) {
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t r = 0; r < nrows; ++r) {
    const int64_t i = rows[r];
    std::vector<float> acc((size_t)n, 0.0f);
    for (int64_t q = 0; q < k; ++q) {
      const float av = bf16_to_f32(a[i * lda + q]);
      const uint16_t *brow = b + q * ldb;
      for (int64_t j = 0; j < n; ++j)
        acc[(size_t)j] += av * bf16_to_f32(brow[j]);
    }
    for (int64_t j = 0; j < n; ++j)
      c[r * ldc + j] = f32_to_bf16(acc[(size_t)j]);
  }
}

/* One entry of a bf16 product in f32, k ascending: the sampled check of
   benchmarks/gpu_gemm/cublas_gemm.cu:84-92. */
float oracle_gemm_bf16_entry(const uint16_t *a, int64_t lda, const uint16_t *b,
                             int64_t ldb, int64_t i, int64_t j, int64_t k) {
  float want = 0.0f;
  for (int64_t q = 0; q < k; ++q)
    want += bf16_to_f32(a[i * lda + q]) * bf16_to_f32(b[q * ldb + j]);
  return want;
}

/* xout[i] = sum_j w[i*n+j] * x[j]: the host loop of
   vx_plugin_dispatch_async_flat, runtime/cuda_dispatch.cpp:1865-1874. */
void oracle_matvec_f32(float *xout, const float *x, const float *w, int n,
                       int d) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < d; ++i) {
    float acc = 0.0f;
    for (int j = 0; j < n; ++j)
      acc += w[(int64_t)i * n + j] * x[j];
    xout[i] = acc;
  }
}

/* ---- the integer mixer of the std::nn parity test ---------------------------
 * tests/optimizations/pass/std_nn_kernels_match_loops_on_the_cpu.vx:45-60.   */
static inline uint32_t mix32(uint32_t x) {
  uint32_t h = x * 2654435761u;
  h ^= h >> 15;
  h *= 2246822519u;
  h ^= h >> 13;
  return h;
}
float oracle_random(uint32_t seed, int32_t i, float scale) {
  return ((float)(mix32(seed * 7919u + (uint32_t)i) >> 8) * 0.00000011920929f -
          1.0f) *
         scale;
}
void oracle_random_f32(float *out, int64_t n, uint32_t seed, float scale) {
  for (int64_t i = 0; i < n; ++i)
    out[i] = oracle_random(seed, (int32_t)i, scale);
}

/* ---- Llama-2 decode in f32, as tests/backend/pass/llama2.vx runs it ---------
 * transformer<D> :218-429, rmsnorm :476-498, sample_argmax :460-474,
 * rope_freq tests/modules/llama_rt.vx:82-85.  Weights in llama2.c order
 * (memory_map_weights :125-147); the classifier shares the embedding table.  */
typedef struct {
  int32_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
} oracle_llama_config;

typedef struct {
  const float *tok, *rms_att, *wq, *wk, *wv, *wo, *rms_ffn, *w1, *w2, *w3,
      *rms_final;
} llama_weights;

static llama_weights map_weights(const float *p, const oracle_llama_config *c) {
  llama_weights w;
  const int64_t dim = c->dim, L = c->n_layers, hs = c->dim / c->n_heads;
  const int64_t kv = c->n_kv_heads * hs, hid = c->hidden_dim;
  w.tok = p;
  p += (int64_t)c->vocab_size * dim;
  w.rms_att = p;
  p += L * dim;
  w.wq = p;
  p += L * dim * dim;
  w.wk = p;
  p += L * dim * kv;
  w.wv = p;
  p += L * dim * kv;
  w.wo = p;
  p += L * dim * dim;
  w.rms_ffn = p;
  p += L * dim;
  w.w1 = p;
  p += L * dim * hid;
  w.w2 = p;
  p += L * hid * dim;
  w.w3 = p;
  p += L * dim * hid;
  w.rms_final = p;
  return w;
}

int64_t oracle_llama_weight_count(const oracle_llama_config *c) {
  const int64_t dim = c->dim, L = c->n_layers, hs = c->dim / c->n_heads;
  const int64_t kv = c->n_kv_heads * hs, hid = c->hidden_dim;
  return (int64_t)c->vocab_size * dim + L * dim + L * dim * dim +
         2 * L * dim * kv + L * dim * dim + L * dim + 3 * L * dim * hid + dim;
}

static void rmsnorm_f32(float *o, const float *x, const float *w, int n) {
  float ss = 0.0f;
  for (int j = 0; j < n; ++j)
    ss += x[j] * x[j];
  ss = ss / (float)n + 0.00001f;
  ss = 1.0f / cr_sqrtf(ss);
  for (int j = 0; j < n; ++j) {
    const float t = ss * x[j];
    o[j] = w[j] * t;
  }
}

/* One token at position pos. key_cache/value_cache are [L, seq_len, kv_dim];
   logits gets vocab_size values. scratch >= 4*dim + 2*hidden + heads*seq_len. */
void oracle_llama_forward(const oracle_llama_config *c, const float *weights,
                          float *key_cache, float *value_cache, int32_t token,
                          int32_t pos, float *logits) {
  const llama_weights w = map_weights(weights, c);
  const int dim = c->dim, hid = c->hidden_dim, heads = c->n_heads;
  const int hs = dim / heads, kv_dim = c->n_kv_heads * hs;
  const int kv_mul = heads / c->n_kv_heads, seq = c->seq_len;
  std::vector<float> x(dim), xb(dim), xb2(dim), q(dim), hb(hid), hb2(hid),
      att((size_t)heads * seq);

  memcpy(x.data(), w.tok + (int64_t)token * dim, sizeof(float) * dim);
  for (int l = 0; l < c->n_layers; ++l) {
    rmsnorm_f32(xb.data(), x.data(), w.rms_att + (int64_t)l * dim, dim);
    float *kp = key_cache + ((int64_t)l * seq + pos) * kv_dim;
    float *vp = value_cache + ((int64_t)l * seq + pos) * kv_dim;
    oracle_matvec_f32(q.data(), xb.data(), w.wq + (int64_t)l * dim * dim, dim,
                      dim);
    oracle_matvec_f32(kp, xb.data(), w.wk + (int64_t)l * dim * kv_dim, dim,
                      kv_dim);
    oracle_matvec_f32(vp, xb.data(), w.wv + (int64_t)l * dim * kv_dim, dim,
                      kv_dim);
    /* RoPE on interleaved pairs; the loop runs over kv_dim as the program's
       does, and turns q and k at the same indices. */
    for (int i = 0; i < kv_dim; i += 2) {
      const int in_head = i % hs;
      const float angle =
          (float)pos * cr_powf(10000.0f, -(float)in_head / (float)hs);
      const float fc = cr_cosf(angle), fs = cr_sinf(angle);
      const float q0 = q[i], q1 = q[i + 1];
      q[i] = q0 * fc - q1 * fs;
      q[i + 1] = q0 * fs + q1 * fc;
      const float k0 = kp[i], k1 = kp[i + 1];
      kp[i] = k0 * fc - k1 * fs;
      kp[i + 1] = k0 * fs + k1 * fc;
    }
    /* With fewer kv heads than heads the program's loop stops at kv_dim, so q
       beyond it is not turned there; turn the rest of q the same way so that
       grouped-query models are still a rotation of every q head. */
    for (int i = kv_dim; i < dim; i += 2) {
      const int in_head = i % hs;
      const float angle =
          (float)pos * cr_powf(10000.0f, -(float)in_head / (float)hs);
      const float fc = cr_cosf(angle), fs = cr_sinf(angle);
      const float q0 = q[i], q1 = q[i + 1];
      q[i] = q0 * fc - q1 * fs;
      q[i + 1] = q0 * fs + q1 * fc;
    }
#pragma omp parallel for schedule(static)
    for (int h = 0; h < heads; ++h) {
      float *a = att.data() + (size_t)h * seq;
      const float *qh = q.data() + h * hs;
      const int64_t base = (int64_t)l * seq * kv_dim + (h / kv_mul) * hs;
      const float factor = 1.0f / cr_sqrtf((float)hs);
      for (int t = 0; t <= pos; ++t) {
        const float *kt = key_cache + base + (int64_t)t * kv_dim;
        float score = 0.0f;
        for (int i = 0; i < hs; ++i)
          score += qh[i] * kt[i];
        a[t] = score * factor;
      }
      float mx = a[0];
      for (int t = 1; t <= pos; ++t)
        if (a[t] > mx)
          mx = a[t];
      float sum = 0.0f;
      for (int t = 0; t <= pos; ++t) {
        a[t] = cr_expf(a[t] - mx);
        sum += a[t];
      }
      for (int t = 0; t <= pos; ++t)
        a[t] = a[t] / sum;
      for (int i = 0; i < hs; ++i) {
        float val = 0.0f;
        for (int t = 0; t <= pos; ++t)
          val += a[t] * value_cache[base + (int64_t)t * kv_dim + i];
        xb[h * hs + i] = val;
      }
    }
    oracle_matvec_f32(xb2.data(), xb.data(), w.wo + (int64_t)l * dim * dim, dim,
                      dim);
    for (int i = 0; i < dim; ++i)
      x[i] = x[i] + xb2[i];
    rmsnorm_f32(xb.data(), x.data(), w.rms_ffn + (int64_t)l * dim, dim);
    oracle_matvec_f32(hb.data(), xb.data(), w.w1 + (int64_t)l * dim * hid, dim,
                      hid);
    oracle_matvec_f32(hb2.data(), xb.data(), w.w3 + (int64_t)l * dim * hid, dim,
                      hid);
    for (int i = 0; i < hid; ++i) {
      const float v = hb[i];
      const float factor = 1.0f / (1.0f + cr_expf(0.0f - v));
      hb[i] = (v * factor) * hb2[i];
    }
    oracle_matvec_f32(xb.data(), hb.data(), w.w2 + (int64_t)l * dim * hid, hid,
                      dim);
    for (int i = 0; i < dim; ++i)
      x[i] = x[i] + xb[i];
  }
  rmsnorm_f32(x.data(), x.data(), w.rms_final, dim);
  oracle_matvec_f32(logits, x.data(), w.tok, dim, c->vocab_size);
}

/* Strict `>`: the first of equal largest values wins (llama2.vx:460-474). */
int32_t oracle_argmax_f32(const float *v, int32_t n) {
  int32_t at = 0;
  float best = v[0];
  for (int32_t i = 1; i < n; ++i)
    if (v[i] > best) {
      best = v[i];
      at = i;
    }
  return at;
}

/* Greedy decode: tokens[0] is given (BOS); fills tokens[1..steps]. When gaps
   is not NULL, gaps[s] is the difference between the two largest logits of
   step s, so a test can say how close a disagreement was. */
void oracle_llama_generate(const oracle_llama_config *c, const float *weights,
                           int32_t *tokens, int32_t steps, float *gaps) {
  const int kv_dim = c->n_kv_heads * (c->dim / c->n_heads);
  std::vector<float> kc((size_t)c->n_layers * c->seq_len * kv_dim, 0.0f),
      vc(kc.size(), 0.0f), logits((size_t)c->vocab_size);
  for (int32_t s = 0; s < steps; ++s) {
    oracle_llama_forward(c, weights, kc.data(), vc.data(), tokens[s], s,
                         logits.data());
    const int32_t best = oracle_argmax_f32(logits.data(), c->vocab_size);
    tokens[s + 1] = best;
    if (gaps) {
      float second = -INFINITY;
      for (int32_t i = 0; i < c->vocab_size; ++i)
        if (i != best && logits[(size_t)i] > second)
          second = logits[(size_t)i];
      gaps[s] = logits[(size_t)best] - second;
    }
  }
}

/* ---- std::nn operators: bf16 weights, f32 everything else -------------------
 * stdlib/std/nn.vx. The dot products follow the kernels' own order: lane l of
 * 128 adds columns l*8..l*8+7, then +1024, ...; the 128 lane sums are then
 * added in lane order (nn.vx:27-47).                                         */
static float lane_dot(const uint16_t *wrow, const float *x, int cols) {
  float total = 0.0f;
  for (int l = 0; l < 128; ++l) {
    float acc = 0.0f;
    for (int c = l * 8; c < cols; c += 1024)
      for (int e = 0; e < 8; ++e)
        acc = acc + bf16_to_f32(wrow[c + e]) * x[c + e];
    total += acc;
  }
  return total;
}

/* nn_matvec :24-51 (mode 0), nn_matvec_add :54-81 and nn_matvec_heads_add
   :86-118 (mode 1: y += ...; a [heads, head_dim] x is the same flat vector). */
void oracle_nn_matvec(float *y, const uint16_t *w, const float *x, int rows,
                      int cols, int add) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const float s = lane_dot(w + (int64_t)r * cols, x, cols);
    y[r] = add ? y[r] + s : s;
  }
}

/* nn_qkv :124-164: rows are q heads, then k heads, then v heads, plus bias. */
void oracle_nn_qkv(float *q, float *k, float *v, const uint16_t *w,
                   const uint16_t *b, const float *x, int q_heads, int kv_heads,
                   int head_dim, int cols) {
  const int rows = (q_heads + 2 * kv_heads) * head_dim;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const float s =
        lane_dot(w + (int64_t)r * cols, x, cols) + bf16_to_f32(b[r]);
    if (r < q_heads * head_dim)
      q[r] = s;
    else if (r < (q_heads + kv_heads) * head_dim)
      k[r - q_heads * head_dim] = s;
    else
      v[r - (q_heads + kv_heads) * head_dim] = s;
  }
}

/* nn_swiglu :169-209: rows of gate, then rows of up; silu(g)*u with
   g / (1 + exp(-g)). */
void oracle_nn_swiglu(float *out, const uint16_t *w, const float *x, int rows,
                      int cols) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const float g = lane_dot(w + (int64_t)r * cols, x, cols);
    const float u = lane_dot(w + (int64_t)(rows + r) * cols, x, cols);
    out[r] = g / (1.0f + cr_expf(0.0f - g)) * u;
  }
}

/* nn_rms_norm :212-239: 1024 lanes each add every 1024th square, the lane sums
   are added in lane order, inv = 1/sqrt(ss/n + eps), y = x*inv*w. */
void oracle_nn_rms_norm(float *y, const float *x, const uint16_t *w, int n,
                        float eps) {
  float ss = 0.0f;
  for (int l = 0; l < 1024; ++l) {
    float s = 0.0f;
    for (int i = l; i < n; i += 1024)
      s = s + x[i] * x[i];
    ss += s;
  }
  const float inv = 1.0f / cr_sqrtf(ss / (float)n + eps);
  for (int i = 0; i < n; ++i)
    y[i] = x[i] * inv * bf16_to_f32(w[i]);
}

/* nn_rope_and_store :245-280: value i pairs with i + head_dim/2; k and v go to
   row pos of caches shaped [max_seq, kv_heads, head_dim]; cos/sin are
   [max_seq, cs_cols] with cs_cols >= head_dim/2. */
void oracle_nn_rope_and_store(float *q_out, float *k_cache, float *v_cache,
                              const float *q, const float *k, const float *v,
                              const float *cos_t, const float *sin_t,
                              int cs_cols, int pos, int q_heads, int kv_heads,
                              int head_dim) {
  const int half = head_dim / 2;
  for (int h = 0; h < q_heads + kv_heads; ++h)
    for (int i = 0; i < head_dim; ++i) {
      const int j = i < half ? i : i - half;
      const float sign = i < half ? -1.0f : 1.0f;
      const int partner = i < half ? i + half : i - half;
      const float c = cos_t[(int64_t)pos * cs_cols + j];
      const float s = sin_t[(int64_t)pos * cs_cols + j];
      if (h < q_heads) {
        const float *qh = q + h * head_dim;
        q_out[h * head_dim + i] = qh[i] * c + sign * qh[partner] * s;
      } else {
        const int g = h - q_heads;
        const float *kh = k + g * head_dim;
        const int64_t at = ((int64_t)pos * kv_heads + g) * head_dim + i;
        k_cache[at] = kh[i] * c + sign * kh[partner] * s;
        v_cache[at] = v[g * head_dim + i];
      }
    }
}

/* nn_attention :349-380 with its parts (:383-821) and merge (:825-866): the
   positions are split in blocks of 32 (pos < 640) or 64; each block gives a
   weighted sum of V, its largest score and its sum of weights; the merge
   rescales by exp(block max - overall max). Same arithmetic, one head at a
   time. */
void oracle_nn_attention(float *out, const float *q, const float *k_cache,
                         const float *v_cache, int pos, int q_heads,
                         int kv_heads, int head_dim) {
  const int group = q_heads / kv_heads;
  const int n_pos = pos >= 640 ? 64 : 32;
  const int splits = (pos + n_pos) / n_pos;
  const float scale = 1.0f / cr_sqrtf((float)head_dim);
#pragma omp parallel for schedule(static)
  for (int h = 0; h < q_heads; ++h) {
    const int g = h / group;
    std::vector<float> part((size_t)splits * (head_dim + 2));
    std::vector<float> wgt((size_t)n_pos);
    for (int c = 0; c < splits; ++c) {
      float big = -3.0e38f;
      for (int l = 0; l < n_pos; ++l) {
        const int t = c * n_pos + l;
        float s = -3.0e38f;
        if (t <= pos) {
          float dot = 0.0f;
          const float *kr = k_cache + ((int64_t)t * kv_heads + g) * head_dim;
          for (int d = 0; d < head_dim; ++d)
            dot = dot + q[h * head_dim + d] * kr[d];
          s = dot * scale;
        }
        wgt[(size_t)l] = s;
        big = fmaxf(big, s);
      }
      float total = 0.0f;
      for (int l = 0; l < n_pos; ++l) {
        wgt[(size_t)l] = cr_expf(wgt[(size_t)l] - big);
        total += wgt[(size_t)l];
      }
      int last = pos - c * n_pos;
      if (last > n_pos - 1)
        last = n_pos - 1;
      float *p = part.data() + (size_t)c * (head_dim + 2);
      for (int d = 0; d < head_dim; ++d) {
        float acc = 0.0f;
        for (int t = 0; t <= last; ++t)
          acc = acc + wgt[(size_t)t] *
                          v_cache[((int64_t)(c * n_pos + t) * kv_heads + g) *
                                      head_dim +
                                  d];
        p[d] = acc;
      }
      p[head_dim] = big;
      p[head_dim + 1] = total;
    }
    float big = -3.0e38f;
    for (int c = 0; c < splits; ++c)
      big = fmaxf(big, part[(size_t)c * (head_dim + 2) + head_dim]);
    for (int d = 0; d < head_dim; ++d) {
      float total = 0.0f, acc = 0.0f;
      for (int c = 0; c < splits; ++c) {
        const float *p = part.data() + (size_t)c * (head_dim + 2);
        const float w = cr_expf(p[head_dim] - big);
        total = total + w * p[head_dim + 1];
        acc = acc + w * p[d];
      }
      out[h * head_dim + d] = acc / total;
    }
  }
}

/* The f64 loop the reference's own test compares nn_attention with
   (std_nn_kernels_match_loops_on_the_cpu.vx:347-390). */
void oracle_attention_f64(double *want, const float *q, const float *k_cache,
                          const float *v_cache, int pos, int q_heads,
                          int kv_heads, int head_dim) {
  const int group = q_heads / kv_heads;
  const double scale = 1.0 / sqrt((double)head_dim);
#pragma omp parallel for schedule(static)
  for (int h = 0; h < q_heads; ++h) {
    const int g = h / group;
    std::vector<double> p((size_t)pos + 1);
    double m = -1.0e300;
    for (int t = 0; t <= pos; ++t) {
      double s = 0.0;
      for (int d = 0; d < head_dim; ++d)
        s += (double)q[h * head_dim + d] *
             (double)k_cache[((int64_t)t * kv_heads + g) * head_dim + d];
      p[(size_t)t] = s * scale;
      m = fmax(m, p[(size_t)t]);
    }
    double total = 0.0;
    for (int t = 0; t <= pos; ++t) {
      p[(size_t)t] = exp(p[(size_t)t] - m);
      total += p[(size_t)t];
    }
    for (int d = 0; d < head_dim; ++d) {
      double acc = 0.0;
      for (int t = 0; t <= pos; ++t)
        acc += p[(size_t)t] *
               (double)v_cache[((int64_t)t * kv_heads + g) * head_dim + d];
      want[h * head_dim + d] = acc / total;
    }
  }
}

/* nn_argmax :870-897: the lowest index wins a tie. */
int32_t oracle_nn_argmax(const float *logits, int32_t n) {
  return oracle_argmax_f32(logits, n);
}

/* nn_embed :942-958. */
void oracle_nn_embed(float *x, const uint16_t *table, int32_t token, int dim) {
  for (int i = 0; i < dim; ++i)
    x[i] = bf16_to_f32(table[(int64_t)token * dim + i]);
}

/* cos/sin tables the way the reference's test makes them
   (std_nn_kernels_match_loops_on_the_cpu.vx:262-272): angle = p / theta^(2i/hd)
   in f64, rounded to f32. */
void oracle_rope_tables(float *cos_t, float *sin_t, int max_seq, int head_dim,
                        double theta) {
  const int half = head_dim / 2;
  for (int p = 0; p < max_seq; ++p)
    for (int i = 0; i < half; ++i) {
      const double angle =
          (double)p / pow(theta, (double)(2 * i) / (double)head_dim);
      cos_t[(int64_t)p * half + i] = (float)cos(angle);
      sin_t[(int64_t)p * half + i] = (float)sin(angle);
    }
}

/* ---- fp8 and Q4_0 weights (nn.vx:1296-1303 and 1645-1663) ---------------------
 * The restatements keep the reference kernels' order of sums; the *_f64
 * functions are the plain loops of the reference's own tests
 * (std_nn_fp8_kernels_match_loops_on_the_cpu.vx:82-103,
 * std_nn_q4_kernels_match_loops_on_the_cpu.vx:119-131), against which those
 * tests accept max |got - want| <= 1e-5 max |want|. */

/* The value of an f8e4m3 code as the kernels' table has it (nn.vx:1316-1326):
   e = 0 gives m * 2^-9; else the bits with 120 added to the exponent. */
static inline float fp8_value(uint32_t code) {
  const uint32_t mag = code & 127u;
  float value;
  if (mag < 8u) {
    value = (float)mag * 0.001953125f;
  } else {
    const uint32_t bits = (mag << 20) + 1006632960u;
    memcpy(&value, &bits, 4);
  }
  return code & 128u ? 0.0f - value : value;
}
static inline double fp8_value_f64(uint32_t code) {
  const int e = (int)((code >> 3) & 15u);
  const double m = (double)(code & 7u);
  double v = e == 0 ? m / 8.0 * ldexp(1.0, -6) : (1.0 + m / 8.0) * ldexp(1.0, e - 7);
  return code >= 128u ? 0.0 - v : v;
}
static inline uint32_t fp8_code(const uint32_t *w, int64_t at) {
  return (w[at / 4] >> (8u * (uint32_t)(at % 4))) & 255u;
}

/* One row of nn_matvec_fp8 (nn.vx:1306-1363): 128 lanes, lane l takes the 8
   columns l*8.. of every 1024; the 8 products are added left to right, the sum
   times the block's scale joins the lane's total; the lanes are added in lane
   order. srow: the row of the scales table (row / 128 of the whole matrix). */
static float fp8_row(const uint32_t *w, int64_t first_code, const float *scales,
                     int srow, const float *x, int cols) {
  const int tiles = cols / 128;
  float total = 0.0f;
  for (int l = 0; l < 128; ++l) {
    float acc = 0.0f;
    for (int c = l * 8; c < cols; c += 1024) {
      float sum = fp8_value(fp8_code(w, first_code + c)) * x[c];
      for (int k = 1; k < 8; ++k)
        sum = sum + fp8_value(fp8_code(w, first_code + c + k)) * x[c + k];
      acc = acc + sum * scales[srow * tiles + c / 128];
    }
    total += acc;
  }
  return total;
}

/* nn_matvec_fp8 :1306, nn_matvec_fp8_add :1367, nn_matvec_fp8_heads_add :1427
   (add = 1); row_base: the row of the whole matrix that row 0 here is. */
void oracle_nn_matvec_fp8(float *y, const uint32_t *w, const float *scales,
                          const float *x, int rows, int cols, int add,
                          int row_base) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const int whole = row_base + r;
    const float s = fp8_row(w, (int64_t)whole * cols, scales, whole / 128, x, cols);
    y[r] = add ? y[r] + s : s;
  }
}
/* nn_swiglu_fp8 :1577-1640 */
void oracle_nn_swiglu_fp8(float *out, const uint32_t *w, const float *scales,
                          const float *x, int rows, int cols) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const float g = fp8_row(w, (int64_t)r * cols, scales, r / 128, x, cols);
    const float u = fp8_row(w, (int64_t)(rows + r) * cols, scales,
                            (rows + r) / 128, x, cols);
    out[r] = g / (1.0f + cr_expf(0.0f - g)) * u;
  }
}
void oracle_fp8_dot_f64(double *want, const uint32_t *w, const float *scales,
                        const float *x, int rows, int cols) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    double sum = 0.0;
    for (int c = 0; c < cols; ++c)
      sum = sum + fp8_value_f64(fp8_code(w, (int64_t)r * cols + c)) *
                      (double)scales[(r / 128) * (cols / 128) + c / 128] *
                      (double)x[c];
    want[r] = sum;
  }
}

/* IEEE half to float (the scales of Q4_0 are f16). */
static inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t e = (h >> 10) & 31u, m = h & 1023u;
  uint32_t bits;
  if (e == 0) {
    if (m == 0) {
      bits = sign;
    } else { /* subnormal: m * 2^-24 */
      float v = (float)m * 5.9604644775390625e-8f;
      memcpy(&bits, &v, 4);
      bits |= sign;
    }
  } else if (e == 31) {
    bits = sign | 0x7F800000u | (m << 13);
  } else {
    bits = sign | ((e + 112u) << 23) | (m << 13);
  }
  float out;
  memcpy(&out, &bits, 4);
  return out;
}

/* One row of nn_matvec_q4 (nn.vx:1666-1744): 32 lanes, lane l takes the two
   words 2l, 2l+1 of every 64 (16 weights, one scale); a code in nibble t
   enters as (word & mask_t) times x / 16^t, the 8 of every code comes off as
   8 times the sum of the 16 values of x; the 16 products are added left to
   right; (dot - sum8) times the scale joins the lane's total; the lanes are
   added in lane order. w: this row's words; scales: this row's. */
static float q4_row(const uint32_t *w, const uint16_t *scales, const float *x,
                    int cols) {
  const int words = cols / 8;
  static const float inv16[8] = {1.0f, 0.0625f, 0.00390625f, 0.000244140625f,
                                 0.0000152587890625f, 0.00000095367431640625f,
                                 0.000000059604644775390625f,
                                 0.0000000037252902984619140625f};
  float total = 0.0f;
  for (int l = 0; l < 32; ++l) {
    float acc = 0.0f;
    for (int i = l * 2; i < words; i += 64) {
      const int c = i * 8;
      float xp[16];
      for (int t = 0; t < 16; ++t)
        xp[t] = x[c + t];
      float sum = xp[0];
      for (int t = 1; t < 16; ++t)
        sum = sum + xp[t];
      const float sum8 = 8.0f * sum;
      for (int t = 0; t < 16; ++t)
        xp[t] = xp[t] * inv16[t & 7];
      float dot = 0.0f;
      for (int t = 0; t < 16; ++t) {
        const uint32_t word = w[i + t / 8];
        const float masked = (float)(word & (15u << (4 * (t & 7))));
        dot = t == 0 ? masked * xp[0] : dot + masked * xp[t];
      }
      acc = acc + (dot - sum8) * f16_to_f32(scales[i / 4]);
    }
    total += acc;
  }
  return total;
}
/* nn_matvec_q4 :1666, _add :1748, _heads_add :1831 */
void oracle_nn_matvec_q4(float *y, const uint32_t *w, const uint16_t *scales,
                         const float *x, int rows, int cols, int add) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const float s = q4_row(w + (int64_t)r * (cols / 8),
                           scales + (int64_t)r * (cols / 32), x, cols);
    y[r] = add ? y[r] + s : s;
  }
}
/* nn_swiglu_q4 :2005-2100 */
void oracle_nn_swiglu_q4(float *out, const uint32_t *w, const uint16_t *scales,
                         const float *x, int rows, int cols) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const float g = q4_row(w + (int64_t)r * (cols / 8),
                           scales + (int64_t)r * (cols / 32), x, cols);
    const float u = q4_row(w + (int64_t)(rows + r) * (cols / 8),
                           scales + (int64_t)(rows + r) * (cols / 32), x, cols);
    out[r] = g / (1.0f + cr_expf(0.0f - g)) * u;
  }
}
void oracle_q4_dot_f64(double *want, const uint32_t *w, const uint16_t *scales,
                       const float *x, int rows, int cols) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    double t = 0.0;
    for (int c = 0; c < cols; ++c) {
      const uint32_t word = w[(int64_t)r * (cols / 8) + c / 8];
      const int code = (int)((word >> (4 * (c % 8))) & 15u);
      t = t + (double)(code - 8) *
                  (double)f16_to_f32(scales[(int64_t)r * (cols / 32) + c / 32]) *
                  (double)x[c];
    }
    want[r] = t;
  }
}
/* The tests' generators: word i of the random tensor `seed` is
   mix(seed * 7919 + i); an fp8 word has no NaN code (0x7f, 0xff): such a byte
   is lowered by one (std_nn_fp8_kernels_match_loops_on_the_cpu.vx:41-50). */
void oracle_random_words(uint32_t *out, int64_t n, uint32_t seed, int fp8) {
  for (int64_t i = 0; i < n; ++i) {
    uint32_t word = mix32(seed * 7919u + (uint32_t)i);
    if (fp8)
      for (int k = 0; k < 4; ++k)
        if (((word >> (8 * k)) & 127u) == 127u)
          word = word - (1u << (8 * k));
    out[i] = word;
  }
}

/* nn_top_k (nn.vx:904-938): keys = the value's bits in an order that keeps the
   order of the values, then 255 - index; sorted descending; the softmax of
   the k first, summed in that order. */
void oracle_nn_top_k(int32_t *ids, float *weights, const float *logits, int n,
                     int k) {
  std::vector<int64_t> keys((size_t)n);
  for (int l = 0; l < n; ++l) {
    int32_t bits;
    memcpy(&bits, &logits[l], 4);
    const int32_t order = bits < 0 ? bits ^ 2147483647 : bits;
    keys[(size_t)l] = (int64_t)order * 4294967296ll + (int64_t)(255 - l);
  }
  for (int a = 1; a < n; ++a) { /* insertion sort, descending */
    const int64_t key = keys[(size_t)a];
    int b = a - 1;
    while (b >= 0 && keys[(size_t)b] < key) {
      keys[(size_t)b + 1] = keys[(size_t)b];
      --b;
    }
    keys[(size_t)b + 1] = key;
  }
  const float m = logits[255 - (int)(keys[0] & 255)];
  float total = 0.0f;
  for (int t = 0; t < k; ++t)
    total = total + cr_expf(logits[255 - (int)(keys[(size_t)t] & 255)] - m);
  for (int l = 0; l < k; ++l) {
    const int id = 255 - (int)(keys[(size_t)l] & 255);
    ids[l] = id;
    weights[l] = cr_expf(logits[id] - m) / total;
  }
}

/* ---- a decoder of std::nn operators (the 7B-shaped configuration) -----------
 * Per layer, in this order: attn_norm[dim], wqkv[(q+2kv)*hd, dim],
 * bqkv[(q+2kv)*hd], wo[dim, q*hd], ffn_norm[dim], w_gate_up[2*hidden, dim],
 * w_down[dim, hidden]; then final_norm[dim], lm_head[vocab, dim]; the
 * embedding table [vocab, dim] is separate. All bf16. */
typedef struct {
  int32_t dim, hidden, n_layers, q_heads, kv_heads, head_dim, vocab, max_seq;
  float eps;
  float rope_theta;
} oracle_nn_config;

int64_t oracle_nn_layer_params(const oracle_nn_config *c) {
  const int64_t qkv = (int64_t)(c->q_heads + 2 * c->kv_heads) * c->head_dim;
  return c->dim + qkv * c->dim + qkv + (int64_t)c->dim * c->q_heads * c->head_dim +
         c->dim + 2 * (int64_t)c->hidden * c->dim + (int64_t)c->dim * c->hidden;
}

/* k_cache/v_cache: [L, max_seq, kv_heads, head_dim] f32. Returns the argmax
   token; logits (vocab) may be NULL. */
int32_t oracle_nn_decode_step(const oracle_nn_config *c, const uint16_t *embed,
                              const uint16_t *layers,
                              const uint16_t *final_norm,
                              const uint16_t *lm_head, const float *cos_t,
                              const float *sin_t, float *k_cache,
                              float *v_cache, int32_t token, int32_t pos,
                              float *logits_out) {
  const int dim = c->dim, hd = c->head_dim, qh = c->q_heads, kvh = c->kv_heads;
  const int qkv_rows = (qh + 2 * kvh) * hd;
  std::vector<float> x(dim), xb(dim), q((size_t)qh * hd), k((size_t)kvh * hd),
      v((size_t)kvh * hd), qr((size_t)qh * hd), att((size_t)qh * hd),
      h((size_t)c->hidden), logits((size_t)c->vocab);
  oracle_nn_embed(x.data(), embed, token, dim);
  const int64_t per_layer = oracle_nn_layer_params(c);
  const int64_t cache_layer = (int64_t)c->max_seq * kvh * hd;
  for (int l = 0; l < c->n_layers; ++l) {
    const uint16_t *p = layers + (int64_t)l * per_layer;
    const uint16_t *attn_norm = p;
    p += dim;
    const uint16_t *wqkv = p;
    p += (int64_t)qkv_rows * dim;
    const uint16_t *bqkv = p;
    p += qkv_rows;
    const uint16_t *wo = p;
    p += (int64_t)dim * qh * hd;
    const uint16_t *ffn_norm = p;
    p += dim;
    const uint16_t *wgu = p;
    p += 2 * (int64_t)c->hidden * dim;
    const uint16_t *wdown = p;
    float *kc = k_cache + l * cache_layer, *vc = v_cache + l * cache_layer;
    oracle_nn_rms_norm(xb.data(), x.data(), attn_norm, dim, c->eps);
    oracle_nn_qkv(q.data(), k.data(), v.data(), wqkv, bqkv, xb.data(), qh, kvh,
                  hd, dim);
    oracle_nn_rope_and_store(qr.data(), kc, vc, q.data(), k.data(), v.data(),
                             cos_t, sin_t, hd / 2, pos, qh, kvh, hd);
    oracle_nn_attention(att.data(), qr.data(), kc, vc, pos, qh, kvh, hd);
    oracle_nn_matvec(x.data(), wo, att.data(), dim, qh * hd, 1);
    oracle_nn_rms_norm(xb.data(), x.data(), ffn_norm, dim, c->eps);
    oracle_nn_swiglu(h.data(), wgu, xb.data(), c->hidden, dim);
    oracle_nn_matvec(x.data(), wdown, h.data(), dim, c->hidden, 1);
  }
  oracle_nn_rms_norm(xb.data(), x.data(), final_norm, dim, c->eps);
  oracle_nn_matvec(logits.data(), lm_head, xb.data(), c->vocab, dim, 0);
  if (logits_out)
    memcpy(logits_out, logits.data(), sizeof(float) * (size_t)c->vocab);
  return oracle_nn_argmax(logits.data(), c->vocab);
}

/* The same step with the four projections of every layer in fp8 (quant 2) or
   Q4_0 (quant 3): nn_qkv_fp8 / nn_matvec_fp8_heads_add / nn_swiglu_fp8 /
   nn_matvec_fp8_add, or their q4 twins, in place of the bf16 kernels. Norms,
   bias, embedding and classifier stay bf16. layer[l * 11 + i]: attn_norm,
   wqkv codes, wqkv scales, bqkv, wo codes, wo scales, ffn_norm, gate/up
   codes, gate/up scales, down codes, down scales. */
int32_t oracle_nn_decode_step_quant(const oracle_nn_config *c, int quant,
                                    const uint16_t *embed,
                                    const void *const *layer,
                                    const uint16_t *final_norm,
                                    const uint16_t *lm_head, const float *cos_t,
                                    const float *sin_t, float *k_cache,
                                    float *v_cache, int32_t token, int32_t pos,
                                    float *logits_out) {
  const int dim = c->dim, hd = c->head_dim, qh = c->q_heads, kvh = c->kv_heads;
  const int qkv_rows = (qh + 2 * kvh) * hd;
  std::vector<float> x(dim), xb(dim), qkv((size_t)qkv_rows), qr((size_t)qh * hd),
      att((size_t)qh * hd), h((size_t)c->hidden), logits((size_t)c->vocab);
  oracle_nn_embed(x.data(), embed, token, dim);
  const int64_t cache_layer = (int64_t)c->max_seq * kvh * hd;
  auto matvec = [&](float *y, const void *w, const void *s, const float *in,
                    int rows, int cols, int add) {
    if (quant == 2)
      oracle_nn_matvec_fp8(y, (const uint32_t *)w, (const float *)s, in, rows,
                           cols, add, 0);
    else
      oracle_nn_matvec_q4(y, (const uint32_t *)w, (const uint16_t *)s, in, rows,
                          cols, add);
  };
  for (int l = 0; l < c->n_layers; ++l) {
    const void *const *p = layer + (int64_t)l * 11;
    float *kc = k_cache + l * cache_layer, *vc = v_cache + l * cache_layer;
    oracle_nn_rms_norm(xb.data(), x.data(), (const uint16_t *)p[0], dim, c->eps);
    matvec(qkv.data(), p[1], p[2], xb.data(), qkv_rows, dim, 0);
    const uint16_t *bias = (const uint16_t *)p[3];
    for (int r = 0; r < qkv_rows; ++r)
      qkv[r] = qkv[r] + bf16_to_f32(bias[r]);
    oracle_nn_rope_and_store(qr.data(), kc, vc, qkv.data(),
                             qkv.data() + (size_t)qh * hd,
                             qkv.data() + (size_t)(qh + kvh) * hd, cos_t, sin_t,
                             hd / 2, pos, qh, kvh, hd);
    oracle_nn_attention(att.data(), qr.data(), kc, vc, pos, qh, kvh, hd);
    matvec(x.data(), p[4], p[5], att.data(), dim, qh * hd, 1);
    oracle_nn_rms_norm(xb.data(), x.data(), (const uint16_t *)p[6], dim, c->eps);
    if (quant == 2)
      oracle_nn_swiglu_fp8(h.data(), (const uint32_t *)p[7], (const float *)p[8],
                           xb.data(), c->hidden, dim);
    else
      oracle_nn_swiglu_q4(h.data(), (const uint32_t *)p[7],
                          (const uint16_t *)p[8], xb.data(), c->hidden, dim);
    matvec(x.data(), p[9], p[10], h.data(), dim, c->hidden, 1);
  }
  oracle_nn_rms_norm(xb.data(), x.data(), final_norm, dim, c->eps);
  oracle_nn_matvec(logits.data(), lm_head, xb.data(), c->vocab, dim, 0);
  if (logits_out)
    memcpy(logits_out, logits.data(), sizeof(float) * (size_t)c->vocab);
  return oracle_nn_argmax(logits.data(), c->vocab);
}

/* ---- attention over whole sequences (the flash-attention configuration) -----
 * softmax(q.k * scale) v with a causal mask, f32 from bf16-rounded inputs: the
 * loop of std_nn_kernels_match_loops_on_the_cpu.vx:347-390 for every query
 * row. q,k,v: [S, D] of one (batch, head); rows: which query rows to compute;
 * out: [nrows, D] f32. */
void oracle_attention_rows(const uint16_t *q, const uint16_t *k,
                           const uint16_t *v, int S, int D, float scale,
                           int causal, const int32_t *rows, int nrows,
                           float *out) {
#pragma omp parallel for schedule(dynamic, 1)
  for (int r = 0; r < nrows; ++r) {
    const int i = rows[r];
    const int last = causal ? i : S - 1;
    std::vector<float> p((size_t)last + 1);
    float m = -INFINITY;
    for (int t = 0; t <= last; ++t) {
      float s = 0.0f;
      for (int d = 0; d < D; ++d)
        s += bf16_to_f32(q[(int64_t)i * D + d]) *
             bf16_to_f32(k[(int64_t)t * D + d]);
      p[(size_t)t] = s * scale;
      m = fmaxf(m, p[(size_t)t]);
    }
    float total = 0.0f;
    for (int t = 0; t <= last; ++t) {
      p[(size_t)t] = cr_expf(p[(size_t)t] - m);
      total += p[(size_t)t];
    }
    for (int d = 0; d < D; ++d) {
      float acc = 0.0f;
      for (int t = 0; t <= last; ++t)
        acc += p[(size_t)t] * bf16_to_f32(v[(int64_t)t * D + d]);
      out[(int64_t)r * D + d] = acc / total;
    }
  }
}

/* ---- collectives: ranks in rank order (vx_collective.h:288-335 for one rank)*/
void oracle_all_reduce_sum_f32(const float *const *inputs, int ranks,
                               float *out, int64_t count) {
  for (int64_t i = 0; i < count; ++i) {
    float s = inputs[0][i];
    for (int r = 1; r < ranks; ++r)
      s += inputs[r][i];
    out[i] = s;
  }
}

} /* extern "C" */
