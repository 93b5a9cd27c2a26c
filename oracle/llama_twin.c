/* llama_twin.c -- TEST INFRASTRUCTURE.  A second, independent CPU restatement of
 * the f32 Llama-2 decode step, after the reference's CPU-only program
 * benchmarks/llama2_100.vx: transformer :206-335, attn :138-204 (ONLINE
 * softmax: a running maximum that starts at -999999, a running sum, and the
 * weighted values rescaled in place), rmsnorm :353-375, matmul :405-421,
 * sample_argmax :337-351, rope_freq tests/modules/llama_rt.vx:82-85.
 *
 * It shares no code with vx_oracle.cpp (which restates
 * tests/backend/pass/llama2.vx with its two-pass softmax): different loops,
 * different buffers, plain C, one thread.  The two programs of the reference
 * are meant to generate the same text; the test that requires the same 100
 * greedy tokens from both restatements is the cross-check of the decode
 * oracle (there is no known-answer token list in the reference tree: its
 * programs need a checkpoint file that is not part of it).
 *
 * Only tests/ load this file.  Built by oracle/build.py with
 * -ffp-contract=off: a multiply and the add after it are two roundings, as in
 * the reference's loops.  exp, sin, cos and pow go through double and are
 * rounded once to float: the reference's CPU math functions are correctly
 * rounded (stdlib/core/num.vx:2404-2479).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
  int32_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
} twin_config;

typedef struct {
  float *x, *xb, *xb2, *hb, *hb2, *q, *logits, *key_cache, *value_cache;
} twin_state;

static float f_exp(float v) { return (float)exp((double)v); }

/* rmsnorm, llama2_100.vx:353-375 */
static void twin_rmsnorm(float *o, const float *x, const float *weight, int size) {
  float ss = 0.0f;
  int j;
  for (j = 0; j < size; ++j) {
    const float val = x[j];
    ss += val * val;
  }
  ss = ss / (float)size + 0.00001f;
  ss = 1.0f / sqrtf(ss);
  for (j = 0; j < size; ++j) {
    const float temp = ss * x[j];
    o[j] = weight[j] * temp;
  }
}

/* matmul, llama2_100.vx:405-421: xout[i] = sum_j w[i*n + j] * x[j] */
static void twin_matmul(float *xout, const float *x, const float *w, int n, int d) {
  int i, j;
  for (i = 0; i < d; ++i) {
    float val = 0.0f;
    const float *row = w + (int64_t)i * n;
    for (j = 0; j < n; ++j)
      val += row[j] * x[j];
    xout[i] = val;
  }
}

/* attn, llama2_100.vx:138-204 */
static void twin_attn(float *xb, const float *q, const float *key_cache,
                      const float *value_cache, int seq_len, int pos, int n_heads,
                      int n_kv_heads, int head_size, int kv_dim, int l) {
  const int kv_mul = n_heads / n_kv_heads;
  int h, t, i;
  for (h = 0; h < n_heads; ++h) {
    const float *qh = q + h * head_size;
    float *out = xb + h * head_size;
    float m = -999999.0f, l_sum = 0.0f;
    for (i = 0; i < head_size; ++i)
      out[i] = 0.0f;
    for (t = 0; t <= pos; ++t) {
      const int64_t off = (int64_t)l * seq_len * kv_dim + (int64_t)t * kv_dim +
                          (h / kv_mul) * head_size;
      const float *k_t = key_cache + off, *v_t = value_cache + off;
      float score = 0.0f, m_new, correction, exp_val;
      for (i = 0; i < head_size; ++i)
        score += qh[i] * k_t[i];
      score = score * (1.0f / sqrtf((float)head_size));
      m_new = score > m ? score : m;
      correction = f_exp(m - m_new);
      exp_val = f_exp(score - m_new);
      l_sum = l_sum * correction + exp_val;
      for (i = 0; i < head_size; ++i)
        out[i] = out[i] * correction + exp_val * v_t[i];
      m = m_new;
    }
    {
      const float inv_l = 1.0f / l_sum;
      for (i = 0; i < head_size; ++i)
        out[i] = out[i] * inv_l;
    }
  }
}

/* transformer, llama2_100.vx:206-335. weights: one flat array in llama2.c
   order (memory_map_weights :98-136), classifier = embedding table. */
static void twin_transformer(int token, int pos, const twin_config *p,
                             twin_state *s, const float *weights) {
  const int dim = p->dim, hidden_dim = p->hidden_dim, n_layers = p->n_layers;
  const int head_size = dim / p->n_heads;
  const int kv_dim = dim * p->n_kv_heads / p->n_heads;
  const int seq_len = p->seq_len;
  const float *tok = weights;
  const float *rms_att = tok + (int64_t)p->vocab_size * dim;
  const float *wq = rms_att + (int64_t)n_layers * dim;
  const float *wk = wq + (int64_t)n_layers * dim * p->n_heads * head_size;
  const float *wv = wk + (int64_t)n_layers * dim * p->n_kv_heads * head_size;
  const float *wo = wv + (int64_t)n_layers * dim * p->n_kv_heads * head_size;
  const float *rms_ffn = wo + (int64_t)n_layers * p->n_heads * head_size * dim;
  const float *w1 = rms_ffn + (int64_t)n_layers * dim;
  const float *w2 = w1 + (int64_t)n_layers * dim * hidden_dim;
  const float *w3 = w2 + (int64_t)n_layers * hidden_dim * dim;
  const float *rms_final = w3 + (int64_t)n_layers * dim * hidden_dim;
  int l, i;

  memcpy(s->x, tok + (int64_t)token * dim, sizeof(float) * (size_t)dim);
  for (l = 0; l < n_layers; ++l) {
    float *s_k = s->key_cache + (int64_t)l * seq_len * kv_dim + (int64_t)pos * kv_dim;
    float *s_v = s->value_cache + (int64_t)l * seq_len * kv_dim + (int64_t)pos * kv_dim;
    twin_rmsnorm(s->xb, s->x, rms_att + (int64_t)l * dim, dim);
    twin_matmul(s->q, s->xb, wq + (int64_t)l * dim * dim, dim, dim);
    twin_matmul(s_k, s->xb, wk + (int64_t)l * dim * kv_dim, dim, kv_dim);
    twin_matmul(s_v, s->xb, wv + (int64_t)l * dim * kv_dim, dim, kv_dim);
    /* RoPE over i in 0..kv_dim, pairs (i, i+1), q and k at the same index
       (:257-281). With n_kv_heads == n_heads that covers every q head. */
    for (i = 0; i + 1 < kv_dim; i += 2) {
      const int in_head = i - (i / head_size) * head_size;
      const float fcr = (float)pos * (float)pow(10000.0, (double)(-(float)in_head /
                                                                   (float)head_size));
      const float fci = (float)cos((double)fcr), fsi = (float)sin((double)fcr);
      const float q0 = s->q[i], q1 = s->q[i + 1];
      const float k0 = s_k[i], k1 = s_k[i + 1];
      s->q[i] = q0 * fci - q1 * fsi;
      s->q[i + 1] = q0 * fsi + q1 * fci;
      s_k[i] = k0 * fci - k1 * fsi;
      s_k[i + 1] = k0 * fsi + k1 * fci;
    }
    twin_attn(s->xb, s->q, s->key_cache, s->value_cache, seq_len, pos, p->n_heads,
              p->n_kv_heads, head_size, kv_dim, l);
    twin_matmul(s->xb2, s->xb, wo + (int64_t)l * dim * dim, dim, dim);
    for (i = 0; i < dim; ++i)
      s->x[i] = s->x[i] + s->xb2[i];
    twin_rmsnorm(s->xb, s->x, rms_ffn + (int64_t)l * dim, dim);
    twin_matmul(s->hb, s->xb, w1 + (int64_t)l * dim * hidden_dim, dim, hidden_dim);
    twin_matmul(s->hb2, s->xb, w3 + (int64_t)l * dim * hidden_dim, dim, hidden_dim);
    for (i = 0; i < hidden_dim; ++i) { /* SwiGLU, :301-311 */
      float val = s->hb[i];
      const float factor = 1.0f / (1.0f + f_exp(0.0f - val));
      val = val * factor;
      s->hb[i] = val * s->hb2[i];
    }
    twin_matmul(s->xb, s->hb, w2 + (int64_t)l * dim * hidden_dim, hidden_dim, dim);
    for (i = 0; i < dim; ++i)
      s->x[i] = s->x[i] + s->xb[i];
  }
  twin_rmsnorm(s->x, s->x, rms_final, dim);
  twin_matmul(s->logits, s->x, tok, dim, p->vocab_size);
}

/* Greedy decode as the program's main loop does it: tokens[0] is given, the
   argmax of step s (strict `>`, :337-351) becomes tokens[s + 1]. Returns 0,
   or -1 when memory ran out. Needs n_kv_heads == n_heads (see the RoPE loop). */
int twin_generate(const twin_config *p, const float *weights, int32_t *tokens,
                  int32_t steps) {
  const int kv_dim = p->dim * p->n_kv_heads / p->n_heads;
  const size_t cache = (size_t)p->n_layers * p->seq_len * kv_dim;
  twin_state s;
  int32_t step;
  int ok;
  s.x = (float *)malloc(sizeof(float) * p->dim);
  s.xb = (float *)malloc(sizeof(float) * p->dim);
  s.xb2 = (float *)malloc(sizeof(float) * p->dim);
  s.hb = (float *)malloc(sizeof(float) * p->hidden_dim);
  s.hb2 = (float *)malloc(sizeof(float) * p->hidden_dim);
  s.q = (float *)malloc(sizeof(float) * p->dim);
  s.logits = (float *)malloc(sizeof(float) * p->vocab_size);
  s.key_cache = (float *)calloc(cache, sizeof(float));
  s.value_cache = (float *)calloc(cache, sizeof(float));
  ok = s.x && s.xb && s.xb2 && s.hb && s.hb2 && s.q && s.logits && s.key_cache &&
       s.value_cache && p->n_kv_heads == p->n_heads;
  for (step = 0; ok && step < steps; ++step) {
    int i, max_i = 0;
    float max_p;
    twin_transformer(tokens[step], step, p, &s, weights);
    max_p = s.logits[0];
    for (i = 1; i < p->vocab_size; ++i)
      if (s.logits[i] > max_p) {
        max_i = i;
        max_p = s.logits[i];
      }
    tokens[step + 1] = max_i;
  }
  free(s.x); free(s.xb); free(s.xb2); free(s.hb); free(s.hb2); free(s.q);
  free(s.logits); free(s.key_cache); free(s.value_cache);
  return ok ? 0 : -1;
}
