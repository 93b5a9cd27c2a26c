/* decoder.cu -- one decoder token as one CUDA graph.
 *
 * The reference runs a Llama-2 token as 43 separate GEMM dispatches with the
 * norms, RoPE, attention and SwiGLU on the host between them
 * (tests/backend/pass/llama2.vx:218-429), or, with std::nn, as about a dozen
 * kernel launches per layer.  Here a token is five fused kernels per layer
 * (q/k/v + RoPE + cache store, attention, output projection + residual,
 * gate/up + SwiGLU, down projection + residual) plus embed, logits and argmax,
 * recorded once into a CUDA graph and replayed: the token fed to the next step
 * and the positions live in device memory, so replaying needs no new
 * parameters.  The attention grid depends on how far the sequence has got, so
 * a graph is recorded per block of 256 positions.
 *
 * Tensor parallel (tp_ranks > 1): every rank holds a slice of the heads and of
 * the MLP rows; the output and down projections produce partial sums that meet
 * either in an NCCL all-reduce inside the graph (tp_reduce 0) or inside the
 * projection kernel itself (tp_reduce 1): each warp stores its finished values
 * into every other rank's memory as (value, call) pairs, waits for the other
 * ranks' pairs of the same rows and adds them to the residual, so a layer is
 * the same five kernels as on one GPU; the logits are split by vocabulary with
 * an exchange of each rank's best (value, index).
 *
 * 8 or 16 sequences per step (head_dim 128): the projections go to the tensor
 * cores (rowdot_umma.cu).  vx_decoder_prefill uses the same kernels to read a
 * one-sequence prompt sixteen positions per pass.
 */
#include "kernels.h"
#include "vx_b200.h"
#include "vx_collective.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <utility>
#include <string>
#include <vector>

namespace vxb {
cudaStream_t caller_stream();
void set_last_error(const char *why);
void note_kernel(const char *name);
vx::NcclCollective *nccl_job();
} // namespace vxb

namespace {

[[noreturn]] void stop(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  fputs("[Vx CUDA] FATAL: ", stderr);
  vfprintf(stderr, fmt, ap);
  fputc('\n', stderr);
  va_end(ap);
  abort();
}
#define CUDA_OK(expr)                                                          \
  do {                                                                         \
    const cudaError_t e_ = (expr);                                             \
    if (e_ != cudaSuccess)                                                     \
      stop("%s failed: %s", #expr, cudaGetErrorString(e_));                    \
  } while (0)

/* pos[i] = first[0] + i: the positions of a run of prompt tokens. */
__global__ void run_positions_kernel(int32_t *pos, const int32_t *first, int n) {
  if ((int)threadIdx.x < n)
    pos[threadIdx.x] = first[0] + threadIdx.x;
}
__global__ void advance_by_kernel(int32_t *pos, int by) {
  if (threadIdx.x == 0)
    pos[0] += by;
}

__global__ void advance_kernel(int32_t *positions, int batch) {
  if (threadIdx.x < batch)
    positions[threadIdx.x] += 1;
}

__global__ void add_kernel(float *x, const float *t, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n)
    x[i] = x[i] + t[i];
}

/* pair[b] = (best local logit, its GLOBAL index as float bits). */
__global__ void best_pair_kernel(float2 *pair, const int32_t *local_best,
                                 const float *logits, int64_t stride,
                                 int vocab_offset) {
  const int b = threadIdx.x;
  const int i = local_best[b];
  pair[b] = make_float2(logits[b * stride + i],
                        __int_as_float(i + vocab_offset));
}
/* gathered: [ranks][batch] pairs; the largest value wins, the lowest index on
   a tie (rank order is index order, so the first rank with the value). */
__global__ void pick_pair_kernel(int32_t *token, const float2 *gathered,
                                 int ranks, int batch) {
  const int b = threadIdx.x;
  if (b >= batch)
    return;
  float best = gathered[b].x;
  int at = __float_as_int(gathered[b].y);
  for (int r = 1; r < ranks; ++r) {
    const float2 p = gathered[r * batch + b];
    if (p.x > best) {
      best = p.x;
      at = __float_as_int(p.y);
    }
  }
  token[b] = at;
}

} // namespace

struct vx_decoder {
  vx_decoder_config c;
  int ranks, q_local, kv_local, hidden_local, vocab_local, vocab_offset;
  std::vector<const void *> attn_norm, wq, wk, wv, bqkv, wo, ffn_norm, w_gate,
      w_up, w_down;
  const void *embed, *final_norm, *lm_head;
  const float *cos_t, *sin_t;
  /* device state */
  float *x, *xn, *q, *att, *h, *tmp, *logits, *k_cache, *v_cache, *scratch;
  bool fused_norm; /* the activations of all sequences fit the projections' shared memory */
  int32_t *tokens, *positions, *counters, *local_best;
  float2 *pair, *pairs_all;
  /* tp_reduce == 1: partial sums exchanged through peer memory */
  bool push;
  vxb::TpPush tp;
  void *recv;                       /* this rank's slots + flags (IPC-shared) */
  void *peer_recv[vxb::kMaxTpRanks];
  int32_t *tp_epoch, *tp_done;
  /* 8 or 16 sequences: the projections run on the tensor cores */
  bool mma;
  void *mma_xs;
  float *mma_scratch;
  /* a one-sequence decoder reading its prompt sixteen positions at a time:
     the same tensor-core projections with the positions as rows */
  float *rows_x, *rows_q, *rows_att, *rows_h;
  int32_t *rows_tokens, *rows_pos;
  int64_t cache_layer_stride, cache_batch_stride;
  int split;
  int host_pos;
  cudaStream_t stream;
  std::map<int, cudaGraphExec_t> graphs;
  int kernels_per_step;
};

namespace {

void need(const char *why, const char *what) {
  if (why)
    stop("vx_decoder: %s: %s", what, why);
}

template <typename T> T *dev_alloc(size_t count) {
  void *p = nullptr;
  if (cudaMalloc(&p, count * sizeof(T)) != cudaSuccess)
    stop("vx_decoder: out of device memory for %zu bytes", count * sizeof(T));
  CUDA_OK(cudaMemset(p, 0, count * sizeof(T)));
  return (T *)p;
}

void all_reduce(vx_decoder *d, float *buf, int64_t count) {
  vx::NcclCollective *job = vxb::nccl_job();
  const int r = job->api()->AllReduce(buf, buf, (size_t)count, vx::NcclFloat32,
                                      vx::NcclSum, job->comm(), d->stream);
  if (r)
    stop("vx_decoder: ncclAllReduce failed: %s", job->api()->GetErrorString(r));
}

/* x += the sum over ranks of the partial projection just computed. With the
   pushed exchange the projection kernel has done it already; else NCCL sums
   d->tmp and a second kernel adds it. Returns the number of launches. */
int add_partials(vx_decoder *d) {
  if (d->ranks == 1 || d->push)
    return 0;
  const int64_t n = (int64_t)d->c.batch * d->c.dim;
  all_reduce(d, d->tmp, n);
  add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, d->stream>>>(d->x, d->tmp, n);
  return 2;
}

/* The receive buffers of the pushed exchange: every rank allocates its slots
   of (value, call) pairs (zero: call numbers start at 1), shares them through CUDA IPC (the handles travel by an NCCL
   all-gather), and maps every other rank's. */
void open_peer_buffers(vx_decoder *d, int rank) {
  const int64_t n = (int64_t)d->c.batch * d->c.dim;
  const size_t bytes = (size_t)2 * d->ranks * n * sizeof(vxb::TpPair);
  CUDA_OK(cudaMalloc(&d->recv, bytes));
  CUDA_OK(cudaMemset(d->recv, 0, bytes));
  d->tp_epoch = dev_alloc<int32_t>(4);
  d->tp_done = d->tp_epoch + 1;
  cudaIpcMemHandle_t mine;
  CUDA_OK(cudaIpcGetMemHandle(&mine, d->recv));
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  float *one = dev_alloc<float>(16), *all = dev_alloc<float>(16 * (size_t)d->ranks);
  CUDA_OK(cudaMemcpy(one, &mine, 64, cudaMemcpyHostToDevice));
  vx::NcclCollective *job = vxb::nccl_job();
  int r = job->api()->AllGather(one, all, 16, vx::NcclFloat32, job->comm(),
                                d->stream);
  if (r)
    stop("vx_decoder: ncclAllGather failed: %s", job->api()->GetErrorString(r));
  CUDA_OK(cudaStreamSynchronize(d->stream));
  std::vector<cudaIpcMemHandle_t> handles(d->ranks);
  CUDA_OK(cudaMemcpy(handles.data(), all, 64 * (size_t)d->ranks,
                     cudaMemcpyDeviceToHost));
  for (int p = 0; p < d->ranks; ++p) {
    if (p == rank) {
      d->peer_recv[p] = d->recv;
    } else {
      const cudaError_t e = cudaIpcOpenMemHandle(
          &d->peer_recv[p], handles[p], cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess)
        stop("vx_decoder: cannot map the receive buffer of rank %d: %s. The "
             "ranks must be GPUs of one machine with peer access.",
             p, cudaGetErrorString(e));
    }
    d->tp.slots[p] = (vxb::TpPair *)d->peer_recv[p];
  }
  d->tp.ranks = d->ranks;
  d->tp.rank = rank;
  d->tp.count = n;
  d->tp.epoch = d->tp_epoch;
  d->tp.done = d->tp_done;
  cudaFree(one);
  cudaFree(all);
  /* Nobody writes into a buffer before everybody has mapped it. */
  all_reduce(d, d->tmp, 1);
  CUDA_OK(cudaStreamSynchronize(d->stream));
}

/* The input of a projection that follows an RMSNorm: x itself when the
   projection kernel applies the norm (its shared memory holds the activations
   of all sequences), else x normalised by a kernel of its own into d->xn. */
const float *normed(vx_decoder *d, const void *norm_w, int &launches) {
  if (d->fused_norm)
    return d->x;
  need(vxb::rms_norm(d->xn, d->x, norm_w, d->c.weights_bf16 != 0, d->c.dim,
                     d->c.eps, d->c.batch, d->c.dim, d->stream),
       "RMSNorm");
  ++launches;
  return d->xn;
}

/* Queue one token on d->stream. */
void record_step(vx_decoder *d, int max_pos) {
  const vx_decoder_config &c = d->c;
  const bool bf = c.weights_bf16 != 0;
  const int B = c.batch, hd = c.head_dim;
  cudaStream_t s = d->stream;
  int launches = 0;

  need(vxb::embed(d->x, d->embed, bf, d->tokens, c.dim, c.vocab, B, c.dim, s),
       "embed");
  ++launches;
  /* 8 or 16 sequences: every projection on the tensor cores */
  auto batched = [&](int mode, const void *w0, const void *w1, const void *w2,
                     int rows, int cols, const float *x, const void *norm_w,
                     float *y, int64_t y_stride, const void *bias, int layer,
                     const char *what, bool terms_ready = false,
                     bool leave_terms = false) {
    vxb::BatchedProj bp{};
    bp.mode = mode;
    bp.w0 = w0;
    bp.w1 = w1;
    bp.w2 = w2;
    bp.rows = rows;
    bp.cols = cols;
    bp.batch = B;
    bp.x = x;
    bp.x_stride = cols;
    bp.norm_w = norm_w;
    bp.eps = c.eps;
    bp.y = y;
    bp.y_stride = y_stride;
    bp.bias = bias;
    bp.q_heads = d->q_local;
    bp.kv_heads = d->kv_local;
    bp.head_dim = hd;
    bp.cos_t = d->cos_t;
    bp.sin_t = d->sin_t;
    bp.positions = d->positions;
    bp.k_cache = d->k_cache + layer * d->cache_layer_stride;
    bp.v_cache = d->v_cache + layer * d->cache_layer_stride;
    bp.cache_batch_stride = d->cache_batch_stride;
    bp.xs = d->mma_xs;
    bp.scratch = d->mma_scratch;
    bp.x_terms_ready = terms_ready;
    bp.next_terms = leave_terms;
    need(vxb::batched_proj(bp, s), what);
    launches += terms_ready ? 2 : 3;
  };
  for (int l = 0; l < c.n_layers; ++l) {
    if (d->mma) {
      batched(4, d->wq[l], d->wk[l], d->wv[l], (d->q_local + 2 * d->kv_local) * hd,
              c.dim, d->x, d->attn_norm[l], d->q, (int64_t)d->q_local * hd,
              d->bqkv[l], l, "q/k/v");
      vxb::AttnArgs ab{};
      ab.q = d->q;
      ab.k_cache = d->k_cache + l * d->cache_layer_stride;
      ab.v_cache = d->v_cache + l * d->cache_layer_stride;
      ab.cache_batch_stride = d->cache_batch_stride;
      ab.out = d->att;
      ab.q_heads = d->q_local;
      ab.kv_heads = d->kv_local;
      ab.head_dim = hd;
      ab.batch = B;
      ab.positions = d->positions;
      ab.max_pos = max_pos;
      ab.scratch = d->scratch;
      ab.counters = d->counters;
      ab.split = d->split;
      ab.rows_settled = 1; /* earlier tokens are earlier graph launches */
      need(vxb::attention_decode(ab, s), "attention");
      ++launches;
      batched(1, d->wo[l], nullptr, nullptr, c.dim, d->q_local * hd, d->att,
              nullptr, d->x, c.dim, nullptr, l, "the output projection");
      /* SwiGLU's finishing kernel leaves the down projection's input as terms */
      batched(3, d->w_gate[l], d->w_up[l], nullptr, d->hidden_local, c.dim, d->x,
              d->ffn_norm[l], d->h, d->hidden_local, nullptr, l, "gate/up", false,
              true);
      batched(1, d->w_down[l], nullptr, nullptr, c.dim, d->hidden_local, d->h,
              nullptr, d->x, c.dim, nullptr, l, "the down projection", true);
      continue;
    }
    vxb::QkvArgs qa{};
    qa.wq = d->wq[l];
    qa.wk = d->wk[l];
    qa.wv = d->wv[l];
    qa.wbf16 = bf;
    qa.bias = d->bqkv[l];
    qa.q_heads = d->q_local;
    qa.kv_heads = d->kv_local;
    qa.head_dim = hd;
    qa.cols = c.dim;
    qa.x = normed(d, d->attn_norm[l], launches);
    qa.x_stride = c.dim;
    qa.batch = B;
    qa.norm_w = d->fused_norm ? d->attn_norm[l] : nullptr;
    qa.norm_bf16 = bf;
    qa.eps = c.eps;
    qa.rope_mode = bf ? 0 : 1;
    qa.cos_t = d->cos_t;
    qa.sin_t = d->sin_t;
    qa.cs_cols = hd / 2;
    qa.theta = c.rope_theta;
    qa.positions = d->positions;
    qa.q_out = d->q;
    qa.k_cache = d->k_cache + l * d->cache_layer_stride;
    qa.v_cache = d->v_cache + l * d->cache_layer_stride;
    qa.cache_batch_stride = d->cache_batch_stride;
    qa.max_seq = c.max_seq;
    need(vxb::qkv_rope_store(qa, s), "q/k/v");

    vxb::AttnArgs aa{};
    aa.q = d->q;
    aa.k_cache = qa.k_cache;
    aa.v_cache = qa.v_cache;
    aa.cache_batch_stride = d->cache_batch_stride;
    aa.out = d->att;
    aa.q_heads = d->q_local;
    aa.kv_heads = d->kv_local;
    aa.head_dim = hd;
    aa.batch = B;
    aa.positions = d->positions;
    aa.max_pos = max_pos;
    aa.scratch = d->scratch;
    aa.counters = d->counters;
    aa.split = d->split;
    aa.rows_settled = 1; /* earlier tokens are earlier graph launches */
    need(vxb::attention_decode(aa, s), "attention");

    vxb::MatvecArgs oa{};
    oa.w = d->wo[l];
    oa.wbf16 = bf;
    oa.rows = c.dim;
    oa.cols = d->q_local * hd;
    oa.x = d->att;
    oa.x_stride = oa.cols;
    oa.batch = B;
    oa.y = d->ranks > 1 && !d->push ? d->tmp : d->x;
    oa.y_stride = c.dim;
    oa.mode = d->push ? 3 : (d->ranks > 1 ? 0 : 1);
    oa.push = &d->tp;
    need(vxb::matvec(oa, s), "the output projection");
    launches += 3;
    launches += add_partials(d);

    vxb::SwigluArgs sa{};
    sa.w = d->w_gate[l];
    sa.w_up = d->w_up[l];
    sa.wbf16 = bf;
    sa.rows = d->hidden_local;
    sa.cols = c.dim;
    sa.x = normed(d, d->ffn_norm[l], launches);
    sa.x_stride = c.dim;
    sa.out = d->h;
    sa.out_stride = d->hidden_local;
    sa.batch = B;
    sa.norm_w = d->fused_norm ? d->ffn_norm[l] : nullptr;
    sa.norm_bf16 = bf;
    sa.eps = c.eps;
    need(vxb::swiglu(sa, s), "gate/up");

    vxb::MatvecArgs da{};
    da.w = d->w_down[l];
    da.wbf16 = bf;
    da.rows = c.dim;
    da.cols = d->hidden_local;
    da.x = d->h;
    da.x_stride = d->hidden_local;
    da.batch = B;
    da.y = d->ranks > 1 && !d->push ? d->tmp : d->x;
    da.y_stride = c.dim;
    da.mode = d->push ? 3 : (d->ranks > 1 ? 0 : 1);
    da.push = &d->tp;
    need(vxb::matvec(da, s), "the down projection");
    launches += 2;
    launches += add_partials(d);
  }

  if (d->mma) {
    batched(0, d->lm_head, nullptr, nullptr, d->vocab_local, c.dim, d->x,
            d->final_norm, d->logits, d->vocab_local, nullptr, 0, "the logits");
  } else {
  vxb::MatvecArgs la{};
  la.w = d->lm_head;
  la.wbf16 = bf;
  la.rows = d->vocab_local;
  la.cols = c.dim;
  la.x = normed(d, d->final_norm, launches);
  la.x_stride = c.dim;
  la.batch = B;
  la.norm_w = d->fused_norm ? d->final_norm : nullptr;
  la.norm_bf16 = bf;
  la.eps = c.eps;
  la.y = d->logits;
  la.y_stride = d->vocab_local;
  la.mode = 0;
  need(vxb::matvec(la, s), "the logits");
  ++launches;
  }
  if (d->ranks == 1) {
    need(vxb::argmax(d->tokens, d->logits, d->vocab_local, B, d->vocab_local, s),
         "argmax");
    launches += 1;
  } else {
    need(vxb::argmax(d->local_best, d->logits, d->vocab_local, B,
                     d->vocab_local, s),
         "argmax");
    best_pair_kernel<<<1, B, 0, s>>>(d->pair, d->local_best, d->logits,
                                     d->vocab_local, d->vocab_offset);
    vx::NcclCollective *job = vxb::nccl_job();
    const int r = job->api()->AllGather(d->pair, d->pairs_all, (size_t)B * 2,
                                        vx::NcclFloat32, job->comm(), s);
    if (r)
      stop("vx_decoder: ncclAllGather failed: %s",
           job->api()->GetErrorString(r));
    pick_pair_kernel<<<1, 32, 0, s>>>(d->tokens, d->pairs_all, d->ranks, B);
    launches += 4;
  }
  advance_kernel<<<1, 32, 0, s>>>(d->positions, B);
  ++launches;
  d->kernels_per_step = launches;
}

cudaGraphExec_t graph_for(vx_decoder *d, int bucket) {
  auto hit = d->graphs.find(bucket);
  if (hit != d->graphs.end())
    return hit->second;
  int max_pos = (bucket + 1) * 256 - 1;
  if (max_pos > d->c.max_seq - 1)
    max_pos = d->c.max_seq - 1;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  CUDA_OK(cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal));
  record_step(d, max_pos);
  CUDA_OK(cudaStreamEndCapture(d->stream, &graph));
  CUDA_OK(cudaGraphInstantiate(&exec, graph, 0));
  CUDA_OK(cudaGraphDestroy(graph));
  d->graphs[bucket] = exec;
  return exec;
}

} // namespace

extern "C" {

vx_decoder *vx_decoder_create(const vx_decoder_config *config,
                              const vx_decoder_weights *w) {
  if (!config || !w)
    stop("vx_decoder_create: a null argument");
  vx_decoder *d = new vx_decoder();
  d->c = *config;
  const vx_decoder_config &c = d->c;
  d->ranks = c.tp_ranks > 1 ? c.tp_ranks : 1;
  if (c.dim <= 0 || c.n_layers <= 0 || c.head_dim <= 0 || c.max_seq <= 0 ||
      c.q_heads % d->ranks || c.kv_heads % d->ranks || c.hidden % d->ranks ||
      c.vocab % d->ranks)
    stop("vx_decoder_create: heads, hidden and vocab must divide by tp_ranks");
  if (c.dim % 8 || c.hidden / d->ranks % 8 || (c.q_heads / d->ranks * c.head_dim) % 8)
    stop("vx_decoder_create: dim, the local hidden size and the local "
         "attention width must be multiples of 8");
  if (c.batch != 1 && c.batch != 2 && c.batch != 4 && c.batch != 8 &&
      c.batch != 16)
    stop("vx_decoder_create: batch must be 1, 2, 4, 8 or 16");
  if (c.weights_bf16 && (!w->cos || !w->sin))
    stop("vx_decoder_create: the std::nn flavour needs cos and sin tables");
  int rank = 0;
  if (d->ranks > 1) {
    vx::NcclCollective *job = vxb::nccl_job();
    if (!job || job->ranks() != d->ranks)
      stop("vx_decoder_create: tp_ranks is %d, but vx_collective_init joined "
           "a job of %d",
           d->ranks, job ? job->ranks() : 0);
    rank = job->rank();
  }
  d->q_local = c.q_heads / d->ranks;
  d->kv_local = c.kv_heads / d->ranks;
  d->hidden_local = c.hidden / d->ranks;
  d->vocab_local = c.vocab / d->ranks;
  d->vocab_offset = rank * d->vocab_local;

  auto copy = [&](std::vector<const void *> &dst, const void *const *src,
                  bool required, const char *name) {
    dst.assign(c.n_layers, nullptr);
    if (!src) {
      if (required)
        stop("vx_decoder_create: weights->%s is null", name);
      return;
    }
    for (int l = 0; l < c.n_layers; ++l)
      dst[l] = src[l];
  };
  copy(d->attn_norm, w->attn_norm, true, "attn_norm");
  copy(d->wq, w->wq, true, "wq");
  copy(d->wk, w->wk, false, "wk");
  copy(d->wv, w->wv, false, "wv");
  copy(d->bqkv, w->bqkv, false, "bqkv");
  copy(d->wo, w->wo, true, "wo");
  copy(d->ffn_norm, w->ffn_norm, true, "ffn_norm");
  copy(d->w_gate, w->w_gate, true, "w_gate");
  copy(d->w_up, w->w_up, false, "w_up");
  copy(d->w_down, w->w_down, true, "w_down");
  d->embed = w->embed;
  d->final_norm = w->final_norm;
  d->lm_head = w->lm_head;
  d->cos_t = w->cos;
  d->sin_t = w->sin;
  if (!d->embed || !d->final_norm || !d->lm_head)
    stop("vx_decoder_create: embed, final_norm and lm_head are required");

  const int B = c.batch;
  const int tiles = d->q_local; /* upper bound on head tiles */
  d->split = (int64_t)tiles * B < 128 ? 32 : 128;
  d->cache_batch_stride = (int64_t)c.max_seq * d->kv_local * c.head_dim;
  d->cache_layer_stride = d->cache_batch_stride * B;
  d->x = dev_alloc<float>((size_t)B * c.dim);
  d->tmp = dev_alloc<float>((size_t)B * c.dim);
  d->xn = dev_alloc<float>((size_t)B * c.dim);
  d->fused_norm = (size_t)B * ((c.dim + 255) / 256 * 256) * sizeof(float) <= 96 * 1024;
  d->q = dev_alloc<float>((size_t)B * d->q_local * c.head_dim);
  d->att = dev_alloc<float>((size_t)B * d->q_local * c.head_dim);
  d->h = dev_alloc<float>((size_t)B * d->hidden_local);
  d->logits = dev_alloc<float>((size_t)B * d->vocab_local);
  d->k_cache = dev_alloc<float>((size_t)d->cache_layer_stride * c.n_layers);
  d->v_cache = dev_alloc<float>((size_t)d->cache_layer_stride * c.n_layers);
  d->scratch = dev_alloc<float>(vxb::attn_scratch_floats(
      B, d->q_local, c.head_dim, c.max_seq, d->split));
  d->counters = dev_alloc<int32_t>((size_t)B * d->q_local + 32);
  d->tokens = dev_alloc<int32_t>(32);
  d->positions = dev_alloc<int32_t>(32);
  d->local_best = dev_alloc<int32_t>(32);
  d->pair = (float2 *)dev_alloc<float>(2 * 32);
  d->pairs_all = (float2 *)dev_alloc<float>(2 * 32 * (size_t)d->ranks);
  d->host_pos = 0;
  d->kernels_per_step = 0;
  CUDA_OK(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
  d->push = false;
  d->recv = nullptr;
  if (d->ranks > 1 && c.tp_reduce == 1) {
    open_peer_buffers(d, rank);
    d->push = true;
  }
  d->rows_x = d->rows_q = d->rows_att = d->rows_h = nullptr;
  d->rows_tokens = d->rows_pos = nullptr;
  d->mma = false;
  d->mma_xs = nullptr;
  d->mma_scratch = nullptr;
  const char *nomma = getenv("VXB_BATCH_MMA");
  if (c.weights_bf16 && d->ranks == 1 && (B == 8 || B == 16) && c.head_dim == 128 &&
      c.dim % 64 == 0 && d->hidden_local % 64 == 0 && !(nomma && nomma[0] == '0')) {
    int widest = c.dim > d->hidden_local ? c.dim : d->hidden_local;
    if (d->q_local * c.head_dim > widest)
      widest = d->q_local * c.head_dim;
    int rows_max = 2 * d->hidden_local;
    if ((d->q_local + 2 * d->kv_local) * c.head_dim > rows_max)
      rows_max = (d->q_local + 2 * d->kv_local) * c.head_dim;
    if (d->vocab_local > rows_max)
      rows_max = d->vocab_local;
    d->mma_xs = dev_alloc<uint16_t>((size_t)48 * widest);
    d->mma_scratch = dev_alloc<float>(vxb::batched_proj_scratch_floats(rows_max, B));
    d->mma = true;
  }
  CUDA_OK(cudaDeviceSynchronize());
  return d;
}

void vx_decoder_destroy(vx_decoder *d) {
  if (!d)
    return;
  cudaStreamSynchronize(d->stream);
  if (d->push) {
    /* No rank unmaps or frees while another may still write into it. */
    all_reduce(d, d->tmp, 1);
    cudaStreamSynchronize(d->stream);
    for (int p = 0; p < d->ranks; ++p)
      if (p != d->tp.rank)
        cudaIpcCloseMemHandle(d->peer_recv[p]);
    cudaFree(d->recv);
    cudaFree(d->tp_epoch);
  }
  for (auto &g : d->graphs)
    cudaGraphExecDestroy(g.second);
  for (void *p : {(void *)d->x, (void *)d->xn, (void *)d->tmp, (void *)d->q, (void *)d->att,
                  (void *)d->h, (void *)d->logits, (void *)d->k_cache,
                  (void *)d->v_cache, (void *)d->scratch, (void *)d->counters,
                  (void *)d->tokens, (void *)d->positions,
                  (void *)d->local_best, (void *)d->pair,
                  (void *)d->pairs_all, d->mma_xs, (void *)d->mma_scratch,
                  (void *)d->rows_x, (void *)d->rows_q, (void *)d->rows_att,
                  (void *)d->rows_h, (void *)d->rows_tokens, (void *)d->rows_pos})
    cudaFree(p);
  cudaStreamDestroy(d->stream);
  delete d;
}

void vx_decoder_reset(vx_decoder *d) {
  CUDA_OK(cudaStreamSynchronize(d->stream));
  CUDA_OK(cudaMemsetAsync(d->positions, 0, 32 * sizeof(int32_t), d->stream));
  CUDA_OK(cudaStreamSynchronize(d->stream));
  d->host_pos = 0;
}

int32_t vx_decoder_step(vx_decoder *d, const int32_t *tokens_in,
                        int32_t *tokens_out) {
  const int pos = d->host_pos;
  if (pos >= d->c.max_seq)
    stop("vx_decoder_step: position %d is past max_seq %d", pos, d->c.max_seq);
  cudaGraphExec_t exec = graph_for(d, pos / 256);
  if (tokens_in)
    CUDA_OK(cudaMemcpyAsync(d->tokens, tokens_in, d->c.batch * sizeof(int32_t),
                            cudaMemcpyHostToDevice, d->stream));
  CUDA_OK(cudaGraphLaunch(exec, d->stream));
  d->host_pos = pos + 1;
  if (tokens_out) {
    CUDA_OK(cudaMemcpyAsync(tokens_out, d->tokens, d->c.batch * sizeof(int32_t),
                            cudaMemcpyDeviceToHost, d->stream));
    const cudaError_t e = cudaStreamSynchronize(d->stream);
    if (e != cudaSuccess)
      stop("a kernel of the decoder faulted: %s", cudaGetErrorString(e));
  }
  return pos;
}

/* A run of prompt tokens of a one-sequence decoder, sixteen positions per
   pass: the projections see the positions as the rows of rowdot_umma.cu (the
   multi-row kernels of nn.vx:2317-3066 are the reference's form of this), every
   row writes its K and V into the one cache at its own position, and row i
   attends positions 0 .. first + i, which are all in the cache by then. No
   logits: the caller feeds the last prompt token through vx_decoder_step.
   Returns the number of tokens taken (a multiple of 16, possibly 0: what is
   left goes through vx_decoder_step), or -1 with vx_b200_last_error() when
   this decoder cannot do it. */
int32_t vx_decoder_prefill(vx_decoder *d, const int32_t *tokens, int32_t count) {
  const vx_decoder_config &c = d->c;
  constexpr int R = 16;
  if (c.batch != 1 || !c.weights_bf16 || d->ranks != 1 || c.head_dim != 128 ||
      c.dim % 64 != 0 || d->hidden_local % 64 != 0) {
    vxb::set_last_error("vx_decoder_prefill: needs one sequence, one rank, bf16 "
                        "weights, head_dim 128 and widths in multiples of 64");
    return -1;
  }
  if (count < 0 || d->host_pos + count > c.max_seq) {
    vxb::set_last_error("vx_decoder_prefill: the prompt does not fit max_seq");
    return -1;
  }
  if (!d->rows_x) {
    int widest = c.dim > d->hidden_local ? c.dim : d->hidden_local;
    if (d->q_local * c.head_dim > widest)
      widest = d->q_local * c.head_dim;
    int rows_max = 2 * d->hidden_local;
    if ((d->q_local + 2 * d->kv_local) * c.head_dim > rows_max)
      rows_max = (d->q_local + 2 * d->kv_local) * c.head_dim;
    d->rows_x = dev_alloc<float>((size_t)R * c.dim);
    d->rows_q = dev_alloc<float>((size_t)R * d->q_local * c.head_dim);
    d->rows_att = dev_alloc<float>((size_t)R * d->q_local * c.head_dim);
    d->rows_h = dev_alloc<float>((size_t)R * d->hidden_local);
    d->rows_tokens = dev_alloc<int32_t>(R);
    d->rows_pos = dev_alloc<int32_t>(R);
    if (!d->mma_xs) {
      d->mma_xs = dev_alloc<uint16_t>((size_t)48 * widest);
      d->mma_scratch = dev_alloc<float>(vxb::batched_proj_scratch_floats(rows_max, R));
    }
  }
  cudaStream_t s = d->stream;
  const int hd = c.head_dim;
  int taken = 0;
  while (count - taken >= R) {
    CUDA_OK(cudaMemcpyAsync(d->rows_tokens, tokens + taken, R * sizeof(int32_t),
                            cudaMemcpyHostToDevice, s));
    run_positions_kernel<<<1, 32, 0, s>>>(d->rows_pos, d->positions, R);
    need(vxb::embed(d->rows_x, d->embed, true, d->rows_tokens, c.dim, c.vocab, R,
                    c.dim, s),
         "embed");
    auto proj = [&](int mode, const void *w0, const void *w1, const void *w2,
                    int rows, int cols, const float *x, const void *norm_w,
                    float *y, int64_t y_stride, const void *bias, int layer,
                    const char *what, bool terms_ready, bool leave_terms) {
      vxb::BatchedProj bp{};
      bp.mode = mode;
      bp.w0 = w0;
      bp.w1 = w1;
      bp.w2 = w2;
      bp.rows = rows;
      bp.cols = cols;
      bp.batch = R;
      bp.x = x;
      bp.x_stride = cols;
      bp.norm_w = norm_w;
      bp.eps = c.eps;
      bp.y = y;
      bp.y_stride = y_stride;
      bp.bias = bias;
      bp.q_heads = d->q_local;
      bp.kv_heads = d->kv_local;
      bp.head_dim = hd;
      bp.cos_t = d->cos_t;
      bp.sin_t = d->sin_t;
      bp.positions = d->rows_pos;
      bp.k_cache = d->k_cache + layer * d->cache_layer_stride;
      bp.v_cache = d->v_cache + layer * d->cache_layer_stride;
      bp.cache_batch_stride = 0; /* every row writes into the one cache */
      bp.xs = d->mma_xs;
      bp.scratch = d->mma_scratch;
      bp.x_terms_ready = terms_ready;
      bp.next_terms = leave_terms;
      need(vxb::batched_proj(bp, s), what);
    };
    for (int l = 0; l < c.n_layers; ++l) {
      proj(4, d->wq[l], d->wk[l], d->wv[l], (d->q_local + 2 * d->kv_local) * hd,
           c.dim, d->rows_x, d->attn_norm[l], d->rows_q, (int64_t)d->q_local * hd,
           d->bqkv[l], l, "q/k/v", false, false);
      vxb::AttnArgs aa{};
      aa.q = d->rows_q;
      aa.k_cache = d->k_cache + l * d->cache_layer_stride;
      aa.v_cache = d->v_cache + l * d->cache_layer_stride;
      aa.cache_batch_stride = 0;
      aa.out = d->rows_att;
      aa.q_heads = d->q_local;
      aa.kv_heads = d->kv_local;
      aa.head_dim = hd;
      aa.batch = R;
      aa.positions = d->rows_pos;
      aa.max_pos = d->host_pos + taken + R - 1;
      aa.fresh_from = d->positions; /* this pass's rows are new */
      aa.scratch = nullptr; /* the cluster form needs none */
      aa.counters = nullptr;
      aa.split = d->split;
      aa.rows_settled = 1; /* rows below fresh_from: earlier passes and steps */
      need(vxb::attention_decode_clustered(aa, s), "attention");
      proj(1, d->wo[l], nullptr, nullptr, c.dim, d->q_local * hd, d->rows_att,
           nullptr, d->rows_x, c.dim, nullptr, l, "the output projection", false,
           false);
      proj(3, d->w_gate[l], d->w_up[l], nullptr, d->hidden_local, c.dim, d->rows_x,
           d->ffn_norm[l], d->rows_h, d->hidden_local, nullptr, l, "gate/up", false,
           true);
      proj(1, d->w_down[l], nullptr, nullptr, c.dim, d->hidden_local, d->rows_h,
           nullptr, d->rows_x, c.dim, nullptr, l, "the down projection", true,
           false);
    }
    advance_by_kernel<<<1, 32, 0, s>>>(d->positions, R);
    taken += R;
  }
  d->host_pos += taken;
  return taken;
}

const float *vx_decoder_logits(const vx_decoder *d) { return d->logits; }
void *vx_decoder_stream(const vx_decoder *d) { return (void *)d->stream; }
int32_t vx_decoder_kernels_per_step(const vx_decoder *d) {
  return d->kernels_per_step;
}

} /* extern "C" */
