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

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
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

__global__ void advance_by_kernel(int32_t *pos, int by) {
  if (threadIdx.x == 0)
    pos[0] += by;
}

__global__ void set_positions_kernel(int32_t *positions, int batch, int to) {
  if (threadIdx.x < batch)
    positions[threadIdx.x] = to;
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

/* The token of a vocabulary-split model: every rank has the best logit of its
   slice (local_best) and all ranks must agree on the best of all. Thread
   (b, r) stores this rank's (value, global index) of sequence b into rank r's
   slots as one 16-byte (value, index, call, call) record -- the two call
   numbers make it its own arrival flag, as in the exchange of the partial
   sums -- and waits (bounded) for rank r's record of sequence b; then the
   largest value wins, the lowest index on a tie (rank order is index order, so
   the first rank with that value). One block; slots: [2 sets][ranks][batch]. */
struct PickSlot {
  float value;
  int32_t index, call, call_again;
};
struct PickPeers {
  PickSlot *slots[vxb::kMaxTpRanks];
};
__global__ void __launch_bounds__(vxb::kMaxTpRanks * 32)
tp_pick_kernel(int32_t *token, const int32_t *local_best, const float *logits,
               int64_t stride, int vocab_offset, PickPeers peers, int ranks,
               int rank, int batch, int32_t *epoch, int32_t *gave_up) {
  __shared__ float values[32][vxb::kMaxTpRanks];
  __shared__ int32_t indices[32][vxb::kMaxTpRanks];
  const int call = *epoch + 1, set = call & 1;
  const int b = threadIdx.x / ranks, r = threadIdx.x % ranks;
  if (b < batch) {
    const int best = local_best[b];
    float v = logits[b * stride + best];
    int32_t idx = best + vocab_offset;
    if (r != rank) {
      PickSlot *to = peers.slots[r] + ((int64_t)set * ranks + rank) * batch + b;
      asm volatile("st.volatile.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(to),
                   "r"(__float_as_uint(v)), "r"(idx), "r"(call), "r"(call)
                   : "memory");
      const PickSlot *from =
          peers.slots[rank] + ((int64_t)set * ranks + r) * batch + b;
      const long long began = clock64();
      for (;;) {
        uint32_t bits;
        int32_t c0, c1;
        asm volatile("ld.volatile.global.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(bits), "=r"(idx), "=r"(c0), "=r"(c1)
                     : "l"(from)
                     : "memory");
        v = __uint_as_float(bits);
        if (c0 == call && c1 == call)
          break;
        if (clock64() - began > (1ll << 31)) { /* about a second */
          atomicCAS(gave_up, 0, 0x54);
          break;
        }
      }
    }
    values[b][r] = v;
    indices[b][r] = idx;
  }
  __syncthreads();
  if ((int)threadIdx.x < batch) {
    float best = values[threadIdx.x][0];
    int32_t at = indices[threadIdx.x][0];
    for (int k = 1; k < ranks; ++k)
      if (values[threadIdx.x][k] > best) {
        best = values[threadIdx.x][k];
        at = indices[threadIdx.x][k];
      }
    token[threadIdx.x] = at;
  }
  if (threadIdx.x == 0)
    *epoch = call;
}

/* The same agreement from an all-gather of (value, index bits) pairs (the
   NCCL form): pair[b] of this rank, then the pick over gathered
   [ranks][batch]. */
__global__ void best_pair_kernel(float2 *pair, const int32_t *local_best,
                                 const float *logits, int64_t stride,
                                 int vocab_offset) {
  const int b = threadIdx.x;
  const int i = local_best[b];
  pair[b] = make_float2(logits[b * stride + i],
                        __int_as_float(i + vocab_offset));
}
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
      w_up, w_down, s_qkv, s_o, s_gate_up, s_down;
  int wfmt; /* 0, or kFmtFp8 / kFmtQ4 for the layers' projections */
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
  int32_t *tp_epoch, *tp_done, *pick_epoch, *pick_gave_up;
  PickPeers pick;
  /* 8 or 16 sequences: the projections run on the tensor cores */
  bool mma;
  void *mma_xs;
  float *mma_scratch;
  /* a one-sequence decoder reading a whole prompt at once (prefill.cu):
     activations of rows_cap positions, their bf16 terms, the GEMMs' partial
     sums */
  float *rows_x, *rows_q, *rows_partials;
  void *rows_terms;
  /* quantised weights: the matrix in hand as two (Q4_0) or three (fp8) bf16
     terms, and the activations' terms spread over six or seven segments */
  void *rows_w_terms, *rows_terms6;
  size_t rows_partial_floats;
  int32_t *rows_tokens;
  int rows_cap;
  int64_t cache_layer_stride, cache_batch_stride;
  int split;
  int host_pos;
  cudaStream_t stream;
  std::map<int, cudaGraphExec_t> graphs;
  int kernels_per_step;
  void *owned_weights; /* a checkpoint this decoder loaded itself, or NULL */
  /* one sequence, bf16 weights, heads of 128 values: all layers and the logits
     of a step are one cooperative launch (step_kernel.cu) */
  bool one_kernel;
  vxb::StepOp *step_ops;
  int n_step_ops;
  float *step_scratch;
  int32_t *arrivals;
  unsigned long long *step_trace; /* VXB_STEP_TRACE=1: clock readings of the last step */
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
  /* the pairs of the partial sums, then the records of the token agreement */
  const size_t pair_bytes = (size_t)2 * d->ranks * n * sizeof(vxb::TpPair);
  const size_t bytes = pair_bytes + (size_t)2 * d->ranks * 32 * sizeof(PickSlot);
  CUDA_OK(cudaMalloc(&d->recv, bytes));
  CUDA_OK(cudaMemset(d->recv, 0, bytes));
  d->tp_epoch = dev_alloc<int32_t>(4);
  d->tp_done = d->tp_epoch + 1;
  d->pick_epoch = d->tp_epoch + 2;
  d->pick_gave_up = d->tp_epoch + 3;
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
    d->pick.slots[p] = (PickSlot *)((char *)d->peer_recv[p] + pair_bytes);
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
/* The projections of a step in the order they run (step_kernel.cu). */
void build_step_ops(vx_decoder *d) {
  const vx_decoder_config &c = d->c;
  const int hd = c.head_dim;
  const int64_t rb = (int64_t)c.dim * 2; /* bytes of a row of dim bf16 values */
  std::vector<vxb::StepOp> ops;
  for (int l = 0; l < c.n_layers; ++l) {
    vxb::StepOp q{};
    q.kind = vxb::kStepQkv;
    q.w0 = d->wq[l];
    q.w1 = d->wk[l] ? d->wk[l] : (const char *)d->wq[l] + (int64_t)d->q_local * hd * rb;
    q.w2 = d->wv[l] ? d->wv[l]
                    : (const char *)d->wq[l] +
                          (int64_t)(d->q_local + d->kv_local) * hd * rb;
    q.norm_w = d->attn_norm[l];
    q.bias = d->bqkv[l];
    q.x = d->x;
    q.k_cache = d->k_cache + l * d->cache_layer_stride;
    q.v_cache = d->v_cache + l * d->cache_layer_stride;
    q.rows = (d->q_local + 2 * d->kv_local) * hd;
    q.items = q.rows / 2;
    q.cols = c.dim;
    ops.push_back(q);
    vxb::StepOp o{};
    o.kind = vxb::kStepAdd;
    o.w0 = d->wo[l];
    o.x = d->att;
    o.y = d->x;
    o.rows = c.dim;
    o.items = (c.dim + 1) / 2;
    o.cols = d->q_local * hd;
    ops.push_back(o);
    vxb::StepOp g{};
    g.kind = vxb::kStepSwiglu;
    g.w0 = d->w_gate[l];
    g.w1 = d->w_up[l] ? d->w_up[l]
                      : (const char *)d->w_gate[l] + (int64_t)d->hidden_local * rb;
    g.norm_w = d->ffn_norm[l];
    g.x = d->x;
    g.y = d->h;
    g.rows = d->hidden_local;
    g.items = d->hidden_local;
    g.cols = c.dim;
    ops.push_back(g);
    vxb::StepOp w{};
    w.kind = vxb::kStepAdd;
    w.w0 = d->w_down[l];
    w.x = d->h;
    w.y = d->x;
    w.rows = c.dim;
    w.items = (c.dim + 1) / 2;
    w.cols = d->hidden_local;
    ops.push_back(w);
  }
  vxb::StepOp head{};
  head.kind = vxb::kStepStore;
  head.w0 = d->lm_head;
  head.norm_w = d->final_norm;
  head.x = d->x;
  head.y = d->logits;
  head.rows = d->vocab_local;
  head.items = (d->vocab_local + 1) / 2;
  head.cols = c.dim;
  ops.push_back(head);
  d->n_step_ops = (int)ops.size();
  d->step_ops = dev_alloc<vxb::StepOp>(ops.size());
  CUDA_OK(cudaMemcpy(d->step_ops, ops.data(), ops.size() * sizeof(vxb::StepOp),
                     cudaMemcpyHostToDevice));
  d->step_scratch = dev_alloc<float>(vxb::step_scratch_floats(d->q_local));
  d->arrivals = dev_alloc<int32_t>(32);
  const char *trace = getenv("VXB_STEP_TRACE");
  if (trace && trace[0] == '1')
    d->step_trace = dev_alloc<unsigned long long>(ops.size() * vxb::kStepTraceSlots);
  d->one_kernel = true;
}

/* The end of a step: the token of every sequence (agreed between the ranks of
   a vocabulary-split model), then the positions move on. */
void record_tail(vx_decoder *d, int launches) {
  const vx_decoder_config &c = d->c;
  const int B = c.batch;
  cudaStream_t s = d->stream;
  if (d->ranks == 1) {
    need(vxb::argmax(d->tokens, d->logits, d->vocab_local, B, d->vocab_local, s),
         "argmax");
    launches += 1;
  } else {
    need(vxb::argmax(d->local_best, d->logits, d->vocab_local, B,
                     d->vocab_local, s),
         "argmax");
    if (d->push) {
      tp_pick_kernel<<<1, d->ranks * 32, 0, s>>>(
          d->tokens, d->local_best, d->logits, d->vocab_local, d->vocab_offset,
          d->pick, d->ranks, d->tp.rank, B, d->pick_epoch, d->pick_gave_up);
      launches += 2;
    } else {
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
  }
  advance_kernel<<<1, 32, 0, s>>>(d->positions, B);
  ++launches;
  d->kernels_per_step = launches;
}

/* One sequence: embed, then every layer and the logits in one launch. */
void record_one_kernel_step(vx_decoder *d) {
  const vx_decoder_config &c = d->c;
  cudaStream_t s = d->stream;
  need(vxb::embed(d->x, d->embed, true, d->tokens, c.dim, c.vocab, 1, c.dim, s),
       "embed");
  CUDA_OK(cudaMemsetAsync(d->arrivals, 0, sizeof(int32_t), s));
  vxb::StepArgs a{};
  a.ops = d->step_ops;
  a.n_ops = d->n_step_ops;
  a.q_heads = d->q_local;
  a.kv_heads = d->kv_local;
  a.head_dim = c.head_dim;
  a.eps = c.eps;
  a.cos_t = d->cos_t;
  a.sin_t = d->sin_t;
  a.positions = d->positions;
  a.q = d->q;
  a.att = d->att;
  a.scratch = d->step_scratch;
  a.counters = d->counters;
  a.arrivals = d->arrivals;
  if (d->push)
    a.tp = d->tp;
  a.trace = d->step_trace;
  need(vxb::decode_step(a, s), "the step kernel");
  record_tail(d, 2);
}

void record_step(vx_decoder *d, int max_pos) {
  if (d->one_kernel) {
    record_one_kernel_step(d);
    return;
  }
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
    qa.wfmt = d->wfmt;
    qa.sq = d->s_qkv[l];
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
    oa.wfmt = d->wfmt;
    oa.scales = d->s_o[l];
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
    sa.wfmt = d->wfmt;
    sa.scales = d->s_gate_up[l];
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
    da.wfmt = d->wfmt;
    da.scales = d->s_down[l];
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
  record_tail(d, launches);
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
  d->wfmt = c.weights_bf16 == 2 ? vxb::kFmtFp8 : c.weights_bf16 == 3 ? vxb::kFmtQ4 : 0;
  copy(d->s_qkv, d->wfmt ? w->s_qkv : nullptr, d->wfmt != 0, "s_qkv");
  copy(d->s_o, d->wfmt ? w->s_o : nullptr, d->wfmt != 0, "s_o");
  copy(d->s_gate_up, d->wfmt ? w->s_gate_up : nullptr, d->wfmt != 0, "s_gate_up");
  copy(d->s_down, d->wfmt ? w->s_down : nullptr, d->wfmt != 0, "s_down");
  if (d->wfmt) {
    if (c.batch != 1 || d->ranks != 1)
      stop("vx_decoder_create: fp8 and Q4_0 weights take one sequence on one rank");
    for (int l = 0; l < c.n_layers; ++l)
      if (d->wk[l] || d->wv[l] || d->w_up[l])
        stop("vx_decoder_create: fp8 and Q4_0 weights need the q, k and v rows in "
             "one matrix (wk, wv NULL) and the gate and up rows in one (w_up NULL)");
    if (c.dim % (d->wfmt == vxb::kFmtFp8 ? 128 : 32) || c.hidden % (d->wfmt == vxb::kFmtFp8 ? 128 : 32))
      stop("vx_decoder_create: fp8 needs dim and hidden in multiples of 128, Q4_0 "
           "of 32");
  }
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
  d->owned_weights = nullptr;
  CUDA_OK(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
  d->push = false;
  d->recv = nullptr;
  if (d->ranks > 1 && c.tp_reduce == 1) {
    open_peer_buffers(d, rank);
    d->push = true;
  }
  d->rows_x = d->rows_q = d->rows_partials = nullptr;
  d->rows_terms = nullptr;
  d->rows_w_terms = d->rows_terms6 = nullptr;
  d->rows_partial_floats = 0;
  d->rows_tokens = nullptr;
  d->rows_cap = 0;
  d->mma = false;
  d->mma_xs = nullptr;
  d->mma_scratch = nullptr;
  const char *nomma = getenv("VXB_BATCH_MMA");
  if (c.weights_bf16 == 1 && d->ranks == 1 && (B == 8 || B == 16) && c.head_dim == 128 &&
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
  d->one_kernel = false;
  d->step_ops = nullptr;
  d->n_step_ops = 0;
  d->step_scratch = nullptr;
  d->arrivals = nullptr;
  d->step_trace = nullptr;
  {
    /* Measured slower than the chain of kernels, which already fills its rings
       ahead of each wait (7B shape, position 520: 90 against 83 us per layer;
       an eighth of it: 40 against 27): it runs only when asked for,
       VXB_STEP_KERNEL=1. */
    const char *on = getenv("VXB_STEP_KERNEL");
    int widest = c.dim > d->hidden_local ? c.dim : d->hidden_local;
    if (d->q_local * c.head_dim > widest)
      widest = d->q_local * c.head_dim;
    if (B == 1 && c.weights_bf16 == 1 && !d->mma && d->fused_norm &&
        c.head_dim == 128 && (d->ranks == 1 || d->push) &&
        widest <= vxb::kStepMaxCols && on && on[0] == '1')
      build_step_ops(d);
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
                  (void *)d->rows_x, (void *)d->rows_q, (void *)d->rows_partials,
                  d->rows_terms, d->rows_w_terms, d->rows_terms6,
                  (void *)d->rows_tokens, (void *)d->step_ops,
                  (void *)d->step_scratch, (void *)d->arrivals,
                  (void *)d->step_trace})
    cudaFree(p);
  cudaFree(d->owned_weights);
  cudaStreamDestroy(d->stream);
  delete d;
}

void vx_decoder_reset(vx_decoder *d) {
  CUDA_OK(cudaStreamSynchronize(d->stream));
  if (d->push) {
    /* a wait for another rank's record that ran out is worth a line: the
       tokens since then are not the model's */
    int32_t gave_up = 0;
    CUDA_OK(cudaMemcpy(&gave_up, d->pick_gave_up, sizeof gave_up,
                       cudaMemcpyDeviceToHost));
    if (gave_up) {
      fprintf(stderr, "[Vx CUDA] vx_decoder: a rank's best token did not arrive "
                      "within a second; the ranks no longer agree\n");
      CUDA_OK(cudaMemset(d->pick_gave_up, 0, sizeof gave_up));
    }
  }
  CUDA_OK(cudaMemsetAsync(d->positions, 0, 32 * sizeof(int32_t), d->stream));
  CUDA_OK(cudaStreamSynchronize(d->stream));
  d->host_pos = 0;
}

int32_t vx_decoder_step(vx_decoder *d, const int32_t *tokens_in,
                        int32_t *tokens_out) {
  const int pos = d->host_pos;
  if (pos >= d->c.max_seq)
    stop("vx_decoder_step: position %d is past max_seq %d", pos, d->c.max_seq);
  cudaGraphExec_t exec = graph_for(d, d->one_kernel ? 0 : pos / 256);
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

/* A run of prompt tokens of a one-sequence decoder, all positions at once: the
   positions are the rows of tensor-core GEMMs (prefill.cu; the reference's form
   of this are the multi-row kernels of nn.vx:2317-3066), every position writes
   its K and V into the cache at its own row, and position t attends rows
   0 .. first + t. No logits: the caller feeds the last prompt token through
   vx_decoder_step. Returns the number of tokens taken (all of them, or 0 when
   there are fewer than 32: single steps are as fast then), or -1 with
   vx_b200_last_error() when this decoder cannot do it. */
int32_t vx_decoder_prefill(vx_decoder *d, const int32_t *tokens, int32_t count) {
  const vx_decoder_config &c = d->c;
  const int hd = c.head_dim;
  const int qkv_rows = (d->q_local + 2 * d->kv_local) * hd, att_cols = d->q_local * hd;
  bool fused = true;
  for (int l = 0; l < c.n_layers; ++l)
    fused = fused && !d->wk[l] && !d->wv[l] && !d->w_up[l];
  const bool q4 = d->wfmt == vxb::kFmtQ4, fp8 = d->wfmt == vxb::kFmtFp8;
  if (c.batch != 1 || (c.weights_bf16 != 1 && !q4 && !fp8) || d->ranks != 1 ||
      hd != 128 || c.dim % 64 != 0 || d->hidden_local % 64 != 0 || !fused ||
      (fp8 && (c.dim % 128 != 0 || d->hidden_local % 128 != 0))) {
    vxb::set_last_error("vx_decoder_prefill: needs one sequence, one rank, bf16, fp8 "
                        "or Q4_0 weights with q/k/v rows in one matrix and gate/up "
                        "rows in one matrix, head_dim 128 and widths in multiples "
                        "of 64 (of 128 for fp8)");
    return -1;
  }
  /* VXB_Q4_PREFILL=mma / VXB_FP8_PREFILL=mma keep the quantised GEMMs on the
     mma.sync kernels (for measurements); the default unpacks a matrix to bf16
     terms and runs the CTA-pair GEMM. */
  const char *route = getenv("VXB_Q4_PREFILL"), *route8 = getenv("VXB_FP8_PREFILL");
  const bool q4_on_pairs = q4 && !(route && strcmp(route, "mma") == 0);
  const bool fp8_on_pairs = fp8 && !(route8 && strcmp(route8, "mma") == 0);
  const bool on_pairs = q4_on_pairs || fp8_on_pairs;
  /* how many bf16 terms a weight becomes, and the segments the activations'
     terms are spread over to meet them */
  const int w_terms = q4_on_pairs ? 2 : 3, segments = q4_on_pairs ? 6 : 7;
  static const int spread_q4[6] = {0, 0, 1, 1, 2, 2};
  static const int spread_fp8[7] = {0, 0, 0, 1, 1, 1, 2};
  /* One GEMM of the prompt, on CTA pairs: bf16 weights as they are, quantised
     ones unpacked to bf16 terms first; or, when asked, Q4_0 on the grouped
     kernel of the experts (one matrix, tiles of sixteen positions) and fp8 on
     its twin (gemm_fp8_rows.cu). Every way sums[run][t][r] for the finishing
     kernels. */
  auto gemm = [&](const void *w, const void *scales, int n, int cols, int *runs) {
    if (!q4 && !fp8)
      return vxb::rows_gemm(d->rows_terms, w, count, n, cols, d->rows_partials, runs,
                            d->stream);
    if (on_pairs) {
      /* Q4_0: exact all the same, two bf16 terms a weight, three an activation,
         six products on tcgen05 instead of three on mma.sync. fp8: the f32
         value code * scale as three terms, the six products of an f32 product
         and one more. */
      const char *why =
          q4 ? vxb::rows_q4_two_terms(d->rows_w_terms, w, scales, n, cols, d->stream)
             : vxb::rows_fp8_three_terms(d->rows_w_terms, w, scales, n, cols, d->stream);
      if (why)
        return why;
      why = vxb::rows_spread_terms(d->rows_terms6, d->rows_terms, count, cols, segments,
                                   q4 ? spread_q4 : spread_fp8, d->stream);
      if (why)
        return why;
      return vxb::rows_gemm_of(d->rows_terms6, segments * (int64_t)cols, d->rows_w_terms,
                               w_terms * (int64_t)cols, count, n, d->rows_partials, runs,
                               d->stream);
    }
    *runs = 1;
    return q4 ? vxb::rows_gemm_q4(d->rows_terms, w, scales, count, n, cols,
                                  d->rows_partials, d->stream)
              : vxb::rows_gemm_fp8(d->rows_terms, w, scales, count, n, cols,
                                   d->rows_partials, d->stream);
  };
  if (count < 0 || d->host_pos + count > c.max_seq) {
    vxb::set_last_error("vx_decoder_prefill: the prompt does not fit max_seq");
    return -1;
  }
  if (count < 32)
    return 0;
  const int T = count;
  int widest = c.dim > d->hidden_local ? c.dim : d->hidden_local;
  if (att_cols > widest)
    widest = att_cols;
  const int shapes[4][2] = {{qkv_rows, c.dim}, {c.dim, att_cols},
                            {2 * d->hidden_local, c.dim}, {c.dim, d->hidden_local}};
  if (T > d->rows_cap || (on_pairs && !d->rows_w_terms)) {
    const int cap = T > d->rows_cap ? T : d->rows_cap;
    for (void *p : {(void *)d->rows_x, (void *)d->rows_q, d->rows_terms,
                    (void *)d->rows_tokens})
      cudaFree(p);
    if (on_pairs) {
      cudaFree(d->rows_w_terms);
      cudaFree(d->rows_terms6);
      size_t widest_matrix = 0;
      for (const auto &sh : shapes)
        if ((size_t)sh[0] * sh[1] > widest_matrix)
          widest_matrix = (size_t)sh[0] * sh[1];
      d->rows_w_terms = dev_alloc<uint16_t>(w_terms * widest_matrix);
      d->rows_terms6 = dev_alloc<uint16_t>((size_t)cap * segments * widest);
    }
    d->rows_x = dev_alloc<float>((size_t)cap * c.dim);
    d->rows_q = dev_alloc<float>((size_t)cap * att_cols);
    d->rows_terms = dev_alloc<uint16_t>((size_t)cap * 3 * widest);
    d->rows_tokens = dev_alloc<int32_t>(cap);
    d->rows_cap = cap;
  }
  /* The sums of this call's GEMMs: the number of runs depends on T, and a
     shorter prompt can ask for more of them than a longer one did. */
  size_t sums = 0;
  for (const auto &sh : shapes) {
    const int64_t k_cols = (on_pairs ? segments : 3) * (int64_t)sh[1];
    const size_t one = (size_t)vxb::rows_gemm_splits_of(T, sh[0], k_cols) * T * sh[0];
    if (one > sums)
      sums = one;
  }
  if (sums > d->rows_partial_floats) {
    cudaFree(d->rows_partials);
    d->rows_partials = dev_alloc<float>(sums);
    d->rows_partial_floats = sums;
  }
  cudaStream_t s = d->stream;
  CUDA_OK(cudaMemcpyAsync(d->rows_tokens, tokens, (size_t)T * sizeof(int32_t),
                          cudaMemcpyHostToDevice, s));
  need(vxb::embed(d->rows_x, d->embed, true, d->rows_tokens, c.dim, c.vocab, T,
                  c.dim, s),
       "embed");
  int splits = 1;
  const bool fuse_norm = c.dim <= 8192;
  need(vxb::rows_norm_terms(d->rows_terms, d->rows_x, d->attn_norm[0], T, c.dim, c.eps,
                            s),
       "RMSNorm");
  for (int l = 0; l < c.n_layers; ++l) {
    /* rows_terms hold the terms of RMSNorm(x) * attn_norm[l] here */
    float *kc = d->k_cache + l * d->cache_layer_stride;
    float *vc = d->v_cache + l * d->cache_layer_stride;
    need(gemm(d->wq[l], d->s_qkv[l], qkv_rows, c.dim, &splits), "q/k/v");
    need(vxb::rows_qkv_finish(d->rows_partials, splits, T, d->q_local, d->kv_local,
                              hd, d->bqkv[l], d->cos_t, d->sin_t, d->positions,
                              d->rows_q, kc, vc, s),
         "RoPE and the cache store");
    /* No logits are computed: once the last layer's K and V are in the cache,
       nothing of what follows them is read by anyone. */
    if (l == c.n_layers - 1)
      break;
    need(vxb::rows_attention(d->rows_terms, d->rows_q, kc, vc, d->positions, T,
                             d->q_local, d->kv_local, hd, s),
         "attention");
    need(gemm(d->wo[l], d->s_o[l], c.dim, att_cols, &splits), "the output projection");
    if (fuse_norm) {
      need(vxb::rows_residual_norm(d->rows_terms, d->rows_x, d->rows_partials, splits,
                                   T, d->ffn_norm[l], c.dim, c.eps, s),
           "the residual add and RMSNorm");
    } else {
      need(vxb::rows_residual_finish(d->rows_x, d->rows_partials, splits, T, c.dim, s),
           "the residual add");
      need(vxb::rows_norm_terms(d->rows_terms, d->rows_x, d->ffn_norm[l], T, c.dim,
                                c.eps, s),
           "RMSNorm");
    }
    need(gemm(d->w_gate[l], d->s_gate_up[l], 2 * d->hidden_local, c.dim, &splits),
         "gate/up");
    need(vxb::rows_swiglu_finish(d->rows_terms, d->rows_partials, splits, T,
                                 d->hidden_local, s),
         "SwiGLU");
    need(gemm(d->w_down[l], d->s_down[l], c.dim, d->hidden_local, &splits),
         "the down projection");
    if (fuse_norm) {
      need(vxb::rows_residual_norm(d->rows_terms, d->rows_x, d->rows_partials, splits,
                                   T, d->attn_norm[l + 1], c.dim, c.eps, s),
           "the residual add and RMSNorm");
    } else {
      need(vxb::rows_residual_finish(d->rows_x, d->rows_partials, splits, T, c.dim, s),
           "the residual add");
      need(vxb::rows_norm_terms(d->rows_terms, d->rows_x, d->attn_norm[l + 1], T, c.dim,
                                c.eps, s),
           "RMSNorm");
    }
  }
  advance_by_kernel<<<1, 32, 0, s>>>(d->positions, T);
  d->host_pos += T;
  return T;
}

/* ---- llama2.c checkpoints ------------------------------------------------------
 * The file the reference's llama programs read (stdlib/rust_core/src/ffi/
 * llama.rs:11-47: vx_load_config takes the first 7 int32, vx_load_weights the
 * f32 values after them; stdlib/std/llama.vx:86-148 gives the order): dim,
 * hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len, then
 * token_embedding_table [vocab, dim], rms_att [L, dim], wq [L, dim, dim],
 * wk, wv [L, kv_dim, dim], wo [L, dim, dim], rms_ffn [L, dim],
 * w1 [L, hidden, dim], w2 [L, dim, hidden], w3 [L, hidden, dim],
 * rms_final [dim]. llama2.c writes a negative vocab_size when the classifier
 * is not the embedding table; it then follows two legacy RoPE tables of
 * seq_len * head_size / 2 values each. */
namespace {
struct MappedFile {
  const unsigned char *data = nullptr;
  size_t bytes = 0;
  int fd = -1;
  ~MappedFile() {
    if (data)
      munmap((void *)data, bytes);
    if (fd >= 0)
      close(fd);
  }
};
const char *map_file(const char *path, MappedFile *f) {
  static thread_local char msg[512];
  f->fd = path ? open(path, O_RDONLY) : -1;
  struct stat st;
  if (f->fd < 0 || fstat(f->fd, &st) != 0) {
    snprintf(msg, sizeof msg, "cannot open the checkpoint %s",
             path ? path : "(null)");
    return msg;
  }
  f->bytes = (size_t)st.st_size;
  if (f->bytes < 28) {
    snprintf(msg, sizeof msg,
             "%s is %zu bytes: shorter than the 7 int32 of a llama2.c header",
             path, f->bytes);
    return msg;
  }
  void *p = mmap(nullptr, f->bytes, PROT_READ, MAP_PRIVATE, f->fd, 0);
  if (p == MAP_FAILED) {
    snprintf(msg, sizeof msg, "cannot map the checkpoint %s", path);
    return msg;
  }
  f->data = (const unsigned char *)p;
  return nullptr;
}
/* The header, checked; `floats` gets how many f32 values the weights take. */
const char *read_llama2c_header(const MappedFile &f, const char *path,
                                vx_llama2c_config *c, bool *shared,
                                int64_t *floats) {
  static thread_local char msg[512];
  memcpy(c, f.data, 28);
  *shared = c->vocab_size > 0;
  if (!*shared)
    c->vocab_size = -c->vocab_size;
  if (c->dim <= 0 || c->hidden_dim <= 0 || c->n_layers <= 0 || c->n_heads <= 0 ||
      c->n_kv_heads <= 0 || c->vocab_size <= 0 || c->seq_len <= 0 ||
      c->dim % c->n_heads != 0 || c->n_heads % c->n_kv_heads != 0) {
    snprintf(msg, sizeof msg,
             "%s does not begin with a llama2.c header (dim %d, hidden_dim %d, "
             "n_layers %d, n_heads %d, n_kv_heads %d, vocab_size %d, seq_len %d)",
             path, c->dim, c->hidden_dim, c->n_layers, c->n_heads, c->n_kv_heads,
             c->vocab_size, c->seq_len);
    return msg;
  }
  const int64_t dim = c->dim, L = c->n_layers, hs = c->dim / c->n_heads;
  const int64_t kv = c->n_kv_heads * hs, hid = c->hidden_dim, vocab = c->vocab_size;
  int64_t n = vocab * dim + L * dim + L * dim * dim + 2 * L * dim * kv +
              L * dim * dim + L * dim + 3 * L * dim * hid + dim;
  if (!*shared)
    n += c->seq_len * hs + vocab * dim; /* two tables of seq_len*hs/2, wcls */
  *floats = n;
  if ((int64_t)f.bytes < 28 + 4 * n) {
    snprintf(msg, sizeof msg,
             "%s holds %zu bytes, and its header describes %lld bytes of "
             "weights after the 28 of the header: the file is cut short or the "
             "header is not this file's",
             path, f.bytes, (long long)(4 * n));
    return msg;
  }
  return nullptr;
}
} // namespace

int32_t vx_b200_llama2c_config(const char *path, vx_llama2c_config *out) {
  MappedFile f;
  bool shared;
  int64_t floats;
  vx_llama2c_config c;
  const char *why = map_file(path, &f);
  if (!why)
    why = read_llama2c_header(f, path, &c, &shared, &floats);
  if (why) {
    vxb::set_last_error(why);
    return -1;
  }
  if (out)
    *out = c;
  return 0;
}

vx_decoder *vx_decoder_from_llama2c(const char *path, int32_t batch,
                                    int32_t max_seq) {
  MappedFile f;
  bool shared;
  int64_t floats;
  vx_llama2c_config c;
  const char *why = map_file(path, &f);
  if (!why)
    why = read_llama2c_header(f, path, &c, &shared, &floats);
  if (why) {
    vxb::set_last_error(why);
    return nullptr;
  }
  /* One device buffer for all weights, filled through a pinned staging buffer
     in pieces, so that neither a second host copy of the model nor a pageable
     copy of it is made. */
  float *dev = nullptr;
  if (cudaMalloc((void **)&dev, (size_t)floats * 4) != cudaSuccess) {
    cudaGetLastError();
    vxb::set_last_error("out of device memory for the checkpoint's weights");
    return nullptr;
  }
  const size_t piece = (size_t)32 << 20;
  void *pinned[2] = {nullptr, nullptr};
  cudaEvent_t landed[2];
  cudaStream_t copy_stream;
  CUDA_OK(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking));
  for (int i = 0; i < 2; ++i) {
    CUDA_OK(cudaMallocHost(&pinned[i], piece));
    CUDA_OK(cudaEventCreateWithFlags(&landed[i], cudaEventDisableTiming));
  }
  const unsigned char *src = f.data + 28;
  const size_t total = (size_t)floats * 4;
  int turn = 0;
  for (size_t at = 0; at < total; at += piece, turn ^= 1) {
    const size_t n = total - at < piece ? total - at : piece;
    CUDA_OK(cudaEventSynchronize(landed[turn])); /* the buffer is free again */
    memcpy(pinned[turn], src + at, n);
    CUDA_OK(cudaMemcpyAsync((char *)dev + at, pinned[turn], n,
                            cudaMemcpyHostToDevice, copy_stream));
    CUDA_OK(cudaEventRecord(landed[turn], copy_stream));
  }
  CUDA_OK(cudaStreamSynchronize(copy_stream));
  for (int i = 0; i < 2; ++i) {
    cudaFreeHost(pinned[i]);
    cudaEventDestroy(landed[i]);
  }
  cudaStreamDestroy(copy_stream);

  const int64_t dim = c.dim, L = c.n_layers, hs = c.dim / c.n_heads;
  const int64_t kv = c.n_kv_heads * hs, hid = c.hidden_dim, vocab = c.vocab_size;
  const float *p = dev;
  const float *tok = p;          p += vocab * dim;
  const float *rms_att = p;      p += L * dim;
  const float *wq = p;           p += L * dim * dim;
  const float *wk = p;           p += L * dim * kv;
  const float *wv = p;           p += L * dim * kv;
  const float *wo = p;           p += L * dim * dim;
  const float *rms_ffn = p;      p += L * dim;
  const float *w1 = p;           p += L * dim * hid;
  const float *w2 = p;           p += L * hid * dim;
  const float *w3 = p;           p += L * dim * hid;
  const float *rms_final = p;    p += dim;
  const float *wcls = shared ? tok : p + (int64_t)c.seq_len * hs;
  std::vector<const void *> a_norm(L), a_wq(L), a_wk(L), a_wv(L), a_wo(L),
      f_norm(L), a_w1(L), a_w2(L), a_w3(L);
  for (int64_t l = 0; l < L; ++l) {
    a_norm[l] = rms_att + l * dim;
    a_wq[l] = wq + l * dim * dim;
    a_wk[l] = wk + l * dim * kv;
    a_wv[l] = wv + l * dim * kv;
    a_wo[l] = wo + l * dim * dim;
    f_norm[l] = rms_ffn + l * dim;
    a_w1[l] = w1 + l * dim * hid;
    a_w2[l] = w2 + l * hid * dim;
    a_w3[l] = w3 + l * dim * hid;
  }
  vx_decoder_weights w{};
  w.embed = tok;
  w.attn_norm = a_norm.data();
  w.wq = a_wq.data();
  w.wk = a_wk.data();
  w.wv = a_wv.data();
  w.wo = a_wo.data();
  w.ffn_norm = f_norm.data();
  w.w_gate = a_w1.data();
  w.w_up = a_w3.data();
  w.w_down = a_w2.data();
  w.final_norm = rms_final;
  w.lm_head = wcls;
  vx_decoder_config cfg{};
  cfg.dim = c.dim;
  cfg.hidden = c.hidden_dim;
  cfg.n_layers = c.n_layers;
  cfg.q_heads = c.n_heads;
  cfg.kv_heads = c.n_kv_heads;
  cfg.head_dim = (int32_t)hs;
  cfg.vocab = c.vocab_size;
  cfg.max_seq = max_seq > 0 ? max_seq : c.seq_len;
  cfg.eps = 1e-5f;
  cfg.rope_theta = 10000.0f;
  cfg.weights_bf16 = 0;
  cfg.batch = batch > 0 ? batch : 1;
  cfg.tp_ranks = 1;
  cfg.tp_reduce = 0;
  vx_decoder *d = vx_decoder_create(&cfg, &w);
  d->owned_weights = dev;
  return d;
}

const float *vx_decoder_logits(const vx_decoder *d) { return d->logits; }

float *vx_decoder_kv_cache(vx_decoder *d, int32_t which) {
  return which == 0 ? d->k_cache : which == 1 ? d->v_cache : nullptr;
}

int64_t vx_decoder_kv_cache_bytes(const vx_decoder *d) {
  return d->cache_layer_stride * d->c.n_layers * (int64_t)sizeof(float);
}

int32_t vx_decoder_adopt_kv(vx_decoder *d, const float *k, const float *v,
                            int32_t positions) {
  if (!k || !v || positions < 0 || positions > d->c.max_seq) {
    vxb::set_last_error("vx_decoder_adopt_kv: needs both caches and 0 <= "
                        "positions <= max_seq");
    return -1;
  }
  /* rows 0 .. positions-1 of every layer and sequence; one copy each (the
     source may be another GPU's memory: unified addressing finds the way) */
  const size_t run = (size_t)positions * d->kv_local * d->c.head_dim * sizeof(float);
  for (int l = 0; l < d->c.n_layers && run; ++l)
    for (int b = 0; b < d->c.batch; ++b) {
      const int64_t at = l * d->cache_layer_stride + b * d->cache_batch_stride;
      CUDA_OK(cudaMemcpyAsync(d->k_cache + at, k + at, run, cudaMemcpyDefault,
                              d->stream));
      CUDA_OK(cudaMemcpyAsync(d->v_cache + at, v + at, run, cudaMemcpyDefault,
                              d->stream));
    }
  set_positions_kernel<<<1, 32, 0, d->stream>>>(d->positions, d->c.batch, positions);
  CUDA_OK(cudaStreamSynchronize(d->stream)); /* the caller may free k and v */
  d->host_pos = positions;
  return positions;
}
void *vx_decoder_stream(const vx_decoder *d) { return (void *)d->stream; }
int32_t vx_decoder_step_trace(vx_decoder *d, uint64_t *out, int32_t capacity) {
  if (!d->step_trace)
    return 0;
  int32_t n = d->n_step_ops * vxb::kStepTraceSlots;
  if (n > capacity)
    n = capacity;
  CUDA_OK(cudaStreamSynchronize(d->stream));
  CUDA_OK(cudaMemcpy(out, d->step_trace, (size_t)n * sizeof(uint64_t),
                     cudaMemcpyDeviceToHost));
  return n;
}

int32_t vx_decoder_kernels_per_step(const vx_decoder *d) {
  return d->kernels_per_step;
}

} /* extern "C" */
