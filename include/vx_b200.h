/* vx_b200.h -- entry points that libvx_cuda_dispatch.so exports on top of the
 * 24 symbols of vx_hardware_runtime.h.  All are additive: a program that uses
 * only the reference interface never calls them.
 *
 *   vx_nn_*        the decode operators of stdlib/std/nn.vx, one C function per
 *                  Vx function, with that function's parameter order and the
 *                  C convention of a Vx `pub fn` (docs/lang/abi.md section 3.6):
 *                  a tensor of rank r arrives as 3 + 2r values -- allocated
 *                  pointer, aligned pointer, offset, r sizes, r strides -- and a
 *                  scalar as one value.  Tensors must be packed and in GPU
 *                  memory.  A shape that the Vx function's `assert` refuses
 *                  stops the program here too.
 *   vx_decoder_*   one whole decoder token (all layers, logits, argmax) as one
 *                  CUDA graph of fused kernels; the host-side counterpart of
 *                  transformer<D> in tests/backend/pass/llama2.vx:218-429 and
 *                  of a program written with std::nn.
 *   vx_b200_*      direct GEMM / flash-attention / utility calls on device
 *                  pointers, for hosts that are not Vx programs.
 *
 * Work is queued on the stream of vx_cuda_set_stream (the legacy default
 * stream when none is set) and the calls do not wait unless they say so.
 */
#ifndef VX_B200_H
#define VX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A tensor parameter in the `pub fn` convention. */
#define VX_TENSOR1(t)                                                          \
  void *t##_allocated, void *t##_aligned, int64_t t##_offset, int64_t t##_n0,  \
      int64_t t##_s0
#define VX_TENSOR2(t)                                                          \
  void *t##_allocated, void *t##_aligned, int64_t t##_offset, int64_t t##_n0,  \
      int64_t t##_n1, int64_t t##_s0, int64_t t##_s1
#define VX_TENSOR3(t)                                                          \
  void *t##_allocated, void *t##_aligned, int64_t t##_offset, int64_t t##_n0,  \
      int64_t t##_n1, int64_t t##_n2, int64_t t##_s0, int64_t t##_s1,          \
      int64_t t##_s2
#define VX_TENSOR4(t)                                                          \
  void *t##_allocated, void *t##_aligned, int64_t t##_offset, int64_t t##_n0,  \
      int64_t t##_n1, int64_t t##_n2, int64_t t##_n3, int64_t t##_s0,          \
      int64_t t##_s1, int64_t t##_s2, int64_t t##_s3

/* ---- std::nn operators (weights bf16, everything else f32) ----------------- */
/* nn_matvec, stdlib/std/nn.vx:24 */
void vx_nn_matvec(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(x), int32_t rows,
                  int32_t cols);
/* nn_matvec_add, nn.vx:54 */
void vx_nn_matvec_add(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(x), int32_t rows,
                      int32_t cols);
/* nn_matvec_heads_add, nn.vx:86 */
void vx_nn_matvec_heads_add(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR2(x),
                            int32_t rows, int32_t heads, int32_t head_dim);
/* nn_qkv, nn.vx:124 */
void vx_nn_qkv(VX_TENSOR2(q), VX_TENSOR2(k), VX_TENSOR2(v), VX_TENSOR1(w),
               VX_TENSOR1(b), VX_TENSOR1(x), int32_t q_heads, int32_t kv_heads,
               int32_t head_dim, int32_t cols);
/* nn_swiglu, nn.vx:169 */
void vx_nn_swiglu(VX_TENSOR1(out), VX_TENSOR1(w), VX_TENSOR1(x), int32_t rows,
                  int32_t cols);
/* nn_rms_norm, nn.vx:212 */
void vx_nn_rms_norm(VX_TENSOR1(y), VX_TENSOR1(x), VX_TENSOR1(w), int32_t n,
                    float eps);
/* nn_rope_and_store, nn.vx:245 */
void vx_nn_rope_and_store(VX_TENSOR2(q_out), VX_TENSOR3(k_cache),
                          VX_TENSOR3(v_cache), VX_TENSOR2(q), VX_TENSOR2(k),
                          VX_TENSOR2(v), VX_TENSOR2(cos), VX_TENSOR2(sin),
                          int32_t pos, int32_t q_heads, int32_t kv_heads,
                          int32_t head_dim);
/* nn_attention, nn.vx:349 (`part` from nn_attention_scratch, nn.vx:370) */
void vx_nn_attention(VX_TENSOR2(out), VX_TENSOR4(part), VX_TENSOR2(q),
                     VX_TENSOR3(k_cache), VX_TENSOR3(v_cache), int32_t pos,
                     int32_t q_heads, int32_t kv_heads, int32_t head_dim);
/* nn_argmax, nn.vx:870 */
void vx_nn_argmax(VX_TENSOR1(out), VX_TENSOR1(logits), int32_t n);
/* nn_embed, nn.vx:942 */
void vx_nn_embed(VX_TENSOR1(x), VX_TENSOR1(table), VX_TENSOR1(token),
                 int32_t dim);

/* The same projections with quantised weights. fp8 (nn.vx:1296-1640): `w` is
   f8e4m3 codes, 4 to a 32-bit word, `scales` one f32 per block of 128 x 128
   weights, [ceil(rows / 128), cols / 128]; rows a multiple of 4, cols of 128.
   Q4_0 (nn.vx:1645-2100): codes of 4 bits, 8 to a word, weight = (code - 8) *
   scale with one f16 scale per 32 weights of a row, [rows, cols / 32]; rows a
   multiple of 4, cols of 32. The bias of the q/k/v projections is bf16. */
/* nn_matvec_fp8 nn.vx:1306, _add :1367, _heads_add :1427, nn_qkv_fp8 :1492,
   nn_swiglu_fp8 :1577 */
void vx_nn_matvec_fp8(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(scales),
                      VX_TENSOR1(x), int32_t rows, int32_t cols);
void vx_nn_matvec_fp8_add(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(scales),
                          VX_TENSOR1(x), int32_t rows, int32_t cols);
void vx_nn_matvec_fp8_heads_add(VX_TENSOR1(y), VX_TENSOR1(w),
                                VX_TENSOR1(scales), VX_TENSOR2(x), int32_t rows,
                                int32_t heads, int32_t head_dim);
void vx_nn_qkv_fp8(VX_TENSOR2(q), VX_TENSOR2(k), VX_TENSOR2(v), VX_TENSOR1(w),
                   VX_TENSOR1(scales), VX_TENSOR1(b), VX_TENSOR1(x),
                   int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                   int32_t cols);
void vx_nn_swiglu_fp8(VX_TENSOR1(out), VX_TENSOR1(w), VX_TENSOR1(scales),
                      VX_TENSOR1(x), int32_t rows, int32_t cols);
/* nn_matvec_q4 nn.vx:1666, _add :1748, _heads_add :1831, nn_qkv_q4 :1912,
   nn_swiglu_q4 :2005 */
void vx_nn_matvec_q4(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(scales),
                     VX_TENSOR1(x), int32_t rows, int32_t cols);
void vx_nn_matvec_q4_add(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(scales),
                         VX_TENSOR1(x), int32_t rows, int32_t cols);
void vx_nn_matvec_q4_heads_add(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(scales),
                               VX_TENSOR2(x), int32_t rows, int32_t heads,
                               int32_t head_dim);
void vx_nn_qkv_q4(VX_TENSOR2(q), VX_TENSOR2(k), VX_TENSOR2(v), VX_TENSOR1(w),
                  VX_TENSOR1(scales), VX_TENSOR1(b), VX_TENSOR1(x),
                  int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                  int32_t cols);
void vx_nn_swiglu_q4(VX_TENSOR1(out), VX_TENSOR1(w), VX_TENSOR1(scales),
                     VX_TENSOR1(x), int32_t rows, int32_t cols);

/* A mixture-of-experts layer: the router and the two expert projections of one
   token, in bf16 and in Q4_0. The experts' matrices sit one after another in
   `w` (and `scales`); `ids` is device memory, normally nn_top_k's output.
   nn_top_k nn.vx:904, nn_moe_swiglu :968, nn_moe_down_add :1019,
   nn_moe_swiglu_q4 :2105, nn_moe_down_q4_add :2190. */
void vx_nn_top_k(VX_TENSOR1(ids), VX_TENSOR1(weights), VX_TENSOR1(logits), int32_t n,
                 int32_t k);
void vx_nn_moe_swiglu(VX_TENSOR2(out), VX_TENSOR1(w), VX_TENSOR1(ids), VX_TENSOR1(x),
                      int32_t k, int32_t rows, int32_t cols, int32_t experts);
void vx_nn_moe_down_add(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(ids),
                        VX_TENSOR1(weights), VX_TENSOR2(h), int32_t k, int32_t rows,
                        int32_t cols, int32_t experts);
void vx_nn_moe_swiglu_q4(VX_TENSOR2(out), VX_TENSOR1(w), VX_TENSOR1(scales),
                         VX_TENSOR1(ids), VX_TENSOR1(x), int32_t k, int32_t rows,
                         int32_t cols, int32_t experts);
void vx_nn_moe_down_q4_add(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(scales),
                           VX_TENSOR1(ids), VX_TENSOR1(weights), VX_TENSOR2(h),
                           int32_t k, int32_t rows, int32_t cols, int32_t experts);

/* Kernels for n positions at once (nn.vx:2312-2950): each is the one-position
   kernel for every row t of its [n, ...] tensors, with bit-identical rows.
   nn_matvec_rows nn.vx:2802, nn_matvec_q4_rows :2317, nn_rms_norm_rows :2835,
   nn_argmax_rows :2866, nn_embed_rows :2933. */
void vx_nn_matvec_rows(VX_TENSOR2(y), VX_TENSOR1(w), VX_TENSOR2(x), int32_t n,
                       int32_t rows, int32_t cols);
void vx_nn_matvec_q4_rows(VX_TENSOR2(y), VX_TENSOR1(w), VX_TENSOR1(scales),
                          VX_TENSOR2(x), int32_t n, int32_t rows, int32_t cols);
void vx_nn_rms_norm_rows(VX_TENSOR2(y), VX_TENSOR2(x), VX_TENSOR1(w), int32_t n,
                         int32_t dim, float eps);
void vx_nn_argmax_rows(VX_TENSOR1(out), VX_TENSOR2(logits), int32_t n,
                       int32_t count);
void vx_nn_embed_rows(VX_TENSOR2(x), VX_TENSOR1(table), VX_TENSOR1(tokens),
                      int32_t n, int32_t dim);
/* nn_top_k_rows nn.vx:2897, nn_matvec_q4_heads_add_rows :2459, nn_qkv_q4_rows
   :2614, nn_moe_swiglu_q4_rows :2958, nn_moe_down_q4_add_rows :3066. ids and
   weights are [n, k]; out and h hold a row for each of the n * k (position,
   slot) pairs, pair t * k + e being slot e of position t. */
void vx_nn_top_k_rows(VX_TENSOR2(ids), VX_TENSOR2(weights), VX_TENSOR2(logits),
                      int32_t n, int32_t count, int32_t k);
void vx_nn_matvec_q4_heads_add_rows(VX_TENSOR2(y), VX_TENSOR1(w), VX_TENSOR1(scales),
                                    VX_TENSOR3(x), int32_t n, int32_t rows,
                                    int32_t heads, int32_t head_dim);
void vx_nn_qkv_q4_rows(VX_TENSOR3(q), VX_TENSOR3(k), VX_TENSOR3(v), VX_TENSOR1(w),
                       VX_TENSOR1(scales), VX_TENSOR1(b), VX_TENSOR2(x), int32_t n,
                       int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                       int32_t cols);
void vx_nn_moe_swiglu_q4_rows(VX_TENSOR2(out), VX_TENSOR1(w), VX_TENSOR1(scales),
                              VX_TENSOR2(ids), VX_TENSOR2(x), int32_t n, int32_t k,
                              int32_t rows, int32_t cols, int32_t experts);
void vx_nn_moe_down_q4_add_rows(VX_TENSOR2(y), VX_TENSOR1(w), VX_TENSOR1(scales),
                                VX_TENSOR2(ids), VX_TENSOR2(weights), VX_TENSOR2(h),
                                int32_t n, int32_t k, int32_t rows, int32_t cols,
                                int32_t experts);

/* The (position, slot) pairs of a mixture-of-experts layer grouped by expert: a
   stable counting sort in three kernels, and all three in nn_moe_group
   (nn_moe_group_count nn.vx:1070, nn_moe_group_offsets :1110,
   nn_moe_group_place :1252, nn_moe_group :1287). ids[p] is the expert of pair
   p. order gets the pairs expert by expert, each group starting at a multiple
   of `align` and padded to one, with n + i at a position i that holds no pair
   (order needs n + experts * (align - 1) positions); starts[e] is where group e
   begins and starts[experts] where the last ends; tile_expert[t] is the expert
   of positions align * t .. align * t + align - 1, or -1 past the last group.
   counts and base are [ceil(n / 256), experts]: the pairs of each expert among
   each 256 pairs, and where the first of them goes. An id that names no expert
   is skipped and reported once by vx_b200_kernel_status() (0x6E). */
void vx_nn_moe_group_count(VX_TENSOR2(counts), VX_TENSOR1(ids), int32_t n,
                           int32_t experts);
void vx_nn_moe_group_offsets(VX_TENSOR2(base), VX_TENSOR1(starts),
                             VX_TENSOR1(tile_expert), VX_TENSOR1(order),
                             VX_TENSOR2(counts), int32_t n, int32_t experts,
                             int32_t align);
void vx_nn_moe_group_place(VX_TENSOR1(order), VX_TENSOR1(ids), VX_TENSOR2(base),
                           int32_t n);
void vx_nn_moe_group(VX_TENSOR1(order), VX_TENSOR2(counts), VX_TENSOR2(base),
                     VX_TENSOR1(starts), VX_TENSOR1(tile_expert), VX_TENSOR1(ids),
                     int32_t experts, int32_t align);

/* ---- a whole decoder token -------------------------------------------------- */
typedef struct {
  int32_t dim, hidden, n_layers, q_heads, kv_heads, head_dim, vocab, max_seq;
  float eps;
  float rope_theta;
  /* 1: bf16 weights, half-split RoPE from tables (std::nn); 0: f32 weights,
     interleaved RoPE computed from the position (llama2.vx); 2 and 3: the
     std::nn flavour with the four projections of every layer in fp8 or in
     Q4_0 (their scales in vx_decoder_weights; norms, embedding and classifier
     stay bf16; one sequence, one rank). */
  int32_t weights_bf16;
  int32_t batch; /* 1, 2, 4, 8 or 16 sequences */
  /* Tensor parallel: this process holds q_heads / tp_ranks query heads,
     kv_heads / tp_ranks KV heads and hidden / tp_ranks MLP rows of every
     layer, and the job of vx_collective_init sums the partial outputs.
     1 = not sharded. The fields above are the WHOLE model's. */
  int32_t tp_ranks;
  /* How the partial sums of the row-split projections are added across ranks:
     0 = an NCCL all-reduce after the projection kernel; 1 = the projection
     kernel itself stores its results into every rank's receive buffer over
     NVLink (peer memory mapped through CUDA IPC) as (value, call number)
     pairs that are their own arrival flags, and a small kernel adds them to
     the residual in rank order (the same order on every rank). */
  int32_t tp_reduce;
} vx_decoder_config;

/* Device pointers, one entry per layer where the field is an array; the caller
   owns the memory. Shapes are this rank's share:
   wq [q_local*hd, dim] (with wk == NULL: q, k and v rows in one matrix),
   wk, wv [kv_local*hd, dim], bqkv bf16 or NULL, wo [dim, q_local*hd],
   w_gate [hidden_local, dim] (with w_up == NULL: gate rows then up rows),
   w_up [hidden_local, dim], w_down [dim, hidden_local]; norms [dim];
   embed, lm_head [vocab, dim]; cos, sin f32 [max_seq, head_dim/2] or NULL. */
typedef struct {
  const void *embed;
  const void *const *attn_norm;
  const void *const *wq;
  const void *const *wk;
  const void *const *wv;
  const void *const *bqkv;
  const void *const *wo;
  const void *const *ffn_norm;
  const void *const *w_gate;
  const void *const *w_up;
  const void *const *w_down;
  const void *final_norm;
  const void *lm_head;
  const float *cos;
  const float *sin;
  /* weights_bf16 2 or 3: the scales of wq (q, k and v rows in one matrix), wo,
     w_gate (gate rows then up rows) and w_down, one entry per layer: f32
     [ceil(rows / 128), cols / 128] for fp8, f16 [rows, cols / 32] for Q4_0.
     Not read otherwise. */
  const void *const *s_qkv;
  const void *const *s_o;
  const void *const *s_gate_up;
  const void *const *s_down;
} vx_decoder_weights;

typedef struct vx_decoder vx_decoder;

/* Allocates the KV cache and the activations on the current GPU. */
vx_decoder *vx_decoder_create(const vx_decoder_config *config,
                              const vx_decoder_weights *weights);
void vx_decoder_destroy(vx_decoder *d);
/* Every sequence back to position 0 (the cache is not cleared: rows past the
   position are never read). */
void vx_decoder_reset(vx_decoder *d);
/* One token for each of the `batch` sequences. tokens_in (host, batch values)
   feeds the step; NULL feeds the argmax of the previous step, which never left
   the GPU. tokens_out (host) receives the argmax of this step when not NULL --
   the call then waits for the GPU. Returns the position the step ran at. */
int32_t vx_decoder_step(vx_decoder *d, const int32_t *tokens_in,
                        int32_t *tokens_out);
/* A run of prompt tokens of a one-sequence decoder, all positions in one pass
   through the layers as rows of tensor-core GEMMs (the reference's multi-row
   kernels, nn.vx:2317-3066: its llama programs feed a prompt one decode step
   at a time). Fills the KV cache and advances the position; computes no
   logits, so the caller gives the last prompt token to vx_decoder_step.
   Returns how many tokens it took (all of them, or 0 when there are fewer
   than 32: the caller steps through those), or -1 with vx_b200_last_error()
   for a decoder that cannot (needs batch 1, one rank, bf16, fp8 or Q4_0
   weights with the q/k/v rows in one matrix and the gate/up rows in one,
   head_dim 128, widths in multiples of 64, of 128 for fp8). Quantised weights
   are unpacked, a matrix at a time, to bf16 terms for the same GEMM (Q4_0: two
   terms, exactly; fp8: the f32 value code * scale as three); with
   VXB_Q4_PREFILL=mma / VXB_FP8_PREFILL=mma in the environment the GEMMs
   unpack the codes in registers instead, once for sixteen positions (the
   kernel of the grouped experts, and its fp8 twin). */
int32_t vx_decoder_prefill(vx_decoder *d, const int32_t *tokens, int32_t count);
/* The logits of the last step: device memory, [batch, vocab] f32. */
const float *vx_decoder_logits(const vx_decoder *d);
/* The K (which = 0) or V (which = 1) cache of this rank: device memory, f32
   [layer][sequence][max_seq][kv_heads][head_dim], vx_decoder_kv_cache_bytes()
   bytes each. What a prefill process hands to a decode process
   (handoff_kv, tests/backend/pass/llama2.vx:431-458: the caches travel by
   vx_plugin_transfer_peer). */
float *vx_decoder_kv_cache(vx_decoder *d, int32_t which);
int64_t vx_decoder_kv_cache_bytes(const vx_decoder *d);
/* The receiving side of that hand-off: copies rows 0 .. positions-1 of every
   layer and sequence from k and v (device memory laid out like this decoder's
   own caches; on this GPU or on another one of the process) into the
   decoder's caches and puts every sequence at `positions`. Returns positions,
   or -1 with vx_b200_last_error(). k and v may be freed when it returns. */
int32_t vx_decoder_adopt_kv(vx_decoder *d, const float *k, const float *v,
                            int32_t positions);
/* The CUDA stream (a CUstream) that the decoder's steps run on, for a host
   that wants to record events around them. */
void *vx_decoder_stream(const vx_decoder *d);
/* How many kernels one step launches (for accounting). */
int32_t vx_decoder_kernels_per_step(const vx_decoder *d);
/* A decoder created with VXB_STEP_TRACE=1 in the environment whose step is one
   launch keeps six nanosecond clock readings per projection of the last step
   (one block's view: loop top, after the barrier, after the input is staged,
   after its rows, before and after the layer's attention); copies up to
   `capacity` of them to `out` and returns how many, 0 when there are none. No
   counterpart in the reference: a measuring aid. */
int32_t vx_decoder_step_trace(vx_decoder *d, uint64_t *out, int32_t capacity);

/* A llama2.c checkpoint: the file the reference's llama programs read through
   vx_load_config and vx_load_weights (stdlib/rust_core/src/ffi/llama.rs:11-47;
   the order of the weights: stdlib/std/llama.vx:86-148). */
typedef struct {
  int32_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
} vx_llama2c_config;
/* Reads and checks the header (a negative vocab_size, llama2.c's mark of a
   classifier of its own, comes back positive). 0, or -1 with the reason in
   vx_b200_last_error(): no such file, a file shorter than its header says. */
int32_t vx_b200_llama2c_config(const char *path, vx_llama2c_config *out);
/* A decoder (f32 weights, interleaved RoPE: the llama2.vx flavour) over the
   weights of the checkpoint, which are copied to the current GPU once and
   belong to the decoder. max_seq 0: the file's seq_len. NULL with the reason in
   vx_b200_last_error() when the file cannot be used. */
vx_decoder *vx_decoder_from_llama2c(const char *path, int32_t batch,
                                    int32_t max_seq);

/* ---- direct calls -------------------------------------------------------------
 * All return 0, or -1 with the reason in vx_b200_last_error(). */
const char *vx_b200_last_error(void);

/* C[m,n] = A[m,k] * B[k,n], row-major device memory, strides in elements.
   dtype is a VX_DTYPE_* code (f32, f64, f16, bf16). route: 0 = as a dispatch
   would run it; for 16-bit types 1 = tcgen05 with B as stored, 2 = tcgen05
   after transposing B into scratch ([n, k] elements), 3 = the plain kernel,
   4 and 5 = 1 and 2 on CTA pairs (256x256 tiles on the two SMs of a TPC). */
int32_t vx_b200_gemm(int32_t dtype, int32_t route, int64_t m, int64_t n,
                     int64_t k, const void *a, int64_t lda, const void *b,
                     int64_t ldb, void *c, int64_t ldc, void *scratch);
/* Waits for the stream, then: 0 when every tensor-core kernel since the last
   call ran to its end, else the code of the first wait that gave up. */
int32_t vx_b200_kernel_status(void);

/* Flash attention forward, bf16 [B, H, S, D] in and out, f32 softmax. */
int32_t vx_b200_flash_attention(const void *q, const void *k, const void *v,
                                void *out, int32_t B, int32_t H, int32_t S,
                                int32_t D, float scale, int32_t causal);

/* The Q4_0 experts of n positions on the tensor cores, fed by the grouping:
   order and tile_expert are vx_nn_moe_group's outputs for the n * k ids (row t
   of a packed [n, k] tensor is pairs t * k .. t * k + k - 1) with `align` 8 or
   16, and tiles the length of tile_expert (tiles * align >= n * k + experts *
   (align - 1)). An expert's sixteen rows are unpacked once for all pairs of a
   tile. Plain device pointers, packed rows: x [n, cols], out [n * k, rows]; for
   the down projection h [n * k, cols], weights [n * k], y [n, rows] (added to,
   a position's k experts in slot order) and a scratch of n * k * rows floats.
   The arithmetic of nn_moe_swiglu_q4_rows / nn_moe_down_q4_add_rows
   (nn.vx:2958, 3066) in another order of sums: results agree with the
   vx_nn_*_rows exports within rounding, not bit for bit. rows a multiple of 8,
   cols of 32 (fastest with cols a multiple of 128). */
/* y[n, rows] = x[n, cols] . W^T for a Q4_0 matrix W [rows, cols] (codes 8 to a
   u32 word, an f16 scale per 32 weights of a row: the layout of nn_matvec_q4,
   nn.vx:1645-1666) and n rows of f32 activations, on the tensor cores: the
   same kernel, one matrix, the rows in tiles of sixteen. What
   vx_nn_matvec_q4_rows computes, in another order of sums. Plain device
   pointers, packed rows; rows a multiple of 8, cols of 32. */
int32_t vx_b200_gemm_q4(float *y, const uint32_t *w, const uint16_t *scales,
                        const float *x, int32_t n, int32_t rows, int32_t cols);
/* The same for an fp8 matrix: f8e4m3 codes 4 to a u32 word and an f32 scale per
   block of 128 x 128, the layout of nn_matvec_fp8 (nn.vx:1296-1306). cols a
   multiple of 128. The reference has no fp8 kernel for n positions; this is
   the product a decoder with fp8 weights reads a prompt with. */
int32_t vx_b200_gemm_fp8(float *y, const uint32_t *w, const float *scales,
                         const float *x, int32_t n, int32_t rows, int32_t cols);
int32_t vx_b200_moe_swiglu_q4_grouped(float *out, const uint32_t *w,
                                      const uint16_t *scales, const int32_t *order,
                                      const int32_t *tile_expert, int32_t tiles,
                                      int32_t align, const float *x, int32_t n,
                                      int32_t k, int32_t rows, int32_t cols,
                                      int32_t experts);
int32_t vx_b200_moe_down_q4_add_grouped(float *y, const uint32_t *w,
                                        const uint16_t *scales, const int32_t *order,
                                        const int32_t *tile_expert, int32_t tiles,
                                        int32_t align, const float *weights,
                                        const float *h, float *scratch, int32_t n,
                                        int32_t k, int32_t rows, int32_t cols,
                                        int32_t experts);

/* Which kernel vx_nn_attention and the decoder's attention run from now on:
   1 = the parts of a head merged inside a thread-block cluster (no scratch
   used; the default), 2 = the reference's scheme (nn.vx:343-368, 823-866):
   one block per 32 or 64 positions, partial results in `part`, merged by the
   block that finishes last; 0 = back to the default. Returns the choice
   before. A decoder takes the choice when it records a token graph. This
   entry point has no counterpart in the reference (which has one kernel). */
int32_t vx_b200_attention_kernel(int32_t which);

/* Decode attention with no allocation of any kind, for hosts that cannot call
   cudaMalloc: processes that handed all device memory to their own pool at
   start-up, and loops that cannot take the device-wide wait an allocation
   implies. The computation of vx_nn_attention on plain device pointers (q, out
   [q_heads, head_dim]; caches [max_seq, kv_heads, head_dim]; f32), always by
   the split kernel, whose partial results and counters live in a fixed array
   inside the library image (68 KiB + 2 MiB per GPU, held until the process
   exits). Limit: pos < 16384, q_heads <= 256 and
   q_heads * (pos / n + 1) * (head_dim + 2) <= 2^19 with n = 32 below position
   640, else 64; beyond it: -1 and a message. All calls on a GPU share the
   array, so calls that overlap on the GPU race: keep them in stream order. The
   first call on a GPU looks up the array's address and fills it in, and should
   come before any stream capture. This entry point has no counterpart in the
   reference. */
int32_t vx_b200_attention_decode_static(float *out, const float *q,
                                        const float *k_cache,
                                        const float *v_cache, int32_t pos,
                                        int32_t q_heads, int32_t kv_heads,
                                        int32_t head_dim);

/* Column-split product for a job of g ranks: this rank holds A [m,k] and
   B_local [k, n_local]; c_full [m, g*n_local] is complete on every rank
   afterwards. c_local [m, n_local] and gathered [g, m, n_local] are scratch. */
int32_t vx_b200_gemm_column_split(int32_t dtype, int64_t m, int64_t n_local,
                                  int64_t k, const void *a, const void *b_local,
                                  void *c_local, void *gathered, void *c_full);

/* A bf16 matrix [rows, cols] in device memory into one of the quantised
   formats of std::nn, for hosts that make such a model out of bf16 weights
   (the reference's programs load theirs already quantised). format 2: fp8,
   `codes` rows * cols bytes, `scales` f32 [ceil(rows/128), cols/128] (the
   block's largest magnitude / 448), cols a multiple of 128. format 3: Q4_0 as
   llama.cpp makes it, `codes` rows * cols / 2 bytes, `scales` f16
   [rows, cols/32], cols a multiple of 32. The numbers are vx_decoder_config's
   weights_bf16 values. */
int32_t vx_b200_quantize(int32_t format, const void *w_bf16, int32_t rows,
                         int32_t cols, void *codes, void *scales);

/* Seeded synthetic data made on the GPU: N(0, sigma^2) or U[lo, hi), written as
   f32 or as bf16 (round to nearest even). */
int32_t vx_b200_fill_normal(void *out, int32_t as_bf16, int64_t n, uint64_t seed,
                            float sigma);
int32_t vx_b200_fill_uniform(void *out, int32_t as_bf16, int64_t n,
                             uint64_t seed, float lo, float hi);

#ifdef __cplusplus
}
#endif

#endif /* VX_B200_H */
