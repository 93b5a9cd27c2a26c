/* nn_api.cu -- the entry points of include/vx_b200.h: the std::nn operator
 * surface in the `pub fn` C convention, the whole-token decoder, and the direct
 * GEMM / attention / utility calls.  Checks here mirror the asserts of the Vx
 * functions in stdlib/std/nn.vx (nn_check_matrix, nn_check_heads,
 * nn_check_cache): a refused shape stops the program with the function's name.
 */
#include "kernels.h"
#include "vx_b200.h"
#include "vx_collective.h"
#include "vx_hardware_runtime.h"

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace vxb {
cudaStream_t caller_stream();
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

thread_local std::string t_error;
int32_t fail(const char *why) {
  t_error = why ? why : "unknown";
  return -1;
}
int32_t done(const char *why, const char *kernel) {
  if (why)
    return fail(why);
  vxb::note_kernel(kernel);
  return 0;
}
void must(const char *why, const char *fn) {
  if (why)
    stop("%s: %s", fn, why);
  vxb::note_kernel(fn);
}

/* A packed tensor's data pointer; a gap between rows is refused as a `pub fn`
   refuses it (docs/lang/abi.md section 3.6, "Packed tensors"). */
template <typename T>
T *packed(const char *fn, const char *name, void *aligned, int64_t offset,
          int rank, const int64_t *sizes, const int64_t *strides) {
  int64_t expect = 1;
  bool empty = false;
  for (int d = 0; d < rank; ++d)
    empty |= sizes[d] == 0;
  for (int d = rank - 1; d >= 0 && !empty; --d) {
    if (sizes[d] != 1 && strides[d] != expect)
      stop("%s: the tensor `%s` has a gap: stride %lld of axis %d, where a "
           "packed tensor has %lld",
           fn, name, (long long)strides[d], d, (long long)expect);
    expect *= sizes[d];
  }
  return (T *)aligned + offset;
}
#define T1(T, t)                                                               \
  packed<T>(FN, #t, t##_aligned, t##_offset, 1, &t##_n0, &t##_s0)
#define T2(T, t)                                                               \
  [&] {                                                                        \
    const int64_t n_[2] = {t##_n0, t##_n1}, s_[2] = {t##_s0, t##_s1};          \
    return packed<T>(FN, #t, t##_aligned, t##_offset, 2, n_, s_);              \
  }()
#define T3(T, t)                                                               \
  [&] {                                                                        \
    const int64_t n_[3] = {t##_n0, t##_n1, t##_n2},                            \
                  s_[3] = {t##_s0, t##_s1, t##_s2};                            \
    return packed<T>(FN, #t, t##_aligned, t##_offset, 3, n_, s_);              \
  }()
#define T4(T, t)                                                               \
  [&] {                                                                        \
    const int64_t n_[4] = {t##_n0, t##_n1, t##_n2, t##_n3},                    \
                  s_[4] = {t##_s0, t##_s1, t##_s2, t##_s3};                    \
    return packed<T>(FN, #t, t##_aligned, t##_offset, 4, n_, s_);              \
  }()
#define UNUSED_ALLOC(t) (void)t##_allocated

/* nn_check_matrix: y has rows values, w rows*cols, x cols; cols % 8 == 0. */
void check_matrix(const char *fn, int64_t y_len, int64_t w_len, int64_t x_len,
                  int rows, int cols) {
  if (rows <= 0 || cols <= 0 || cols % 8 != 0)
    stop("%s: rows and cols must be positive, and cols a multiple of 8", fn);
  if (y_len < rows || w_len < (int64_t)rows * cols || x_len < cols)
    stop("%s: a tensor is smaller than rows and cols say", fn);
}
void check_heads(const char *fn, int64_t e0, int64_t e1, int heads, int hd) {
  if (heads <= 0 || hd <= 0 || hd % 8 != 0 || hd > 128 || e0 < heads || e1 != hd)
    stop("%s: a tensor of heads must be [heads, head_dim], with head_dim a "
         "multiple of 8 and at most 128",
         fn);
}
void check_cache(const char *fn, int64_t e0, int64_t e1, int64_t e2, int pos,
                 int kv_heads, int hd) {
  if (pos < 0 || pos >= e0 || e1 != kv_heads || e2 != hd)
    stop("%s: the KV cache must be [max_seq, kv_heads, head_dim] with a row "
         "for `pos`",
         fn);
}

/* Zeroed counters for the attention kernel's "last block merges" step, one
   buffer per GPU, kept for the life of the process. */
int32_t *attention_counters() {
  static std::mutex mu;
  static std::map<int, int32_t *> per_device;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  int32_t *&p = per_device[dev];
  if (!p) {
    if (cudaMalloc(&p, 16384 * sizeof(int32_t)) != cudaSuccess ||
        cudaMemset(p, 0, 16384 * sizeof(int32_t)) != cudaSuccess)
      stop("out of device memory for the attention counters");
  }
  return p;
}

int32_t *device_i32(int value) {
  /* A position that a kernel reads from device memory. One slot per GPU and
     value would be wasteful; positions up to 64 Ki are made once per GPU. */
  static std::mutex mu;
  static std::map<int, int32_t *> per_device;
  constexpr int kMost = 1 << 16;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  int32_t *&p = per_device[dev];
  if (!p) {
    std::vector<int32_t> iota(kMost);
    for (int i = 0; i < kMost; ++i)
      iota[i] = i;
    if (cudaMalloc(&p, kMost * sizeof(int32_t)) != cudaSuccess ||
        cudaMemcpy(p, iota.data(), kMost * sizeof(int32_t),
                   cudaMemcpyHostToDevice) != cudaSuccess)
      stop("out of device memory for the position table");
  }
  if (value < 0 || value >= kMost)
    stop("a position of %d is outside 0..65535", value);
  return p + value;
}

} // namespace

namespace vxb {
void set_last_error(const char *why) { t_error = why ? why : "unknown"; }
} // namespace vxb

extern "C" {

const char *vx_b200_last_error(void) { return t_error.c_str(); }

/* ------------------------------------------------------------------ std::nn */
#define FN "nn_matvec"
void vx_nn_matvec(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(x), int32_t rows,
                  int32_t cols) {
  UNUSED_ALLOC(y); UNUSED_ALLOC(w); UNUSED_ALLOC(x);
  check_matrix(FN, y_n0, w_n0, x_n0, rows, cols);
  vxb::MatvecArgs a{};
  a.w = T1(uint16_t, w);
  a.wbf16 = true;
  a.rows = rows;
  a.cols = cols;
  a.x = T1(float, x);
  a.x_stride = cols;
  a.y = T1(float, y);
  a.y_stride = rows;
  a.batch = 1;
  a.mode = 0;
  must(vxb::matvec(a, vxb::caller_stream()), FN);
}
#undef FN

#define FN "nn_matvec_add"
void vx_nn_matvec_add(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(x), int32_t rows,
                      int32_t cols) {
  UNUSED_ALLOC(y); UNUSED_ALLOC(w); UNUSED_ALLOC(x);
  check_matrix(FN, y_n0, w_n0, x_n0, rows, cols);
  vxb::MatvecArgs a{};
  a.w = T1(uint16_t, w);
  a.wbf16 = true;
  a.rows = rows;
  a.cols = cols;
  a.x = T1(float, x);
  a.x_stride = cols;
  a.y = T1(float, y);
  a.y_stride = rows;
  a.batch = 1;
  a.mode = 1;
  must(vxb::matvec(a, vxb::caller_stream()), FN);
}
#undef FN

#define FN "nn_matvec_heads_add"
void vx_nn_matvec_heads_add(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR2(x),
                            int32_t rows, int32_t heads, int32_t head_dim) {
  UNUSED_ALLOC(y); UNUSED_ALLOC(w); UNUSED_ALLOC(x);
  const int cols = heads * head_dim;
  check_heads(FN, x_n0, x_n1, heads, head_dim);
  check_matrix(FN, y_n0, w_n0, cols, rows, cols);
  vxb::MatvecArgs a{};
  a.w = T1(uint16_t, w);
  a.wbf16 = true;
  a.rows = rows;
  a.cols = cols;
  a.x = T2(float, x); /* packed [heads, head_dim] is the flat vector */
  a.x_stride = cols;
  a.y = T1(float, y);
  a.y_stride = rows;
  a.batch = 1;
  a.mode = 1;
  must(vxb::matvec(a, vxb::caller_stream()), FN);
}
#undef FN

#define FN "nn_qkv"
void vx_nn_qkv(VX_TENSOR2(q), VX_TENSOR2(k), VX_TENSOR2(v), VX_TENSOR1(w),
               VX_TENSOR1(b), VX_TENSOR1(x), int32_t q_heads, int32_t kv_heads,
               int32_t head_dim, int32_t cols) {
  UNUSED_ALLOC(q); UNUSED_ALLOC(k); UNUSED_ALLOC(v);
  UNUSED_ALLOC(w); UNUSED_ALLOC(b); UNUSED_ALLOC(x);
  const int heads = q_heads + 2 * kv_heads;
  check_heads(FN, q_n0, q_n1, q_heads, head_dim);
  check_heads(FN, k_n0, k_n1, kv_heads, head_dim);
  check_heads(FN, v_n0, v_n1, kv_heads, head_dim);
  check_matrix(FN, b_n0, w_n0, x_n0, heads * head_dim, cols);
  /* Three row ranges of one matrix, each with its slice of the bias. */
  const uint16_t *wp = T1(uint16_t, w), *bp = T1(uint16_t, b);
  const float *xp = T1(float, x);
  float *outs[3] = {T2(float, q), T2(float, k), T2(float, v)};
  const int counts[3] = {q_heads, kv_heads, kv_heads};
  int64_t row = 0;
  for (int part = 0; part < 3; ++part) {
    vxb::MatvecArgs a{};
    a.w = wp + row * cols;
    a.wbf16 = true;
    a.rows = counts[part] * head_dim;
    a.cols = cols;
    a.x = xp;
    a.x_stride = cols;
    a.y = outs[part];
    a.y_stride = a.rows;
    a.batch = 1;
    a.mode = 2;
    a.bias = bp + row;
    must(vxb::matvec(a, vxb::caller_stream()), FN);
    row += a.rows;
  }
}
#undef FN

#define FN "nn_swiglu"
void vx_nn_swiglu(VX_TENSOR1(out), VX_TENSOR1(w), VX_TENSOR1(x), int32_t rows,
                  int32_t cols) {
  UNUSED_ALLOC(out); UNUSED_ALLOC(w); UNUSED_ALLOC(x);
  check_matrix(FN, out_n0, w_n0 / 2, x_n0, rows, cols);
  vxb::SwigluArgs a{};
  a.w = T1(uint16_t, w);
  a.wbf16 = true;
  a.rows = rows;
  a.cols = cols;
  a.x = T1(float, x);
  a.x_stride = cols;
  a.out = T1(float, out);
  a.out_stride = rows;
  a.batch = 1;
  must(vxb::swiglu(a, vxb::caller_stream()), FN);
}
#undef FN

#define FN "nn_rms_norm"
void vx_nn_rms_norm(VX_TENSOR1(y), VX_TENSOR1(x), VX_TENSOR1(w), int32_t n,
                    float eps) {
  UNUSED_ALLOC(y); UNUSED_ALLOC(x); UNUSED_ALLOC(w);
  if (n <= 0 || y_n0 < n || x_n0 < n || w_n0 < n)
    stop("nn_rms_norm: a tensor has fewer than n values");
  must(vxb::rms_norm(T1(float, y), T1(float, x), T1(uint16_t, w), true, n, eps,
                     1, n, vxb::caller_stream()),
       FN);
}
#undef FN

#define FN "nn_rope_and_store"
void vx_nn_rope_and_store(VX_TENSOR2(q_out), VX_TENSOR3(k_cache),
                          VX_TENSOR3(v_cache), VX_TENSOR2(q), VX_TENSOR2(k),
                          VX_TENSOR2(v), VX_TENSOR2(cos), VX_TENSOR2(sin),
                          int32_t pos, int32_t q_heads, int32_t kv_heads,
                          int32_t head_dim) {
  UNUSED_ALLOC(q_out); UNUSED_ALLOC(k_cache); UNUSED_ALLOC(v_cache);
  UNUSED_ALLOC(q); UNUSED_ALLOC(k); UNUSED_ALLOC(v);
  UNUSED_ALLOC(cos); UNUSED_ALLOC(sin);
  const int half = head_dim / 2;
  check_heads(FN, q_n0, q_n1, q_heads, head_dim);
  check_heads(FN, q_out_n0, q_out_n1, q_heads, head_dim);
  check_heads(FN, k_n0, k_n1, kv_heads, head_dim);
  check_heads(FN, v_n0, v_n1, kv_heads, head_dim);
  check_cache(FN, k_cache_n0, k_cache_n1, k_cache_n2, pos, kv_heads, head_dim);
  check_cache(FN, v_cache_n0, v_cache_n1, v_cache_n2, pos, kv_heads, head_dim);
  if (pos >= cos_n0 || pos >= sin_n0 || half > cos_n1 || half > sin_n1 ||
      cos_n1 != sin_n1)
    stop("nn_rope_and_store: `cos` and `sin` need a row for `pos` with "
         "head_dim / 2 values");
  must(vxb::rope_and_store(T2(float, q_out), T3(float, k_cache),
                           T3(float, v_cache), T2(float, q), T2(float, k),
                           T2(float, v), T2(float, cos), T2(float, sin),
                           (int)cos_n1, pos, q_heads, kv_heads, head_dim,
                           vxb::caller_stream()),
       FN);
}
#undef FN

#define FN "nn_attention"
void vx_nn_attention(VX_TENSOR2(out), VX_TENSOR4(part), VX_TENSOR2(q),
                     VX_TENSOR3(k_cache), VX_TENSOR3(v_cache), int32_t pos,
                     int32_t q_heads, int32_t kv_heads, int32_t head_dim) {
  UNUSED_ALLOC(out); UNUSED_ALLOC(part); UNUSED_ALLOC(q);
  UNUSED_ALLOC(k_cache); UNUSED_ALLOC(v_cache);
  check_heads(FN, q_n0, q_n1, q_heads, head_dim);
  check_heads(FN, out_n0, out_n1, q_heads, head_dim);
  check_cache(FN, k_cache_n0, k_cache_n1, k_cache_n2, pos, kv_heads, head_dim);
  check_cache(FN, v_cache_n0, v_cache_n1, v_cache_n2, pos, kv_heads, head_dim);
  if (kv_heads <= 0 || q_heads % kv_heads != 0)
    stop("nn_attention: q_heads must be a multiple of kv_heads");
  if (head_dim % 32 != 0 || head_dim > 128)
    stop("nn_attention: head_dim must be a multiple of 32, and at most 128");
  /* The reference splits the positions 32 to a block below 640 and 64 from
     there on, and sizes `part` for that (nn.vx:356-361); the same split keeps
     this kernel inside the same scratch. */
  const int n_pos = pos >= 640 ? 64 : 32;
  const int group = q_heads / kv_heads;
  if (part_n0 < (int64_t)kv_heads * ((group + 7) / 8) ||
      part_n1 < (pos + n_pos) / n_pos || part_n2 < 8 || part_n3 < head_dim + 2)
    stop("nn_attention: `part` is too small for this position. Make it with "
         "nn_attention_scratch");
  vxb::AttnArgs a{};
  a.q = T2(float, q);
  a.k_cache = T3(float, k_cache);
  a.v_cache = T3(float, v_cache);
  a.cache_batch_stride = 0;
  a.out = T2(float, out);
  a.q_heads = q_heads;
  a.kv_heads = kv_heads;
  a.head_dim = head_dim;
  a.batch = 1;
  a.positions = device_i32(pos);
  a.max_pos = pos;
  a.scratch = T4(float, part);
  a.counters = attention_counters();
  a.split = n_pos;
  must(vxb::attention_decode(a, vxb::caller_stream()), FN);
}
#undef FN

#define FN "nn_argmax"
void vx_nn_argmax(VX_TENSOR1(out), VX_TENSOR1(logits), int32_t n) {
  UNUSED_ALLOC(out); UNUSED_ALLOC(logits);
  if (n <= 0 || logits_n0 < n || out_n0 < 1)
    stop("nn_argmax: `logits` has fewer than n values, or `out` is empty");
  must(vxb::argmax(T1(int32_t, out), T1(float, logits), n, 1, n,
                   vxb::caller_stream()),
       FN);
}
#undef FN

#define FN "nn_embed"
void vx_nn_embed(VX_TENSOR1(x), VX_TENSOR1(table), VX_TENSOR1(token),
                 int32_t dim) {
  UNUSED_ALLOC(x); UNUSED_ALLOC(table); UNUSED_ALLOC(token);
  if (dim <= 0 || x_n0 < dim || token_n0 < 1)
    stop("nn_embed: `x` has fewer than dim values, or `token` is empty");
  must(vxb::embed(T1(float, x), T1(uint16_t, table), true, T1(int32_t, token),
                  dim, (int)(table_n0 / dim), 1, dim, vxb::caller_stream()),
       FN);
}
#undef FN

} /* extern "C" */

/* ------------------------------------------------ fp8 and Q4_0 projections
 * (nn.vx:1296-1640 and 1645-2100). One body for both formats: `quant` is
 * kFmtFp8 (codes 4 to a u32 word, f32 scales per 128 x 128 block) or kFmtQ4
 * (codes 8 to a word, an f16 scale per 32 weights of a row). The checks are
 * nn_check_fp8 and nn_check_q4 (nn.vx:2267-2284). */
namespace {
void check_quant(const char *fn, int quant, int64_t w_len, int64_t s_len,
                 int64_t x_len, int rows, int cols) {
  if (quant == vxb::kFmtFp8) {
    if (rows <= 0 || rows % 4 != 0 || cols <= 0 || cols % 128 != 0)
      stop("%s: rows must be a multiple of 4, and cols a multiple of 128", fn);
    if (x_len < cols)
      stop("%s: the input has fewer values than cols", fn);
    if (rows > w_len / (cols / 4) ||
        s_len < (int64_t)((rows + 127) / 128) * (cols / 128))
      stop("%s: the codes or the scales are too few for rows x cols", fn);
  } else {
    if (rows <= 0 || rows % 4 != 0 || cols <= 0 || cols % 32 != 0)
      stop("%s: rows must be a multiple of 4, and cols a multiple of 32", fn);
    if (x_len < cols)
      stop("%s: the input has fewer values than cols", fn);
    if (rows > w_len / (cols / 8) || rows > s_len / (cols / 32))
      stop("%s: the codes or the scales are too few for rows x cols", fn);
  }
}
void quant_matvec(const char *fn, int quant, float *y, int64_t y_len,
                  const void *w, int64_t w_len, const void *scales,
                  int64_t s_len, const float *x, int64_t x_len, int rows,
                  int cols, int mode) {
  check_quant(fn, quant, w_len, s_len, x_len, rows, cols);
  if (y_len < rows)
    stop("%s: the output has fewer values than rows", fn);
  vxb::MatvecArgs a{};
  a.w = w;
  a.wfmt = quant;
  a.scales = scales;
  a.rows = rows;
  a.cols = cols;
  a.x = x;
  a.x_stride = cols;
  a.y = y;
  a.y_stride = rows;
  a.batch = 1;
  a.mode = mode;
  must(vxb::matvec(a, vxb::caller_stream()), fn);
}
void quant_qkv(const char *fn, int quant, float *q, float *k, float *v,
               const void *w, int64_t w_len, const void *scales, int64_t s_len,
               const uint16_t *bias, int64_t b_len, const float *x,
               int64_t x_len, int q_heads, int kv_heads, int head_dim, int cols) {
  const int rows_all = (q_heads + 2 * kv_heads) * head_dim;
  check_quant(fn, quant, w_len, s_len, x_len, rows_all, cols);
  if (b_len < rows_all)
    stop("%s: the bias has fewer values than rows", fn);
  float *outs[3] = {q, k, v};
  const int counts[3] = {q_heads, kv_heads, kv_heads};
  const int64_t row_bytes = quant == vxb::kFmtFp8 ? cols : cols / 2;
  int row = 0;
  for (int part = 0; part < 3; ++part) {
    vxb::MatvecArgs a{};
    a.w = (const char *)w + row * row_bytes;
    a.wfmt = quant;
    a.scales = scales; /* of the whole matrix: row_base says where we are */
    a.row_base = row;
    a.rows = counts[part] * head_dim;
    a.cols = cols;
    a.x = x;
    a.x_stride = cols;
    a.y = outs[part];
    a.y_stride = a.rows;
    a.batch = 1;
    a.mode = 2;
    a.bias = bias + row;
    must(vxb::matvec(a, vxb::caller_stream()), fn);
    row += a.rows;
  }
}
void quant_swiglu(const char *fn, int quant, float *out, int64_t out_len,
                  const void *w, int64_t w_len, const void *scales,
                  int64_t s_len, const float *x, int64_t x_len, int rows,
                  int cols) {
  check_quant(fn, quant, w_len, s_len, x_len, 2 * rows, cols);
  if (out_len < rows)
    stop("%s: the output has fewer values than rows", fn);
  vxb::SwigluArgs a{};
  a.w = w;
  a.wfmt = quant;
  a.scales = scales;
  a.rows = rows;
  a.cols = cols;
  a.x = x;
  a.x_stride = cols;
  a.out = out;
  a.out_stride = rows;
  a.batch = 1;
  must(vxb::swiglu(a, vxb::caller_stream()), fn);
}
} // namespace

#define QUANT_EXPORTS(SUFFIX, QUANT, SCALE_T, TAG)                             \
  void vx_nn_matvec_##SUFFIX(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(scales), \
                             VX_TENSOR1(x), int32_t rows, int32_t cols) {      \
    static const char FN[] = "nn_matvec_" TAG;                                 \
    UNUSED_ALLOC(y); UNUSED_ALLOC(w); UNUSED_ALLOC(scales); UNUSED_ALLOC(x);   \
    quant_matvec(FN, QUANT, T1(float, y), y_n0, T1(uint32_t, w), w_n0,         \
                 T1(SCALE_T, scales), scales_n0, T1(float, x), x_n0, rows,     \
                 cols, 0);                                                     \
  }                                                                            \
  void vx_nn_matvec_##SUFFIX##_add(VX_TENSOR1(y), VX_TENSOR1(w),               \
                                   VX_TENSOR1(scales), VX_TENSOR1(x),          \
                                   int32_t rows, int32_t cols) {               \
    static const char FN[] = "nn_matvec_" TAG "_add";                          \
    UNUSED_ALLOC(y); UNUSED_ALLOC(w); UNUSED_ALLOC(scales); UNUSED_ALLOC(x);   \
    quant_matvec(FN, QUANT, T1(float, y), y_n0, T1(uint32_t, w), w_n0,         \
                 T1(SCALE_T, scales), scales_n0, T1(float, x), x_n0, rows,     \
                 cols, 1);                                                     \
  }                                                                            \
  void vx_nn_matvec_##SUFFIX##_heads_add(                                      \
      VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(scales), VX_TENSOR2(x),         \
      int32_t rows, int32_t heads, int32_t head_dim) {                         \
    static const char FN[] = "nn_matvec_" TAG "_heads_add";                    \
    UNUSED_ALLOC(y); UNUSED_ALLOC(w); UNUSED_ALLOC(scales); UNUSED_ALLOC(x);   \
    check_heads(FN, x_n0, x_n1, heads, head_dim);                              \
    quant_matvec(FN, QUANT, T1(float, y), y_n0, T1(uint32_t, w), w_n0,         \
                 T1(SCALE_T, scales), scales_n0, T2(float, x),                 \
                 (int64_t)heads * head_dim, rows, heads * head_dim, 1);        \
  }                                                                            \
  void vx_nn_qkv_##SUFFIX(VX_TENSOR2(q), VX_TENSOR2(k), VX_TENSOR2(v),         \
                          VX_TENSOR1(w), VX_TENSOR1(scales), VX_TENSOR1(b),    \
                          VX_TENSOR1(x), int32_t q_heads, int32_t kv_heads,    \
                          int32_t head_dim, int32_t cols) {                    \
    static const char FN[] = "nn_qkv_" TAG;                                    \
    UNUSED_ALLOC(q); UNUSED_ALLOC(k); UNUSED_ALLOC(v); UNUSED_ALLOC(w);        \
    UNUSED_ALLOC(scales); UNUSED_ALLOC(b); UNUSED_ALLOC(x);                    \
    check_heads(FN, q_n0, q_n1, q_heads, head_dim);                            \
    check_heads(FN, k_n0, k_n1, kv_heads, head_dim);                           \
    check_heads(FN, v_n0, v_n1, kv_heads, head_dim);                           \
    quant_qkv(FN, QUANT, T2(float, q), T2(float, k), T2(float, v),             \
              T1(uint32_t, w), w_n0, T1(SCALE_T, scales), scales_n0,           \
              T1(uint16_t, b), b_n0, T1(float, x), x_n0, q_heads, kv_heads,    \
              head_dim, cols);                                                 \
  }                                                                            \
  void vx_nn_swiglu_##SUFFIX(VX_TENSOR1(out), VX_TENSOR1(w),                   \
                             VX_TENSOR1(scales), VX_TENSOR1(x), int32_t rows,  \
                             int32_t cols) {                                   \
    static const char FN[] = "nn_swiglu_" TAG;                                 \
    UNUSED_ALLOC(out); UNUSED_ALLOC(w); UNUSED_ALLOC(scales); UNUSED_ALLOC(x); \
    quant_swiglu(FN, QUANT, T1(float, out), out_n0, T1(uint32_t, w), w_n0,     \
                 T1(SCALE_T, scales), scales_n0, T1(float, x), x_n0, rows,     \
                 cols);                                                        \
  }

extern "C" {
QUANT_EXPORTS(fp8, vxb::kFmtFp8, float, "fp8")
QUANT_EXPORTS(q4, vxb::kFmtQ4, uint16_t, "q4")
}
#undef QUANT_EXPORTS


/* ------------------------------------------------ a mixture-of-experts layer
 * nn_top_k nn.vx:904, nn_moe_swiglu :968, nn_moe_down_add :1019 (bf16), and
 * nn_moe_swiglu_q4 :2105, nn_moe_down_q4_add :2190. The experts' matrices sit
 * one after another in `w`; `ids` (device memory, from nn_top_k) names the k
 * that a token uses. One projection launch per expert slot; the down
 * projection adds the experts to y in slot order. */
namespace {
void moe_swiglu(const char *fn, int quant, float *out, int64_t out_rows,
                int64_t out_pitch, const void *w, int64_t w_len,
                const void *scales, const int32_t *ids, int64_t ids_len,
                const float *x, int64_t x_len, int k, int rows, int cols,
                int experts) {
  const int per = quant ? 32 : 8;
  if (k <= 0 || ids_len < k || out_rows < k || out_pitch < rows)
    stop("%s: `ids` needs k values, and `out` a row of rows values for each", fn);
  if (cols % per != 0 || x_len < cols || rows <= 0 || experts <= 0 ||
      (quant ? w_len / (cols / 8) : w_len / cols) / 2 / rows < experts)
    stop("%s: `w` needs 2 * rows rows of cols values for each expert", fn);
  for (int e = 0; e < k; ++e) {
    vxb::SwigluArgs a{};
    a.w = w;
    a.wbf16 = true;
    a.wfmt = quant;
    a.scales = scales;
    a.rows = rows;
    a.cols = cols;
    a.x = x;
    a.x_stride = cols;
    a.out = out + (int64_t)e * out_pitch;
    a.out_stride = out_pitch;
    a.batch = 1;
    a.expert_ids = ids;
    a.expert_slot = e;
    a.experts = experts;
    must(vxb::swiglu(a, vxb::caller_stream()), fn);
  }
}
void moe_down_add(const char *fn, int quant, float *y, int64_t y_len,
                  const void *w, int64_t w_len, const void *scales,
                  const int32_t *ids, int64_t ids_len, const float *weights,
                  int64_t weights_len, const float *h, int64_t h_rows,
                  int64_t h_pitch, int k, int rows, int cols, int experts) {
  const int per = quant ? 32 : 8;
  if (k <= 0 || ids_len < k || weights_len < k || h_rows < k || h_pitch < cols)
    stop("%s: `ids` and `weights` need k values, and `h` a row of cols values for "
         "each", fn);
  if (cols % per != 0 || y_len < rows || rows <= 0 || experts <= 0 ||
      (quant ? w_len / (cols / 8) : w_len / cols) / rows < experts)
    stop("%s: `w` needs rows rows of cols values for each expert", fn);
  for (int e = 0; e < k; ++e) {
    vxb::MatvecArgs a{};
    a.w = w;
    a.wbf16 = true;
    a.wfmt = quant;
    a.scales = scales;
    a.rows = rows;
    a.cols = cols;
    a.x = h + (int64_t)e * h_pitch;
    a.x_stride = h_pitch;
    a.y = y;
    a.y_stride = rows;
    a.batch = 1;
    a.mode = 1;
    a.expert_ids = ids;
    a.expert_slot = e;
    a.experts = experts;
    a.add_scale = weights + e;
    must(vxb::matvec(a, vxb::caller_stream()), fn);
  }
}
} // namespace

extern "C" {

#define FN "nn_top_k"
void vx_nn_top_k(VX_TENSOR1(ids), VX_TENSOR1(weights), VX_TENSOR1(logits), int32_t n,
                 int32_t k) {
  UNUSED_ALLOC(ids); UNUSED_ALLOC(weights); UNUSED_ALLOC(logits);
  if (n <= 0 || n > 256 || k <= 0 || k > n)
    stop("nn_top_k: n must be 1 to 256, and k must be 1 to n");
  if (logits_n0 < n || ids_n0 < k || weights_n0 < k)
    stop("nn_top_k: a tensor has too few values");
  must(vxb::top_k(T1(int32_t, ids), T1(float, weights), T1(float, logits), n, k,
                  vxb::caller_stream()),
       FN);
}
#undef FN

#define FN "nn_moe_swiglu"
void vx_nn_moe_swiglu(VX_TENSOR2(out), VX_TENSOR1(w), VX_TENSOR1(ids), VX_TENSOR1(x),
                      int32_t k, int32_t rows, int32_t cols, int32_t experts) {
  UNUSED_ALLOC(out); UNUSED_ALLOC(w); UNUSED_ALLOC(ids); UNUSED_ALLOC(x);
  moe_swiglu(FN, 0, T2(float, out), out_n0, out_n1, T1(uint16_t, w), w_n0, nullptr,
             T1(int32_t, ids), ids_n0, T1(float, x), x_n0, k, rows, cols, experts);
}
#undef FN

#define FN "nn_moe_down_add"
void vx_nn_moe_down_add(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(ids),
                        VX_TENSOR1(weights), VX_TENSOR2(h), int32_t k, int32_t rows,
                        int32_t cols, int32_t experts) {
  UNUSED_ALLOC(y); UNUSED_ALLOC(w); UNUSED_ALLOC(ids); UNUSED_ALLOC(weights);
  UNUSED_ALLOC(h);
  moe_down_add(FN, 0, T1(float, y), y_n0, T1(uint16_t, w), w_n0, nullptr,
               T1(int32_t, ids), ids_n0, T1(float, weights), weights_n0,
               T2(float, h), h_n0, h_n1, k, rows, cols, experts);
}
#undef FN

#define FN "nn_moe_swiglu_q4"
void vx_nn_moe_swiglu_q4(VX_TENSOR2(out), VX_TENSOR1(w), VX_TENSOR1(scales),
                         VX_TENSOR1(ids), VX_TENSOR1(x), int32_t k, int32_t rows,
                         int32_t cols, int32_t experts) {
  UNUSED_ALLOC(out); UNUSED_ALLOC(w); UNUSED_ALLOC(scales); UNUSED_ALLOC(ids);
  UNUSED_ALLOC(x);
  if (scales_n0 < (int64_t)experts * 2 * rows * (cols / 32))
    stop("nn_moe_swiglu_q4: the scales are too few for the experts");
  moe_swiglu(FN, vxb::kFmtQ4, T2(float, out), out_n0, out_n1, T1(uint32_t, w), w_n0,
             T1(uint16_t, scales), T1(int32_t, ids), ids_n0, T1(float, x), x_n0, k,
             rows, cols, experts);
}
#undef FN

#define FN "nn_moe_down_q4_add"
void vx_nn_moe_down_q4_add(VX_TENSOR1(y), VX_TENSOR1(w), VX_TENSOR1(scales),
                           VX_TENSOR1(ids), VX_TENSOR1(weights), VX_TENSOR2(h),
                           int32_t k, int32_t rows, int32_t cols, int32_t experts) {
  UNUSED_ALLOC(y); UNUSED_ALLOC(w); UNUSED_ALLOC(scales); UNUSED_ALLOC(ids);
  UNUSED_ALLOC(weights); UNUSED_ALLOC(h);
  if (scales_n0 < (int64_t)experts * rows * (cols / 32))
    stop("nn_moe_down_q4_add: the scales are too few for the experts");
  moe_down_add(FN, vxb::kFmtQ4, T1(float, y), y_n0, T1(uint32_t, w), w_n0,
               T1(uint16_t, scales), T1(int32_t, ids), ids_n0, T1(float, weights),
               weights_n0, T2(float, h), h_n0, h_n1, k, rows, cols, experts);
}
#undef FN

} /* extern "C" */

/* ---------------------------------------------- kernels for n positions
 * (nn.vx:2312-2950: "the kernel of the same name without _rows ... for each
 * position ... row t of the output is bit-identical to the one-position kernel
 * on x[t]"). The projections take the positions 16, 8, 4, 2 or 1 at a time
 * through the one-position kernel's own code (every sequence of a launch is
 * summed in the order a single one is), so that property holds here too. */
namespace {
template <typename F> void in_chunks(int n, F &&run) {
  int t = 0;
  for (int chunk = 16; chunk >= 1; chunk /= 2)
    while (n - t >= chunk) {
      run(t, chunk);
      t += chunk;
    }
}
void check_rows(const char *fn, int n, int64_t x_rows, int64_t y_rows) {
  if (n <= 0 || x_rows < n || y_rows < n)
    stop("%s: the input and the output need n rows", fn);
}
} // namespace

extern "C" {

#define FN "nn_matvec_rows"
void vx_nn_matvec_rows(VX_TENSOR2(y), VX_TENSOR1(w), VX_TENSOR2(x), int32_t n,
                       int32_t rows, int32_t cols) {
  UNUSED_ALLOC(y); UNUSED_ALLOC(w); UNUSED_ALLOC(x);
  check_matrix(FN, y_n1, w_n0, x_n1, rows, cols);
  check_rows(FN, n, x_n0, y_n0);
  float *yp = T2(float, y);
  const float *xp = T2(float, x);
  const uint16_t *wp = T1(uint16_t, w);
  in_chunks(n, [&](int t, int chunk) {
    vxb::MatvecArgs a{};
    a.w = wp;
    a.wbf16 = true;
    a.rows = rows;
    a.cols = cols;
    a.x = xp + (int64_t)t * x_n1;
    a.x_stride = x_n1;
    a.y = yp + (int64_t)t * y_n1;
    a.y_stride = y_n1;
    a.batch = chunk;
    a.mode = 0;
    must(vxb::matvec(a, vxb::caller_stream()), FN);
  });
}
#undef FN

#define FN "nn_matvec_q4_rows"
void vx_nn_matvec_q4_rows(VX_TENSOR2(y), VX_TENSOR1(w), VX_TENSOR1(scales),
                          VX_TENSOR2(x), int32_t n, int32_t rows, int32_t cols) {
  UNUSED_ALLOC(y); UNUSED_ALLOC(w); UNUSED_ALLOC(scales); UNUSED_ALLOC(x);
  check_rows(FN, n, x_n0, y_n0);
  float *yp = T2(float, y);
  const float *xp = T2(float, x);
  for (int t = 0; t < n; ++t)
    quant_matvec(FN, vxb::kFmtQ4, yp + (int64_t)t * y_n1, y_n1, T1(uint32_t, w),
                 w_n0, T1(uint16_t, scales), scales_n0, xp + (int64_t)t * x_n1,
                 x_n1, rows, cols, 0);
}
#undef FN

#define FN "nn_rms_norm_rows"
void vx_nn_rms_norm_rows(VX_TENSOR2(y), VX_TENSOR2(x), VX_TENSOR1(w), int32_t n,
                         int32_t dim, float eps) {
  UNUSED_ALLOC(y); UNUSED_ALLOC(x); UNUSED_ALLOC(w);
  if (dim <= 0 || y_n1 < dim || x_n1 < dim || w_n0 < dim)
    stop("nn_rms_norm_rows: a row has fewer than dim values");
  check_rows(FN, n, x_n0, y_n0);
  float *yp = T2(float, y);
  const float *xp = T2(float, x);
  if (y_n1 == x_n1) {
    must(vxb::rms_norm(yp, xp, T1(uint16_t, w), true, dim, eps, n, x_n1,
                       vxb::caller_stream()),
         FN);
    return;
  }
  for (int t = 0; t < n; ++t)
    must(vxb::rms_norm(yp + (int64_t)t * y_n1, xp + (int64_t)t * x_n1,
                       T1(uint16_t, w), true, dim, eps, 1, dim,
                       vxb::caller_stream()),
         FN);
}
#undef FN

#define FN "nn_argmax_rows"
void vx_nn_argmax_rows(VX_TENSOR1(out), VX_TENSOR2(logits), int32_t n,
                       int32_t count) {
  UNUSED_ALLOC(out); UNUSED_ALLOC(logits);
  if (count <= 0 || logits_n1 < count)
    stop("nn_argmax_rows: a row of `logits` has fewer than count values");
  if (n <= 0 || logits_n0 < n || out_n0 < n)
    stop("nn_argmax_rows: `logits` needs n rows, and `out` n values");
  must(vxb::argmax(T1(int32_t, out), T2(float, logits), count, n, logits_n1,
                   vxb::caller_stream()),
       FN);
}
#undef FN

#define FN "nn_embed_rows"
void vx_nn_embed_rows(VX_TENSOR2(x), VX_TENSOR1(table), VX_TENSOR1(tokens),
                      int32_t n, int32_t dim) {
  UNUSED_ALLOC(x); UNUSED_ALLOC(table); UNUSED_ALLOC(tokens);
  if (dim <= 0 || x_n1 < dim || n <= 0 || x_n0 < n || tokens_n0 < n)
    stop("nn_embed_rows: `x` needs n rows of dim values, and `tokens` n values");
  must(vxb::embed(T2(float, x), T1(uint16_t, table), true, T1(int32_t, tokens),
                  dim, (int)(table_n0 / dim), n, x_n1, vxb::caller_stream()),
       FN);
}
#undef FN

#define FN "nn_top_k_rows"
void vx_nn_top_k_rows(VX_TENSOR2(ids), VX_TENSOR2(weights), VX_TENSOR2(logits),
                      int32_t n, int32_t count, int32_t k) {
  UNUSED_ALLOC(ids); UNUSED_ALLOC(weights); UNUSED_ALLOC(logits);
  if (count <= 0 || count > 256 || k <= 0 || k > count)
    stop("nn_top_k_rows: count must be 1 to 256, and k must be 1 to count");
  if (logits_n1 < count || ids_n1 < k || weights_n1 < k)
    stop("nn_top_k_rows: a row has too few values");
  if (n <= 0 || logits_n0 < n || ids_n0 < n || weights_n0 < n)
    stop("nn rows: each tensor needs n rows");
  must(vxb::top_k_rows(T2(int32_t, ids), T2(float, weights), T2(float, logits), n,
                       count, k, ids_n1, weights_n1, logits_n1,
                       vxb::caller_stream()),
       FN);
}
#undef FN

#define FN "nn_matvec_q4_heads_add_rows"
void vx_nn_matvec_q4_heads_add_rows(VX_TENSOR2(y), VX_TENSOR1(w), VX_TENSOR1(scales),
                                    VX_TENSOR3(x), int32_t n, int32_t rows,
                                    int32_t heads, int32_t head_dim) {
  UNUSED_ALLOC(y); UNUSED_ALLOC(w); UNUSED_ALLOC(scales); UNUSED_ALLOC(x);
  check_heads(FN, x_n1, x_n2, heads, head_dim);
  check_rows(FN, n, x_n0, y_n0);
  float *yp = T2(float, y);
  const float *xp = T3(float, x);
  for (int t = 0; t < n; ++t)
    quant_matvec(FN, vxb::kFmtQ4, yp + (int64_t)t * y_n1, y_n1, T1(uint32_t, w),
                 w_n0, T1(uint16_t, scales), scales_n0,
                 xp + (int64_t)t * x_n1 * x_n2, (int64_t)heads * head_dim, rows,
                 heads * head_dim, 1);
}
#undef FN

#define FN "nn_qkv_q4_rows"
void vx_nn_qkv_q4_rows(VX_TENSOR3(q), VX_TENSOR3(k), VX_TENSOR3(v), VX_TENSOR1(w),
                       VX_TENSOR1(scales), VX_TENSOR1(b), VX_TENSOR2(x), int32_t n,
                       int32_t q_heads, int32_t kv_heads, int32_t head_dim,
                       int32_t cols) {
  UNUSED_ALLOC(q); UNUSED_ALLOC(k); UNUSED_ALLOC(v); UNUSED_ALLOC(w);
  UNUSED_ALLOC(scales); UNUSED_ALLOC(b); UNUSED_ALLOC(x);
  check_heads(FN, q_n1, q_n2, q_heads, head_dim);
  check_heads(FN, k_n1, k_n2, kv_heads, head_dim);
  check_heads(FN, v_n1, v_n2, kv_heads, head_dim);
  if (n <= 0 || x_n0 < n || q_n0 < n || k_n0 < n || v_n0 < n)
    stop("nn rows: `x`, `q`, `k` and `v` need n rows");
  float *qp = T3(float, q), *kp = T3(float, k), *vp = T3(float, v);
  const float *xp = T2(float, x);
  for (int t = 0; t < n; ++t)
    quant_qkv(FN, vxb::kFmtQ4, qp + (int64_t)t * q_n1 * q_n2,
              kp + (int64_t)t * k_n1 * k_n2, vp + (int64_t)t * v_n1 * v_n2,
              T1(uint32_t, w), w_n0, T1(uint16_t, scales), scales_n0,
              T1(uint16_t, b), b_n0, xp + (int64_t)t * x_n1, x_n1, q_heads,
              kv_heads, head_dim, cols);
}
#undef FN

/* The experts of n positions (nn.vx:2952-3155). Position t runs the
   one-position projections on ids[t], x[t] and h[t * k ..]: row t is the
   one-position kernel's own result, bit for bit. */
#define FN "nn_moe_swiglu_q4_rows"
void vx_nn_moe_swiglu_q4_rows(VX_TENSOR2(out), VX_TENSOR1(w), VX_TENSOR1(scales),
                              VX_TENSOR2(ids), VX_TENSOR2(x), int32_t n, int32_t k,
                              int32_t rows, int32_t cols, int32_t experts) {
  UNUSED_ALLOC(out); UNUSED_ALLOC(w); UNUSED_ALLOC(scales); UNUSED_ALLOC(ids);
  UNUSED_ALLOC(x);
  if (k <= 0 || n <= 0 || ids_n0 < n || ids_n1 < k || x_n0 < n ||
      out_n0 < (int64_t)n * k || out_n1 < rows)
    stop("nn_moe_swiglu_q4_rows: `ids` needs n rows of k values, `x` n rows, and "
         "`out` a row of rows values for each of the n * k");
  if (cols <= 0 || cols % 32 != 0 ||
      scales_n0 < (int64_t)experts * 2 * rows * (cols / 32))
    stop("nn_moe_swiglu_q4_rows: the scales are too few for the experts");
  float *op = T2(float, out);
  const int32_t *ip = T2(int32_t, ids);
  const float *xp = T2(float, x);
  for (int t = 0; t < n; ++t)
    moe_swiglu(FN, vxb::kFmtQ4, op + (int64_t)t * k * out_n1, k, out_n1,
               T1(uint32_t, w), w_n0, T1(uint16_t, scales), ip + (int64_t)t * ids_n1,
               ids_n1, xp + (int64_t)t * x_n1, x_n1, k, rows, cols, experts);
}
#undef FN

#define FN "nn_moe_down_q4_add_rows"
void vx_nn_moe_down_q4_add_rows(VX_TENSOR2(y), VX_TENSOR1(w), VX_TENSOR1(scales),
                                VX_TENSOR2(ids), VX_TENSOR2(weights), VX_TENSOR2(h),
                                int32_t n, int32_t k, int32_t rows, int32_t cols,
                                int32_t experts) {
  UNUSED_ALLOC(y); UNUSED_ALLOC(w); UNUSED_ALLOC(scales); UNUSED_ALLOC(ids);
  UNUSED_ALLOC(weights); UNUSED_ALLOC(h);
  if (k <= 0 || n <= 0 || ids_n0 < n || ids_n1 < k || weights_n0 < n ||
      weights_n1 < k || h_n0 < (int64_t)n * k || h_n1 < cols || y_n0 < n)
    stop("nn_moe_down_q4_add_rows: `ids` and `weights` need n rows of k values, `h` "
         "a row of cols values for each of the n * k, and `y` n rows");
  if (cols <= 0 || cols % 32 != 0 ||
      scales_n0 < (int64_t)experts * rows * (cols / 32))
    stop("nn_moe_down_q4_add_rows: the scales are too few for the experts");
  float *yp = T2(float, y);
  const int32_t *ip = T2(int32_t, ids);
  const float *wp = T2(float, weights), *hp = T2(float, h);
  for (int t = 0; t < n; ++t)
    moe_down_add(FN, vxb::kFmtQ4, yp + (int64_t)t * y_n1, y_n1, T1(uint32_t, w),
                 w_n0, T1(uint16_t, scales), ip + (int64_t)t * ids_n1, ids_n1,
                 wp + (int64_t)t * weights_n1, weights_n1,
                 hp + (int64_t)t * k * h_n1, k, h_n1, k, rows, cols, experts);
}
#undef FN

/* ------------------------------------------- pairs grouped by expert
 * nn_moe_group_count nn.vx:1070, nn_moe_group_offsets :1110,
 * nn_moe_group_place :1252, nn_moe_group :1287. The asserts of those functions
 * are the checks here. */
#define FN "nn_moe_group_count"
void vx_nn_moe_group_count(VX_TENSOR2(counts), VX_TENSOR1(ids), int32_t n,
                           int32_t experts) {
  UNUSED_ALLOC(counts); UNUSED_ALLOC(ids);
  if (experts <= 0 || experts > 1024 || n < 0 || n > ids_n0)
    stop("nn_moe_group_count: `experts` must be 1 to 1024, and `ids` needs n values");
  if (counts_n0 * 256 < n || counts_n1 < experts)
    stop("nn_moe_group_count: `counts` needs a row for each 256 pairs, and a column "
         "for each expert");
  must(vxb::moe_group_count(T2(int32_t, counts), counts_n1, T1(int32_t, ids), n,
                            experts, vxb::caller_stream()),
       FN);
}
#undef FN

#define FN "nn_moe_group_offsets"
void vx_nn_moe_group_offsets(VX_TENSOR2(base), VX_TENSOR1(starts),
                             VX_TENSOR1(tile_expert), VX_TENSOR1(order),
                             VX_TENSOR2(counts), int32_t n, int32_t experts,
                             int32_t align) {
  UNUSED_ALLOC(base); UNUSED_ALLOC(starts); UNUSED_ALLOC(tile_expert);
  UNUSED_ALLOC(order); UNUSED_ALLOC(counts);
  if (experts <= 0 || experts > 1024 || align <= 0 || n < 0)
    stop("nn_moe_group_offsets: `experts` must be 1 to 1024, and `align` above 0");
  if (starts_n0 <= experts || counts_n0 * 256 < n || counts_n1 < experts ||
      base_n0 * 256 < n || base_n1 < experts)
    stop("nn_moe_group_offsets: `starts` needs experts + 1 values, and `counts` and "
         "`base` a row for each 256 pairs");
  if (order_n0 < (int64_t)n + (int64_t)experts * (align - 1) ||
      tile_expert_n0 * align < order_n0 || order_n0 > INT32_MAX ||
      tile_expert_n0 > INT32_MAX)
    stop("nn_moe_group_offsets: `order` needs n + experts * (align - 1) positions, "
         "and `tile_expert` one for each align of them");
  must(vxb::moe_group_offsets(T2(int32_t, base), base_n1, T1(int32_t, starts),
                              T1(int32_t, tile_expert), (int)tile_expert_n0,
                              T1(int32_t, order), (int)order_n0,
                              T2(int32_t, counts), counts_n1, n, experts, align,
                              vxb::caller_stream()),
       FN);
}
#undef FN

#define FN "nn_moe_group_place"
void vx_nn_moe_group_place(VX_TENSOR1(order), VX_TENSOR1(ids), VX_TENSOR2(base),
                           int32_t n) {
  UNUSED_ALLOC(order); UNUSED_ALLOC(ids); UNUSED_ALLOC(base);
  if (n < 0 || n > ids_n0 || base_n0 * 256 < n || order_n0 < n ||
      order_n0 > INT32_MAX)
    stop("nn_moe_group_place: `ids` needs n values, and `base` a row for each 256 "
         "pairs");
  /* the columns of `base` bound the ids; nn_moe_group_count has refused an id
     that names no expert */
  const int experts = base_n1 > 1024 ? 1024 : (int)base_n1;
  must(vxb::moe_group_place(T1(int32_t, order), (int)order_n0, T1(int32_t, ids),
                            T2(int32_t, base), base_n1, n, experts,
                            vxb::caller_stream()),
       FN);
}
#undef FN

#define PASS1(t) t##_allocated, t##_aligned, t##_offset, t##_n0, t##_s0
#define PASS2(t) t##_allocated, t##_aligned, t##_offset, t##_n0, t##_n1, t##_s0, t##_s1
void vx_nn_moe_group(VX_TENSOR1(order), VX_TENSOR2(counts), VX_TENSOR2(base),
                     VX_TENSOR1(starts), VX_TENSOR1(tile_expert), VX_TENSOR1(ids),
                     int32_t experts, int32_t align) {
  if (ids_n0 > INT32_MAX)
    stop("nn_moe_group: too many pairs");
  const int32_t n = (int32_t)ids_n0;
  vx_nn_moe_group_count(PASS2(counts), PASS1(ids), n, experts);
  vx_nn_moe_group_offsets(PASS2(base), PASS1(starts), PASS1(tile_expert),
                          PASS1(order), PASS2(counts), n, experts, align);
  vx_nn_moe_group_place(PASS1(order), PASS1(ids), PASS2(base), n);
}
#undef PASS1
#undef PASS2

} /* extern "C" */

extern "C" {

/* --------------------------------------------------------------- direct calls */
int32_t vx_b200_gemm(int32_t dtype, int32_t route, int64_t m, int64_t n,
                     int64_t k, const void *a, int64_t lda, const void *b,
                     int64_t ldb, void *c, int64_t ldc, void *scratch) {
  cudaStream_t s = vxb::caller_stream();
  switch (dtype) {
  case VX_DTYPE_F32:
    return done(vxb::gemm_f32((const float *)a, lda, (const float *)b, ldb,
                              (float *)c, ldc, m, n, k, s),
                "a GEMM");
  case VX_DTYPE_F64:
    return done(vxb::gemm_f64((const double *)a, lda, (const double *)b, ldb,
                              (double *)c, ldc, m, n, k, s),
                "a GEMM");
  case VX_DTYPE_F16:
  case VX_DTYPE_BF16: {
    const bool bf = dtype == VX_DTYPE_BF16;
    return done(route == 0 ? vxb::gemm_16(bf, a, lda, b, ldb, c, ldc, m, n, k, s)
                           : vxb::gemm_16_route(route, bf, a, lda, b, ldb, c,
                                                ldc, m, n, k, scratch, s),
                "a GEMM");
  }
  default:
    return fail("vx_b200_gemm takes f32, f64, f16 or bf16");
  }
}

int32_t vx_b200_gemm_q4(float *y, const uint32_t *w, const uint16_t *scales,
                        const float *x, int32_t n, int32_t rows, int32_t cols) {
  return done(vxb::gemm_q4(y, w, scales, x, n, rows, cols, vxb::caller_stream()),
              "gemm_q4");
}

int32_t vx_b200_gemm_fp8(float *y, const uint32_t *w, const float *scales,
                         const float *x, int32_t n, int32_t rows, int32_t cols) {
  return done(vxb::gemm_fp8(y, w, scales, x, n, rows, cols, vxb::caller_stream()),
              "gemm_fp8");
}

int32_t vx_b200_moe_swiglu_q4_grouped(float *out, const uint32_t *w,
                                      const uint16_t *scales, const int32_t *order,
                                      const int32_t *tile_expert, int32_t tiles,
                                      int32_t align, const float *x, int32_t n,
                                      int32_t k,
                                      int32_t rows, int32_t cols, int32_t experts) {
  vxb::MoeGroupedArgs m{};
  m.w = w;
  m.scales = scales;
  m.order = order;
  m.tile_expert = tile_expert;
  m.tiles = tiles;
  m.align = align;
  m.x = x;
  m.x_pitch = cols;
  m.out = out;
  m.out_pitch = rows;
  m.n = n;
  m.k = k;
  m.rows = rows;
  m.cols = cols;
  m.experts = experts;
  return done(vxb::moe_swiglu_q4_grouped(m, vxb::caller_stream()),
              "moe_swiglu_q4_grouped");
}

int32_t vx_b200_moe_down_q4_add_grouped(float *y, const uint32_t *w,
                                        const uint16_t *scales, const int32_t *order,
                                        const int32_t *tile_expert, int32_t tiles,
                                        int32_t align, const float *weights,
                                        const float *h,
                                        float *scratch, int32_t n, int32_t k,
                                        int32_t rows, int32_t cols, int32_t experts) {
  vxb::MoeGroupedArgs m{};
  m.w = w;
  m.scales = scales;
  m.order = order;
  m.tile_expert = tile_expert;
  m.tiles = tiles;
  m.align = align;
  m.x = h;
  m.x_pitch = cols;
  m.y = y;
  m.y_pitch = rows;
  m.pair_weights = weights;
  m.scratch = scratch;
  m.n = n;
  m.k = k;
  m.rows = rows;
  m.cols = cols;
  m.experts = experts;
  return done(vxb::moe_down_q4_add_grouped(m, vxb::caller_stream()),
              "moe_down_q4_add_grouped");
}

int32_t vx_b200_kernel_status(void) {
  const int g = vxb::gemm_status(vxb::caller_stream());
  const int f = vxb::flash_status(vxb::caller_stream());
  const int t = vxb::tp_status(vxb::caller_stream());
  const int m = vxb::batched_proj_status(vxb::caller_stream());
  const int r = vxb::rows_status();
  const int s = vxb::step_status(vxb::caller_stream());
  const int e = vxb::moe_group_status(vxb::caller_stream());
  return g ? g : (f ? f : (t ? t : (m ? m : (r ? r : (s ? s : e)))));
}

int32_t vx_b200_attention_kernel(int32_t which) {
  return vxb::attention_kernel_choice(which);
}

int32_t vx_b200_flash_attention(const void *q, const void *k, const void *v,
                                void *out, int32_t B, int32_t H, int32_t S,
                                int32_t D, float scale, int32_t causal) {
  return done(vxb::flash_attention_fwd(q, k, v, out, B, H, S, D, scale,
                                       causal != 0, vxb::caller_stream()),
              "flash attention");
}

int32_t vx_b200_gemm_column_split(int32_t dtype, int64_t m, int64_t n_local,
                                  int64_t k, const void *a, const void *b_local,
                                  void *c_local, void *gathered, void *c_full) {
  if (dtype != VX_DTYPE_BF16)
    return fail("the column-split product takes bf16");
  cudaStream_t s = vxb::caller_stream();
  if (const char *why = vxb::gemm_16(true, a, k, b_local, n_local, c_local,
                                     n_local, m, n_local, k, s))
    return fail(why);
  vx::NcclCollective *job = vxb::nccl_job();
  const int ranks = job ? job->ranks() : 0;
  if (ranks < 1)
    return fail("vx_collective_init has not run");
  const std::string why =
      job->all_gather(c_local, gathered, m * n_local, vx::NcclBfloat16,
                      "vx_b200_gemm_column_split");
  if (!why.empty())
    return fail(why.c_str());
  return done(vxb::interleave_gathered(gathered, c_full, ranks, m, n_local, 2, s),
              "a column-split GEMM");
}

int32_t vx_b200_quantize(int32_t format, const void *w_bf16, int32_t rows,
                         int32_t cols, void *codes, void *scales) {
  if (format == 2)
    return done(vxb::quantize_fp8(w_bf16, rows, cols, codes, (float *)scales,
                                  vxb::caller_stream()),
                "a quantisation");
  if (format == 3)
    return done(vxb::quantize_q4(w_bf16, rows, cols, codes, scales,
                                 vxb::caller_stream()),
                "a quantisation");
  return fail("vx_b200_quantize takes format 2 (fp8) or 3 (Q4_0)");
}

int32_t vx_b200_fill_normal(void *out, int32_t as_bf16, int64_t n, uint64_t seed,
                            float sigma) {
  return done(vxb::fill_normal(out, as_bf16 != 0, n, seed, sigma,
                               vxb::caller_stream()),
              "a fill");
}
int32_t vx_b200_fill_uniform(void *out, int32_t as_bf16, int64_t n,
                             uint64_t seed, float lo, float hi) {
  return done(vxb::fill_uniform(out, as_bf16 != 0, n, seed, lo, hi,
                                vxb::caller_stream()),
              "a fill");
}

} /* extern "C" */
