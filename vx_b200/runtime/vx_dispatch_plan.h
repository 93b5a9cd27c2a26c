/* vx_dispatch_plan.h -- read a `kind=matmul` dispatch as C[m,n] = A[m,k]*B[k,n].
 *
 * Vendor-free, so the decision "which argument is A, which is B, where does
 * the result go" is testable without a GPU.  Behaviour follows the reference's
 * runtime/vx_dispatch_plan.h:55-305 (same names, same refusals): nothing is
 * inferred from shapes, and anything that does not line up is a refusal (0),
 * never a guess.
 */
#ifndef VX_DISPATCH_PLAN_H
#define VX_DISPATCH_PLAN_H

#include "vx_hardware_runtime.h"

#include <stdlib.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  VX_GEMM_OUT_BUFFER = 0, /* fill the buffer the kernel was handed          */
  VX_GEMM_OUT_SLOT = 1    /* allocate, then publish a descriptor in a slot   */
};

/* Row-major operands; a row stride is in elements and may exceed the width. */
typedef struct {
  int32_t dtype;
  int64_t m, n, k;
  const void *a_data;
  const void *b_data;
  int64_t a_row_stride;
  int64_t b_row_stride;
  int32_t out_kind;
  void *out_data; /* NULL for a slot */
  int64_t out_row_stride;
  void *out_desc; /* slot only: where the descriptor goes */
} vx_gemm_plan;

/* "a:<i>,b:<j>,out:<k>" in any order, each role exactly once. */
static inline int vx_parse_roles(const char *roles, int *a, int *b, int *out) {
  static const struct {
    const char *name;
    size_t len;
  } known[3] = {{"a:", 2}, {"b:", 2}, {"out:", 4}};
  int *dest[3];
  unsigned have = 0;
  const char *p = roles;
  if (!roles || !a || !b || !out || !*roles)
    return 0;
  dest[0] = a;
  dest[1] = b;
  dest[2] = out;
  for (;;) {
    int which = -1, r;
    char *stop = NULL;
    long index;
    for (r = 0; r < 3; ++r)
      if (strncmp(p, known[r].name, known[r].len) == 0)
        which = r;
    if (which < 0 || (have & (1u << which)))
      return 0;
    p += known[which].len;
    index = strtol(p, &stop, 10);
    if (stop == p || index < 0)
      return 0;
    *dest[which] = (int)index;
    have |= 1u << which;
    p = stop;
    if (*p == '\0')
      break;
    if (*p != ',' || p[1] == '\0')
      return 0;
    ++p;
  }
  return have == 7u;
}

static inline int vx_gemm_dtype_supported(int32_t dtype) {
  return dtype == VX_DTYPE_F32 || dtype == VX_DTYPE_F64 ||
         dtype == VX_DTYPE_F16 || dtype == VX_DTYPE_BF16;
}

/* The descriptor behind argument idx: the argument itself, or, for a slot,
   the descriptor that the slot's storage holds. */
static inline const void *vx_operand_desc(void **device_args,
                                          const int32_t *arg_tags, int idx) {
  const void *d = *(const void **)device_args[idx];
  return (d && VX_ABI_IS_SLOT(arg_tags[idx])) ? vx_memref_aligned(d) : d;
}

static inline int vx_plan_is_matrix_tag(int32_t tag, int32_t dtype) {
  return VX_ABI_KIND(tag) == VX_ABI_KIND_MEMREF && VX_ABI_RANK(tag) == 2 &&
         (int32_t)VX_ABI_ELEM(tag) == dtype;
}

/* 1 and a filled plan, or 0 when the region must take another route. */
static inline int vx_gemm_plan_decode(const void *payload, size_t payload_size,
                                      void **device_args,
                                      const int32_t *arg_tags, int64_t num_args,
                                      vx_gemm_plan *plan) {
  const char *text;
  const void *da, *db, *dc;
  const int64_t *as, *bs, *at, *bt;
  int ia = -1, ib = -1, ic = -1, to_slot;
  int32_t dtype;

  if (!plan || !device_args || !arg_tags)
    return 0;
  text = vx_payload_field(payload, payload_size, "kind=");
  if (!text || strcmp(text, "matmul") != 0)
    return 0;
  if (!vx_parse_roles(vx_payload_field(payload, payload_size, "roles="), &ia,
                      &ib, &ic))
    return 0;
  if (ia >= num_args || ib >= num_args || ic >= num_args || ia == ib ||
      ia == ic || ib == ic)
    return 0;
  text = vx_payload_field(payload, payload_size, "outkind=");
  if (!text)
    return 0;
  if (strcmp(text, "slot") == 0)
    to_slot = 1;
  else if (strcmp(text, "buffer") == 0)
    to_slot = 0;
  else
    return 0;

  dtype = VX_ABI_ELEM(arg_tags[ia]);
  if (!vx_gemm_dtype_supported(dtype) ||
      !vx_plan_is_matrix_tag(arg_tags[ia], dtype) ||
      !vx_plan_is_matrix_tag(arg_tags[ib], dtype) ||
      !vx_plan_is_matrix_tag(arg_tags[ic], dtype))
    return 0;

  da = vx_operand_desc(device_args, arg_tags, ia);
  db = vx_operand_desc(device_args, arg_tags, ib);
  dc = vx_operand_desc(device_args, arg_tags, ic);
  if (!da || !db || !dc)
    return 0;
  as = vx_memref_sizes(da);
  bs = vx_memref_sizes(db);
  at = vx_memref_strides(da, 2);
  bt = vx_memref_strides(db, 2);
  /* Rows must be contiguous; a permuted operand would need a transposed
     product, which the roles cannot say. */
  if (at[1] != 1 || bt[1] != 1)
    return 0;
  if (as[0] <= 0 || as[1] <= 0 || bs[1] <= 0 || bs[0] != as[1])
    return 0;

  plan->dtype = dtype;
  plan->m = as[0];
  plan->k = as[1];
  plan->n = bs[1];
  plan->a_data = vx_memref_data(da, dtype); /* base + offset: views count */
  plan->b_data = vx_memref_data(db, dtype);
  plan->a_row_stride = at[0];
  plan->b_row_stride = bt[0];
  plan->out_kind = to_slot ? VX_GEMM_OUT_SLOT : VX_GEMM_OUT_BUFFER;
  plan->out_data = NULL;
  plan->out_desc = NULL;
  plan->out_row_stride = plan->n;

  if (to_slot) {
    if (!VX_ABI_IS_SLOT(arg_tags[ic]))
      return 0; /* nowhere to write a descriptor */
    plan->out_desc = (void *)dc;
  } else {
    const int64_t *cs = vx_memref_sizes(dc);
    const int64_t *ct = vx_memref_strides(dc, 2);
    if (ct[1] != 1 || cs[0] != plan->m || cs[1] != plan->n)
      return 0;
    plan->out_data = vx_memref_data(dc, dtype);
    plan->out_row_stride = ct[0];
    if (!plan->out_data)
      return 0;
  }
  return plan->a_data && plan->b_data;
}

/* Hand a freshly allocated m x n result back through the slot. */
static inline void vx_gemm_publish_slot(const vx_gemm_plan *plan, void *data) {
  const int64_t shape[2] = {plan->m, plan->n};
  vx_memref_write_desc(plan->out_desc, data, 2, shape);
}

#ifdef __cplusplus
}
#endif

#endif /* VX_DISPATCH_PLAN_H */
