/* vx_collective_cpu.h -- the eight vx_collective_* entry points for a build
 * with no GPU: a job of one rank, where all-reduce and all-gather are copies.
 * Same exports and messages as the reference's runtime/vx_collective_cpu.h
 * :26-76. The CUDA dispatch library does not include this; it is what the test
 * oracle for the collectives links.
 */
#ifndef VX_COLLECTIVE_CPU_H
#define VX_COLLECTIVE_CPU_H

#include "vx_collective.h"

static vx::OneRankCollective vx_one_rank;

#ifndef VX_COLLECTIVE_CPU_BEFORE_COPY
#define VX_COLLECTIVE_CPU_BEFORE_COPY(input, output, bytes) ((void)0)
#endif

static void vx_collective_cpu_check(const std::string &why) {
  if (why.empty())
    return;
  fprintf(stderr, "[Vx] FATAL: %s\n", why.c_str());
  abort();
}

#define VX_COLLECTIVE_CPU_COPY(fn, type, width)                                \
  void fn(const type *input, type *output, int64_t count) {                    \
    VX_COLLECTIVE_CPU_BEFORE_COPY(input, output, count *width);                \
    vx_collective_cpu_check(vx_one_rank.copy(input, output, count, width, #fn)); \
  }

extern "C" {
void vx_collective_init(int32_t rank, int32_t ranks) {
  vx_collective_cpu_check(vx_one_rank.init(rank, ranks));
}
void vx_collective_finish(void) {
  vx_collective_cpu_check(vx_one_rank.finish());
}
int32_t vx_collective_rank(void) { return vx_one_rank.rank(); }
int32_t vx_collective_ranks(void) { return vx_one_rank.ranks(); }
VX_COLLECTIVE_CPU_COPY(vx_collective_all_reduce_sum_f32, float, 4)
VX_COLLECTIVE_CPU_COPY(vx_collective_all_reduce_sum_bf16, uint16_t, 2)
VX_COLLECTIVE_CPU_COPY(vx_collective_all_gather_f32, float, 4)
VX_COLLECTIVE_CPU_COPY(vx_collective_all_gather_bf16, uint16_t, 2)
} /* extern "C" */

#endif /* VX_COLLECTIVE_CPU_H */
