/* vx_stream_policy.h -- what a wait or a free may do, given whether the host
 * program set a stream (vx_cuda_set_stream) and whether that stream is
 * recording a CUDA graph.  Pure decisions, no CUDA calls, so the truth table
 * is testable anywhere.  Same enumerators and answers as the reference's
 * runtime/vx_stream_policy.h:20-63.
 */
#ifndef VX_STREAM_POLICY_H
#define VX_STREAM_POLICY_H

typedef enum {
  VX_WAIT_DEVICE, /* no caller stream: wait for the whole device        */
  VX_WAIT_STREAM, /* wait for the caller's stream only                   */
  VX_WAIT_REFUSE  /* the stream records a graph, which cannot hold a wait */
} vx_wait_action;

static inline vx_wait_action vx_wait_action_for(int has_stream, int recording) {
  if (!has_stream)
    return VX_WAIT_DEVICE;
  return recording ? VX_WAIT_REFUSE : VX_WAIT_STREAM;
}

typedef enum {
  VX_FREE_AFTER_DEVICE_WAIT, /* device wait, then cudaFree                  */
  VX_FREE_AFTER_STREAM_WAIT, /* stream wait, then cudaFree                  */
  VX_FREE_ON_STREAM,         /* cudaFreeAsync where the memory came from    */
  VX_FREE_REFUSE             /* recording, and the memory needs a wait first */
} vx_free_action;

/* on_stream: the memory came from cudaMallocAsync on a caller's stream; it is
   freed in order on that stream even if no stream is set any more. */
static inline vx_free_action vx_free_action_for(int has_stream, int recording,
                                                int on_stream) {
  if (on_stream)
    return VX_FREE_ON_STREAM;
  switch (vx_wait_action_for(has_stream, recording)) {
  case VX_WAIT_DEVICE:
    return VX_FREE_AFTER_DEVICE_WAIT;
  case VX_WAIT_STREAM:
    return VX_FREE_AFTER_STREAM_WAIT;
  default:
    return VX_FREE_REFUSE;
  }
}

#endif /* VX_STREAM_POLICY_H */
