/* vx_hardware_runtime.h -- the C boundary between a compiled Vx program and
 * the dispatch library that serves its `spawn on(Topology::GPU[i])` regions.
 *
 * This is the B200 dispatch library's statement of the interface that the
 * reference declares in include/vx_hardware_runtime.h (the whole file): the
 * same entry points, tag bits, descriptor layout, payload format, topology
 * bands and control opcodes, so that an object file produced by vxc links
 * against either library.  Line references below are to that reference file.
 */
#ifndef VX_HARDWARE_RUNTIME_H
#define VX_HARDWARE_RUNTIME_H

#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- what the machine model said about host access (ref :23-34) ---------- */
typedef enum {
  VX_SPACE_ACCESS_UNKNOWN = 0,      /* caller does not know; nothing checked */
  VX_SPACE_ACCESS_EXPLICIT = 1,     /* `managed: explicit`: device memory ok  */
  VX_SPACE_ACCESS_HOST_READABLE = 2 /* model claims the host may read it      */
} vx_space_access;

/* ---- argument tags (ref :53-130) -----------------------------------------
 * bits 7:0 kind (0 = memref descriptor, else scalar type code)
 * bits 15:8 element type of a memref, bits 23:16 its rank,
 * bit 24 "slot": the argument is storage holding a descriptor.            */
#define VX_ABI_KIND(tag) ((tag) & 0xFF)
#define VX_ABI_ELEM(tag) (((tag) >> 8) & 0xFF)
#define VX_ABI_RANK(tag) (((tag) >> 16) & 0xFF)
#define VX_ABI_IS_SLOT(tag) (((tag) >> 24) & 1)
#define VX_ABI_SLOT_BIT (1 << 24)
#define VX_ABI_MEMREF_TAG(elem, rank)                                          \
  (((int32_t)(rank) << 16) | ((int32_t)(elem) << 8))
#define VX_ABI_SLOT_TAG(elem, rank)                                            \
  (VX_ABI_SLOT_BIT | VX_ABI_MEMREF_TAG(elem, rank))
#define VX_ABI_MAX_RANK 8

enum {
  VX_ABI_KIND_MEMREF = 0,
  VX_ABI_KIND_I1,
  VX_ABI_KIND_I8,
  VX_ABI_KIND_I16,
  VX_ABI_KIND_I32,
  VX_ABI_KIND_I64,
  VX_ABI_KIND_F32,
  VX_ABI_KIND_F64
};

enum {
  VX_DTYPE_UNKNOWN = 0,
  VX_DTYPE_I1,
  VX_DTYPE_I8,
  VX_DTYPE_I16,
  VX_DTYPE_I32,
  VX_DTYPE_I64,
  VX_DTYPE_F32,
  VX_DTYPE_F64,
  VX_DTYPE_F16,
  VX_DTYPE_BF16
};
#define VX_DTYPE_MAX_BYTES 8

static inline size_t vx_dtype_bytes(int32_t code) {
  static const unsigned char width[10] = {0, 1, 1, 2, 4, 8, 4, 8, 2, 2};
  return (code >= 0 && code < 10) ? width[code] : 0;
}

static inline const char *vx_dtype_name(int32_t code) {
  static const char *const names[10] = {"?",   "i1",  "i8",  "i16", "i32",
                                        "i64", "f32", "f64", "f16", "bf16"};
  return (code > 0 && code < 10) ? names[code] : "?";
}

/* ---- memref descriptors (ref :182-341) -----------------------------------
 * {allocated, aligned, offset, sizes[rank], strides[rank]}, all 8 bytes.  */
static inline const int64_t *vx_memref_sizes(const void *desc) {
  return (const int64_t *)desc + 3;
}
static inline const int64_t *vx_memref_strides(const void *desc, int32_t rank) {
  return (const int64_t *)desc + 3 + rank;
}
static inline void *vx_memref_aligned(const void *desc) {
  return ((void *const *)desc)[1];
}
static inline int64_t vx_memref_offset(const void *desc) {
  return ((const int64_t *)desc)[2];
}
static inline void *vx_memref_data(const void *desc, int32_t dtype) {
  return (char *)vx_memref_aligned(desc) +
         vx_memref_offset(desc) * (int64_t)vx_dtype_bytes(dtype);
}

enum {
  VX_VIEW_OK = 0,
  VX_VIEW_UNKNOWN_ELEMENT,
  VX_VIEW_NEGATIVE,
  VX_VIEW_TOO_MANY_ELEMENTS,
  VX_VIEW_TOO_MANY_BYTES
};

/* Bytes from the first element of a view to one past the last it reaches. */
static inline int vx_memref_view_span(const int64_t *sizes,
                                      const int64_t *strides, int32_t rank,
                                      int32_t elem, uint64_t *bytes,
                                      int32_t *dim) {
  const uint64_t width = vx_dtype_bytes(elem);
  uint64_t reach = 0, count = 0;
  int32_t d;
  int any_empty = 0;
  if (width == 0)
    return VX_VIEW_UNKNOWN_ELEMENT;
  for (d = 0; d < rank; ++d) {
    if (sizes[d] < 0 || strides[d] < 0) {
      *dim = d;
      return VX_VIEW_NEGATIVE;
    }
    if (sizes[d] == 0)
      any_empty = 1;
  }
  if (any_empty) {
    *bytes = 0;
    return VX_VIEW_OK;
  }
  for (d = 0; d < rank; ++d) {
    uint64_t far_end;
    if (__builtin_mul_overflow((uint64_t)(sizes[d] - 1), (uint64_t)strides[d],
                               &far_end) ||
        __builtin_add_overflow(reach, far_end, &reach))
      return VX_VIEW_TOO_MANY_ELEMENTS;
  }
  if (__builtin_add_overflow(reach, (uint64_t)1, &count))
    return VX_VIEW_TOO_MANY_ELEMENTS;
  if (__builtin_mul_overflow(count, width, bytes))
    return VX_VIEW_TOO_MANY_BYTES;
  return VX_VIEW_OK;
}

/* As above, but a broken descriptor stops the program (ref :282-312). */
static inline uint64_t vx_memref_view_bytes(const int64_t *sizes,
                                            const int64_t *strides,
                                            int32_t rank, int32_t elem) {
  uint64_t bytes = 0;
  int32_t d = 0;
  const int why = vx_memref_view_span(sizes, strides, rank, elem, &bytes, &d);
  if (why == VX_VIEW_OK)
    return bytes;
  if (why == VX_VIEW_UNKNOWN_ELEMENT)
    fprintf(stderr,
            "[Vx] FATAL: a tensor with element type code %d cannot be copied: "
            "the runtime does not know the size of that element (code 0 is "
            "what index and pointer elements get)\n",
            elem);
  else if (why == VX_VIEW_NEGATIVE)
    fprintf(stderr, "[Vx] FATAL: dimension %d of a tensor view has the negative %s %lld\n",
            d, sizes[d] < 0 ? "size" : "stride",
            (long long)(sizes[d] < 0 ? sizes[d] : strides[d]));
  else if (why == VX_VIEW_TOO_MANY_ELEMENTS)
    fprintf(stderr, "[Vx] FATAL: a tensor view spans 2^64 elements or more\n");
  else
    fprintf(stderr, "[Vx] FATAL: a tensor view spans 2^64 bytes or more\n");
  abort();
}

/* Fill `desc` as a dense row-major view of `data`. */
static inline void vx_memref_write_desc(void *desc, void *data, int32_t rank,
                                        const int64_t *sizes) {
  int64_t *f = (int64_t *)desc;
  int64_t step = 1;
  int32_t d;
  ((void **)desc)[0] = data;
  ((void **)desc)[1] = data;
  f[2] = 0;
  for (d = rank - 1; d >= 0; --d) {
    f[3 + d] = sizes[d];
    f[3 + rank + d] = step;
    step *= sizes[d];
  }
}

/* ---- dispatch payload (ref :343-563) --------------------------------------
 * name NUL key=value NUL ... [empty entry NUL, u64le length, image bytes]   */
#define VX_PAYLOAD_ABI 1

static inline size_t vx_payload_text_end(const void *payload,
                                         size_t payload_size) {
  const char *base = (const char *)payload;
  size_t at = 0;
  int first = 1;
  if (!payload || payload_size == 0)
    return 0;
  while (at < payload_size) {
    const char *nul = (const char *)memchr(base + at, '\0', payload_size - at);
    if (!nul)
      return payload_size;
    if (!first && nul == base + at)
      return at + 1;
    first = 0;
    at = (size_t)(nul - base) + 1;
  }
  return payload_size;
}

static inline const char *
vx_payload_field(const void *payload, size_t payload_size, const char *key) {
  const char *base = (const char *)payload;
  const char *nul;
  size_t key_len, at;
  int closed;
  if (!payload || payload_size == 0 || !key)
    return NULL;
  key_len = strlen(key);
  closed = base[payload_size - 1] == '\0';
  nul = (const char *)memchr(base, '\0', payload_size);
  if (!nul)
    return NULL;
  for (at = (size_t)(nul - base) + 1; at < payload_size;) {
    const char *entry = base + at;
    const size_t left = payload_size - at;
    size_t len;
    /* With a closing NUL every entry ends inside the blob, so a hit can
       answer before its end is searched for (an image= entry is long). */
    if (closed && left > key_len && memcmp(entry, key, key_len) == 0)
      return entry + key_len;
    nul = (const char *)memchr(entry, '\0', left);
    if (!nul)
      return NULL;
    len = (size_t)(nul - entry);
    if (len == 0)
      return NULL; /* the text part ended; a section follows */
    if (len >= key_len && memcmp(entry, key, key_len) == 0)
      return entry + key_len;
    at += len + 1;
  }
  return NULL;
}

static inline int32_t vx_payload_abi(const void *payload, size_t payload_size) {
  const char *v = vx_payload_field(payload, payload_size, "abi=");
  int64_t n = 0;
  if (!v || !*v)
    return -1;
  for (; *v; ++v) {
    if (*v < '0' || *v > '9')
      return -1;
    n = n * 10 + (*v - '0');
    if (n > INT32_MAX)
      return -1;
  }
  return (int32_t)n;
}

/* Length of the binary section and its start in *out; -1 none, -2 malformed,
   -3 out is NULL. */
static inline int64_t
vx_payload_section(const void *payload, size_t payload_size, const void **out) {
  const unsigned char *p;
  uint64_t length = 0;
  size_t start;
  int i;
  if (!out)
    return -3;
  if (!payload)
    return -1;
  start = vx_payload_text_end(payload, payload_size);
  if (start == payload_size)
    return -1;
  if (payload_size - start < 8)
    return -2;
  p = (const unsigned char *)payload + start;
  for (i = 0; i < 8; ++i)
    length |= (uint64_t)p[i] << (8 * i);
  if (length != payload_size - start - 8)
    return -2;
  *out = p + 8;
  return (int64_t)length;
}

/* ---- topology ids (ref :565-640) ---------------------------------------- */
#define VX_TOPO_CPU 0
#define VX_TOPO_NPU_BASE 100
#define VX_TOPO_ACCCORE_BASE 200
#define VX_TOPO_AMX 300
#define VX_TOPO_ANE 400
#define VX_TOPO_GPU_BASE 500
#define VX_TOPO_CPU_AVX512 600
#define VX_TOPO_CPU_NEON 700
#define VX_TOPO_NIC_BASE 800
#define VX_TOPO_REMOTE_BASE 900
#define VX_TOPO_SPIRV_BASE 1000
#define VX_TOPO_NUMA_BASE 1100
#define VX_TOPO_SLICE_BASE 2000
#define VX_TOPO_NAME_BASE 3000
#define VX_TOPO_BAND 100

static inline int vx_topology_device_index(int32_t topology_id, int32_t base) {
  const int32_t i = topology_id - base;
  return (topology_id >= base && i < VX_TOPO_BAND) ? (int)i : -1;
}

static inline int vx_topology_numa_node(int32_t topology_id) {
  return (topology_id >= VX_TOPO_NUMA_BASE && topology_id < VX_TOPO_SLICE_BASE)
             ? (int)(topology_id - VX_TOPO_NUMA_BASE)
             : -1;
}

static inline int32_t vx_payload_topology(const void *payload,
                                          size_t payload_size) {
  const char *v = vx_payload_field(payload, payload_size, "topo=");
  return (v && *v) ? (int32_t)strtol(v, NULL, 10) : -1;
}

/* ---- entry points (ref :36-51, :642-702) --------------------------------- */
void *vx_plugin_alloc_and_transfer(size_t bytes, void *host_ptr,
                                   uint32_t topology_id, uint32_t space_access);
void *vx_plugin_alloc_and_transfer_async(size_t bytes, void *host_ptr,
                                         uint32_t topology_id,
                                         uint32_t space_access);
uint64_t vx_plugin_dispatch_async(const void *binary_payload,
                                  size_t payload_size, void **device_args,
                                  const int32_t *arg_tags, int64_t num_args);
uint64_t vx_plugin_dispatch_async_flat(float *xout, float *x, float *w, int n,
                                       int d);
void vx_plugin_await_future(uint64_t future_id);
int32_t vx_plugin_transfer_device_to_host(void *device_ptr, void *host_ptr,
                                          size_t bytes, uint32_t topology_id);
void *vx_plugin_transfer_peer(void *src_device_ptr, uint32_t src_topology_id,
                              uint32_t dst_topology_id, size_t bytes);
void vx_plugin_free(void *device_ptr, uint32_t topology_id);
void *vx_plugin_arrivals_take(const void *site, size_t bytes, void *zeros,
                              uint32_t topology_id, uint32_t space_access);
void vx_plugin_arrivals_give(const void *site, void *count, size_t bytes,
                             uint32_t topology_id);
void vx_plugin_release_future(uint64_t future_id);
int32_t vx_plugin_control(uint32_t opcode, void *payload);

#define VX_CTRL_INIT_DEVICE 0x01
#define VX_CTRL_SHUTDOWN 0x02
#define VX_CTRL_GET_DEVICE_COUNT 0x03
#define VX_CTRL_LOCAL_DEVICE 0x04 /* payload: int32 declared id, builtin id */
#define VX_CTRL_WAIT 0x05         /* payload: int32 topology id */
#define VX_CTRL_WAIT_FOR_TENSORS 0x06 /* payload: vx_wait_for_tensors */
#define VX_CTRL_WAIT_FOR_THREAD 0x07  /* payload: int32 topology id */
#define VX_CTRL_VENDOR_BASE 0x1000

typedef struct vx_wait_for_tensors {
  int32_t topology;
  int32_t count;
  void **args;
  const int32_t *tags;
} vx_wait_for_tensors;

#ifdef __cplusplus
}
#endif

#endif /* VX_HARDWARE_RUNTIME_H */
