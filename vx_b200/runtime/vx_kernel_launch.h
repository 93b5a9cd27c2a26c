/* vx_kernel_launch.h -- turn a dispatch's arguments into the parameter list of
 * a compiler-emitted kernel, read that kernel's signature, and size its launch.
 *
 * Nothing here touches a vendor API, so the marshalling is checked on a
 * machine with no GPU.  Behaviour follows the reference's
 * runtime/vx_kernel_launch.h:57-484: a rank-r memref becomes 3+2r parameters
 * (allocated, aligned, offset, sizes, strides) that point INTO the caller's
 * descriptor, a scalar is one parameter, a slot is refused.
 */
#ifndef VX_KERNEL_LAUNCH_H
#define VX_KERNEL_LAUNCH_H

#include "vx_hardware_runtime.h"

#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define VX_LAUNCH_MAX_PARAMS 128

typedef struct {
  void *params[VX_LAUNCH_MAX_PARAMS];
  int count;
} vx_launch_params;

/* How many kernel parameters one argument becomes; 0 = cannot be passed. */
static inline int vx_launch_param_width(int32_t tag) {
  if (VX_ABI_IS_SLOT(tag))
    return 0; /* a descriptor that does not exist yet has no address */
  if (VX_ABI_KIND(tag) != VX_ABI_KIND_MEMREF)
    return vx_dtype_bytes(VX_ABI_KIND(tag)) != 0;
  return VX_ABI_RANK(tag) <= VX_ABI_MAX_RANK ? 3 + 2 * (int)VX_ABI_RANK(tag)
                                             : 0;
}

static inline int vx_launch_build_params(void *const *device_args,
                                         const int32_t *arg_tags,
                                         int64_t num_args,
                                         vx_launch_params *out) {
  int n = 0;
  int64_t i;
  if (!device_args || !arg_tags || !out || num_args < 0)
    return 0;
  out->count = 0;
  for (i = 0; i < num_args; ++i) {
    const int width = vx_launch_param_width(arg_tags[i]);
    if (width == 0 || n + width > VX_LAUNCH_MAX_PARAMS || !device_args[i])
      return 0;
    if (width == 1 && VX_ABI_KIND(arg_tags[i]) != VX_ABI_KIND_MEMREF) {
      out->params[n++] = (void *)device_args[i];
    } else {
      /* device_args[i] points at a pointer to the descriptor; every field of
         the descriptor is 8 bytes, so field f sits at byte 8*f. */
      char *fields = (char *)*(void *const *)device_args[i];
      int f;
      if (!fields)
        return 0;
      for (f = 0; f < width; ++f)
        out->params[n++] = fields + 8 * f;
    }
  }
  out->count = n;
  return 1;
}

/* The parenthesised parameter list of `.entry <entry>` in PTX text. */
static inline int vx_launch_entry_signature(const char *ptx, const char *entry,
                                            const char **open,
                                            const char **close) {
  size_t len;
  const char *at;
  if (!ptx || !entry)
    return 0;
  len = strlen(entry);
  for (at = strstr(ptx, ".entry "); at; at = strstr(at, ".entry ")) {
    at += 7;
    at += strspn(at, " \t");
    /* whole-name match only: kernel_1 must not answer for kernel_10 */
    if (strncmp(at, entry, len) != 0 || !strchr("( \t\n", at[len]) ||
        at[len] == '\0')
      continue;
    *open = strchr(at, '(');
    if (!*open)
      return 0;
    *close = strchr(*open, ')');
    return *close != NULL;
  }
  return 0;
}

static inline int vx_launch_entry_param_count(const char *ptx,
                                              const char *entry) {
  const char *open, *close, *p;
  int n = 0;
  if (!vx_launch_entry_signature(ptx, entry, &open, &close))
    return -1;
  for (p = open; p < close; ++p)
    n += strncmp(p, ".param", 6) == 0;
  return n;
}

static inline uint32_t vx_spirv_word(const unsigned char *module,
                                     size_t index) {
  const unsigned char *b = module + 4 * index;
  return (uint32_t)b[0] | (uint32_t)b[1] << 8 | (uint32_t)b[2] << 16 |
         (uint32_t)b[3] << 24;
}

/* Parameters of the function that OpEntryPoint `entry` names, or -1. Kept so
   that a payload for another vendor's device is still read the same way. */
static inline int vx_launch_entry_param_count_spirv(const void *image,
                                                    size_t image_size,
                                                    const char *entry) {
  const unsigned char *m = (const unsigned char *)image;
  size_t words, at;
  uint32_t fn = 0;
  if (!image || !entry || image_size < 20 || (image_size & 3))
    return -1;
  if (vx_spirv_word(m, 0) != 0x07230203u)
    return -1;
  words = image_size / 4;
  /* pass 1: the id that the entry point instruction (opcode 15) gives */
  for (at = 5; at < words;) {
    const uint32_t head = vx_spirv_word(m, at);
    const uint32_t len = head >> 16, op = head & 0xFFFF;
    if (len == 0 || at + len > words)
      return -1;
    if (op == 15 && len >= 4) {
      const size_t room = (size_t)(len - 3) * 4, need = strlen(entry) + 1;
      if (need <= room && memcmp(m + 4 * (at + 3), entry, need) == 0)
        fn = vx_spirv_word(m, at + 2);
    }
    at += len;
  }
  if (!fn)
    return -1;
  /* pass 2: OpFunction (54) with that id, then its run of parameters (55) */
  for (at = 5; at < words;) {
    const uint32_t head = vx_spirv_word(m, at);
    const uint32_t len = head >> 16, op = head & 0xFFFF;
    if (len == 0 || at + len > words)
      return -1;
    if (op == 54 && len >= 3 && vx_spirv_word(m, at + 2) == fn) {
      int n = 0;
      size_t q = at + len;
      while (q < words) {
        const uint32_t h2 = vx_spirv_word(m, q);
        if ((h2 >> 16) == 0 || q + (h2 >> 16) > words || (h2 & 0xFFFF) != 55)
          break;
        ++n;
        q += h2 >> 16;
      }
      return n;
    }
    at += len;
  }
  return -1;
}

/* align[k] = the `.align N` of pointer parameter k, 0 for the others. */
static inline int vx_launch_param_aligns(const char *ptx, const char *entry,
                                         long *align, int max) {
  const char *open, *close, *p;
  int k = 0;
  if (!align || !vx_launch_entry_signature(ptx, entry, &open, &close))
    return 0;
  for (p = open; p < close && k < max; ++p) {
    const char *end, *is_ptr, *al;
    if (strncmp(p, ".param", 6) != 0)
      continue;
    end = strchr(p + 6, ',');
    if (!end || end > close)
      end = close;
    is_ptr = strstr(p, ".ptr");
    al = strstr(p, ".align ");
    align[k++] = (is_ptr && is_ptr < end && al && al < end)
                     ? strtol(al + 7, NULL, 10)
                     : 0;
  }
  return 1;
}

/* Index of the first pointer value that breaks its declared alignment. */
static inline int vx_launch_misaligned(const vx_launch_params *params,
                                       const long *align, int count) {
  int k;
  for (k = 0; k < count && k < params->count; ++k) {
    uintptr_t value;
    if (align[k] <= 1)
      continue;
    memcpy(&value, params->params[k], sizeof value);
    if (value % (uintptr_t)align[k])
      return k;
  }
  return -1;
}

static inline int vx_launch_takes_assert_flag(const void *payload,
                                              size_t payload_size) {
  const char *v = vx_payload_field(payload, payload_size, "assert_flag=");
  return v && v[0] == '1' && v[1] == '\0';
}

/* One size from a shape text: a number, or `$j` = launch value j, an i32 that
   sits after the kernel's num_args arguments.  -1 when it is not an i32. */
static inline long vx_launch_size(const char **text, void *const *device_args,
                                  const int32_t *arg_tags, int64_t num_args) {
  char *stop = NULL;
  long v;
  if (**text == '$') {
    const long j = strtol(*text + 1, &stop, 10);
    if (j < 0 || j > 3 || arg_tags[num_args + j] != VX_ABI_KIND_I32)
      return -1;
    v = *(const int32_t *)device_args[num_args + j];
  } else {
    v = strtol(*text, &stop, 10);
  }
  *text = (*stop == ',') ? stop + 1 : stop;
  return v;
}

/* `launch=` : trip count (and threads for the two-level `B,T` form). */
static inline long vx_launch_trip(const void *payload, size_t payload_size,
                                  void *const *device_args,
                                  const int32_t *arg_tags, int64_t num_args,
                                  long *threads) {
  const char *text = vx_payload_field(payload, payload_size, "launch=");
  long trip;
  *threads = 0;
  if (!text)
    return 0;
  trip = vx_launch_size(&text, device_args, arg_tags, num_args);
  if (trip >= 0 && *text)
    *threads = vx_launch_size(&text, device_args, arg_tags, num_args);
  return trip;
}

/* `grid=` + `block=`: 1 filled, 0 absent, -1 not launchable (reason in why).
   With `grid_loops=` the kernel strides over blocks, so a grid is clamped to
   what the GPU launches instead of refused. */
static inline int vx_launch_shape(const void *payload, size_t payload_size,
                                  void *const *device_args,
                                  const int32_t *arg_tags, int64_t num_args,
                                  unsigned grid[3], unsigned *block, char *why,
                                  size_t why_size) {
  static const long most[3] = {2147483647L, 65535L, 65535L};
  const char *g = vx_payload_field(payload, payload_size, "grid=");
  const char *b = vx_payload_field(payload, payload_size, "block=");
  int clamp, axis;
  long t;
  if (!g || !b)
    return 0;
  clamp = vx_payload_field(payload, payload_size, "grid_loops=") != NULL;
  for (axis = 0; axis < 3; ++axis) {
    long n = *g ? vx_launch_size(&g, device_args, arg_tags, num_args) : 1;
    if (clamp) {
      if (n < 1)
        n = 1;
      if (n > most[axis])
        n = most[axis];
    } else if (n < 1 || n > most[axis]) {
      snprintf(why, why_size,
               "grid axis %d has %ld blocks, and a GPU launches 1 to %ld on "
               "that axis",
               axis, n, most[axis]);
      return -1;
    }
    grid[axis] = (unsigned)n;
  }
  t = vx_launch_size(&b, device_args, arg_tags, num_args);
  if (t < 1 || t > 1024) {
    snprintf(why, why_size,
             "a block of %ld threads, and a block holds 1 to 1024 threads", t);
    return -1;
  }
  *block = (unsigned)t;
  return 1;
}

#endif /* VX_KERNEL_LAUNCH_H */
