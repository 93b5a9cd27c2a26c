/* vx_nccl_binding.h -- NCCL as this library sees it: a table of entry points
 * resolved with dlsym at run time, and the file through which rank 0 hands the
 * job's NCCL id to the other ranks.
 *
 * Nothing here includes an NCCL header; the handful of types and constants the
 * calls need are restated with NCCL's published values.
 */
#ifndef VX_NCCL_BINDING_H
#define VX_NCCL_BINDING_H

#include <dlfcn.h>
#include <errno.h>
#include <fcntl.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <chrono>
#include <memory>
#include <string>
#include <thread>

namespace vx {

/* ncclUniqueId, ncclComm_t, ncclDataType_t, ncclRedOp_t */
struct NcclUniqueId {
  char internal[128];
};
typedef void *NcclComm;
enum NcclDataType : int { NcclFloat32 = 7, NcclBfloat16 = 9 };
enum NcclRedOp : int { NcclSum = 0 };

typedef int (*NcclReduceFn)(const void *send, void *recv, size_t count,
                            int type, int op_or_root, NcclComm comm,
                            void *stream);
typedef int (*NcclGatherFn)(const void *send, void *recv, size_t count,
                            int type, NcclComm comm, void *stream);

/* Every slot is one pointer wide, which is what lets load_nccl() fill the
   struct from a table of names. */
struct NcclApi {
  int (*GetUniqueId)(NcclUniqueId *) = nullptr;
  int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  NcclReduceFn AllReduce = nullptr;
  NcclGatherFn AllGather = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  /* From here on a library may lack the entry; users check for nullptr. */
  NcclReduceFn ReduceScatter = nullptr;
  NcclReduceFn Broadcast = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
};

namespace nccl_binding {

struct Entry {
  const char *symbol;
  size_t slot; /* offsetof the member in NcclApi */
  bool must_have;
};

inline const Entry *entries(size_t *n) {
  static const Entry table[] = {
      {"ncclGetUniqueId", offsetof(NcclApi, GetUniqueId), true},
      {"ncclCommInitRank", offsetof(NcclApi, CommInitRank), true},
      {"ncclCommDestroy", offsetof(NcclApi, CommDestroy), true},
      {"ncclAllReduce", offsetof(NcclApi, AllReduce), true},
      {"ncclAllGather", offsetof(NcclApi, AllGather), true},
      {"ncclGetErrorString", offsetof(NcclApi, GetErrorString), true},
      {"ncclReduceScatter", offsetof(NcclApi, ReduceScatter), false},
      {"ncclBroadcast", offsetof(NcclApi, Broadcast), false},
      {"ncclGroupStart", offsetof(NcclApi, GroupStart), false},
      {"ncclGroupEnd", offsetof(NcclApi, GroupEnd), false},
  };
  *n = sizeof table / sizeof table[0];
  return table;
}

inline bool exists(const char *path) {
  struct stat st;
  return lstat(path, &st) == 0;
}

inline std::string os_error() { return std::string(strerror(errno)) + "."; }

} // namespace nccl_binding

/* Opens `path` and resolves the table above. On failure the answer is null
   and *why holds one sentence for the user. The handle is never closed: the
   communicator lives as long as the process may use it. */
inline std::unique_ptr<const NcclApi> load_nccl(const char *path,
                                                std::string *why) {
  static_assert(sizeof(void *) == sizeof(NcclReduceFn),
                "function and data pointers of one width");
  why->clear();
  void *handle = dlopen(path, RTLD_LOCAL | RTLD_NOW);
  if (handle == nullptr) {
    why->assign("Vx cannot load NCCL: ");
    why->append(dlerror());
    why->append(". Install NCCL, or set VX_NCCL_LIB to the path of "
                "libnccl.so.2.");
    return nullptr;
  }
  std::unique_ptr<NcclApi> table(new NcclApi);
  size_t n = 0;
  const nccl_binding::Entry *e = nccl_binding::entries(&n);
  for (size_t i = 0; i < n; ++i) {
    void *address = dlsym(handle, e[i].symbol);
    if (address == nullptr && e[i].must_have) {
      why->assign(path);
      why->append(" has no ");
      why->append(e[i].symbol);
      why->append(".");
      return nullptr;
    }
    memcpy(reinterpret_cast<char *>(table.get()) + e[i].slot, &address,
           sizeof address);
  }
  return std::unique_ptr<const NcclApi>(table.release());
}

/* Rank 0's half of the hand-over. The 128 bytes are written under a
   temporary name and renamed into place, so whoever finds `path` finds all of
   them. A `path` that exists before the job starts is left alone and the job
   refused: it would be read as this job's id by a rank that started early. */
inline std::string write_unique_id(const char *path, const NcclUniqueId &id) {
  using nccl_binding::os_error;
  if (nccl_binding::exists(path)) {
    std::string s("the file ");
    s += path;
    s += " is already there. It may hold the id of an earlier job. Remove it "
         "before you start the ranks.";
    return s;
  }
  std::string tmp(path);
  tmp += ".partial";
  const int fd = open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0)
    return "rank 0 cannot write " + tmp + ": " + os_error();
  const char *bytes = id.internal;
  size_t left = sizeof id.internal;
  while (left > 0) {
    const ssize_t put = write(fd, bytes, left);
    if (put < 0 && errno == EINTR)
      continue;
    if (put <= 0) {
      const std::string why = "rank 0 cannot write " + tmp + ": " + os_error();
      close(fd);
      return why;
    }
    bytes += put;
    left -= (size_t)put;
  }
  if (close(fd) != 0)
    return "rank 0 cannot write " + tmp + ": " + os_error();
  if (rename(tmp.c_str(), path) != 0)
    return "rank 0 cannot rename " + tmp + ": " + os_error();
  return std::string();
}

/* The other ranks' half: look for the file every 10 ms for at most `wait`. */
inline std::string read_unique_id(const char *path, NcclUniqueId *id,
                                  std::chrono::milliseconds wait) {
  typedef std::chrono::steady_clock Clock;
  const Clock::time_point give_up = Clock::now() + wait;
  while (!nccl_binding::exists(path)) {
    if (Clock::now() > give_up) {
      std::string s("rank 0 did not write ");
      s += path;
      s += " in " + std::to_string(wait.count() / 1000) + " s.";
      return s;
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(10));
  }
  size_t got = 0;
  const int fd = open(path, O_RDONLY);
  while (fd >= 0 && got < sizeof id->internal) {
    const ssize_t n = read(fd, id->internal + got, sizeof id->internal - got);
    if (n < 0 && errno == EINTR)
      continue;
    if (n <= 0)
      break;
    got += (size_t)n;
  }
  if (fd >= 0)
    close(fd);
  if (got == sizeof id->internal)
    return std::string();
  return std::string("cannot read the NCCL id from ") + path + ".";
}

} // namespace vx

#endif /* VX_NCCL_BINDING_H */
