/* vx_collective.h -- the job of ranks behind the vx_collective_* entry points.
 *
 * One process per GPU.  NCCL is found at run time (dlopen), rank 0 passes the
 * NCCL id to the others through a file, and every operation is queued on the
 * caller's stream.  Each method answers "" or one sentence saying why not; the
 * exported C functions turn a sentence into a FATAL line and abort().
 *
 * Same interface and refusals as the reference's runtime/vx_collective.h
 * (NcclApi :63-90, id file :95-132, NcclCollective :138-286,
 * OneRankCollective :288-335), so its collective_test.cpp runs against this
 * file with its fake NCCL.  The optional NCCL entries (group calls, send/recv,
 * reduce-scatter, broadcast) are what the tensor-parallel helpers use when the
 * loaded library has them; a library with only the six required symbols still
 * loads.
 */
#ifndef VX_COLLECTIVE_H
#define VX_COLLECTIVE_H

#include <dlfcn.h>
#include <errno.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <chrono>
#include <memory>
#include <string>
#include <thread>

namespace vx {

struct NcclUniqueId {
  char internal[128];
};
using NcclComm = void *;
enum NcclDataType : int { NcclFloat32 = 7, NcclBfloat16 = 9 };
enum NcclRedOp : int { NcclSum = 0 };

struct NcclApi {
  /* required */
  int (*GetUniqueId)(NcclUniqueId *) = nullptr;
  int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*AllReduce)(const void *, void *, size_t, int, int, NcclComm,
                   void *) = nullptr;
  int (*AllGather)(const void *, void *, size_t, int, NcclComm,
                   void *) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  /* optional */
  int (*ReduceScatter)(const void *, void *, size_t, int, int, NcclComm,
                       void *) = nullptr;
  int (*Broadcast)(const void *, void *, size_t, int, int, NcclComm,
                   void *) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
};

inline std::unique_ptr<const NcclApi> load_nccl(const char *path,
                                                std::string *why) {
  why->clear();
  void *lib = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!lib) {
    *why = std::string("Vx cannot load NCCL: ") + dlerror() +
           ". Install NCCL, or set VX_NCCL_LIB to the path of libnccl.so.2.";
    return nullptr;
  }
  auto api = std::make_unique<NcclApi>();
  auto bind = [&](auto &fn, const char *symbol, bool required) {
    fn = reinterpret_cast<std::decay_t<decltype(fn)>>(dlsym(lib, symbol));
    if (!fn && required && why->empty())
      *why = std::string(path) + " has no " + symbol + ".";
  };
  bind(api->GetUniqueId, "ncclGetUniqueId", true);
  bind(api->CommInitRank, "ncclCommInitRank", true);
  bind(api->CommDestroy, "ncclCommDestroy", true);
  bind(api->AllReduce, "ncclAllReduce", true);
  bind(api->AllGather, "ncclAllGather", true);
  bind(api->GetErrorString, "ncclGetErrorString", true);
  bind(api->ReduceScatter, "ncclReduceScatter", false);
  bind(api->Broadcast, "ncclBroadcast", false);
  bind(api->GroupStart, "ncclGroupStart", false);
  bind(api->GroupEnd, "ncclGroupEnd", false);
  if (!why->empty())
    return nullptr;
  return api;
}

/* Rank 0 publishes the id under `path`. The bytes go to `path`.partial first
   and reach `path` by one rename, so a reader never sees half an id. A file
   that is already there belongs to some earlier job and is refused. */
inline std::string write_unique_id(const char *path, const NcclUniqueId &id) {
  if (access(path, F_OK) == 0)
    return std::string("the file ") + path +
           " is already there. It may hold the id of an earlier job. Remove "
           "it before you start the ranks.";
  const std::string staging = std::string(path) + ".partial";
  FILE *f = fopen(staging.c_str(), "wb");
  bool ok = f != nullptr;
  if (f) {
    ok = fwrite(&id, sizeof id, 1, f) == 1;
    ok = (fclose(f) == 0) && ok;
  }
  if (!ok)
    return "rank 0 cannot write " + staging + ": " + strerror(errno) + ".";
  if (rename(staging.c_str(), path) != 0)
    return "rank 0 cannot rename " + staging + ": " + strerror(errno) + ".";
  return "";
}

/* The other ranks poll for the file until `timeout`. */
inline std::string read_unique_id(const char *path, NcclUniqueId *id,
                                  std::chrono::milliseconds timeout) {
  const auto deadline = std::chrono::steady_clock::now() + timeout;
  for (;;) {
    if (access(path, F_OK) == 0)
      break;
    if (std::chrono::steady_clock::now() > deadline)
      return std::string("rank 0 did not write ") + path + " in " +
             std::to_string(timeout.count() / 1000) + " s.";
    std::this_thread::sleep_for(std::chrono::milliseconds(10));
  }
  FILE *f = fopen(path, "rb");
  const bool ok = f && fread(id, sizeof *id, 1, f) == 1;
  if (f)
    fclose(f);
  return ok ? "" : std::string("cannot read the NCCL id from ") + path + ".";
}

/* What the job needs from the GPU runtime, as plain functions, so that a test
   supplies fakes. */
struct CollectiveDevice {
  void *(*stream)();
  bool (*recording)();
  bool (*device_memory)(const void *ptr);
  int (*current_device)();
  void (*set_device)(int);
};

class NcclCollective {
public:
  explicit NcclCollective(CollectiveDevice device) : dev_(device) {}

  std::string init(int32_t rank, int32_t ranks, const char *nccl_lib,
                   const char *id_file, std::chrono::milliseconds timeout) {
    if (comm_)
      return "vx_collective_init ran a second time. Call vx_collective_finish "
             "first.";
    if (rank < 0 || rank >= ranks)
      return "vx_collective_init needs 0 <= rank < ranks, but rank is " +
             std::to_string(rank) + " and ranks is " + std::to_string(ranks) +
             ".";
    if (dev_.recording())
      return "vx_collective_init ran while the stream records a CUDA graph. "
             "Call it before the recording.";
    std::string why;
    if (!api_) {
      api_ = load_nccl(nccl_lib, &why);
      if (!api_)
        return why;
    }
    NcclUniqueId id;
    const bool makes_id = ranks == 1 || rank == 0;
    if (ranks > 1 && (!id_file || !*id_file))
      return "a job with more than one rank needs VX_NCCL_ID_FILE, a path that "
             "every rank can read. Rank 0 writes the NCCL id there.";
    if (makes_id) {
      if (int r = api_->GetUniqueId(&id))
        return failed("ncclGetUniqueId", r);
      if (ranks > 1 && !(why = write_unique_id(id_file, id)).empty())
        return why;
    } else if (!(why = read_unique_id(id_file, &id, timeout)).empty()) {
      return why;
    }
    home_ = dev_.current_device();
    if (int r = api_->CommInitRank(&comm_, ranks, id, rank)) {
      comm_ = nullptr;
      return failed("ncclCommInitRank", r);
    }
    rank_ = rank;
    ranks_ = ranks;
    return "";
  }

  std::string finish() {
    if (!comm_)
      return "vx_collective_finish ran before vx_collective_init.";
    const int r = api_->CommDestroy(comm_);
    comm_ = nullptr;
    rank_ = -1;
    ranks_ = 0;
    return r ? failed("ncclCommDestroy", r) : "";
  }

  int32_t rank() const { return rank_; }
  int32_t ranks() const { return ranks_; }
  /* For the tensor-parallel helpers, which queue their own NCCL calls. */
  NcclComm comm() const { return comm_; }
  const NcclApi *api() const { return api_.get(); }
  int home_device() const { return home_; }

  std::string all_reduce_sum(const void *input, void *output, int64_t count,
                             NcclDataType type, const char *name) {
    std::string why = refusal(input, output, count, name);
    if (!why.empty())
      return why;
    return at_home(name, [&](void *s) {
      return api_->AllReduce(input, output, (size_t)count, type, NcclSum, comm_,
                             s);
    });
  }

  std::string all_gather(const void *input, void *output, int64_t count,
                         NcclDataType type, const char *name) {
    std::string why = refusal(input, output, count, name);
    if (!why.empty())
      return why;
    return at_home(name, [&](void *s) {
      return api_->AllGather(input, output, (size_t)count, type, comm_, s);
    });
  }

private:
  std::string refusal(const void *input, const void *output, int64_t count,
                      const char *name) const {
    if (!comm_)
      return std::string(name) + " ran before vx_collective_init.";
    if (count < 0)
      return std::string(name) + " got a count of " + std::to_string(count) +
             ".";
    if (count > 0 && !(dev_.device_memory(input) && dev_.device_memory(output)))
      return std::string(name) +
             " needs tensors in GPU memory. Transfer them to the GPU first.";
    return "";
  }

  /* Run `call` with the GPU that joined the job current, then put back the
     GPU that was current. */
  template <typename Call> std::string at_home(const char *name, Call call) {
    const int was = dev_.current_device();
    if (was != home_)
      dev_.set_device(home_);
    const int r = call(dev_.stream());
    if (was != home_)
      dev_.set_device(was);
    return r ? failed(name, r) : "";
  }

  std::string failed(const char *what, int r) const {
    return std::string(what) + " failed: " + api_->GetErrorString(r) + ".";
  }

  CollectiveDevice dev_;
  std::unique_ptr<const NcclApi> api_;
  NcclComm comm_ = nullptr;
  int home_ = 0;
  int32_t rank_ = -1;
  int32_t ranks_ = 0;
};

/* A job of one rank on a machine with no GPU: every collective is a copy. */
class OneRankCollective {
public:
  std::string init(int32_t rank, int32_t ranks) {
    if (joined_)
      return "vx_collective_init ran a second time. Call vx_collective_finish "
             "first.";
    if (ranks != 1 || rank != 0)
      return "vx_collective_init got rank " + std::to_string(rank) + " of " +
             std::to_string(ranks) +
             " ranks, but this process runs a job of one rank only: this "
             "backend has no library that joins several ranks.";
    joined_ = true;
    return "";
  }
  std::string finish() {
    if (!joined_)
      return "vx_collective_finish ran before vx_collective_init.";
    joined_ = false;
    return "";
  }
  int32_t rank() const { return joined_ ? 0 : -1; }
  int32_t ranks() const { return joined_ ? 1 : 0; }
  std::string copy(const void *input, void *output, int64_t count,
                   size_t element, const char *name) const {
    if (!joined_)
      return std::string(name) + " ran before vx_collective_init.";
    if (count < 0)
      return std::string(name) + " got a count of " + std::to_string(count) +
             ".";
    if (input != output)
      memmove(output, input, (size_t)count * element);
    return "";
  }

private:
  bool joined_ = false;
};

} // namespace vx

#endif /* VX_COLLECTIVE_H */
