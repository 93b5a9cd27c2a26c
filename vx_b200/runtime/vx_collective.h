/* vx_collective.h -- what stands behind the vx_collective_* exports: one
 * process per GPU, all of them members of one NCCL communicator.
 *
 * Contract (the reference's runtime/vx_collective.h :138-335 has the same one,
 * and its tests/runtime/collective_test.cpp is run against this header with a
 * fake NCCL): a method returns an empty string when it did its work, else a
 * sentence for the user that the exported C function prints as a FATAL line
 * before abort(). NCCL itself comes from vx_nccl_binding.h. Work is queued on
 * whatever stream the caller has made current, on the GPU that joined.
 */
#ifndef VX_COLLECTIVE_H
#define VX_COLLECTIVE_H

#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <memory>
#include <string>

#include "vx_nccl_binding.h"

namespace vx {

/* The five questions the job asks of the GPU runtime. Plain function
   pointers: the dispatch library fills them with CUDA calls, a test with
   fakes. */
struct CollectiveDevice {
  void *(*stream)();
  bool (*recording)();
  bool (*device_memory)(const void *ptr);
  int (*current_device)();
  void (*set_device)(int);
};

/* Sentences both kinds of job use. */
namespace collective_words {

inline std::string joined_twice() {
  return "vx_collective_init ran a second time. Call vx_collective_finish "
         "first.";
}

inline std::string never_joined(const char *who) {
  std::string s(who);
  s += " ran before vx_collective_init.";
  return s;
}

inline std::string bad_count(const char *who, int64_t count) {
  std::string s(who);
  s += " got a count of ";
  s += std::to_string(count);
  s += ".";
  return s;
}

} // namespace collective_words

class NcclCollective {
public:
  explicit NcclCollective(CollectiveDevice device) : gpu_(device) {}

  int32_t rank() const { return member_.comm ? member_.rank : -1; }
  int32_t ranks() const { return member_.comm ? member_.ranks : 0; }

  /* The tensor-parallel decoder queues NCCL calls of its own on these. */
  NcclComm comm() const { return member_.comm; }
  const NcclApi *api() const { return nccl_.get(); }
  int home_device() const { return member_.gpu; }

  /* Joins the communicator. With ranks > 1, rank 0 creates the id and leaves
     it in `id_file`; the others wait up to `patience` for it. */
  std::string init(int32_t rank, int32_t ranks, const char *nccl_lib,
                   const char *id_file, std::chrono::milliseconds patience) {
    std::string why = may_join(rank, ranks, id_file);
    if (!why.empty())
      return why;
    if (!nccl_ && !(nccl_ = load_nccl(nccl_lib, &why)))
      return why;

    NcclUniqueId id;
    const bool creates = rank == 0;
    if (creates) {
      const int err = nccl_->GetUniqueId(&id);
      if (err)
        return nccl_said("ncclGetUniqueId", err);
      if (ranks > 1)
        why = write_unique_id(id_file, id);
    } else {
      why = read_unique_id(id_file, &id, patience);
    }
    if (!why.empty())
      return why;

    Member m;
    m.gpu = gpu_.current_device();
    m.rank = rank;
    m.ranks = ranks;
    const int err = nccl_->CommInitRank(&m.comm, ranks, id, rank);
    if (err)
      return nccl_said("ncclCommInitRank", err);
    member_ = m;
    return std::string();
  }

  std::string finish() {
    if (!member_.comm)
      return "vx_collective_finish ran before vx_collective_init.";
    const NcclComm leaving = member_.comm;
    member_ = Member();
    const int err = nccl_->CommDestroy(leaving);
    return err ? nccl_said("ncclCommDestroy", err) : std::string();
  }

  std::string all_reduce_sum(const void *input, void *output, int64_t count,
                             NcclDataType type, const char *name) {
    Op op = {name, input, output, count, type, /*reduce=*/true};
    return queue(op);
  }

  std::string all_gather(const void *input, void *output, int64_t count,
                         NcclDataType type, const char *name) {
    Op op = {name, input, output, count, type, /*reduce=*/false};
    return queue(op);
  }

private:
  struct Member {
    NcclComm comm = nullptr;
    int32_t rank = -1;
    int32_t ranks = 0;
    int gpu = 0; /* the GPU that was current at init */
  };

  struct Op {
    const char *name;
    const void *from;
    void *to;
    int64_t count;
    NcclDataType type;
    bool reduce;
  };

  std::string may_join(int32_t rank, int32_t ranks, const char *id_file) const {
    if (member_.comm)
      return collective_words::joined_twice();
    if (!(0 <= rank && rank < ranks)) {
      char line[160];
      snprintf(line, sizeof line,
               "vx_collective_init needs 0 <= rank < ranks, but rank is %d and "
               "ranks is %d.",
               (int)rank, (int)ranks);
      return line;
    }
    if (gpu_.recording())
      return "vx_collective_init ran while the stream records a CUDA graph. "
             "Call it before the recording.";
    if (ranks > 1 && (id_file == nullptr || id_file[0] == '\0'))
      return "a job with more than one rank needs VX_NCCL_ID_FILE, a path that "
             "every rank can read. Rank 0 writes the NCCL id there.";
    return std::string();
  }

  /* Checks the operation, then issues it with the joining GPU current and
     restores the caller's GPU. An empty operation may name any memory. */
  std::string queue(const Op &op) {
    if (!member_.comm)
      return collective_words::never_joined(op.name);
    if (op.count < 0)
      return collective_words::bad_count(op.name, op.count);
    const bool on_gpu =
        op.count == 0 ||
        (gpu_.device_memory(op.from) && gpu_.device_memory(op.to));
    if (!on_gpu) {
      std::string s(op.name);
      s += " needs tensors in GPU memory. Transfer them to the GPU first.";
      return s;
    }
    const int callers_gpu = gpu_.current_device();
    const bool away = callers_gpu != member_.gpu;
    if (away)
      gpu_.set_device(member_.gpu);
    void *stream = gpu_.stream();
    const size_t n = (size_t)op.count;
    const int err =
        op.reduce ? nccl_->AllReduce(op.from, op.to, n, op.type, NcclSum,
                                     member_.comm, stream)
                  : nccl_->AllGather(op.from, op.to, n, op.type, member_.comm,
                                     stream);
    if (away)
      gpu_.set_device(callers_gpu);
    return err ? nccl_said(op.name, err) : std::string();
  }

  std::string nccl_said(const char *call, int err) const {
    std::string s(call);
    s += " failed: ";
    s += nccl_->GetErrorString(err);
    s += ".";
    return s;
  }

  CollectiveDevice gpu_;
  std::unique_ptr<const NcclApi> nccl_;
  Member member_;
};

/* The job a build without a GPU library can offer: exactly one rank, for
   which a sum over ranks and a gather from ranks are both the input itself. */
class OneRankCollective {
public:
  int32_t rank() const { return in_job_ ? 0 : -1; }
  int32_t ranks() const { return in_job_ ? 1 : 0; }

  std::string init(int32_t rank, int32_t ranks) {
    if (in_job_)
      return collective_words::joined_twice();
    if (rank == 0 && ranks == 1) {
      in_job_ = true;
      return std::string();
    }
    char line[240];
    snprintf(line, sizeof line,
             "vx_collective_init got rank %d of %d ranks, but this process "
             "runs a job of one rank only: this backend has no library that "
             "joins several ranks.",
             (int)rank, (int)ranks);
    return line;
  }

  std::string finish() {
    const bool was = in_job_;
    in_job_ = false;
    return was ? std::string()
               : "vx_collective_finish ran before vx_collective_init.";
  }

  std::string copy(const void *input, void *output, int64_t count,
                   size_t element, const char *name) const {
    if (!in_job_)
      return collective_words::never_joined(name);
    if (count < 0)
      return collective_words::bad_count(name, count);
    if (output != input && count > 0)
      memmove(output, input, element * (size_t)count);
    return std::string();
  }

private:
  bool in_job_ = false;
};

} // namespace vx

#endif /* VX_COLLECTIVE_H */
