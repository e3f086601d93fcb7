// c10d backend "stragglar": straggler-aware collectives for PyTorch.
//
//   import stragglar_b200.parallel            # registers the backend
//   dist.init_process_group("stragglar")      # or "cpu:gloo,cuda:stragglar"
//
// AllReduce runs the compiled StragglAR table (or ring / rhd / direct / ...)
// with the persistent peer-memory kernel on a communication stream of its own;
// the 1/world_size of ReduceOp.AVG (the DDP gradient average) is fused into the
// kernel.  Tensors that live in the backend's symmetric heap
// (`alloc_symmetric`) are reduced in place; any other tensor is staged through
// the arena.  broadcast, all_gather, reduce_scatter, reduce, gather, scatter,
// all_to_all, barrier and send/recv are provided through the same arenas, so
// that `DistributedDataParallel` can be built on the backend.  Work objects
// carry CUDA events and real futures.  CPU tensors are served by the host
// executor over POSIX shared memory with the same tables and flag protocol.
//
// The reference backend ("dummy", implementation/custom_backend/src/dummy.cpp)
// implements allreduce only (fp32, world size 8, straggler fixed at rank 6),
// fakes allgather and reports every Work as complete immediately
// (dummy.cpp:137-151,233-247,717-811).
#pragma once
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>

#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAStream.h>

#include <atomic>
#include <exception>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <string>

#include "../core/plan.h"
#include "transport.h"

namespace sarpg {

struct BackendOptions {
  std::string alg = "stragglar";   // stragglar | stragglar_a2a | ring | rhd | direct | rsag | auto
  int straggler = -1;              // physical rank that is persistently late (-1: the last rank)
  int path = 1;                    // 0 simt, 1 tma, 2 simta (see SarPath)
  int blocks = 0, threads = 0;
  uint32_t tile_bytes = 0;
  double timeout_s = 30.0;         // bound of every device-side wait
  size_t arena_bytes = 0;          // data region per rank (0: STRAGGLAR_ARENA_MB or 1 GiB on CUDA, 64 MiB on CPU)
  size_t staging_bytes = 0;        // part of the arena used to stage foreign tensors (0: a quarter, at most 256 MiB)
  std::string schedule_text;       // overrides the built-in StragglAR schedule
  bool check_args = false;         // STRAGGLAR_CHECK_ARGS=1: every AllReduce first compares, through the Store, what the
                                   // ranks passed (element count, dtypes, symmetric offset or "ordinary tensor"); a
                                   // mismatch raises on every rank instead of producing wrong sums.  A debugging aid:
                                   // it costs a Store round trip per collective.
};

// The failure word of one device side of a process group, shared with the Work objects it hands out.
// `reported`: a Work has already raised for the failure that the word shows, so the process group clears
// it silently before its next collective instead of raising a second time.
struct FailureState {
  std::shared_ptr<uint32_t> word;   // pinned host memory written by the device (see Transport::status)
  std::atomic<bool> reported{false};
};

class WorkStragglar : public c10d::Work {
 public:
  WorkStragglar(int rank, c10d::OpType op, std::vector<at::Tensor> outputs, bool cuda);
  bool isCompleted() override;
  bool isSuccess() const override;
  bool wait(std::chrono::milliseconds timeout = kNoTimeout) override;
  void synchronize() override;
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override;
  std::vector<at::Tensor> result() override { return outputs_; }

 private:
  friend class ProcessGroupStragglar;
  std::vector<at::Tensor> outputs_;
  bool cuda_;
  void check_failure();             // raises when the device has recorded a failed wait
  std::shared_ptr<at::cuda::CUDAEvent> end_;
  c10::intrusive_ptr<c10::ivalue::Future> future_;
  std::shared_ptr<FailureState> fail_;
  std::exception_ptr error_;        // a failure that happened while the work was issued (CPU tensors run at once)
};

class ProcessGroupStragglar : public c10d::Backend {
 public:
  ProcessGroupStragglar(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                        std::chrono::milliseconds timeout, BackendOptions opts);
  ~ProcessGroupStragglar() override;

  const std::string getBackendName() const override { return "stragglar"; }

  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors, const c10d::BroadcastOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors, const c10d::AllreduceOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor>& tensors,
                                                     const c10d::AllreduceCoalescedOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                           const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& output, at::Tensor& input,
                                                 const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(std::vector<at::Tensor>& outputs,
                                                                 std::vector<at::Tensor>& inputs,
                                                                 const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                        const c10d::GatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor>& outputs, std::vector<std::vector<at::Tensor>>& inputs,
                                         const c10d::ScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor>& outputs,
                                                std::vector<std::vector<at::Tensor>>& inputs,
                                                const c10d::ReduceScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor& output, at::Tensor& input,
                                                      const c10d::ReduceScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& outputs,
                                                                 std::vector<at::Tensor>& inputs,
                                                                 const c10d::ReduceScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allgather_coalesced(std::vector<std::vector<at::Tensor>>& output_lists,
                                                     std::vector<at::Tensor>& inputs,
                                                     const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& output, at::Tensor& input, std::vector<int64_t>& out_splits,
                                               std::vector<int64_t>& in_splits, const c10d::AllToAllOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
                                          const c10d::AllToAllOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dst, int tag) override;
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int src, int tag) override;
  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& opts) override;

  // ---- beyond c10d
  // AllReduce with an explicit communication dtype: the cast to `comm_dtype`
  // (and the 1/world_size of `average`) happens while the tensor is staged in,
  // the cast back while it is staged out.
  c10::intrusive_ptr<c10d::Work> allreduce_ex(at::Tensor& tensor, bool average, std::optional<at::ScalarType> comm_dtype);
  // A tensor inside the symmetric heap: collectives on it (or on views of it)
  // run in place without staging.  Collective call: every rank must allocate
  // the same sizes in the same order.
  at::Tensor alloc_symmetric(int64_t numel, at::ScalarType dtype, bool cuda, int device);
  void set_straggler(int physical_rank);     // re-labels the schedule; takes effect at the next collective
  void set_algorithm(const std::string& alg);
  int straggler() const { return opts_.straggler; }
  std::string algorithm() const { return opts_.alg; }
  // The algorithm an AllReduce of `bytes` runs: the configured one, or the choice of "auto".
  std::string algorithm_for(size_t bytes) const;
  // Waits for the communication stream and returns the device status word
  // (a SarStatus; 0 = ok), clearing a recorded failure.
  int64_t check_status(bool cuda);
  int64_t launches() const { return launches_; }   // kernels of this library launched so far
  // True while the canary bytes around this rank's data region (symmetric heap + staging) are intact.
  bool check_guards(bool cuda);
  // %globaltimer stamps (ns) of the last collective kernel of this rank: when it arrived and
  // when it left.  Their difference is the time the rank spent inside the collective; the
  // persistent straggler is the rank that spends the least (it arrives last and waits for nobody).
  std::pair<int64_t, int64_t> last_trace();

 private:
  struct Side {   // per device type
    std::unique_ptr<Transport> t;
    std::optional<c10::cuda::CUDAStream> stream;
    std::shared_ptr<FailureState> fail;
    int device = -1;
    std::vector<std::shared_ptr<void>> dev_tables;   // keeps uploaded tables alive
    std::map<std::pair<const void*, int>, std::pair<void*, void*>> uploaded;  // (table, rank) -> ops, round_begin
  };
  Side& side(const at::Tensor& like);
  Side& side(bool cuda, int device);
  const sar::Program& program(size_t bytes = 0);
  // `user` (CUDA, single-phase programs): staged mode -- the kernel reads the input from and writes the result to
  // `user` (elements of SarDtype `user_dtype`), the arena range at data_off only serves the peers
  void run_program(Side& s, const sar::Program& prog, size_t data_off, uint64_t count, at::ScalarType dtype, float scale,
                   void* user = nullptr, int user_dtype = 0);
  void device_barrier(Side& s);
  c10::intrusive_ptr<WorkStragglar> begin(Side& s, c10d::OpType op, std::vector<at::Tensor> outputs);
  void finish(Side& s, const c10::intrusive_ptr<WorkStragglar>& w);
  // CPU tensors are reduced inside the call: a failure there (a rank that never joined) becomes the Work's
  // error, raised by wait(), as it is for CUDA tensors
  c10::intrusive_ptr<c10d::Work> failed(Side& s, const c10::intrusive_ptr<WorkStragglar>& w);
  void recover_if_failed(Side& s);  // raises for a failure nobody has been told about, then clears it
  void clear_failure(Side& s);
  void copy_local(Side& s, void* dst, const void* src, size_t bytes);
  void pull(Side& s, const std::vector<std::tuple<int, size_t, void*, size_t>>& segs);  // (peer, offset in data region, dst, bytes)
  void allreduce_impl(Side& s, at::Tensor& t, float scale, std::optional<at::ScalarType> comm_dtype);
  void allreduce_generic(Side& s, at::Tensor& t, const c10d::ReduceOp& op);   // any dtype / op: gather + local reduce
  void gather_all(Side& s, void* out, const void* in, size_t bytes);

  c10::intrusive_ptr<c10d::Store> store_;
  BackendOptions opts_;
  std::chrono::milliseconds timeout_;
  std::string prefix_;
  Side cuda_, cpu_;
  std::map<std::string, sar::Program> programs_;
  std::mutex mu_;
  int64_t launches_ = 0;
  uint64_t alloc_seq_ = 0;
  uint64_t check_seq_ = 0;
  void check_same_arguments(uint64_t count, int tensor_dtype, int comm_dtype, int64_t heap_off);
  std::map<std::pair<bool, int>, uint32_t> send_seq_, recv_seq_;   // (cuda?, peer) -> handshakes so far
};

}  // namespace sarpg
