#include "process_group_stragglar.h"

#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <pybind11/chrono.h>
#include <torch/extension.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <thread>

#include "../core/c_api.h"
#include "../core/host_exec.h"
#include "../kernels/sar_cuda.h"
#include "../kernels/sar_params.h"

namespace sarpg {

#define SAR_CUDA_CHECK(x)                                                                    \
  do {                                                                                       \
    cudaError_t e_ = (cudaError_t)(x);                                                       \
    TORCH_CHECK(e_ == cudaSuccess, "stragglar backend: ", #x, ": ", cudaGetErrorString(e_)); \
  } while (0)

namespace {
// NVTX range around the host side of every collective (visible in Nsight Systems)
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
};
constexpr int kBarrierChannel = 2;   // control words of barrier() and the staged collectives
constexpr int kP2PChannel = 3;       // flag words of send/recv handshakes

int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return SAR_F32;
    case at::kBFloat16: return SAR_BF16;
    case at::kHalf: return SAR_F16;
    default: TORCH_CHECK(false, "stragglar backend reduces float32, bfloat16 and float16 tensors, got ", t);
  }
}
size_t env_mb(const char* name, size_t dflt_mb) {
  const char* v = getenv(name);
  return ((v && *v) ? (size_t)strtoull(v, nullptr, 10) : dflt_mb) << 20;
}
std::atomic<uint32_t>* as_atomic(uint32_t* p) { return reinterpret_cast<std::atomic<uint32_t>*>(p); }

void check_contiguous(const at::Tensor& t) {
  TORCH_CHECK(t.is_contiguous(), "stragglar backend needs contiguous tensors");
  TORCH_CHECK(t.is_cuda() || t.is_cpu(), "stragglar backend serves CUDA and CPU tensors");
}
}  // namespace

// ------------------------------------------------------------------------ Work
WorkStragglar::WorkStragglar(int rank, c10d::OpType op, std::vector<at::Tensor> outputs, bool cuda)
    : c10d::Work(rank, op), outputs_(std::move(outputs)), cuda_(cuda) {}

bool WorkStragglar::isCompleted() { return !cuda_ || !end_ || end_->query(); }
bool WorkStragglar::isSuccess() const {
  if (error_) return false;
  if (!cuda_ || !end_ || !fail_ || !end_->query()) return !cuda_ || !end_;   // CUDA work in flight: not known yet
  return *(volatile uint32_t*)fail_->word.get() == 0;
}
void WorkStragglar::check_failure() {
  if (!fail_) return;
  const uint32_t st = *(volatile uint32_t*)fail_->word.get();
  if (!st) return;
  fail_->reported.store(true);
  TORCH_CHECK(false, "stragglar backend: a collective failed on rank ", rank_, ": ", sar_status_string(st),
              " (a device-side wait ran out; the result is incomplete)");
}
// Makes the caller's stream wait for the collective (the c10d contract for CUDA work).  With a timeout the host
// waits too, at most that long.  Whenever the collective is known to have ended, a failure that the device
// recorded (a wait that ran out because a peer was late or never came) is raised here.
bool WorkStragglar::wait(std::chrono::milliseconds timeout) {
  if (error_) std::rethrow_exception(error_);
  if (cuda_ && end_) {
    end_->block(c10::cuda::getCurrentCUDAStream(end_->device_index()));
    if (timeout != kNoTimeout) {
      const auto deadline = std::chrono::steady_clock::now() + timeout;
      while (!end_->query()) {
        TORCH_CHECK(std::chrono::steady_clock::now() < deadline, "stragglar backend: the collective did not finish within ",
                    timeout.count(), " ms");
        std::this_thread::sleep_for(std::chrono::microseconds(50));
      }
    }
    if (end_->query()) check_failure();
  }
  return true;
}
void WorkStragglar::synchronize() {
  wait();
  if (cuda_ && end_) { end_->synchronize(); check_failure(); }
}
c10::intrusive_ptr<c10::ivalue::Future> WorkStragglar::getFuture() { return future_; }

// --------------------------------------------------------------- process group
ProcessGroupStragglar::ProcessGroupStragglar(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                                             std::chrono::milliseconds timeout, BackendOptions opts)
    : c10d::Backend(rank, size), store_(store), opts_(std::move(opts)), timeout_(timeout) {
  TORCH_CHECK(size >= 1 && size <= SAR_MAX_RANKS, "stragglar backend supports 1..", SAR_MAX_RANKS, " ranks");
  TORCH_CHECK(opts_.straggler < size, "straggler rank out of range");
  prefix_ = "sar";
  if (const char* a = getenv("STRAGGLAR_ALG")) if (*a) opts_.alg = a;
  if (const char* s = getenv("STRAGGLAR_STRAGGLER")) if (*s) opts_.straggler = atoi(s);
  if (const char* p = getenv("STRAGGLAR_PATH")) if (*p) opts_.path = !strcmp(p, "simt") ? SAR_PATH_SIMT : !strcmp(p, "simta") ? SAR_PATH_SIMTA : SAR_PATH_TMA;
  if (const char* b = getenv("STRAGGLAR_BLOCKS")) if (*b) opts_.blocks = atoi(b);
  if (const char* b = getenv("STRAGGLAR_THREADS")) if (*b) opts_.threads = atoi(b);
  if (const char* b = getenv("STRAGGLAR_TILE_BYTES")) if (*b) opts_.tile_bytes = (uint32_t)atoi(b);
  if (const char* b = getenv("STRAGGLAR_TIMEOUT_MS")) if (*b) opts_.timeout_s = atof(b) / 1e3;
  if (const char* b = getenv("STRAGGLAR_CHECK_ARGS")) if (*b) opts_.check_args = atoi(b) != 0;
  (void)program();   // fail early on a bad algorithm / rank count
}

ProcessGroupStragglar::~ProcessGroupStragglar() {
  if (cuda_.t) {
    cudaSetDevice(cuda_.device);
    cudaDeviceSynchronize();
    for (auto& kv : cuda_.uploaded) { cudaFree(kv.second.first); cudaFree(kv.second.second); }
  }
}

// "auto" picks per call, from what every rank knows (message size, declared straggler), so all ranks agree.
// With a declared straggler: stragglar_a2a, whose pre-phase hides in the straggler's delay and whose ranks then
// move exactly S bytes per direction (8 x B200, net of a 5 ms delay: 25 MiB 0.145 ms, 100 MiB 0.274, 1 GiB 1.79,
// against 0.137 / 0.319 / 2.58 for NCCL and 2.21 for the faithful schedule at 1 GiB).  With nobody declared late the
// pre-phase would be on the critical path (1 GiB: 4.66 ms), so the one-shot reduce-scatter + all-gather serves up to
// 512 MiB (1 / 4 / 25 / 100 MiB: 0.068 / 0.075 / 0.134 / 0.326 ms on symmetric tensors) and the ring above, where
// the two are level (2.86 / 2.85 ms at 1 GiB).
std::string ProcessGroupStragglar::algorithm_for(size_t bytes) const {
  if (opts_.alg != "auto") return opts_.alg;
  const int n = getSize();
  if (opts_.straggler >= 0 && n >= 2 && n % 2 == 0) return "stragglar_a2a";
  return bytes < (512ull << 20) ? "rsag" : "ring";
}

const sar::Program& ProcessGroupStragglar::program(size_t bytes) {
  std::string alg = algorithm_for(bytes);
  static const char* const kKnown[] = {"stragglar", "stragglar_a2a", "ring", "rhd", "direct", "rsag"};
  bool known = false;
  for (const char* k : kKnown) known = known || alg == k;
  TORCH_CHECK(known, "stragglar backend: unknown algorithm '", alg,
              "' (stragglar, stragglar_a2a, ring, rhd, direct, rsag or auto)");
  const std::string key = alg + "/" + std::to_string(opts_.straggler);
  auto it = programs_.find(key);
  if (it != programs_.end()) return it->second;
  sar::Schedule sched;
  const sar::Schedule* sp = nullptr;
  if (!opts_.schedule_text.empty()) { sched = sar::parse_schedule(opts_.schedule_text); sp = &sched; }
  try {
    return programs_.emplace(key, sar::build_program(alg, getSize(), true, opts_.straggler, sp)).first->second;
  } catch (const std::exception& e) {
    // StragglAR schedules exist for even rank counts (and halving-doubling for powers of two);
    // a group of another size, e.g. a sub-group of three ranks, is served by the ring instead
    if (alg != "ring" && opts_.schedule_text.empty()) {
      try {
        auto& p = programs_.emplace(key, sar::build_program("ring", getSize(), true, opts_.straggler, nullptr)).first->second;
        TORCH_WARN_ONCE("stragglar backend: '", alg, "' is not available for ", getSize(), " ranks (", e.what(),
                        "); using ring for this group");
        return p;
      } catch (const std::exception&) {
      }
    }
    TORCH_CHECK(false, "stragglar backend: cannot build '", alg, "' for ", getSize(), " ranks: ", e.what());
  }
}

void ProcessGroupStragglar::set_straggler(int r) {
  TORCH_CHECK(r >= -1 && r < getSize(), "straggler rank out of range");
  std::lock_guard<std::mutex> lk(mu_);
  const int old = opts_.straggler;
  opts_.straggler = r;
  try { (void)program(); } catch (...) { opts_.straggler = old; throw; }
}
void ProcessGroupStragglar::set_algorithm(const std::string& alg) {
  std::lock_guard<std::mutex> lk(mu_);   // collectives read the options and the program cache under this lock
  const std::string old = opts_.alg;
  opts_.alg = alg;
  try { (void)program(); } catch (...) { opts_.alg = old; throw; }
}

ProcessGroupStragglar::Side& ProcessGroupStragglar::side(const at::Tensor& like) {
  return side(like.is_cuda(), like.is_cuda() ? like.get_device() : -1);
}

ProcessGroupStragglar::Side& ProcessGroupStragglar::side(bool cuda, int device) {
  Side& s = cuda ? cuda_ : cpu_;
  if (s.t) {
    TORCH_CHECK(!cuda || s.device == device, "stragglar backend is bound to cuda:", s.device, ", got a tensor on cuda:", device);
    return s;
  }
  size_t arena = opts_.arena_bytes ? opts_.arena_bytes : env_mb(cuda ? "STRAGGLAR_ARENA_MB" : "STRAGGLAR_CPU_ARENA_MB", cuda ? 1024 : 64);
  size_t staging = opts_.staging_bytes ? opts_.staging_bytes : env_mb("STRAGGLAR_STAGING_MB", 0);
  if (!staging) staging = cuda ? std::min<size_t>(arena / 4, (size_t)256 << 20) : arena / 2;
  s.device = device;
  s.t = std::make_unique<Transport>(cuda, device, getRank(), getSize(), arena, staging, store_, prefix_ + (cuda ? "/cuda" : "/cpu"));
  if (cuda) {
    s.stream = c10::cuda::getStreamFromPool(/*isHighPriority=*/true, (c10::DeviceIndex)device);
    s.fail = std::make_shared<FailureState>();
    s.fail->word = s.t->status_owner();
  }
  return s;
}

c10::intrusive_ptr<WorkStragglar> ProcessGroupStragglar::begin(Side& s, c10d::OpType op, std::vector<at::Tensor> outputs) {
  recover_if_failed(s);
  auto w = c10::make_intrusive<WorkStragglar>(getRank(), op, std::move(outputs), s.t->cuda());
  w->fail_ = s.fail;
  if (s.t->cuda()) {
    // the communication stream picks up after whatever the caller has queued
    at::cuda::CUDAEvent ready;
    ready.record(c10::cuda::getCurrentCUDAStream((c10::DeviceIndex)s.device));
    ready.block(*s.stream);
    SAR_CUDA_CHECK(cudaSetDevice(s.device));
  }
  return w;
}

void ProcessGroupStragglar::finish(Side& s, const c10::intrusive_ptr<WorkStragglar>& w) {
  if (s.t->cuda()) {
    w->end_ = std::make_shared<at::cuda::CUDAEvent>();
    w->end_->record(*s.stream);
    for (auto& t : w->outputs_)
      if (t.defined() && t.is_cuda()) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), *s.stream);
    c10::cuda::CUDAStreamGuard g(*s.stream);
    w->future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()),
                                                          std::vector<c10::Device>{c10::Device(c10::kCUDA, (c10::DeviceIndex)s.device)});
    w->future_->markCompleted(at::IValue(w->outputs_));
  } else {
    w->future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
    w->future_->markCompleted(at::IValue(w->outputs_));
  }
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::failed(Side& s, const c10::intrusive_ptr<WorkStragglar>& w) {
  if (s.t->cuda()) throw;   // CUDA launches fail for host-side reasons only (bad arguments): raise at once
  w->error_ = std::current_exception();
  w->future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
  w->future_->setError(w->error_);
  return w;
}

void ProcessGroupStragglar::clear_failure(Side& s) {
  SAR_CUDA_CHECK(cudaSetDevice(s.device));
  SAR_CUDA_CHECK(cudaStreamSynchronize(s.stream->stream()));   // every block of the failed launch has returned
  *(volatile uint32_t*)s.t->status() = 0;
  for (int ch = 0; ch < SAR_NUM_CHANNELS; ++ch) {
    SAR_CUDA_CHECK(cudaMemset(&s.t->ctrl(getRank(), ch)->abort_flag, 0, 4));
    SAR_CUDA_CHECK(cudaMemset(&s.t->ctrl(getRank(), ch)->blocks_done, 0, 4));
    SAR_CUDA_CHECK(cudaMemset(&s.t->ctrl(getRank(), ch)->items_done, 0, 8));
  }
}

void ProcessGroupStragglar::recover_if_failed(Side& s) {
  if (!s.t || !s.t->cuda() || !s.fail) return;
  const uint32_t st = *(volatile uint32_t*)s.t->status();
  if (!st) return;
  clear_failure(s);
  if (s.fail->reported.exchange(false)) return;   // a Work has raised for it already
  TORCH_CHECK(false, "stragglar backend: an earlier collective failed on rank ", getRank(), ": ", sar_status_string(st),
              " (a device-side wait ran out; its result is incomplete)");
}

void ProcessGroupStragglar::copy_local(Side& s, void* dst, const void* src, size_t bytes) {
  if (!bytes || dst == src) return;
  if (s.t->cuda()) SAR_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s.stream->stream()));
  else memcpy(dst, src, bytes);
}

void ProcessGroupStragglar::pull(Side& s, const std::vector<std::tuple<int, size_t, void*, size_t>>& segs) {
  Transport& t = *s.t;
  if (t.cuda()) {
    std::vector<SarCopySeg> v;
    for (auto& g : segs) {
      if (!std::get<3>(g)) continue;
      v.push_back(SarCopySeg{t.data(std::get<0>(g)) + std::get<1>(g), std::get<2>(g), std::get<3>(g)});
      if ((int)v.size() == SAR_MAX_RANKS) { SAR_CUDA_CHECK(sar_cuda_copy_segments(v.data(), (int)v.size(), s.stream->stream())); ++launches_; v.clear(); }
    }
    if (!v.empty()) { SAR_CUDA_CHECK(sar_cuda_copy_segments(v.data(), (int)v.size(), s.stream->stream())); ++launches_; }
  } else {
    for (auto& g : segs) memcpy(std::get<2>(g), t.data(std::get<0>(g)) + std::get<1>(g), std::get<3>(g));
  }
}

void ProcessGroupStragglar::device_barrier(Side& s) {
  Transport& t = *s.t;
  const int n = getSize(), me = getRank();
  const uint32_t ep = t.next_barrier_epoch();
  if (n == 1) return;
  if (t.cuda()) {
    SarCtrl* ctrl[SAR_MAX_RANKS];
    for (int r = 0; r < n; ++r) ctrl[r] = t.ctrl(r, kBarrierChannel);
    SAR_CUDA_CHECK(sar_cuda_barrier(ctrl, me, n, (n >= 32 ? 0xffffffffu : (1u << n) - 1u), ep, (uint64_t)(opts_.timeout_s * 1e9), t.status(), s.stream->stream()));
    ++launches_;
  } else {
    std::atomic_thread_fence(std::memory_order_seq_cst);
    as_atomic(&t.ctrl(me, kBarrierChannel)->arrival)->store(ep, std::memory_order_release);
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(opts_.timeout_s);
    for (int r = 0; r < n; ++r) {
      if (r == me) continue;
      unsigned spins = 0;
      while (!sar_reached(as_atomic(&t.ctrl(r, kBarrierChannel)->arrival)->load(std::memory_order_acquire), ep)) {
        if ((++spins & 255) == 0) {
          TORCH_CHECK(std::chrono::steady_clock::now() < deadline, "stragglar backend: barrier timed out waiting for rank ", r);
          std::this_thread::yield();
        }
      }
    }
  }
}

void ProcessGroupStragglar::run_program(Side& s, const sar::Program& prog, size_t data_off, uint64_t count,
                                        at::ScalarType dtype, float scale, void* user, int user_dtype) {
  Transport& t = *s.t;
  const int n = getSize(), me = getRank();
  const int dt = dtype_code(dtype);
  const uint32_t esize = dt == SAR_F32 ? 4 : 2;
  for (const sar::Compiled& c : prog.phases) {
    const uint64_t epoch64 = t.next_epoch(c.channel);   // every rank counts, participant or not
    const uint32_t epoch = (uint32_t)epoch64;
    if (!(c.participants >> me & 1)) continue;
    int blocks = t.cuda() ? (opts_.blocks > 0 ? opts_.blocks : sar_cuda_pick_blocks(opts_.path, count * esize)) : 1;
    if (t.cuda() && opts_.blocks <= 0 && c.blocks_hint > 0 && c.blocks_hint < blocks) blocks = c.blocks_hint;
    if (t.cuda() && opts_.blocks <= 0 && n == 1 && blocks == 128) blocks = 148;   // a lone rank: one block per SM
    const bool gated = c.gate_rounds && count * esize >= sar::gate_min_bytes();
    // staged launches poll a flag over the link for every tile they read from a peer, version 0 included: larger tiles
    const uint32_t tile_max = opts_.tile_bytes ? opts_.tile_bytes
                            : (t.cuda() ? ((gated || user) ? sar::gate_tile_bytes() : sar_cuda_default_tile_bytes(opts_.path)) : (128u << 10));
    const uint32_t tile_elems = sar::pick_tile_elems(count, esize, (uint32_t)c.num_chunks, (uint32_t)blocks, 2048, tile_max);
    const SarGeom g = sar::make_geom(count, esize, (uint32_t)c.num_chunks, tile_elems);
    TORCH_CHECK((uint64_t)g.tiles_per_chunk * g.num_chunks <= SAR_FLAG_CAPACITY, "tensor too large for the flag array");
    const sar::RankTable& rt = c.ranks[me];
    if (t.cuda()) {
      auto key = std::make_pair((const void*)&c, me);
      auto it = s.uploaded.find(key);
      if (it == s.uploaded.end()) {
        const std::string why = sar::validate_rank_table(rt, me, n, c.num_chunks);
        TORCH_CHECK(why.empty(), "stragglar backend: refusing to launch a malformed table: ", why);
        void *d_ops = nullptr, *d_rb = nullptr;
        SAR_CUDA_CHECK(cudaMalloc(&d_ops, std::max<size_t>(1, rt.ops.size()) * sizeof(SarOp)));
        SAR_CUDA_CHECK(cudaMalloc(&d_rb, std::max<size_t>(1, rt.round_begin.size()) * sizeof(uint16_t)));
        if (!rt.ops.empty()) SAR_CUDA_CHECK(cudaMemcpy(d_ops, rt.ops.data(), rt.ops.size() * sizeof(SarOp), cudaMemcpyHostToDevice));
        if (!rt.round_begin.empty()) SAR_CUDA_CHECK(cudaMemcpy(d_rb, rt.round_begin.data(), rt.round_begin.size() * sizeof(uint16_t), cudaMemcpyHostToDevice));
        it = s.uploaded.emplace(key, std::make_pair(d_ops, d_rb)).first;
      }
      SarLaunchParams P;
      memset(&P, 0, sizeof P);
      for (int r = 0; r < n; ++r) {
        P.comm.flags[r] = t.flags(r, c.channel);
        P.comm.ctrl[r] = t.ctrl(r, c.channel);
        P.comm.buf[r] = t.data(r) + data_off;
      }
      P.ops = (const SarOp*)it->second.first;
      P.round_begin = (const uint16_t*)it->second.second;
      P.num_rounds = rt.round_begin.empty() ? 0 : (uint32_t)rt.round_begin.size() - 1;
      P.geom = g; P.rank = me; P.nranks = n; P.participants = c.participants;
      P.epoch_base = epoch; P.scale = scale; P.dtype = dt;
      P.timeout_ns = (uint64_t)(opts_.timeout_s * 1e9);
      P.status = t.status(); P.trace = t.trace_words(); P.delay_ns = 0;
      if (user) {
        // staged mode: the kernel copies the caller's tensor in and out itself (see sar_params.h)
        P.user_in = user; P.user_out = user; P.user_dtype = user_dtype;
        for (size_t ch = 0; ch < rt.final_ver.size() && ch < SAR_MAX_CHUNKS; ++ch) P.final_ver[ch] = rt.final_ver[ch];
      }
      P.gate_rounds = gated ? 1u : 0u;
      P.gate_base = epoch64; P.gate_slack = sar::gate_slack(g.tiles_per_chunk);
      P.stages = (uint32_t)c.stages_hint;
      P.lane1_eighths = (uint32_t)c.lane1_eighths;
      int launch_blocks = blocks;
      if (user) {
        // staging blocks on top of the table's: local copies need many blocks to run at memory speed
        const int extra = std::max(1, std::min(64, 144 - blocks));
        P.staging_blocks = (uint32_t)extra;
        launch_blocks = blocks + extra;
      }
      SAR_CUDA_CHECK(sar_cuda_launch(&P, opts_.path, launch_blocks, opts_.threads, s.stream->stream()));
      ++launches_;
    } else {
      sar::HostRankView v;
      v.rank = me; v.nranks = n;
      for (int r = 0; r < n; ++r) {
        v.buf[r] = t.data(r) + data_off;
        v.flags[r] = as_atomic(t.flags(r, c.channel));
        v.ctrl[r] = as_atomic(reinterpret_cast<uint32_t*>(t.ctrl(r, c.channel)));
      }
      sar::HostLaunch l;
      l.geom = g; l.dtype = (SarDtype)dt; l.scale = scale; l.epoch_base = epoch; l.timeout_s = opts_.timeout_s;
      l.participants = c.participants;
      l.gate_rounds = gated;
      l.gate_base = epoch64; l.gate_slack = sar::gate_slack(g.tiles_per_chunk);
      l.lane1_eighths = (uint32_t)c.lane1_eighths;
      const uint32_t st = sar::host_run_block(v, rt, l, 0, 1);
      if (st != SAR_OK) {
        as_atomic(&t.ctrl(me, c.channel)->abort_flag)->store(0);
        as_atomic(&t.ctrl(me, c.channel)->blocks_done)->store(0);
        TORCH_CHECK(false, "stragglar backend: collective failed on rank ", me, " (status ", st, ")");
      }
    }
  }
}

int64_t ProcessGroupStragglar::check_status(bool cuda) {
  Side& s = cuda ? cuda_ : cpu_;
  if (!s.t || !cuda) return 0;
  SAR_CUDA_CHECK(cudaSetDevice(s.device));
  SAR_CUDA_CHECK(cudaStreamSynchronize(s.stream->stream()));
  const uint32_t st = *(volatile uint32_t*)s.t->status();
  if (st) { clear_failure(s); s.fail->reported.store(false); }
  return st;
}

bool ProcessGroupStragglar::check_guards(bool cuda) {
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = cuda ? cuda_ : cpu_;
  return !s.t || s.t->check_guards();
}

std::pair<int64_t, int64_t> ProcessGroupStragglar::last_trace() {
  Side& s = cuda_;
  if (!s.t) return {0, 0};
  SAR_CUDA_CHECK(cudaSetDevice(s.device));
  SAR_CUDA_CHECK(cudaStreamSynchronize(s.stream->stream()));
  uint64_t v[2] = {0, 0};
  SAR_CUDA_CHECK(cudaMemcpy(v, s.t->trace_words(), 16, cudaMemcpyDeviceToHost));
  return {(int64_t)v[0], (int64_t)v[1]};
}

// The in-place path hands the kernel this rank's heap offset for every peer, and the staged path waits for tile
// flags where the in-place path waits for arrival words: ranks that pass different kinds of tensors (or different
// sizes) to one collective compute garbage or time out.  With check_args every rank publishes what it was given and
// compares it with everybody else's before anything is launched.
void ProcessGroupStragglar::check_same_arguments(uint64_t count, int tensor_dtype, int comm_dtype, int64_t heap_off) {
  const int n = getSize(), me = getRank();
  if (n == 1) return;
  const uint64_t seq = check_seq_++;
  const std::string mine = std::to_string(count) + "/" + std::to_string(tensor_dtype) + "/" + std::to_string(comm_dtype) +
                           "/" + (heap_off >= 0 ? "symmetric@" + std::to_string(heap_off) : std::string("ordinary"));
  const std::string base = prefix_ + "/chk/" + std::to_string(seq) + "/";
  store_->set(base + std::to_string(me), std::vector<uint8_t>(mine.begin(), mine.end()));
  for (int r = 0; r < n; ++r) {
    if (r == me) continue;
    auto v = store_->get(base + std::to_string(r));
    const std::string theirs(v.begin(), v.end());
    TORCH_CHECK(theirs == mine, "stragglar backend: ranks passed different arguments to one AllReduce (count/tensor dtype/"
                "wire dtype/placement): rank ", me, " has ", mine, ", rank ", r, " has ", theirs,
                ". Every rank must pass a tensor of the same size and kind (the same symmetric allocation at the same "
                "offset, or an ordinary tensor everywhere).");
  }
}

// ------------------------------------------------------------------- allreduce
void ProcessGroupStragglar::allreduce_impl(Side& s, at::Tensor& tensor, float scale, std::optional<at::ScalarType> comm_dtype) {
  Transport& t = *s.t;
  const at::ScalarType tdt = tensor.scalar_type();
  const at::ScalarType cdt = comm_dtype.value_or(tdt);
  (void)dtype_code(tdt);
  const int cdc = dtype_code(cdt);
  const uint64_t count = (uint64_t)tensor.numel();
  if (count == 0) return;
  const size_t csize = cdc == SAR_F32 ? 4 : 2;
  const sar::Program& prog = program(count * csize);
  char* ptr = (char*)tensor.data_ptr();
  const int64_t hoff = (cdt == tdt) ? t.heap_offset(ptr, count * csize) : -1;
  if (opts_.check_args) check_same_arguments(count, dtype_code(tdt), cdc, (hoff >= 0 && (((uintptr_t)ptr) & 15) == 0) ? hoff : -1);
  if (hoff >= 0 && (((uintptr_t)ptr) & 15) == 0) {
    run_program(s, prog, (size_t)hoff, count, cdt, scale);   // in place, no staging
    return;
  }
  const size_t tsize = tensor.element_size();
  uint64_t piece = t.staging_bytes() / csize;
  piece = piece / 256 * 256;
  TORCH_CHECK(piece > 0, "staging area too small");
  char* stage = t.data(getRank()) + t.staging_off();
  if (t.cuda() && prog.phases.size() == 1) {
    // Any other CUDA tensor (a DDP bucket, say): the staging area only serves the peers.  One kernel per piece
    // copies the tensor in tile by tile (casting to the communication dtype), reduces, and copies every finished
    // tile back (casting again); no separate copy or cast launches.  Every rank must pass the same kind of tensor.
    for (uint64_t off = 0; off < count; off += piece) {
      const uint64_t k = std::min<uint64_t>(piece, count - off);
      run_program(s, prog, t.staging_off(), k, cdt, scale, ptr + off * tsize, dtype_code(tdt));
    }
    return;
  }
  for (uint64_t off = 0; off < count; off += piece) {
    const uint64_t k = std::min<uint64_t>(piece, count - off);
    if (cdt == tdt) copy_local(s, stage, ptr + off * tsize, k * tsize);
    else if (t.cuda()) { SAR_CUDA_CHECK(sar_cuda_scale_cast(stage, cdc, ptr + off * tsize, dtype_code(tdt), k, 1.0f, s.stream->stream())); ++launches_; }
    else {
      at::Tensor src = tensor.view({-1}).narrow(0, (int64_t)off, (int64_t)k);
      at::Tensor dst = at::from_blob(stage, {(int64_t)k}, at::TensorOptions().dtype(cdt));
      dst.copy_(src);
    }
    run_program(s, prog, t.staging_off(), k, cdt, scale);
    if (cdt == tdt) copy_local(s, ptr + off * tsize, stage, k * tsize);
    else if (t.cuda()) { SAR_CUDA_CHECK(sar_cuda_scale_cast(ptr + off * tsize, dtype_code(tdt), stage, cdc, k, 1.0f, s.stream->stream())); ++launches_; }
    else {
      at::Tensor dst = tensor.view({-1}).narrow(0, (int64_t)off, (int64_t)k);
      at::Tensor src = at::from_blob(stage, {(int64_t)k}, at::TensorOptions().dtype(cdt));
      dst.copy_(src);
    }
  }
}

// what the table kernels reduce themselves; everything else takes allreduce_generic
static bool table_dtype(at::ScalarType t) { return t == at::kFloat || t == at::kBFloat16 || t == at::kHalf; }
static bool table_op(const c10d::ReduceOp& op) { return op == c10d::ReduceOp::SUM || op == c10d::ReduceOp::AVG; }

static float scale_for(const c10d::ReduceOp& op, int n) {
  if (op == c10d::ReduceOp::SUM) return 1.0f;
  if (op == c10d::ReduceOp::AVG) return 1.0f / (float)n;
  TORCH_CHECK(false, "stragglar backend supports ReduceOp.SUM and ReduceOp.AVG");
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::allreduce(std::vector<at::Tensor>& tensors, const c10d::AllreduceOptions& opts) {
  NvtxRange nvtx_range("stragglar::allreduce");
  TORCH_CHECK(tensors.size() == 1, "stragglar backend takes one tensor per rank");
  check_contiguous(tensors[0]);
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(tensors[0]);
  auto w = begin(s, c10d::OpType::ALLREDUCE, tensors);
  try {
    if (table_dtype(tensors[0].scalar_type()) && table_op(opts.reduceOp))
      allreduce_impl(s, tensors[0], scale_for(opts.reduceOp, getSize()), std::nullopt);
    else
      allreduce_generic(s, tensors[0], opts.reduceOp);
  } catch (const std::exception&) {
    return failed(s, w);
  }
  finish(s, w);
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::allreduce_ex(at::Tensor& tensor, bool average, std::optional<at::ScalarType> comm_dtype) {
  NvtxRange nvtx_range("stragglar::allreduce_ex");
  check_contiguous(tensor);
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(tensor);
  auto w = begin(s, c10d::OpType::ALLREDUCE, {tensor});
  try {
    allreduce_impl(s, tensor, average ? 1.0f / (float)getSize() : 1.0f, comm_dtype);
  } catch (const std::exception&) {
    return failed(s, w);
  }
  finish(s, w);
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::allreduce_coalesced(std::vector<at::Tensor>& tensors, const c10d::AllreduceCoalescedOptions& opts) {
  TORCH_CHECK(!tensors.empty(), "no tensors");
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(tensors[0]);
  auto w = begin(s, c10d::OpType::ALLREDUCE_COALESCED, tensors);
  for (auto& t : tensors) {
    check_contiguous(t);
    if (table_dtype(t.scalar_type()) && table_op(opts.reduceOp)) allreduce_impl(s, t, scale_for(opts.reduceOp, getSize()), std::nullopt);
    else allreduce_generic(s, t, opts.reduceOp);
  }
  finish(s, w);
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& opts) {
  TORCH_CHECK(tensors.size() == 1, "stragglar backend takes one tensor per rank");
  check_contiguous(tensors[0]);
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(tensors[0]);
  auto w = begin(s, c10d::OpType::REDUCE, tensors);
  if (!(table_dtype(tensors[0].scalar_type()) && table_op(opts.reduceOp))) {
    // the gather-based path reduces on every rank; only the root keeps the result
    std::optional<c10::cuda::CUDAStreamGuard> guard;
    if (s.t->cuda()) guard.emplace(*s.stream);     // the scratch copy is made (and lives) on the communication stream
    at::Tensor x = getRank() == opts.rootRank ? tensors[0] : tensors[0].clone();
    allreduce_generic(s, x, opts.reduceOp);
    finish(s, w);
    return w;
  }
  // everybody computes the sum on a staged copy; only the root keeps it
  Transport& t = *s.t;
  at::Tensor& x = tensors[0];
  const size_t es = x.element_size();
  uint64_t piece = t.staging_bytes() / es / 256 * 256;
  TORCH_CHECK(piece > 0, "staging area too small");
  char* stage = t.data(getRank()) + t.staging_off();
  const float scale = scale_for(opts.reduceOp, getSize());
  for (uint64_t off = 0; off < (uint64_t)x.numel(); off += piece) {
    const uint64_t k = std::min<uint64_t>(piece, x.numel() - off);
    copy_local(s, stage, (char*)x.data_ptr() + off * es, k * es);
    run_program(s, program((size_t)x.numel() * es), t.staging_off(), k, x.scalar_type(), scale);
    if (getRank() == opts.rootRank) copy_local(s, (char*)x.data_ptr() + off * es, stage, k * es);
  }
  finish(s, w);
  return w;
}

// --------------------------------------------------- staged data-movement ops
c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::broadcast(std::vector<at::Tensor>& tensors, const c10d::BroadcastOptions& opts) {
  NvtxRange nvtx_range("stragglar::broadcast");
  TORCH_CHECK(tensors.size() == 1, "stragglar backend takes one tensor per rank");
  check_contiguous(tensors[0]);
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(tensors[0]);
  auto w = begin(s, c10d::OpType::BROADCAST, tensors);
  Transport& t = *s.t;
  const int root = (int)opts.rootRank;
  char* p = (char*)tensors[0].data_ptr();
  const size_t bytes = tensors[0].nbytes(), piece = t.staging_bytes();
  for (size_t off = 0; off < bytes; off += piece) {
    const size_t k = std::min(piece, bytes - off);
    if (getRank() == root) copy_local(s, t.data(root) + t.staging_off(), p + off, k);
    device_barrier(s);
    if (getRank() != root) pull(s, {{root, t.staging_off(), p + off, k}});
    device_barrier(s);
  }
  finish(s, w);
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::_allgather_base(at::Tensor& output, at::Tensor& input, const c10d::AllgatherOptions&) {
  NvtxRange nvtx_range("stragglar::allgather");
  check_contiguous(output); check_contiguous(input);
  const int n = getSize();
  TORCH_CHECK(output.nbytes() == input.nbytes() * n, "all_gather output must be world_size times the input");
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(input);
  auto w = begin(s, c10d::OpType::_ALLGATHER_BASE, {output});
  gather_all(s, output.data_ptr(), input.data_ptr(), input.nbytes());
  finish(s, w);
  return w;
}

// out[r * bytes ...] = rank r's `in`, on every rank, through the staging area
void ProcessGroupStragglar::gather_all(Side& s, void* out, const void* in, size_t bytes) {
  Transport& t = *s.t;
  const int n = getSize();
  const size_t piece = t.staging_bytes();
  for (size_t off = 0; off < bytes || (bytes == 0 && off == 0); off += piece) {
    const size_t k = std::min(piece, bytes - off);
    copy_local(s, t.data(getRank()) + t.staging_off(), (const char*)in + off, k);
    device_barrier(s);
    std::vector<std::tuple<int, size_t, void*, size_t>> segs;
    for (int r = 0; r < n; ++r) segs.push_back({r, t.staging_off(), (char*)out + (size_t)r * bytes + off, k});
    pull(s, segs);
    device_barrier(s);
    if (bytes == 0) break;
  }
}

// What the table kernels do not cover -- integer, fp64 and bool tensors, MIN / MAX / PRODUCT and
// the bitwise operations: every rank gathers all contributions and reduces them itself with
// ATen, on the communication stream.  Meant for the small control tensors frameworks
// all-reduce besides the gradients (DDP's bitmap of unused parameters, found-inf flags,
// counters); the bytes on the wire are world_size times those of a real all-reduce.

void ProcessGroupStragglar::allreduce_generic(Side& s, at::Tensor& tensor, const c10d::ReduceOp& op) {
  const int n = getSize();
  const int64_t numel = tensor.numel();
  if (numel == 0) return;
  std::optional<c10::cuda::CUDAStreamGuard> guard;
  if (s.t->cuda()) guard.emplace(*s.stream);      // allocation and the ATen kernels below on the communication stream
  at::Tensor all = at::empty({(int64_t)n, numel}, tensor.options());
  gather_all(s, all.data_ptr(), tensor.data_ptr(), tensor.nbytes());
  at::Tensor flat = tensor.view({-1});
  at::Tensor r;
  if (op == c10d::ReduceOp::SUM) r = all.sum(0, false, tensor.scalar_type());
  else if (op == c10d::ReduceOp::AVG) {
    TORCH_CHECK(at::isFloatingType(tensor.scalar_type()), "ReduceOp.AVG needs a floating-point tensor");
    r = all.sum(0) / (double)n;
  } else if (op == c10d::ReduceOp::MIN) r = all.amin(0);
  else if (op == c10d::ReduceOp::MAX) r = all.amax(0);
  else if (op == c10d::ReduceOp::PRODUCT) r = all.prod(0, false, tensor.scalar_type());
  else if (op == c10d::ReduceOp::BAND || op == c10d::ReduceOp::BOR || op == c10d::ReduceOp::BXOR) {
    TORCH_CHECK(at::isIntegralType(tensor.scalar_type(), /*includeBool=*/true), "bitwise reductions need an integer tensor");
    r = all[0].clone();
    for (int k = 1; k < n; ++k) {
      if (op == c10d::ReduceOp::BAND) r.bitwise_and_(all[k]);
      else if (op == c10d::ReduceOp::BOR) r.bitwise_or_(all[k]);
      else r.bitwise_xor_(all[k]);
    }
  } else {
    TORCH_CHECK(false, "stragglar backend: unsupported ReduceOp");
  }
  flat.copy_(r.to(tensor.scalar_type()));
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::allgather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs, const c10d::AllgatherOptions& opts) {
  TORCH_CHECK(inputs.size() == 1 && outputs.size() == 1, "stragglar backend takes one tensor per rank");
  const int n = getSize();
  TORCH_CHECK((int)outputs[0].size() == n, "all_gather needs world_size output tensors");
  check_contiguous(inputs[0]);
  at::Tensor flat = at::empty({(int64_t)n * inputs[0].numel()}, inputs[0].options());
  auto w = _allgather_base(flat, inputs[0], opts);
  // the copies into the caller's tensors are ordered after the gather on the communication stream
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(inputs[0]);
  for (int r = 0; r < n; ++r) {
    check_contiguous(outputs[0][r]);
    TORCH_CHECK(outputs[0][r].nbytes() == inputs[0].nbytes(), "all_gather tensors must have one size");
    copy_local(s, outputs[0][r].data_ptr(), (char*)flat.data_ptr() + (size_t)r * inputs[0].nbytes(), inputs[0].nbytes());
  }
  auto w2 = c10::make_intrusive<WorkStragglar>(getRank(), c10d::OpType::ALLGATHER, outputs[0], s.t->cuda());
  if (s.t->cuda()) c10::cuda::CUDACachingAllocator::recordStream(flat.storage().data_ptr(), *s.stream);
  finish(s, w2);
  return w2;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::allgather_into_tensor_coalesced(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs, const c10d::AllgatherOptions& opts) {
  TORCH_CHECK(outputs.size() == inputs.size(), "size mismatch");
  c10::intrusive_ptr<c10d::Work> w;
  for (size_t i = 0; i < inputs.size(); ++i) w = _allgather_base(outputs[i], inputs[i], opts);
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::_reduce_scatter_base(at::Tensor& output, at::Tensor& input, const c10d::ReduceScatterOptions& opts) {
  NvtxRange nvtx_range("stragglar::reduce_scatter");
  check_contiguous(output); check_contiguous(input);
  const int n = getSize(), me = getRank();
  TORCH_CHECK(input.numel() == output.numel() * n, "reduce_scatter input must be world_size times the output");
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(input);
  auto w = begin(s, c10d::OpType::_REDUCE_SCATTER_BASE, {output});
  Transport& t = *s.t;
  const int dt = dtype_code(input.scalar_type());
  const size_t es = input.element_size();
  const float scale = scale_for(opts.reduceOp, n);
  const uint64_t per = (uint64_t)output.numel();
  uint64_t piece = t.staging_bytes() / es / (uint64_t)n / 64 * 64;   // elements per rank-slot per pass
  TORCH_CHECK(piece > 0, "staging area too small");
  for (uint64_t off = 0; off < per; off += piece) {
    const uint64_t k = std::min<uint64_t>(piece, per - off);
    for (int q = 0; q < n; ++q)
      copy_local(s, t.data(me) + t.staging_off() + (size_t)q * piece * es, (char*)input.data_ptr() + ((size_t)q * per + off) * es, k * es);
    device_barrier(s);
    if (t.cuda()) {
      const void* srcs[SAR_MAX_RANKS];
      for (int p = 0; p < n; ++p) srcs[p] = t.data(p) + t.staging_off() + (size_t)me * piece * es;
      SAR_CUDA_CHECK(sar_cuda_reduce_segments((char*)output.data_ptr() + off * es, srcs, n, k, dt, scale, s.stream->stream()));
      ++launches_;
    } else {
      at::Tensor acc = at::zeros({(int64_t)k}, at::TensorOptions().dtype(at::kFloat));
      for (int p = 0; p < n; ++p)
        acc += at::from_blob(t.data(p) + t.staging_off() + (size_t)me * piece * es, {(int64_t)k}, input.options().device(at::kCPU)).to(at::kFloat);
      output.view({-1}).narrow(0, (int64_t)off, (int64_t)k).copy_(acc * scale);
    }
    device_barrier(s);
  }
  finish(s, w);
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::reduce_scatter(std::vector<at::Tensor>& outputs, std::vector<std::vector<at::Tensor>>& inputs, const c10d::ReduceScatterOptions& opts) {
  TORCH_CHECK(outputs.size() == 1 && inputs.size() == 1, "stragglar backend takes one tensor per rank");
  TORCH_CHECK((int)inputs[0].size() == getSize(), "reduce_scatter needs world_size input tensors");
  at::Tensor flat = at::cat(inputs[0]).contiguous();
  if (flat.is_cuda()) {
    // at::cat ran on the current stream; begin() orders the communication stream after it
  }
  auto w = _reduce_scatter_base(outputs[0], flat, opts);
  if (flat.is_cuda()) c10::cuda::CUDACachingAllocator::recordStream(flat.storage().data_ptr(), *cuda_.stream);
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs, const c10d::ReduceScatterOptions& opts) {
  TORCH_CHECK(outputs.size() == inputs.size() && !inputs.empty(), "size mismatch");
  c10::intrusive_ptr<c10d::Work> w;
  for (size_t i = 0; i < inputs.size(); ++i) w = _reduce_scatter_base(outputs[i], inputs[i], opts);
  return w;   // the operations run in order on the communication stream: the last one's completion covers all
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::allgather_coalesced(std::vector<std::vector<at::Tensor>>& output_lists, std::vector<at::Tensor>& inputs, const c10d::AllgatherOptions& opts) {
  TORCH_CHECK(output_lists.size() == inputs.size() && !inputs.empty(), "size mismatch");
  c10::intrusive_ptr<c10d::Work> w;
  for (size_t i = 0; i < inputs.size(); ++i) {
    std::vector<std::vector<at::Tensor>> outs{output_lists[i]};
    std::vector<at::Tensor> in{inputs[i]};
    w = allgather(outs, in, opts);
  }
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::gather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs, const c10d::GatherOptions& opts) {
  TORCH_CHECK(inputs.size() == 1, "stragglar backend takes one tensor per rank");
  check_contiguous(inputs[0]);
  const int n = getSize(), me = getRank(), root = (int)opts.rootRank;
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(inputs[0]);
  Transport& t = *s.t;
  const size_t bytes = inputs[0].nbytes();
  TORCH_CHECK(bytes <= t.staging_bytes(), "gather: tensor larger than the staging area");
  auto w = begin(s, c10d::OpType::GATHER, me == root ? outputs[0] : std::vector<at::Tensor>{});
  copy_local(s, t.data(me) + t.staging_off(), inputs[0].data_ptr(), bytes);
  device_barrier(s);
  if (me == root) {
    TORCH_CHECK(outputs.size() == 1 && (int)outputs[0].size() == n, "gather needs world_size output tensors on the root");
    std::vector<std::tuple<int, size_t, void*, size_t>> segs;
    for (int r = 0; r < n; ++r) { check_contiguous(outputs[0][r]); segs.push_back({r, t.staging_off(), outputs[0][r].data_ptr(), bytes}); }
    pull(s, segs);
  }
  device_barrier(s);
  finish(s, w);
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::scatter(std::vector<at::Tensor>& outputs, std::vector<std::vector<at::Tensor>>& inputs, const c10d::ScatterOptions& opts) {
  TORCH_CHECK(outputs.size() == 1, "stragglar backend takes one tensor per rank");
  check_contiguous(outputs[0]);
  const int n = getSize(), me = getRank(), root = (int)opts.rootRank;
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(outputs[0]);
  Transport& t = *s.t;
  const size_t bytes = outputs[0].nbytes();
  const size_t slot = t.staging_bytes() / n / 256 * 256;
  TORCH_CHECK(bytes <= slot, "scatter: tensor larger than a staging slot");
  auto w = begin(s, c10d::OpType::SCATTER, outputs);
  if (me == root) {
    TORCH_CHECK(inputs.size() == 1 && (int)inputs[0].size() == n, "scatter needs world_size input tensors on the root");
    for (int r = 0; r < n; ++r) { check_contiguous(inputs[0][r]); copy_local(s, t.data(me) + t.staging_off() + (size_t)r * slot, inputs[0][r].data_ptr(), bytes); }
  }
  device_barrier(s);
  pull(s, {{root, t.staging_off() + (size_t)me * slot, outputs[0].data_ptr(), bytes}});
  device_barrier(s);
  finish(s, w);
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::alltoall_base(at::Tensor& output, at::Tensor& input, std::vector<int64_t>& out_splits, std::vector<int64_t>& in_splits, const c10d::AllToAllOptions&) {
  check_contiguous(output); check_contiguous(input);
  const int n = getSize(), me = getRank();
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(input);
  Transport& t = *s.t;
  const size_t row_in = input.dim() ? input.nbytes() / std::max<int64_t>(1, input.size(0)) : input.nbytes();
  const size_t row_out = output.dim() ? output.nbytes() / std::max<int64_t>(1, output.size(0)) : output.nbytes();
  std::vector<size_t> ib(n), ob(n);
  for (int r = 0; r < n; ++r) {
    ib[r] = in_splits.empty() ? input.nbytes() / n : (size_t)in_splits[r] * row_in;
    ob[r] = out_splits.empty() ? output.nbytes() / n : (size_t)out_splits[r] * row_out;
  }
  const size_t slot = t.staging_bytes() / n / 256 * 256;
  auto w = begin(s, c10d::OpType::ALLTOALL_BASE, {output});
  size_t off = 0;
  for (int r = 0; r < n; ++r) {
    TORCH_CHECK(ib[r] <= slot && ob[r] <= slot, "all_to_all: a segment is larger than a staging slot");
    copy_local(s, t.data(me) + t.staging_off() + (size_t)r * slot, (char*)input.data_ptr() + off, ib[r]);
    off += ib[r];
  }
  device_barrier(s);
  std::vector<std::tuple<int, size_t, void*, size_t>> segs;
  off = 0;
  for (int p = 0; p < n; ++p) { segs.push_back({p, t.staging_off() + (size_t)me * slot, (char*)output.data_ptr() + off, ob[p]}); off += ob[p]; }
  pull(s, segs);
  device_barrier(s);
  finish(s, w);
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::alltoall(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs, const c10d::AllToAllOptions&) {
  const int n = getSize(), me = getRank();
  TORCH_CHECK((int)outputs.size() == n && (int)inputs.size() == n, "all_to_all needs world_size tensors");
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(inputs[0]);
  Transport& t = *s.t;
  const size_t slot = t.staging_bytes() / n / 256 * 256;
  auto w = begin(s, c10d::OpType::ALLTOALL, outputs);
  for (int r = 0; r < n; ++r) {
    check_contiguous(inputs[r]); check_contiguous(outputs[r]);
    TORCH_CHECK(inputs[r].nbytes() <= slot && outputs[r].nbytes() <= slot, "all_to_all: a tensor is larger than a staging slot");
    copy_local(s, t.data(me) + t.staging_off() + (size_t)r * slot, inputs[r].data_ptr(), inputs[r].nbytes());
  }
  device_barrier(s);
  std::vector<std::tuple<int, size_t, void*, size_t>> segs;
  for (int p = 0; p < n; ++p) segs.push_back({p, t.staging_off() + (size_t)me * slot, outputs[p].data_ptr(), outputs[p].nbytes()});
  pull(s, segs);
  device_barrier(s);
  finish(s, w);
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::barrier(const c10d::BarrierOptions& opts) {
  NvtxRange nvtx_range("stragglar::barrier");
  std::lock_guard<std::mutex> lk(mu_);
  bool cuda = cuda_.t != nullptr;
  int device = cuda_.device;
  if (!cuda && !cpu_.t) {
    // nothing has run yet: pick the device the way the NCCL backend does
    if (opts.device.has_value() && opts.device->is_cuda()) { cuda = true; device = opts.device->index(); }
    else if (!opts.device_ids.empty()) { cuda = true; device = (int)opts.device_ids[0]; }
    else if (torch::cuda::is_available() && !(opts.device.has_value() && opts.device->is_cpu())) {
      cuda = true;
      int d = 0; SAR_CUDA_CHECK(cudaGetDevice(&d)); device = d;
    }
  }
  Side& s = side(cuda, device);
  auto w = begin(s, c10d::OpType::BARRIER, {});
  device_barrier(s);
  finish(s, w);
  if (s.t->cuda()) w->end_->synchronize();   // a barrier is a host-visible rendezvous
  return w;
}

// ------------------------------------------------------------------ send/recv
c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::send(std::vector<at::Tensor>& tensors, int dst, int /*tag*/) {
  TORCH_CHECK(tensors.size() == 1, "stragglar backend takes one tensor per rank");
  check_contiguous(tensors[0]);
  TORCH_CHECK(dst >= 0 && dst < getSize() && dst != getRank(), "bad destination rank");
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(tensors[0]);
  Transport& t = *s.t;
  const int me = getRank();
  auto w = begin(s, c10d::OpType::SEND, {});
  char* p = (char*)tensors[0].data_ptr();
  const size_t bytes = tensors[0].nbytes(), piece = t.staging_bytes();
  uint32_t& seq = send_seq_[{t.cuda(), dst}];
  for (size_t off = 0; off < bytes || off == 0; off += piece) {
    const size_t k = std::min(piece, bytes - off);
    copy_local(s, t.data(me) + t.staging_off(), p + off, k);
    ++seq;
    uint32_t* ready = t.flags(dst, kP2PChannel) + me;                    // at the receiver: "rank me has staged piece seq"
    uint32_t* ack = t.flags(me, kP2PChannel) + SAR_MAX_RANKS + dst;      // here: "rank dst has taken piece seq"
    if (t.cuda()) {
      SAR_CUDA_CHECK(sar_cuda_signal_wait(ready, seq, ack, seq, (uint64_t)(opts_.timeout_s * 1e9), &t.ctrl(me, kP2PChannel)->abort_flag, t.status(), s.stream->stream()));
      ++launches_;
    } else {
      as_atomic(ready)->store(seq, std::memory_order_release);
      const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(opts_.timeout_s);
      while (!sar_reached(as_atomic(ack)->load(std::memory_order_acquire), seq)) {
        TORCH_CHECK(std::chrono::steady_clock::now() < deadline, "stragglar backend: send to rank ", dst, " timed out");
        std::this_thread::yield();
      }
    }
    if (bytes == 0) break;
  }
  finish(s, w);
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupStragglar::recv(std::vector<at::Tensor>& tensors, int src, int /*tag*/) {
  TORCH_CHECK(tensors.size() == 1, "stragglar backend takes one tensor per rank");
  check_contiguous(tensors[0]);
  TORCH_CHECK(src >= 0 && src < getSize() && src != getRank(), "bad source rank");
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(tensors[0]);
  Transport& t = *s.t;
  const int me = getRank();
  auto w = begin(s, c10d::OpType::RECV, tensors);
  char* p = (char*)tensors[0].data_ptr();
  const size_t bytes = tensors[0].nbytes(), piece = t.staging_bytes();
  uint32_t& seq = recv_seq_[{t.cuda(), src}];
  for (size_t off = 0; off < bytes || off == 0; off += piece) {
    const size_t k = std::min(piece, bytes - off);
    ++seq;
    uint32_t* ready = t.flags(me, kP2PChannel) + src;
    uint32_t* ack = t.flags(src, kP2PChannel) + SAR_MAX_RANKS + me;
    if (t.cuda()) {
      SAR_CUDA_CHECK(sar_cuda_signal_wait(nullptr, 0, ready, seq, (uint64_t)(opts_.timeout_s * 1e9), &t.ctrl(me, kP2PChannel)->abort_flag, t.status(), s.stream->stream()));
      pull(s, {{src, t.staging_off(), p + off, k}});
      SAR_CUDA_CHECK(sar_cuda_signal_wait(ack, seq, nullptr, 0, 0, &t.ctrl(me, kP2PChannel)->abort_flag, t.status(), s.stream->stream()));
      launches_ += 2;
    } else {
      const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(opts_.timeout_s);
      while (!sar_reached(as_atomic(ready)->load(std::memory_order_acquire), seq)) {
        TORCH_CHECK(std::chrono::steady_clock::now() < deadline, "stragglar backend: recv from rank ", src, " timed out");
        std::this_thread::yield();
      }
      memcpy(p + off, t.data(src) + t.staging_off(), k);
      as_atomic(ack)->store(seq, std::memory_order_release);
    }
    if (bytes == 0) break;
  }
  finish(s, w);
  return w;
}

// -------------------------------------------------------------- symmetric heap
at::Tensor ProcessGroupStragglar::alloc_symmetric(int64_t numel, at::ScalarType dtype, bool cuda, int device) {
  std::lock_guard<std::mutex> lk(mu_);
  Side& s = side(cuda, device);
  Transport& t = *s.t;
  const size_t bytes = (size_t)numel * c10::elementSize(dtype);
  const int64_t off = t.heap_alloc(bytes);
  TORCH_CHECK(off >= 0, "stragglar backend: symmetric heap exhausted (", bytes, " bytes requested of ", t.heap_bytes(),
              "); raise STRAGGLAR_ARENA_MB");
  // the offsets must agree on every rank
  const std::string key = prefix_ + (cuda ? "/cuda" : "/cpu") + "/alloc/" + std::to_string(alloc_seq_++);
  const std::string mine = std::to_string(off) + ":" + std::to_string(bytes);
  store_->set(key + "/" + std::to_string(getRank()), std::vector<uint8_t>(mine.begin(), mine.end()));
  for (int r = 0; r < getSize(); ++r) {
    auto v = store_->get(key + "/" + std::to_string(r));
    TORCH_CHECK(std::string(v.begin(), v.end()) == mine, "alloc_symmetric: rank ", r, " allocated ",
                std::string(v.begin(), v.end()), " but rank ", getRank(), " allocated ", mine,
                " (every rank must allocate the same sizes in the same order)");
  }
  std::shared_ptr<Heap> heap = t.heap();
  auto opts = at::TensorOptions().dtype(dtype);
  opts = cuda ? opts.device(at::kCUDA, (c10::DeviceIndex)device) : opts.device(at::kCPU);
  // the block returns to the heap when the tensor dies; the arena outlives the tensors of a well-formed program
  return at::from_blob(t.data(getRank()) + off, {numel}, [heap, off](void*) { heap->free(off); }, opts);
}

// -------------------------------------------------------------------- bindings
static c10::intrusive_ptr<c10d::Backend> create_backend(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                                                        const std::chrono::duration<float>& timeout, const py::dict& options) {
  BackendOptions o;
  if (options.contains("alg")) o.alg = options["alg"].cast<std::string>();
  if (options.contains("straggler")) o.straggler = options["straggler"].cast<int>();
  if (options.contains("path")) {
    const std::string p = options["path"].cast<std::string>();
    TORCH_CHECK(p == "simt" || p == "tma" || p == "simta", "stragglar backend: unknown path '", p, "' (simt, tma or simta)");
    o.path = p == "simt" ? SAR_PATH_SIMT : p == "simta" ? SAR_PATH_SIMTA : SAR_PATH_TMA;
  }
  if (options.contains("blocks")) o.blocks = options["blocks"].cast<int>();
  if (options.contains("threads")) o.threads = options["threads"].cast<int>();
  if (options.contains("tile_bytes")) o.tile_bytes = options["tile_bytes"].cast<uint32_t>();
  if (options.contains("timeout_s")) o.timeout_s = options["timeout_s"].cast<double>();
  if (options.contains("arena_bytes")) o.arena_bytes = options["arena_bytes"].cast<size_t>();
  if (options.contains("staging_bytes")) o.staging_bytes = options["staging_bytes"].cast<size_t>();
  if (options.contains("schedule_text")) o.schedule_text = options["schedule_text"].cast<std::string>();
  if (options.contains("check_args")) o.check_args = options["check_args"].cast<bool>();
  return c10::make_intrusive<ProcessGroupStragglar>(
      store, rank, size, std::chrono::duration_cast<std::chrono::milliseconds>(timeout), o);
}

static ProcessGroupStragglar* cast(const c10::intrusive_ptr<c10d::Backend>& b) {
  auto* p = dynamic_cast<ProcessGroupStragglar*>(b.get());
  TORCH_CHECK(p, "not a stragglar backend");
  return p;
}

}  // namespace sarpg

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  using namespace sarpg;
  m.doc() = "c10d backend 'stragglar'";
  m.def("create_backend", &create_backend, py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("timeout"),
        py::arg("options") = py::dict());
  m.def("allreduce_ex", [](const c10::intrusive_ptr<c10d::Backend>& b, at::Tensor t, bool average, py::object comm_dtype) {
    std::optional<at::ScalarType> cd;
    if (!comm_dtype.is_none()) cd = torch::python::detail::py_object_to_dtype(comm_dtype);
    return cast(b)->allreduce_ex(t, average, cd);
  }, py::arg("backend"), py::arg("tensor"), py::arg("average") = false, py::arg("comm_dtype") = py::none());
  m.def("alloc_symmetric", [](const c10::intrusive_ptr<c10d::Backend>& b, int64_t numel, py::object dtype, bool cuda, int device) {
    return cast(b)->alloc_symmetric(numel, torch::python::detail::py_object_to_dtype(dtype), cuda, device);
  });
  m.def("set_straggler", [](const c10::intrusive_ptr<c10d::Backend>& b, int r) { cast(b)->set_straggler(r); });
  m.def("set_algorithm", [](const c10::intrusive_ptr<c10d::Backend>& b, const std::string& a) { cast(b)->set_algorithm(a); });
  m.def("get_straggler", [](const c10::intrusive_ptr<c10d::Backend>& b) { return cast(b)->straggler(); });
  m.def("get_algorithm", [](const c10::intrusive_ptr<c10d::Backend>& b) { return cast(b)->algorithm(); });
  m.def("algorithm_for", [](const c10::intrusive_ptr<c10d::Backend>& b, size_t bytes) { return cast(b)->algorithm_for(bytes); });
  m.def("check_status", [](const c10::intrusive_ptr<c10d::Backend>& b, bool cuda) { return cast(b)->check_status(cuda); },
        py::arg("backend"), py::arg("cuda") = true, py::call_guard<py::gil_scoped_release>());
  m.def("launches", [](const c10::intrusive_ptr<c10d::Backend>& b) { return cast(b)->launches(); });
  m.def("check_guards", [](const c10::intrusive_ptr<c10d::Backend>& b, bool cuda) { return cast(b)->check_guards(cuda); },
        py::arg("backend"), py::arg("cuda") = true, py::call_guard<py::gil_scoped_release>());
  m.def("last_trace", [](const c10::intrusive_ptr<c10d::Backend>& b) { return cast(b)->last_trace(); },
        py::call_guard<py::gil_scoped_release>());
}
