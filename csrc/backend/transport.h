// Symmetric arenas of a process group, as one rank sees them.
//
// Every rank owns one region with the same layout:
//   [control words | status | flags (all channels) | guard | data | guard]
// (the guards are canary bytes on both sides of the data region; check_guards() tells whether a
// kernel or a copy has written outside the region)
// and maps every peer's region into its own address space: CUDA IPC handles
// for device memory, POSIX shared memory for host memory.  The handles (or
// names) travel through the c10d Store the process group was given; the
// reference backend instead opened its own TCP socket on a fixed port and
// ignored the Store (implementation/custom_backend/src/dummy.cpp:170-211,813-819).
#pragma once
#include <c10/util/intrusive_ptr.h>
#include <torch/csrc/distributed/c10d/Store.hpp>

#include <atomic>
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../core/table.h"

namespace sarpg {

struct ArenaLayout {
  static constexpr size_t kCtrlOff = 0;
  static constexpr size_t kStatusOff = 2048;
  static constexpr size_t kFlagsOff = 4096;
  static constexpr size_t kFlagsBytes = sizeof(uint32_t) * (size_t)SAR_NUM_CHANNELS * SAR_FLAG_CAPACITY;
  static constexpr size_t kGuardBytes = 256;
  static constexpr unsigned char kGuardByte = 0xA5;
  static constexpr size_t kDataOff = kFlagsOff + kFlagsBytes + kGuardBytes;
};

// Bookkeeping of the symmetric heap.  Shared with the deleters of the tensors handed out, so that a
// tensor outliving its process group only returns its block to a dead book instead of touching freed memory.
class Heap {
 public:
  explicit Heap(size_t bytes) { blocks_.push_back({0, bytes, false}); }
  int64_t alloc(size_t bytes);
  void free(int64_t off);
 private:
  struct Block { size_t off, bytes; bool used; };
  std::vector<Block> blocks_;
  std::mutex mu_;
};

class Transport {
 public:
  Transport(bool cuda, int device, int rank, int n, size_t data_bytes, size_t staging_bytes,
            const c10::intrusive_ptr<c10d::Store>& store, const std::string& key_prefix);
  ~Transport();
  Transport(const Transport&) = delete;

  bool cuda() const { return cuda_; }
  int device() const { return device_; }
  int rank() const { return rank_; }
  int size() const { return n_; }
  char* base(int r) const { return base_[r]; }
  char* data(int r) const { return base_[r] + ArenaLayout::kDataOff; }
  uint32_t* flags(int r, int channel) const {
    return reinterpret_cast<uint32_t*>(base_[r] + ArenaLayout::kFlagsOff) + (size_t)channel * SAR_FLAG_CAPACITY;
  }
  SarCtrl* ctrl(int r, int channel) const { return reinterpret_cast<SarCtrl*>(base_[r] + ArenaLayout::kCtrlOff) + channel; }
  // This rank's failure word (a SarStatus; 0 = ok).  On CUDA it lives in pinned host memory that the device
  // writes through a mapped pointer, so the host can look at it at any time without a CUDA call; kernels write
  // it only when a wait runs out.
  uint32_t* status() const { return host_status_ ? host_status_.get() : reinterpret_cast<uint32_t*>(base_[rank_] + ArenaLayout::kStatusOff); }
  std::shared_ptr<uint32_t> status_owner() const { return host_status_; }
  // arrival / end stamps of the last collective kernel (device memory on CUDA)
  uint64_t* trace_words() const { return reinterpret_cast<uint64_t*>(base_[rank_] + ArenaLayout::kStatusOff + 16); }
  size_t data_bytes() const { return data_bytes_; }
  size_t staging_bytes() const { return staging_bytes_; }
  size_t staging_off() const { return data_bytes_ - staging_bytes_; }   // staging sits at the end of the data region
  size_t heap_bytes() const { return data_bytes_ - staging_bytes_; }

  // True while the canary bytes before and after this rank's data region are intact (waits for the
  // device first).  A false answer means something wrote outside the region it was given.
  bool check_guards() const;

  // next epoch base of a channel (every rank calls this in the same order)
  // (64-bit: the low word is the flag epoch, the whole value the base of the round-gate words)
  uint64_t next_epoch(int channel) { return epoch_[channel] += SAR_VER_STRIDE; }
  uint32_t next_barrier_epoch() { return ++barrier_epoch_; }

  // offset into the data region if p lies inside this rank's heap, else -1
  int64_t heap_offset(const void* p, size_t bytes) const;
  // symmetric heap: the same call sequence on every rank yields the same offsets
  int64_t heap_alloc(size_t bytes) { return heap_->alloc(bytes); }
  void heap_free(int64_t off) { heap_->free(off); }
  std::shared_ptr<Heap> heap() const { return heap_; }

 private:
  void open_arenas(const c10::intrusive_ptr<c10d::Store>& store, const std::string& key_prefix);
  void release();
  bool cuda_;
  int device_, rank_, n_;
  size_t data_bytes_, staging_bytes_, total_bytes_;
  char* base_[SAR_MAX_RANKS] = {};
  uint64_t epoch_[SAR_NUM_CHANNELS] = {};
  uint32_t barrier_epoch_ = 0;
  std::string shm_name_;
  std::shared_ptr<Heap> heap_;
  std::shared_ptr<uint32_t> host_status_;   // CUDA: pinned, mapped
};

}  // namespace sarpg
