#include "transport.h"

#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <c10/util/Exception.h>

#include <cstring>
#include <random>

namespace sarpg {

#define SAR_CUDA_CHECK(x)                                                            \
  do {                                                                               \
    cudaError_t e_ = (x);                                                            \
    TORCH_CHECK(e_ == cudaSuccess, "stragglar backend: ", #x, ": ", cudaGetErrorString(e_)); \
  } while (0)

static std::vector<uint8_t> to_bytes(const void* p, size_t n) {
  return std::vector<uint8_t>((const uint8_t*)p, (const uint8_t*)p + n);
}

Transport::Transport(bool cuda, int device, int rank, int n, size_t data_bytes, size_t staging_bytes,
                     const c10::intrusive_ptr<c10d::Store>& store, const std::string& prefix)
    : cuda_(cuda), device_(device), rank_(rank), n_(n) {
  TORCH_CHECK(n >= 1 && n <= SAR_MAX_RANKS, "stragglar backend supports up to ", SAR_MAX_RANKS, " ranks, got ", n);
  data_bytes_ = (data_bytes + 4095) / 4096 * 4096;
  staging_bytes_ = std::min(data_bytes_, (staging_bytes + 4095) / 4096 * 4096);
  total_bytes_ = ArenaLayout::kDataOff + data_bytes_ + ArenaLayout::kGuardBytes;
  heap_ = std::make_shared<Heap>(heap_bytes());
  try {
    open_arenas(store, prefix);
  } catch (...) {
    // e.g. a peer that never published its handle: give back what was mapped so far
    if (!shm_name_.empty()) shm_unlink(shm_name_.c_str());
    release();
    throw;
  }
}

void Transport::open_arenas(const c10::intrusive_ptr<c10d::Store>& store, const std::string& prefix) {
  const int rank = rank_, n = n_, device = device_;
  const std::string me = prefix + "/arena/" + std::to_string(rank);
  if (cuda_) {
    SAR_CUDA_CHECK(cudaSetDevice(device));
    void* p = nullptr;
    SAR_CUDA_CHECK(cudaMalloc(&p, total_bytes_));
    SAR_CUDA_CHECK(cudaMemset(p, 0, ArenaLayout::kDataOff));
    SAR_CUDA_CHECK(cudaMemset((char*)p + ArenaLayout::kDataOff - ArenaLayout::kGuardBytes, ArenaLayout::kGuardByte, ArenaLayout::kGuardBytes));
    SAR_CUDA_CHECK(cudaMemset((char*)p + ArenaLayout::kDataOff + data_bytes_, ArenaLayout::kGuardByte, ArenaLayout::kGuardBytes));
    SAR_CUDA_CHECK(cudaDeviceSynchronize());
    base_[rank] = (char*)p;
    {
      void* hs = nullptr;
      SAR_CUDA_CHECK(cudaHostAlloc(&hs, 64, cudaHostAllocMapped | cudaHostAllocPortable));
      memset(hs, 0, 64);
      host_status_ = std::shared_ptr<uint32_t>((uint32_t*)hs, [](uint32_t* q) { cudaFreeHost(q); });
    }
    if (n > 1) {
      cudaIpcMemHandle_t h;
      SAR_CUDA_CHECK(cudaIpcGetMemHandle(&h, p));
      store->set(me, to_bytes(&h, sizeof h));
      for (int r = 0; r < n; ++r) {
        if (r == rank) continue;
        auto v = store->get(prefix + "/arena/" + std::to_string(r));
        TORCH_CHECK(v.size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle from rank ", r);
        cudaIpcMemHandle_t ph;
        memcpy(&ph, v.data(), sizeof ph);
        void* q = nullptr;
        SAR_CUDA_CHECK(cudaIpcOpenMemHandle(&q, ph, cudaIpcMemLazyEnablePeerAccess));
        base_[r] = (char*)q;
      }
    }
  } else {
    std::random_device rd;
    shm_name_ = "/sar_" + std::to_string((unsigned)getpid()) + "_" + std::to_string(rd()) + "_" + std::to_string(rank);
    int fd = shm_open(shm_name_.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    TORCH_CHECK(fd >= 0, "shm_open(", shm_name_, ") failed: ", strerror(errno));
    TORCH_CHECK(ftruncate(fd, (off_t)total_bytes_) == 0, "ftruncate failed: ", strerror(errno));
    void* p = mmap(nullptr, total_bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    TORCH_CHECK(p != MAP_FAILED, "mmap failed: ", strerror(errno));
    base_[rank] = (char*)p;   // fresh shared memory reads as zero
    memset((char*)p + ArenaLayout::kDataOff - ArenaLayout::kGuardBytes, ArenaLayout::kGuardByte, ArenaLayout::kGuardBytes);
    memset((char*)p + ArenaLayout::kDataOff + data_bytes_, ArenaLayout::kGuardByte, ArenaLayout::kGuardBytes);
    store->set(me, to_bytes(shm_name_.data(), shm_name_.size()));
    for (int r = 0; r < n; ++r) {
      if (r == rank) continue;
      auto v = store->get(prefix + "/arena/" + std::to_string(r));
      std::string name(v.begin(), v.end());
      int pfd = shm_open(name.c_str(), O_RDWR, 0600);
      TORCH_CHECK(pfd >= 0, "shm_open(", name, ") failed: ", strerror(errno));
      void* q = mmap(nullptr, total_bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, pfd, 0);
      close(pfd);
      TORCH_CHECK(q != MAP_FAILED, "mmap of peer arena failed: ", strerror(errno));
      base_[r] = (char*)q;
    }
  }
  // nobody touches a peer's arena before everybody has mapped everything
  store->set(prefix + "/mapped/" + std::to_string(rank), std::vector<uint8_t>{1});
  for (int r = 0; r < n; ++r) store->get(prefix + "/mapped/" + std::to_string(r));
  if (!cuda_) shm_unlink(shm_name_.c_str());   // the mappings keep the memory alive
}

Transport::~Transport() { release(); }

void Transport::release() {
  if (cuda_) {
    cudaSetDevice(device_);
    cudaDeviceSynchronize();
    for (int r = 0; r < n_; ++r)
      if (r != rank_ && base_[r]) cudaIpcCloseMemHandle(base_[r]);
    if (base_[rank_]) cudaFree(base_[rank_]);
  } else {
    for (int r = 0; r < n_; ++r)
      if (base_[r]) munmap(base_[r], total_bytes_);
  }
  for (int r = 0; r < n_; ++r) base_[r] = nullptr;
}

bool Transport::check_guards() const {
  unsigned char g[2 * ArenaLayout::kGuardBytes];
  const char* lo = base_[rank_] + ArenaLayout::kDataOff - ArenaLayout::kGuardBytes;
  const char* hi = base_[rank_] + ArenaLayout::kDataOff + data_bytes_;
  if (cuda_) {
    if (cudaSetDevice(device_) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) return false;
    if (cudaMemcpy(g, lo, ArenaLayout::kGuardBytes, cudaMemcpyDeviceToHost) != cudaSuccess) return false;
    if (cudaMemcpy(g + ArenaLayout::kGuardBytes, hi, ArenaLayout::kGuardBytes, cudaMemcpyDeviceToHost) != cudaSuccess) return false;
  } else {
    memcpy(g, lo, ArenaLayout::kGuardBytes);
    memcpy(g + ArenaLayout::kGuardBytes, hi, ArenaLayout::kGuardBytes);
  }
  for (unsigned char b : g)
    if (b != ArenaLayout::kGuardByte) return false;
  return true;
}

int64_t Transport::heap_offset(const void* p, size_t bytes) const {
  const char* c = (const char*)p;
  const char* lo = data(rank_);
  if (c < lo || c + bytes > lo + heap_bytes()) return -1;
  return c - lo;
}

int64_t Heap::alloc(size_t bytes) {
  std::lock_guard<std::mutex> lk(mu_);
  bytes = (bytes + 255) / 256 * 256;
  if (bytes == 0) bytes = 256;
  for (size_t i = 0; i < blocks_.size(); ++i) {
    if (blocks_[i].used || blocks_[i].bytes < bytes) continue;
    if (blocks_[i].bytes > bytes) {
      Block rest{blocks_[i].off + bytes, blocks_[i].bytes - bytes, false};
      blocks_[i].bytes = bytes;
      blocks_.insert(blocks_.begin() + i + 1, rest);
    }
    blocks_[i].used = true;
    return (int64_t)blocks_[i].off;
  }
  return -1;
}

void Heap::free(int64_t off) {
  std::lock_guard<std::mutex> lk(mu_);
  for (size_t i = 0; i < blocks_.size(); ++i) {
    if ((int64_t)blocks_[i].off != off || !blocks_[i].used) continue;
    blocks_[i].used = false;
    if (i + 1 < blocks_.size() && !blocks_[i + 1].used) { blocks_[i].bytes += blocks_[i + 1].bytes; blocks_.erase(blocks_.begin() + i + 1); }
    if (i > 0 && !blocks_[i - 1].used) { blocks_[i - 1].bytes += blocks_[i].bytes; blocks_.erase(blocks_.begin() + i); }
    return;
  }
}

}  // namespace sarpg
