// Kernel entry points and launchers for the table executor and its helpers.
#include "exec_table.cuh"
#include "sar_cuda.h"

#include <cooperative_groups.h>

using namespace sar_dev;

extern __shared__ __align__(128) unsigned char sar_smem[];

template <typename T>
__global__ void __launch_bounds__(512, 1) sar_exec_simt_kernel(const __grid_constant__ SarLaunchParams P) {
  run_rank_simt<T>(P, blockIdx.x, gridDim.x);
}

template <typename T>
__global__ void __launch_bounds__(tma::kThreads, 1) sar_exec_tma_kernel(const __grid_constant__ SarLaunchParams P) {
  run_rank_tma<T>(P, blockIdx.x, gridDim.x, *reinterpret_cast<tma::Shared*>(sar_smem));
}

template <typename T>
__global__ void __launch_bounds__(simta::kThreads, 1) sar_exec_simta_kernel(const __grid_constant__ SarLaunchParams P) {
  __shared__ simta::Shared S;
  run_rank_simta<T>(P, blockIdx.x, gridDim.x, S);
}

// All ranks of a collective in one launch on one device (tests, profiling).
// Blocks of different ranks wait on one another, so they must be co-resident:
// launched cooperatively.
template <typename T>
__global__ void __launch_bounds__(512, 1) sar_emul_simt_kernel(const SarLaunchParams* params, int blocks_per_rank) {
  __shared__ SarLaunchParams P;
  const int r = blockIdx.x / blocks_per_rank;
  for (uint32_t i = threadIdx.x; i < sizeof(SarLaunchParams) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(&P)[i] = reinterpret_cast<const uint32_t*>(params + r)[i];
  __syncthreads();
  if (!(P.participants >> P.rank & 1)) return;
  run_rank_simt<T>(P, blockIdx.x % blocks_per_rank, blocks_per_rank);
}

template <typename T>
__global__ void __launch_bounds__(simta::kThreads, 1) sar_emul_simta_kernel(const SarLaunchParams* params, int blocks_per_rank) {
  __shared__ SarLaunchParams P;
  __shared__ simta::Shared S;
  const int r = blockIdx.x / blocks_per_rank;
  for (uint32_t i = threadIdx.x; i < sizeof(SarLaunchParams) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(&P)[i] = reinterpret_cast<const uint32_t*>(params + r)[i];
  __syncthreads();
  if (!(P.participants >> P.rank & 1)) return;
  run_rank_simta<T>(P, blockIdx.x % blocks_per_rank, blocks_per_rank, S);
}

template <typename T>
__global__ void __launch_bounds__(tma::kThreads, 1) sar_emul_tma_kernel(const SarLaunchParams* params, int blocks_per_rank) {
  __shared__ SarLaunchParams P;
  const int r = blockIdx.x / blocks_per_rank;
  for (uint32_t i = threadIdx.x; i < sizeof(SarLaunchParams) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(&P)[i] = reinterpret_cast<const uint32_t*>(params + r)[i];
  __syncthreads();
  if (!(P.participants >> P.rank & 1)) return;
  run_rank_tma<T>(P, blockIdx.x % blocks_per_rank, blocks_per_rank, *reinterpret_cast<tma::Shared*>(sar_smem));
}

static_assert(sizeof(SarLaunchParams) % 4 == 0, "params are copied word by word");

__global__ void sar_barrier_kernel(SarDevComm comm, int rank, int nranks, uint32_t participants, uint32_t epoch,
                                   uint64_t timeout_ns, uint32_t* status) {
  if (threadIdx.x != 0) return;
  WaitCtx w;
  w.deadline = globaltimer() + timeout_ns;
  w.abort_flag = &comm.ctrl[rank]->abort_flag;
  w.status = status;
  fence_sys();
  st_release_sys(&comm.ctrl[rank]->arrival, epoch);
  for (int r = 0; r < nranks; ++r) {
    if (r == rank || !(participants >> r & 1)) continue;
    if (!wait_word(&comm.ctrl[r]->arrival, epoch, w, SAR_TIMEOUT_ARRIVAL)) return;
  }
}

__global__ void sar_signal_wait_kernel(uint32_t* set_ptr, uint32_t set_val, const uint32_t* wait_ptr, uint32_t wait_val,
                                       uint64_t timeout_ns, uint32_t* abort_flag, uint32_t* status) {
  if (threadIdx.x != 0) return;
  if (set_ptr) { fence_sys(); st_release_sys(set_ptr, set_val); }
  if (wait_ptr) {
    WaitCtx w;
    w.deadline = globaltimer() + timeout_ns;
    w.abort_flag = abort_flag;
    w.status = status;
    wait_word(wait_ptr, wait_val, w, SAR_TIMEOUT_FLAG);
  }
}

__global__ void sar_delay_kernel(uint64_t ns) {
  const uint64_t t0 = globaltimer();
  while (globaltimer() - t0 < ns) __nanosleep(200);
}

__host__ __device__ inline float sar_uniform(uint64_t seed, uint64_t i) {
  uint64_t x = (i + 1) * 0x9E3779B97F4A7C15ull + seed * 0xD1B54A32D192ED03ull;
  x ^= x >> 32; x *= 0xD6E8FEB86659FD93ull; x ^= x >> 32; x *= 0xD6E8FEB86659FD93ull; x ^= x >> 32;
  return (float)(uint32_t)(x >> 40) * (2.0f / 16777216.0f) - 1.0f;
}

template <typename T> __device__ inline T from_float(float v);
template <> __device__ inline float from_float<float>(float v) { return v; }
template <> __device__ inline __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ inline __half from_float<__half>(float v) { return __float2half_rn(v); }
__device__ inline float to_float(float v) { return v; }
__device__ inline float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ inline float to_float(__half v) { return __half2float(v); }

template <typename T>
__global__ void sar_fill_uniform_kernel(T* dst, uint64_t count, uint64_t seed) {
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x)
    dst[i] = from_float<T>(sar_uniform(seed, i));
}
template <typename T>
__global__ void sar_fill_const_kernel(T* dst, uint64_t count, float v) {
  const T t = from_float<T>(v);
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x)
    dst[i] = t;
}
template <typename TD, typename TS>
__global__ void sar_scale_cast_kernel(TD* dst, const TS* src, uint64_t count, float scale) {
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x)
    dst[i] = from_float<TD>(to_float(src[i]) * scale);
}
// converting fast path: eight elements per thread and turn, 16-byte accesses on the 2-byte side and 2 x 16 bytes
// on the 4-byte side (both pointers 16-byte aligned)
template <typename TD, typename TS>
__global__ void sar_scale_cast_vec8_kernel(TD* dst, const TS* src, uint64_t ngroups, float scale) {
  for (uint64_t g = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; g < ngroups; g += (uint64_t)gridDim.x * blockDim.x) {
    float f[8];
    if constexpr (sizeof(TS) == 4) {
      const float4 a = reinterpret_cast<const float4*>(src)[2 * g], b = reinterpret_cast<const float4*>(src)[2 * g + 1];
      f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
      Vec<TS>::unpack(reinterpret_cast<const uint4*>(src)[g], f);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] *= scale;
    if constexpr (sizeof(TD) == 4) {
      reinterpret_cast<float4*>(dst)[2 * g] = make_float4(f[0], f[1], f[2], f[3]);
      reinterpret_cast<float4*>(dst)[2 * g + 1] = make_float4(f[4], f[5], f[6], f[7]);
    } else {
      reinterpret_cast<uint4*>(dst)[g] = Vec<TD>::pack(f);
    }
  }
}
// same-type fast path: 16 bytes per thread
template <typename T>
__global__ void sar_scale_vec_kernel(uint4* dst, const uint4* src, uint64_t nvec, float scale) {
  constexpr int N = Vec<T>::N;
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < nvec; i += (uint64_t)gridDim.x * blockDim.x) {
    float f[N];
    Vec<T>::unpack(src[i], f);
#pragma unroll
    for (int k = 0; k < N; ++k) f[k] *= scale;
    dst[i] = Vec<T>::pack(f);
  }
}

struct SeedList { uint64_t s[SAR_MAX_RANKS]; int n; };
template <typename T>
__global__ void sar_verify_kernel(const T* buf, uint64_t begin, uint64_t end, SeedList seeds, float scale, float atol,
                                  float rtol, uint32_t* result) {
  uint32_t bad = 0;
  float worst = 0.f;
  for (uint64_t i = begin + blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < end; i += (uint64_t)gridDim.x * blockDim.x) {
    double want = 0.0;
    for (int r = 0; r < seeds.n; ++r) {
      // the inputs are stored in T: sum what was actually stored
      want += (double)to_float(from_float<T>(sar_uniform(seeds.s[r], i)));
    }
    want *= scale;
    const float err = fabsf((float)((double)to_float(buf[i]) - want));
    if (!(err <= atol + rtol * fabsf((float)want))) ++bad;
    worst = fmaxf(worst, err);
  }
  if (bad) atomicAdd(&result[0], bad);
  atomicMax(&result[1], __float_as_uint(worst));   // non-negative floats order like their bits
}

template <typename T>
__global__ void sar_fill_uniform_sum_kernel(T* dst, uint64_t begin, uint64_t end, SeedList seeds) {
  for (uint64_t i = begin + blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < end; i += (uint64_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < seeds.n; ++r) acc += to_float(from_float<T>(sar_uniform(seeds.s[r], i)));
    dst[i] = from_float<T>(acc);
  }
}

struct SegList { SarCopySeg s[SAR_MAX_RANKS]; int n; };
__global__ void sar_copy_segments_kernel(SegList L) {
  for (int k = 0; k < L.n; ++k) {
    const char* src = (const char*)L.s[k].src;
    char* dst = (char*)L.s[k].dst;
    const uint64_t bytes = L.s[k].bytes;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, t = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    if ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
      const uint64_t nvec = bytes / 16;
      for (uint64_t i = t; i < nvec; i += stride) st_vec(dst + i * 16, ld_vec_sys(src + i * 16));
      for (uint64_t i = nvec * 16 + t; i < bytes; i += stride) dst[i] = *(volatile const char*)(src + i);
    } else {
      for (uint64_t i = t; i < bytes; i += stride) dst[i] = *(volatile const char*)(src + i);
    }
  }
}
struct SrcList { const void* p[SAR_MAX_RANKS]; int n; };
template <typename T>
__global__ void sar_reduce_segments_kernel(T* dst, SrcList L, uint64_t begin, uint64_t count, float scale) {
  for (uint64_t i = begin + blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < L.n; ++k) acc += Vec<T>::load1((const char*)L.p[k] + i * sizeof(T));
    dst[i] = from_float<T>(acc * scale);
  }
}
// 16 bytes per thread and source (all pointers 16-byte aligned); the sources may be peer memory
template <typename T>
__global__ void sar_reduce_segments_vec_kernel(uint4* dst, SrcList L, uint64_t nvec, float scale) {
  constexpr int N = Vec<T>::N;
  for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < nvec; i += (uint64_t)gridDim.x * blockDim.x) {
    float acc[N];
#pragma unroll
    for (int k = 0; k < N; ++k) acc[k] = 0.f;
    for (int s = 0; s < L.n; ++s) {
      float f[N];
      Vec<T>::unpack(ld_vec_sys((const char*)L.p[s] + i * 16), f);
#pragma unroll
      for (int k = 0; k < N; ++k) acc[k] += f[k];
    }
#pragma unroll
    for (int k = 0; k < N; ++k) acc[k] *= scale;
    dst[i] = Vec<T>::pack(acc);
  }
}

// -------------------------------------------------------------------- launchers
namespace {
template <typename F> int with_dtype(int dtype, F&& f) {
  switch (dtype) {
    case SAR_F32: return f(float{});
    case SAR_BF16: return f(__nv_bfloat16{});
    case SAR_F16: return f(__half{});
    default: return (int)cudaErrorInvalidValue;
  }
}
int grid_for(uint64_t count, int threads) {
  uint64_t b = (count + threads - 1) / threads;
  return (int)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}
template <typename K> int allow_smem(K kernel, size_t bytes) {
  return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}
}  // namespace

extern "C" {

int sar_cuda_default_blocks(int path) { return path == SAR_PATH_TMA ? 32 : 64; }
int sar_cuda_pick_blocks(int path, uint64_t bytes) {
  // 8 x B200: 16 blocks cost 20-30 % at 16-64 MiB (0.132 ms against 0.104 at 16 MiB), 32 or more are level
  const uint64_t b = bytes / (1ull << 20);
  const int lo = 32, hi = 128;
  (void)path;
  return (int)(b < (uint64_t)lo ? lo : (b > (uint64_t)hi ? hi : b));
}
uint32_t sar_cuda_default_tile_bytes(int path) { return path == SAR_PATH_TMA ? (64u << 10) : (128u << 10); }

int sar_cuda_launch(const SarLaunchParams* p, int path, int blocks, int threads, void* stream) {
  if (blocks <= 0) blocks = sar_cuda_default_blocks(path);
  cudaStream_t st = (cudaStream_t)stream;
  return with_dtype(p->dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    if (path == SAR_PATH_TMA) {
      int e = allow_smem(sar_exec_tma_kernel<T>, sizeof(tma::Shared));
      if (e) return e;
      sar_exec_tma_kernel<T><<<blocks, tma::kThreads, sizeof(tma::Shared), st>>>(*p);
    } else if (path == SAR_PATH_SIMTA) {
      sar_exec_simta_kernel<T><<<blocks, simta::kThreads, 0, st>>>(*p);
    } else {
      if (threads <= 0) threads = 512;
      sar_exec_simt_kernel<T><<<blocks, threads, 0, st>>>(*p);
    }
    return (int)cudaGetLastError();
  });
}

int sar_cuda_max_emulated_blocks(int dtype, int path, int threads) {
  int dev = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&dev) || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) return 0;
  with_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    if (path == SAR_PATH_TMA) {
      allow_smem(sar_emul_tma_kernel<T>, sizeof(tma::Shared));
      return (int)cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sar_emul_tma_kernel<T>, tma::kThreads, sizeof(tma::Shared));
    }
    if (path == SAR_PATH_SIMTA)
      return (int)cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sar_emul_simta_kernel<T>, simta::kThreads, 0);
    return (int)cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sar_emul_simt_kernel<T>, threads <= 0 ? 512 : threads, 0);
  });
  return sms * per_sm;
}

int sar_cuda_launch_emulated(const SarLaunchParams* d_params, int n, int dtype, int path, int blocks_per_rank,
                             int threads, void* stream) {
  if (blocks_per_rank <= 0) blocks_per_rank = 4;
  cudaStream_t st = (cudaStream_t)stream;
  return with_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    void* args[] = {(void*)&d_params, (void*)&blocks_per_rank};
    if (path == SAR_PATH_TMA) {
      int e = allow_smem(sar_emul_tma_kernel<T>, sizeof(tma::Shared));
      if (e) return e;
      return (int)cudaLaunchCooperativeKernel((void*)sar_emul_tma_kernel<T>, dim3(n * blocks_per_rank), dim3(tma::kThreads),
                                              args, sizeof(tma::Shared), st);
    }
    if (path == SAR_PATH_SIMTA)
      return (int)cudaLaunchCooperativeKernel((void*)sar_emul_simta_kernel<T>, dim3(n * blocks_per_rank), dim3(simta::kThreads), args, 0, st);
    if (threads <= 0) threads = 512;
    return (int)cudaLaunchCooperativeKernel((void*)sar_emul_simt_kernel<T>, dim3(n * blocks_per_rank), dim3(threads), args, 0, st);
  });
}

int sar_cuda_barrier(SarCtrl* const* ctrl, int rank, int nranks, uint32_t participants, uint32_t epoch,
                     uint64_t timeout_ns, uint32_t* status, void* stream) {
  SarDevComm c{};
  for (int r = 0; r < nranks && r < SAR_MAX_RANKS; ++r) c.ctrl[r] = ctrl[r];
  sar_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(c, rank, nranks, participants, epoch, timeout_ns, status);
  return (int)cudaGetLastError();
}

int sar_cuda_delay(uint64_t ns, void* stream) {
  if (ns > 10000000000ull) ns = 10000000000ull;
  sar_delay_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(ns);
  return (int)cudaGetLastError();
}

int sar_cuda_fill_uniform(void* dst, uint64_t count, int dtype, uint64_t seed, void* stream) {
  return with_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    sar_fill_uniform_kernel<T><<<grid_for(count, 256), 256, 0, (cudaStream_t)stream>>>((T*)dst, count, seed);
    return (int)cudaGetLastError();
  });
}

int sar_cuda_fill_uniform_sum(void* dst, uint64_t begin, uint64_t end, int dtype, const uint64_t* seeds, int nseeds,
                              void* stream) {
  if (nseeds > SAR_MAX_RANKS) return (int)cudaErrorInvalidValue;
  if (end <= begin) return 0;
  SeedList sl{};
  sl.n = nseeds;
  for (int i = 0; i < nseeds; ++i) sl.s[i] = seeds[i];
  return with_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    sar_fill_uniform_sum_kernel<T><<<grid_for(end - begin, 256), 256, 0, (cudaStream_t)stream>>>((T*)dst, begin, end, sl);
    return (int)cudaGetLastError();
  });
}

int sar_cuda_fill_const(void* dst, uint64_t count, int dtype, float value, void* stream) {
  return with_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    sar_fill_const_kernel<T><<<grid_for(count, 256), 256, 0, (cudaStream_t)stream>>>((T*)dst, count, value);
    return (int)cudaGetLastError();
  });
}

int sar_cuda_scale_cast(void* dst, int dst_dtype, const void* src, int src_dtype, uint64_t count, float scale,
                        void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (count == 0) return 0;
  if (dst_dtype == src_dtype) {
    return with_dtype(dst_dtype, [&](auto tag) -> int {
      using T = decltype(tag);
      const bool aligned = (((uintptr_t)dst | (uintptr_t)src) & 15) == 0;
      const uint64_t nvec = aligned ? count / Vec<T>::N : 0;
      if (nvec) sar_scale_vec_kernel<T><<<grid_for(nvec, 256), 256, 0, st>>>((uint4*)dst, (const uint4*)src, nvec, scale);
      const uint64_t done = nvec * Vec<T>::N;
      if (done < count)
        sar_scale_cast_kernel<T, T><<<grid_for(count - done, 256), 256, 0, st>>>((T*)dst + done, (const T*)src + done, count - done, scale);
      return (int)cudaGetLastError();
    });
  }
  return with_dtype(dst_dtype, [&](auto dtag) -> int {
    using TD = decltype(dtag);
    return with_dtype(src_dtype, [&](auto stag) -> int {
      using TS = decltype(stag);
      const bool aligned = (((uintptr_t)dst | (uintptr_t)src) & 15) == 0;
      const uint64_t groups = aligned ? count / 8 : 0;
      if (groups) sar_scale_cast_vec8_kernel<TD, TS><<<grid_for(groups, 256), 256, 0, st>>>((TD*)dst, (const TS*)src, groups, scale);
      const uint64_t done = groups * 8;
      if (done < count)
        sar_scale_cast_kernel<TD, TS><<<grid_for(count - done, 256), 256, 0, st>>>((TD*)dst + done, (const TS*)src + done, count - done, scale);
      return (int)cudaGetLastError();
    });
  });
}

int sar_cuda_verify_uniform_sum(const void* buf, uint64_t begin, uint64_t end, int dtype, const uint64_t* seeds,
                                int nseeds, float scale, float atol, float rtol, uint32_t* result, void* stream) {
  if (nseeds > SAR_MAX_RANKS) return (int)cudaErrorInvalidValue;
  SeedList sl{};
  sl.n = nseeds;
  for (int i = 0; i < nseeds; ++i) sl.s[i] = seeds[i];
  cudaStream_t st = (cudaStream_t)stream;
  int e = (int)cudaMemsetAsync(result, 0, 8, st);
  if (e) return e;
  if (end <= begin) return 0;
  return with_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    sar_verify_kernel<T><<<grid_for(end - begin, 256), 256, 0, st>>>((const T*)buf, begin, end, sl, scale, atol, rtol, result);
    return (int)cudaGetLastError();
  });
}

int sar_cuda_copy_segments(const SarCopySeg* segs, int nseg, void* stream) {
  if (nseg < 0 || nseg > SAR_MAX_RANKS) return (int)cudaErrorInvalidValue;
  if (nseg == 0) return 0;
  SegList L{};
  L.n = nseg;
  uint64_t mx = 0;
  for (int i = 0; i < nseg; ++i) { L.s[i] = segs[i]; mx = segs[i].bytes > mx ? segs[i].bytes : mx; }
  sar_copy_segments_kernel<<<grid_for(mx / 16 + 1, 256), 256, 0, (cudaStream_t)stream>>>(L);
  return (int)cudaGetLastError();
}

int sar_cuda_reduce_segments(void* dst, const void* const* srcs, int nsrc, uint64_t count, int dtype, float scale,
                             void* stream) {
  if (nsrc < 1 || nsrc > SAR_MAX_RANKS) return (int)cudaErrorInvalidValue;
  if (count == 0) return 0;
  SrcList L{};
  L.n = nsrc;
  for (int i = 0; i < nsrc; ++i) L.p[i] = srcs[i];
  return with_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    bool aligned = (((uintptr_t)dst) & 15) == 0;
    for (int i = 0; i < nsrc; ++i) aligned = aligned && (((uintptr_t)srcs[i]) & 15) == 0;
    const uint64_t nvec = aligned ? count / Vec<T>::N : 0;
    if (nvec) sar_reduce_segments_vec_kernel<T><<<grid_for(nvec, 256), 256, 0, (cudaStream_t)stream>>>((uint4*)dst, L, nvec, scale);
    const uint64_t done = nvec * Vec<T>::N;
    if (done < count)
      sar_reduce_segments_kernel<T><<<grid_for(count - done, 256), 256, 0, (cudaStream_t)stream>>>((T*)dst, L, done, count, scale);
    return (int)cudaGetLastError();
  });
}

int sar_cuda_signal_wait(uint32_t* set_ptr, uint32_t set_val, const uint32_t* wait_ptr, uint32_t wait_val,
                         uint64_t timeout_ns, uint32_t* abort_flag, uint32_t* status, void* stream) {
  sar_signal_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(set_ptr, set_val, wait_ptr, wait_val, timeout_ns, abort_flag, status);
  return (int)cudaGetLastError();
}

float sar_host_uniform(uint64_t seed, uint64_t index) { return sar_uniform(seed, index); }
}
