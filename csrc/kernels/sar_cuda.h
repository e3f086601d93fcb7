// Host interface of the CUDA kernels (C linkage; usable from C++, ctypes and
// the torch extension).  All functions return a cudaError_t value as int
// (0 = success) unless stated otherwise; they never allocate.
#pragma once
#include <stdint.h>

#include "../core/table.h"

struct SarLaunchParams;

#ifdef __cplusplus
extern "C" {
#endif

// simt: every thread moves vectors and takes part in the control flow; tma: bulk-copy pipeline;
// simta: the simt data path with control and signalling in threads of their own
enum SarPath { SAR_PATH_SIMT = 0, SAR_PATH_TMA = 1, SAR_PATH_SIMTA = 2 };

// blocks <= 0 picks the default for the path.  threads is used by the simt
// path only (<= 0: 512).
int sar_cuda_launch(const struct SarLaunchParams* p, int path, int blocks, int threads, void* stream);
// n ranks emulated on the current device by ONE cooperative launch: d_params
// points to n SarLaunchParams in device memory; rank r is run by blocks
// [r*blocks_per_rank, (r+1)*blocks_per_rank).  Fails with
// cudaErrorCooperativeLaunchTooLarge when the blocks cannot all be resident.
int sar_cuda_launch_emulated(const struct SarLaunchParams* d_params, int n, int dtype, int path, int blocks_per_rank,
                             int threads, void* stream);
int sar_cuda_default_blocks(int path);
// blocks per rank for a buffer of `bytes`: few for small messages (latency bound, and the SMs
// are left to the compute that overlaps the collective), up to 128 for large ones
int sar_cuda_pick_blocks(int path, uint64_t bytes);
uint32_t sar_cuda_default_tile_bytes(int path);
int sar_cuda_max_emulated_blocks(int dtype, int path, int threads);   // resident blocks on the current device

// Barrier across ranks on control channel `channel`: announces `epoch` and
// waits (bounded) until every rank in `participants` has announced it.
int sar_cuda_barrier(SarCtrl* const* ctrl /*host array of nranks device ptrs*/, int rank, int nranks,
                     uint32_t participants, uint32_t epoch, uint64_t timeout_ns, uint32_t* status, void* stream);

// Busy-wait on the device for `ns` nanoseconds of %globaltimer (at most 10 s):
// the injected straggler delay (cf. gpu_sleep_kernel, stragglar/allreduce_8GPU.cu:36-39,
// which counts SM clocks and so depends on the clock the GPU happens to run at).
int sar_cuda_delay(uint64_t ns, void* stream);
// dst[i] = uniform[-1, 1) from a counter hash of (seed, i); same values as sar_host_uniform.
int sar_cuda_fill_uniform(void* dst, uint64_t count, int dtype, uint64_t seed, void* stream);
// dst[i] = (T)(sum over r of (float)(T)uniform(seeds[r], i)) for i in [begin, end): what a
// reduce-scatter over inputs made by sar_cuda_fill_uniform leaves in a chunk (fp32
// accumulation, one rounding).  Used to emulate a finished pre-phase.
int sar_cuda_fill_uniform_sum(void* dst, uint64_t begin, uint64_t end, int dtype, const uint64_t* seeds, int nseeds,
                              void* stream);
int sar_cuda_fill_const(void* dst, uint64_t count, int dtype, float value, void* stream);
// dst[i] = (dst_dtype)(src[i] * scale); src and dst may alias when the dtypes agree.
int sar_cuda_scale_cast(void* dst, int dst_dtype, const void* src, int src_dtype, uint64_t count, float scale,
                        void* stream);
// Checks buf[i] against scale * sum over r of uniform(seeds[r], i) for i in
// [begin, end); result[0] = number of elements off by more than
// atol + rtol*|want|, result[1] = max abs error as float bits.  result is
// device memory (2 x uint32) and is zeroed by the call.
int sar_cuda_verify_uniform_sum(const void* buf, uint64_t begin, uint64_t end, int dtype, const uint64_t* seeds,
                                int nseeds, float scale, float atol, float rtol, uint32_t* result, void* stream);
// Plain data movement for the backend's staged collectives (broadcast,
// all-gather, ...): up to SAR_MAX_RANKS segments per launch, each copied from
// `src` (local or peer memory, read with system-scope loads) to local `dst`.
struct SarCopySeg { const void* src; void* dst; uint64_t bytes; };
int sar_cuda_copy_segments(const struct SarCopySeg* segs, int nseg, void* stream);
// dst[i] = scale * sum over k of srcs[k][i]  (fp32 accumulation, one rounding)
int sar_cuda_reduce_segments(void* dst, const void* const* srcs, int nsrc, uint64_t count, int dtype, float scale,
                             void* stream);
// One thread: release-store set_val to *set_ptr (if set_ptr), then wait
// (bounded) until *wait_ptr has reached wait_val (if wait_ptr).  The building
// block of the backend's point-to-point send/recv handshake.
int sar_cuda_signal_wait(uint32_t* set_ptr, uint32_t set_val, const uint32_t* wait_ptr, uint32_t wait_val,
                         uint64_t timeout_ns, uint32_t* abort_flag, uint32_t* status, void* stream);
float sar_host_uniform(uint64_t seed, uint64_t index);

#ifdef __cplusplus
}
#endif
