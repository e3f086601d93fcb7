// The allocation-free AllReduce entry point (see noalloc.h).
#include "noalloc.h"

#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>

#include "../core/host_exec.h"
#include "../core/table.h"
#include "sar_params.h"

// A private copy of the executor's device code: the definitions in
// exec_table.cuh have external linkage and are already part of exec_table.cu.
namespace sar_noalloc_impl {
#include "exec_table.cuh"
}
using sar_noalloc_impl::sar_dev::run_rank_simt;

// All scratch of this entry point.  Zero at load time.  Layout (bytes):
//   [0, 64 KiB)            launch parameters, one per rank
//   [64 KiB, 192 KiB)      op tables: SAR_MAX_OPS ops per rank
//   [192 KiB, 200 KiB)     round offsets: 512 uint16 per rank
//   [200 KiB, 204 KiB)     control words, one SarCtrl per rank
//   [256 KiB, 768 KiB)     flags: SAR_NOALLOC_MAX_TILES words per rank
static __device__ __align__(256) unsigned char sar_noalloc_scratch[SAR_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr size_t kParamsOff = 0;
constexpr size_t kOpsOff = 64u << 10;
constexpr size_t kRoundsOff = 192u << 10;
constexpr size_t kCtrlOff = 200u << 10;
constexpr size_t kFlagsOff = 256u << 10;
static_assert(sizeof(SarLaunchParams) * SAR_NOALLOC_MAX_RANKS <= kOpsOff, "parameters do not fit");
static_assert(kOpsOff + sizeof(SarOp) * SAR_MAX_OPS * SAR_NOALLOC_MAX_RANKS <= kRoundsOff, "op tables do not fit");
static_assert(kRoundsOff + 2 * 512 * SAR_NOALLOC_MAX_RANKS <= kCtrlOff, "round offsets do not fit");
static_assert(kCtrlOff + sizeof(SarCtrl) * SAR_NOALLOC_MAX_RANKS <= kFlagsOff, "control words do not fit");
static_assert(kFlagsOff + 4ull * SAR_NOALLOC_MAX_TILES * SAR_NOALLOC_MAX_RANKS <= SAR_NOALLOC_SCRATCH_BYTES, "flags do not fit");

// device address of the scratch array, per device (0 = not looked up yet)
unsigned char* g_scratch[64] = {};

template <typename T>
__global__ void __launch_bounds__(512, 1) sar_noalloc_kernel(const SarLaunchParams* params, int blocks_per_rank) {
  __shared__ SarLaunchParams P;
  const int r = blockIdx.x / blocks_per_rank;
  for (uint32_t i = threadIdx.x; i < sizeof(SarLaunchParams) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(&P)[i] = reinterpret_cast<const uint32_t*>(params + r)[i];
  __syncthreads();
  run_rank_simt<T>(P, blockIdx.x % blocks_per_rank, blocks_per_rank);
}

int fail(char* err, int errlen, int code, const char* msg) {
  if (err && errlen > 0) snprintf(err, (size_t)errlen, "%s", msg);
  return code;
}
}  // namespace

extern "C" int sar_emulated_allreduce_noalloc(const sar_table* table, void* const* bufs, uint64_t count, int dtype,
                                              float scale, int blocks_per_rank, uint32_t* device_status, void* stream,
                                              char* err, int errlen) {
  if (!table || !bufs) return fail(err, errlen, 1, "table and bufs must not be null");
  if (dtype != SAR_F32 && dtype != SAR_BF16 && dtype != SAR_F16) return fail(err, errlen, 1, "unsupported dtype");
  const int n = sar_table_nranks(table);
  if (n > SAR_NOALLOC_MAX_RANKS) return fail(err, errlen, 2, "too many ranks for the static scratch array (max 8)");
  if (blocks_per_rank <= 0) blocks_per_rank = 4;
  {
    // The parameter and table copies below read host memory that lives only as long as this call;
    // recorded into a graph they would read it when the graph runs.  Refuse instead.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing((cudaStream_t)stream, &cap) != cudaSuccess) { cudaGetLastError(); cap = cudaStreamCaptureStatusNone; }
    if (cap != cudaStreamCaptureStatusNone)
      return fail(err, errlen, 1, "not capturable: the stream is being captured; call this entry point outside stream capture");
  }
  const uint32_t esize = dtype == SAR_F32 ? 4 : 2;
  const uint32_t nch = (uint32_t)sar_table_num_chunks(table);
  for (int r = 0; r < n; ++r) {
    if (!bufs[r] || ((uintptr_t)bufs[r] & 15)) return fail(err, errlen, 1, "buffers must be non-null and 16-byte aligned");
    if (sar_table_num_ops(table, r) > SAR_MAX_OPS || sar_table_num_round_begin(table, r) > 512)
      return fail(err, errlen, 2, "op table too large for the static scratch array");
  }
  // tiles of at most 1 MiB; the flags of one rank (all chunks) must fit SAR_NOALLOC_MAX_TILES words
  const uint32_t tile_elems = sar::pick_tile_elems(count, esize, nch, (uint32_t)blocks_per_rank, 2048, 128u << 10);
  SarGeom g = sar::make_geom(count, esize, nch, tile_elems);
  while ((uint64_t)g.tiles_per_chunk * g.num_chunks > SAR_NOALLOC_MAX_TILES) {
    if ((uint64_t)g.tile_elems * esize >= (1u << 20))
      return fail(err, errlen, 2, "buffer too large: it needs more than 16384 one-MiB tiles, the capacity of the static flag array");
    g = sar::make_geom(count, esize, nch, g.tile_elems * 2);
  }

  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(err, errlen, (int)e, cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(err, errlen, 1, "device index out of range");
  if (!g_scratch[dev]) {
    // once per device, with that device current: the array's name is only a host-side handle
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, sar_noalloc_scratch);
    if (e != cudaSuccess) return fail(err, errlen, (int)e, cudaGetErrorString(e));
    g_scratch[dev] = (unsigned char*)p;
  }
  unsigned char* S = g_scratch[dev];
  cudaStream_t st = (cudaStream_t)stream;

  // the array keeps the previous call's contents: flags and control words start at zero
  const size_t flag_words = (size_t)g.tiles_per_chunk * g.num_chunks;
  for (int r = 0; r < n; ++r) {
    e = cudaMemsetAsync(S + kFlagsOff + 4ull * SAR_NOALLOC_MAX_TILES * r, 0, 4 * flag_words, st);
    if (e != cudaSuccess) return fail(err, errlen, (int)e, cudaGetErrorString(e));
  }
  e = cudaMemsetAsync(S + kCtrlOff, 0, sizeof(SarCtrl) * SAR_NOALLOC_MAX_RANKS, st);
  if (e != cudaSuccess) return fail(err, errlen, (int)e, cudaGetErrorString(e));

  SarLaunchParams hp[SAR_NOALLOC_MAX_RANKS];
  memset(hp, 0, sizeof hp);
  for (int r = 0; r < n; ++r) {
    const int nops = sar_table_num_ops(table, r), nrb = sar_table_num_round_begin(table, r);
    SarOp* d_ops = reinterpret_cast<SarOp*>(S + kOpsOff) + (size_t)SAR_MAX_OPS * r;
    uint16_t* d_rb = reinterpret_cast<uint16_t*>(S + kRoundsOff) + 512 * r;
    if (nops) {
      e = cudaMemcpyAsync(d_ops, sar_table_ops(table, r), sizeof(SarOp) * nops, cudaMemcpyHostToDevice, st);
      if (e != cudaSuccess) return fail(err, errlen, (int)e, cudaGetErrorString(e));
    }
    if (nrb) {
      e = cudaMemcpyAsync(d_rb, sar_table_round_begin(table, r), sizeof(uint16_t) * nrb, cudaMemcpyHostToDevice, st);
      if (e != cudaSuccess) return fail(err, errlen, (int)e, cudaGetErrorString(e));
    }
    SarLaunchParams& P = hp[r];
    for (int q = 0; q < n; ++q) {
      P.comm.flags[q] = reinterpret_cast<uint32_t*>(S + kFlagsOff) + (size_t)SAR_NOALLOC_MAX_TILES * q;
      P.comm.ctrl[q] = reinterpret_cast<SarCtrl*>(S + kCtrlOff) + q;
      P.comm.buf[q] = bufs[q];
    }
    P.ops = d_ops; P.round_begin = d_rb; P.num_rounds = nrb > 0 ? (uint32_t)(nrb - 1) : 0;
    P.geom = g; P.rank = r; P.nranks = n; P.participants = sar_table_participants(table);
    P.epoch_base = SAR_VER_STRIDE; P.scale = scale; P.dtype = dtype;
    P.timeout_ns = 10000000000ull;
    P.status = device_status; P.trace = nullptr; P.delay_ns = 0;
  }
  e = cudaMemcpyAsync(S + kParamsOff, hp, sizeof(SarLaunchParams) * n, cudaMemcpyHostToDevice, st);
  if (e != cudaSuccess) return fail(err, errlen, (int)e, cudaGetErrorString(e));

  const SarLaunchParams* d_params = reinterpret_cast<const SarLaunchParams*>(S + kParamsOff);
  void* args[] = {(void*)&d_params, (void*)&blocks_per_rank};
  const void* fn = dtype == SAR_F32 ? (const void*)sar_noalloc_kernel<float>
                 : dtype == SAR_BF16 ? (const void*)sar_noalloc_kernel<__nv_bfloat16>
                                     : (const void*)sar_noalloc_kernel<__half>;
  e = cudaLaunchCooperativeKernel(fn, dim3(n * blocks_per_rank), dim3(512), args, 0, st);
  if (e != cudaSuccess) return fail(err, errlen, (int)e, cudaGetErrorString(e));
  return 0;
}
