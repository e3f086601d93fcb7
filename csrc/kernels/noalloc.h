// An AllReduce entry point for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference.
//
// Some hosts of this library are not allowed to call cudaMalloc: code that
// runs inside another framework's memory budget (every byte on the device is
// owned by that framework's allocator), plugins loaded into a process whose
// CUDA context has no memory headroom left, and tools that must not disturb
// the allocation pattern of the program they are attached to.  The regular
// entry points (sar_local_run, the c10d backend) allocate their flag arrays,
// control words and device copies of the op tables with cudaMalloc.  This
// variant keeps all of that scratch in one file-scope device array of
// SAR_NOALLOC_SCRATCH_BYTES (1 MiB) that is part of the library image: every
// GPU that loads the library holds it until the process exits.  The caller
// passes only its own input/output buffers.
#pragma once
#include <stdint.h>

#include "../core/c_api.h"

#ifdef __cplusplus
extern "C" {
#endif

#define SAR_NOALLOC_SCRATCH_BYTES (1u << 20)
#define SAR_NOALLOC_MAX_RANKS 8
#define SAR_NOALLOC_MAX_TILES 16384u   // flag words per rank

// Runs the single-phase collective `table` for all of its ranks (at most
// SAR_NOALLOC_MAX_RANKS) on the CURRENT device in one cooperative launch on
// `stream`: bufs[r] is rank r's buffer of `count` elements of `dtype`
// (SarDtype), reduced in place; `scale` multiplies the result where the table
// says so.  Same kernel code as the emulated mode of sar_local_run (simt data
// path), but flags, control words, launch parameters and the device copy of
// the op table live in the static scratch array.
//
// Returns 0, or a non-zero code with a message in `err`: 1 = bad argument
// (this includes a call made while `stream` is being captured, see below),
// 2 = the request does not fit the scratch array (too many ranks, or a buffer
// that needs more than SAR_NOALLOC_MAX_TILES tiles of 1 MiB per rank, all
// chunks together), other values = a cudaError_t.  It calls no cudaMalloc,
// cudaFree or allocating library routine.
//
// The first call on a device looks up the scratch array's device address
// (cudaGetSymbolAddress); make that first call before any stream capture.
// The entry point itself must not be called while `stream` is capturing: it
// copies its launch parameters and the op table from host memory that is only
// valid during the call, so a captured copy would read freed memory when the
// graph runs.  Such a call is refused with code 1 and nothing is enqueued.
// All calls on a device share the array, which keeps the previous call's
// contents: the words that must start at zero are cleared on `stream` at the
// start of every call, so calls that overlap on the GPU (different streams,
// no ordering between them) race and must not be issued.
// *device_status (optional, device memory owned by the caller, 4 bytes, zeroed
// by the caller) receives a SarStatus if a device-side wait runs out.
int sar_emulated_allreduce_noalloc(const sar_table* table, void* const* bufs, uint64_t count, int dtype, float scale,
                                   int blocks_per_rank, uint32_t* device_status, void* stream, char* err, int errlen);

#ifdef __cplusplus
}
#endif
