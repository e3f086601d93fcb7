// Single-process communicator: n ranks driven by one host thread, either one
// rank per CUDA device (peer access over NVLink) or all ranks emulated on one
// device by a single cooperative launch (tests and profiling on one GPU).
// Used by the allreduce / reducescatter benchmark programs and, through
// ctypes, by the Python tests.  The multi-process equivalent lives in the
// c10d backend and shares the kernels.
#pragma once
#include <stdint.h>

#include "../core/c_api.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct sar_local_comm sar_local_comm;

struct sar_run_opts {
  int path;               // SAR_PATH_SIMT / SAR_PATH_TMA
  int blocks;             // thread blocks per rank (<= 0: default of the path)
  int threads;            // simt path: threads per block (<= 0: 512)
  uint32_t tile_bytes;    // upper bound of the tile size (0: 128 KiB)
  double timeout_s;       // bound of every device-side wait (<= 0: 10 s)
  float scale;            // fused multiplier of the result
  int timed;              // 1: bracket every rank's work with events after a device-side start barrier
};

// devices[r] is the CUDA device of rank r.  emulate != 0 places every rank on
// devices[0] and runs collectives as one cooperative launch.
sar_local_comm* sar_local_create(int n, const int* devices, int emulate, char* err, int errlen);
void sar_local_destroy(sar_local_comm* c);
int sar_local_nranks(const sar_local_comm* c);
void* sar_local_stream(sar_local_comm* c, int rank);
// Enqueues the program on every participating rank.  bufs[r] is rank r's buffer
// (count elements of dtype, 16-byte aligned).  delay_ns may be NULL; a non-zero
// entry delays that rank on the device before its first phase.  Returns 0 or a
// cudaError_t; err receives a message.
int sar_local_run(sar_local_comm* c, const sar_program* prog, void* const* bufs, uint64_t count, int dtype,
                  const struct sar_run_opts* opts, const uint64_t* delay_ns, char* err, int errlen);
// Waits for all ranks; fills ms[r] with rank r's device time of the last timed
// run (if ms != NULL) and returns the worst SarStatus over ranks (0 = ok),
// clearing the failure state so that the communicator can be used again.
uint32_t sar_local_sync(sar_local_comm* c, float* ms);
// per rank: %globaltimer stamps {arrival, end} of the last phase it ran
int sar_local_trace(sar_local_comm* c, uint64_t* out /* 2*n */);

#ifdef __cplusplus
}
#endif
