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
  int trace_rounds;       // 1: keep per-round statistics of this run (see sar_local_round_trace)
  int stages;             // bulk-copy path: shared-memory ring stages per block (<= 0: all six)
  int store_window;       // bulk-copy path: store groups a block keeps in flight: 3, 8 or 16 (<= 0: default)
  // Staged mode (single-phase programs): bufs[r] only serves as the buffer peers can reach; rank r's input is read
  // from user_in[r] and its result written to user_out[r] (elements of user_dtype, converted to and from the
  // collective's dtype) by the collective kernel itself.  NULL: off.
  void* const* user_in;
  void* const* user_out;
  int user_dtype;
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
// Per rank and schedule round of the last run made with trace_rounds = 1 (all phases of the
// program together): out[(r * 3 + k) * SAR_MAX_ROUNDS + round] with k = 0: %globaltimer ns when the
// round's first item started (UINT64_MAX: the rank had none), 1: when its last item was announced,
// 2: ns the round's items spent waiting for their operands, summed over the items.
int sar_local_round_trace(sar_local_comm* c, uint64_t* out /* n * 3 * SAR_MAX_ROUNDS */);

// Symmetric buffers: `bytes` on every rank's device, bufs[r] = rank r's.  mode 0: plain device
// memory; 1: virtual-memory allocations bound to NVLink multicast objects (an error where the
// devices or the driver do not offer multicast, or when the ranks share a device); 2: multicast
// when available, else plain.  `sub_members` names the ranks of a second multicast group (e.g. the
// non-stragglers; 0: none).  When a collective runs on the simt path over buffers that lie at the
// same offset inside such an allocation, reductions over and pushes to all members of a group go
// through the switch (multimem.ld_reduce / multimem.st) instead of one transfer per peer.
int sar_local_alloc(sar_local_comm* c, size_t bytes, int mode, uint32_t sub_members, void** bufs, char* err, int errlen);
// Frees the allocation whose rank-0 buffer is buf0 (after waiting for the devices).  0 if found.
int sar_local_free(sar_local_comm* c, void* buf0);
// Bit g set: multicast group g (0: all ranks, 1: sub_members) serves the allocation holding buf0.
int sar_local_multicast_groups(sar_local_comm* c, const void* buf0);
// 1 when every device of the communicator offers NVLink multicast (and the ranks do not share devices)
int sar_local_multicast_supported(sar_local_comm* c);

#ifdef __cplusplus
}
#endif
