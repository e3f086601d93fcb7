// Symmetric buffers for the single-process communicator, with optional NVLink
// multicast (NVLS) views.
//
// A symmetric allocation is one buffer of the same size on every rank's device.
// With multicast, the buffers are created with the virtual memory API, bound at
// offset 0 to a multicast object over all ranks (group 0) and, optionally, to a
// second object over a subset of the ranks (group 1, e.g. the non-stragglers),
// and every member rank gets a mapping of each object.  A multimem.ld_reduce on
// such a mapping returns the sum over the members' buffers, a multimem.st writes
// all of them: the switch does the reduction and the replication, and a rank
// moves S bytes per direction for an AllReduce of S bytes instead of 2 S (n-1)/n.
//
// The driver entry points are looked up at run time (cudaGetDriverEntryPoint),
// so the library has no link-time dependency on the driver and loads on machines
// without one.  The reference has no counterpart: it reaches NVLS only through
// NCCL's own algorithms (ncclReduceScatter / ncclAllReduce on its sub-communicator,
// stragglar/allreduce_8GPU.cu:132,893).
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "../core/table.h"

namespace sar {

struct SymmAlloc {
  int n = 0;
  size_t bytes = 0;                      // usable bytes per rank (as requested)
  size_t mapped = 0;                     // bytes mapped per rank (rounded up to the granularity)
  int dev[SAR_MAX_RANKS] = {};
  void* uc[SAR_MAX_RANKS] = {};          // rank r's buffer (accessible from every rank's device)
  bool vmm = false;                      // created with the virtual memory API (else cudaMalloc)
  // multicast groups: 0 = all ranks, 1 = `members[1]`
  uint32_t members[2] = {0, 0};
  void* mc[2][SAR_MAX_RANKS] = {};       // rank r's mapping of group g (nullptr: none)
  // opaque driver handles
  unsigned long long mem_handle[SAR_MAX_RANKS] = {};
  unsigned long long mc_handle[2] = {0, 0};
  bool bound[2][SAR_MAX_RANKS] = {};
};

enum SymmMode {
  SYMM_PLAIN = 0,       // cudaMalloc on every device
  SYMM_MULTICAST = 1,   // virtual memory + multicast; an error if the devices or the driver do not offer it
  SYMM_TRY_MULTICAST = 2,  // multicast when available, else plain
};

// 1 when every listed device reports multicast support and the driver entry points exist.
bool multicast_supported(int n, const int* devices);

// Allocates `bytes` on every device.  `sub_members`: ranks of the second multicast group (0: none).
// Returns 0 on success; on failure everything created so far is released and `err` says why.
int symm_alloc(SymmAlloc* a, int n, const int* devices, size_t bytes, int mode, uint32_t sub_members, char* err, int errlen);
void symm_free(SymmAlloc* a);

}  // namespace sar
