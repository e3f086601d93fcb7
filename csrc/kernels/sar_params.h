// Launch parameters of the table-executing kernels (plain data, shared by
// host and device code).
#pragma once
#include <stdint.h>

#include "../core/table.h"

struct SarDevComm {
  uint32_t* flags[SAR_MAX_RANKS];  // this collective's channel of every rank's flag array
  SarCtrl* ctrl[SAR_MAX_RANKS];    // this collective's channel of every rank's control words
  void* buf[SAR_MAX_RANKS];        // every rank's data buffer (same layout)
};

// An NVLink multicast (NVLS) view of the data buffers: `base` is this rank's mapping of a
// multicast object to which the buffers of the ranks in `members` are bound at the same offsets,
// so that one multimem.ld_reduce at base + x returns the sum of the members' values at x and one
// multimem.st writes all of them.  base == nullptr: not available.
struct SarMcGroup {
  void* base;
  uint32_t members;
  uint32_t pad;
};

struct SarLaunchParams {
  SarDevComm comm;
  const SarOp* ops;
  const uint16_t* round_begin;  // num_rounds + 1 entries
  uint32_t num_rounds;
  SarGeom geom;
  int32_t rank, nranks;
  uint32_t participants;
  uint32_t epoch_base;
  float scale;
  int32_t dtype;
  uint64_t timeout_ns;
  uint32_t* status;       // first failure of this launch (0 = ok); may be mapped host memory
  uint64_t* trace;        // optional: [0] = arrival time, [1] = end time (%globaltimer ns), else nullptr
  uint32_t trace_rounds;  // != 0: trace holds SAR_TRACE_WORDS words and the per-round statistics are kept
  uint32_t gate_rounds;   // != 0: the rounds run one after the other (every rank of the launch agrees; see table.h)
  uint32_t lane1_eighths; // share of the blocks of lane 1, in eighths (0 or 4: half; see sar_lane_of_block)
  uint32_t gate_slack;    // round gating: items of a round that may still be running when the next round opens
  uint64_t gate_base;     // round gating: value that stands for round 0 of this launch (grows by >= 32 per launch)
  uint32_t stages;        // bulk-copy path: ring stages in use (0 or > the ring size: all)
  uint32_t store_window;  // bulk-copy path: store groups a block keeps in flight (3, 8 or 16; 0: 3)
  // Staged mode (all three null/zero: off).  The caller's tensor is not reachable by peers: the kernel itself copies
  // it tile by tile into this rank's buffer before the table's ops (announcing every tile as version 0 through its
  // flag, so that nobody waits for the whole copy) and copies every tile that has reached its final version out
  // again, converting between the caller's element type and the wire type on the way.  Every rank of the
  // collective must run in the same mode: in staged mode version 0 of a peer's tile is waited for through the
  // tile's flag, otherwise through the peer's arrival word.
  const void* user_in;
  void* user_out;
  int32_t user_dtype;     // SarDtype of user_in / user_out
  uint8_t final_ver[SAR_MAX_CHUNKS];   // version of this rank's slot of every chunk when the table is done
  uint32_t staging_blocks; // blocks of the launch (the last ones) that only stage; 0: a quarter of the blocks
  uint64_t delay_ns;      // spin this long before arriving (a late rank when ranks share one launch)
  SarMcGroup mc[2];       // multicast views (simt path): all ranks, and e.g. the non-stragglers
};

