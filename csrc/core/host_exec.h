// Host executor of round tables.
//
// Walks a rank's table exactly as the CUDA kernels do (same item order, same
// flag protocol with epochs, arrival and exit words, bounded waits), but with
// host threads and std::atomic flags.  It is the CPU oracle for the kernels,
// lets the flag protocol be exercised under real concurrency on a machine
// without a GPU, and backs the c10d backend for CPU tensors (ranks in
// different processes share the flag and data arenas through POSIX shm).
#pragma once
#include <atomic>
#include <cstdint>

#include "plan.h"
#include "table.h"

namespace sar {

struct HostRankView {           // what one rank can see of every rank
  int rank = 0, nranks = 0;
  void* buf[SAR_MAX_RANKS] = {};                       // data buffers (same layout on every rank)
  std::atomic<uint32_t>* flags[SAR_MAX_RANKS] = {};    // the launch's channel: SAR_FLAG_CAPACITY words each
  std::atomic<uint32_t>* ctrl[SAR_MAX_RANKS] = {};     // the launch's channel: laid out as SarCtrl
};

struct HostLaunch {
  SarGeom geom{};
  SarDtype dtype = SAR_F32;
  float scale = 1.0f;
  uint32_t epoch_base = SAR_VER_STRIDE;   // must grow by SAR_VER_STRIDE per collective
  double timeout_s = 10.0;
  double delay_ms = 0.0;                  // sleep before arriving (an injected straggler delay)
  uint32_t participants = 0;              // ranks that run this collective (exit barrier set)
  bool gate_rounds = false;               // rounds one after the other (every rank of the launch must agree)
  uint32_t gate_slack = 0;                // items of a round that may still run when the next round opens (0: full barrier)
  uint64_t gate_base = SAR_VER_STRIDE;    // stands for round 0 of this launch; grows with epoch_base and never wraps
  uint32_t lane1_eighths = 4;             // share of the blocks of lane 1 (see sar_lane_of_block)
};

// Executes block `block` of `nblocks` of this rank's table.  Every block of
// every rank must be run (concurrently).  Returns a SarStatus.
uint32_t host_run_block(const HostRankView& v, const RankTable& t, const HostLaunch& l, int block, int nblocks);

// Convenience: all ranks in this process, `blocks` threads per rank.
// bufs[r] is rank r's buffer of `count` elements.  delay_ms may be null.
uint32_t host_execute(const Compiled& c, void* const* bufs, uint64_t count, SarDtype dtype, uint32_t tile_elems,
                      float scale, int blocks, const double* delay_ms, double timeout_s, int repeats);

// A whole program (one or two phases), every rank's phases in stream order.
uint32_t host_execute_program(const Program& p, void* const* bufs, uint64_t count, SarDtype dtype, uint32_t tile_elems,
                              float scale, int blocks, const double* delay_ms, double timeout_s);

// Round gating costs a hand-shake per round and pays once a round's chunk takes much longer than that on the
// link: a gated table is launched with gating for buffers of at least this many bytes (STRAGGLAR_GATE_MIN_BYTES,
// default 128 MiB; measured on 8 x B200: gated rounds win at 256 MiB and 1 GiB and lose at 64 MiB).  Every rank of
// a launch sees the same size, hence the same answer.
uint64_t gate_min_bytes();
// Items of a round that may still be running when the next round opens: STRAGGLAR_GATE_SLACK if set (0 = full
// barrier between rounds), else three tenths of a chunk's tiles, the middle of a flat optimum measured on 8 x B200
// (1 GiB: 2.17-2.25 ms for slacks of 5-45 % of a chunk against 2.33-2.40 ms with the full barrier).
uint32_t gate_slack(uint32_t tiles_per_chunk);
// Upper bound of the tile size of a gated launch on the GPU: with the rounds kept apart there is little to gain
// from fine-grained pipelining across rounds, and larger tiles mean fewer flag polls over the link.
inline uint32_t gate_tile_bytes() { return 256u << 10; }

uint32_t pick_tile_elems(uint64_t count, uint32_t esize, uint32_t num_chunks, uint32_t blocks, uint32_t min_bytes,
                         uint32_t max_bytes);
SarGeom make_geom(uint64_t count, uint32_t esize, uint32_t num_chunks, uint32_t tile_elems);

}  // namespace sar
