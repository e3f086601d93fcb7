// Round table: the device-resident form of a collective schedule.
//
// A collective on n ranks over a buffer of `count` elements is a list of ops
// per rank.  The buffer is cut into `num_chunks` chunks (n-1 for StragglAR,
// n for ring / halving-doubling); a chunk is cut into tiles of `tile_elems`
// elements.  Every op works on one chunk (or on one of `parts` equal tile
// ranges of it) and is executed tile by tile by the rank that owns the table.
// Reductions are *pulls* (the executing rank loads its peers' tiles), which makes
// them safe in place without temporary buffers; copies are pulls or pushes.
//
//   SAR_COPY         own[chunk] = peer[chunk]
//   SAR_REDUCE       own[chunk] = (own[chunk] +) sum over nsrc peers
//   SAR_REDUCE_PUSH  own[chunk] = peer[chunk] = own[chunk] + peer[chunk]
//                    (the executing rank also stores the sum into the peer)
//   SAR_PUSH         peer[chunk] = own[chunk] for nsrc peers (a copy executed by
//                    its source: posted stores instead of loads over the link;
//                    the source polls its own flags, loads a tile once and
//                    stores it to every destination, whose flags it sets remotely)
//
// Synchronisation is one 32-bit flag per (rank, chunk, tile), living in the
// memory of the rank that owns the slot.  A flag holds `epoch_base + version`,
// where the version counts how often the slot was rewritten in this
// collective (0 = the caller's input) and `epoch_base` grows by
// SAR_VER_STRIDE per collective, so flags never need clearing.  An op names,
// for every operand, the version it needs; version 0 of a peer slot is covered
// by that peer's arrival word.  The table is independent of `count`: tile
// ranges are derived from the chunk geometry at launch.
//
// The helpers below are shared by the CUDA kernels and the host executor so
// that both walk a table in exactly the same order.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define SAR_HD __host__ __device__ __forceinline__
#else
#define SAR_HD inline
#endif

#define SAR_MAX_RANKS 16
#define SAR_MAX_CHUNKS 16
#define SAR_MAX_OPS 256
#define SAR_MAX_ROUNDS 64
// Trace words of a launch (uint64, %globaltimer ns): [0] arrival, [1] end; with round tracing on,
// three arrays of SAR_MAX_ROUNDS follow: first item started, last item announced, time spent
// waiting for operands (summed over the items of the round).
#define SAR_TRACE_WORDS (2 + 3 * SAR_MAX_ROUNDS)
#define SAR_VER_STRIDE 32u
#define SAR_NUM_CHANNELS 4               // independent flag/control sets (0: all ranks, 1: the non-stragglers)
#define SAR_FLAG_CAPACITY (1u << 18)     // flags per rank and channel
#define SAR_VEC_BYTES 16

enum SarOpKind : uint8_t { SAR_COPY = 0, SAR_REDUCE = 1, SAR_REDUCE_PUSH = 2, SAR_PUSH = 3,
                           // Never in a table: the executors add them around a table when the caller's tensor is not the
                           // buffer that peers can reach.  STAGE_IN copies a tile of the caller's input into the own
                           // slot (casting to the wire type) and announces it as version 0; STAGE_OUT copies a tile
                           // whose slot has reached its final version into the caller's output (casting back).
                           SAR_STAGE_IN = 4, SAR_STAGE_OUT = 5 };
enum SarOpFlag : uint8_t {
  SAR_F_SCALE = 1,  // multiply the result by the launch's scale (fused AVG / pre-division)
  SAR_F_LOCAL = 2,  // REDUCE: the own slot is one of the addends
};
enum SarDtype : int32_t { SAR_F32 = 0, SAR_BF16 = 1, SAR_F16 = 2 };

// status codes written to the launch's status word (0 = ok)
enum SarStatus : uint32_t {
  SAR_OK = 0,
  SAR_TIMEOUT_ARRIVAL = 1,   // a peer never entered the collective
  SAR_TIMEOUT_FLAG = 2,      // a tile some op depends on never became ready
  SAR_TIMEOUT_EXIT = 3,      // a peer never left the collective
  SAR_TIMEOUT_PIPE = 4,      // an on-chip pipeline barrier never completed
  SAR_BAD_TABLE = 5,
  SAR_ABORTED = 6,           // another block of this rank gave up first
};

struct SarOp {
  uint8_t kind;        // SarOpKind
  uint8_t flags;       // SarOpFlag bits
  uint8_t round;       // schedule round (ops of a rank are sorted by it)
  uint8_t chunk;
  uint8_t part;        // this op covers tile range `part` of `parts`
  uint8_t parts;
  uint8_t nsrc;        // peers read (1 for COPY / REDUCE_PUSH); PUSH: the destinations src[0..nsrc)
  uint8_t local_ver;   // version the own slot must have before it is read or overwritten
  uint8_t post_ver;    // version of the own slot after this op
  uint8_t push_ver;    // REDUCE_PUSH / PUSH: version of the peer slot after this op
  uint8_t lane;        // 0 or 1: which group of blocks executes the op (see sar_lane_of_block)
  uint8_t pad;
  uint8_t src[SAR_MAX_RANKS];      // peer ranks (physical)
  uint8_t src_ver[SAR_MAX_RANKS];  // version needed of each peer's slot (PUSH: the version it replaces)
};
static_assert(sizeof(SarOp) == 12 + 2 * SAR_MAX_RANKS, "SarOp layout");

// Control words of one rank (in its own memory, read by peers).
struct SarCtrl {
  uint32_t arrival;    // epoch_base of the newest collective this rank has entered
  uint32_t exited;     // epoch_base of the newest collective this rank has left
  uint32_t abort_flag; // set by any block that timed out; makes the others return
  uint32_t blocks_done;// local counter to find the last block of a launch
  // round gating (local words, reset by the last block of a launch): items this rank has finished in
  // the launch, and the newest round it has announced to its peers
  uint32_t items_done;
  uint32_t announced;
  uint32_t reserved[26];
  // round gating: gate[q] is written by rank q into THIS rank's memory (so that waiting for a round
  // polls local memory only) and holds gate_base + R once rank q has finished its items of every
  // round before R.  64-bit and raised with a max-reduction: announcements of different rounds may
  // overtake one another on the way, and the value never wraps.
  uint64_t gate[SAR_MAX_RANKS];
  // Mirrors, written by the other ranks into THIS rank's memory so that waiting polls local memory instead of
  // crossing the link once per peer: arrival_m[q] / exited_m[q] = rank q's `arrival` / `exited` word.  The CUDA
  // kernels write and read the mirrors; the host executor, whose ranks share host memory, reads the words themselves.
  uint32_t arrival_m[SAR_MAX_RANKS];
  uint32_t exited_m[SAR_MAX_RANKS];
};
static_assert(sizeof(SarCtrl) == 384, "SarCtrl layout");
#define SAR_CTRL_WORDS (sizeof(SarCtrl) / 4)
// Round gating.  The rounds of a matching-based schedule are contention-free one at a time: in
// every round a rank sends at most one chunk and receives at most one.  When the rounds overlap
// freely, a rank that holds a finished chunk serves the readers of several rounds at once, each
// at a fraction of the link rate, and what depends on them is late.  With gating, an item of
// round r >= 1 starts only when every participant has announced r, i.e. has finished its items of
// all rounds before r (a rank without items in a round skips it when it announces).  The first
// round is not gated: a pre-phase among the early ranks must not wait for a late rank's arrival.
// With `gate_slack` = 0 the gate is a full barrier between rounds, every operand of a gated item is
// known to be complete, and the item skips its flag waits (no polling of peer memory at all);
// with a slack of s items a rank announces a round when all but s of the items before it are
// done, the tail of a round overlaps the head of the next, and items wait for their flags as
// usual.  Tiles still pipeline inside a round.  SAR_GATE_ALL_DONE is announced after the last
// round; it bounds the number of rounds a gated table may have (< SAR_VER_STRIDE).
#define SAR_GATE_ALL_DONE 31u

// Chunk geometry for `count` elements of `esize` bytes in `num_chunks` chunks.
// Chunks are contiguous, start on 16-byte boundaries and differ by at most one
// 16-byte vector; the sub-vector tail of the buffer belongs to the last chunk.
struct SarGeom {
  uint64_t count;
  uint32_t esize;
  uint32_t num_chunks;
  uint32_t tile_elems;       // multiple of the vector width
  uint32_t tiles_per_chunk;  // max over chunks (flag stride)
};

SAR_HD uint64_t sar_chunk_begin(const SarGeom& g, uint32_t c) {
  const uint64_t vw = SAR_VEC_BYTES / g.esize;
  const uint64_t nvec = g.count / vw;
  const uint64_t q = nvec / g.num_chunks, r = nvec % g.num_chunks;
  if (c >= g.num_chunks) return g.count;
  return (q * c + (c < r ? c : r)) * vw;
}
SAR_HD uint64_t sar_chunk_len(const SarGeom& g, uint32_t c) {
  return sar_chunk_begin(g, c + 1) - sar_chunk_begin(g, c);
}
SAR_HD uint32_t sar_chunk_tiles(const SarGeom& g, uint32_t c) {
  const uint64_t len = sar_chunk_len(g, c);
  return (uint32_t)((len + g.tile_elems - 1) / g.tile_elems);
}
// tile range [t0, t1) of chunk tiles covered by part `part` of `parts`
SAR_HD void sar_part_range(uint32_t tiles, uint32_t part, uint32_t parts, uint32_t* t0, uint32_t* t1) {
  *t0 = (uint32_t)(((uint64_t)tiles * part) / parts);
  *t1 = (uint32_t)(((uint64_t)tiles * (part + 1)) / parts);
}
SAR_HD uint32_t sar_op_tiles(const SarGeom& g, const SarOp& op) {
  uint32_t t0, t1;
  sar_part_range(sar_chunk_tiles(g, op.chunk), op.part, op.parts, &t0, &t1);
  return t1 - t0;
}
SAR_HD uint32_t sar_flag_index(const SarGeom& g, uint32_t chunk, uint32_t tile) {
  return chunk * g.tiles_per_chunk + tile;
}
// Lanes.  A table may put its ops in two lanes (0: reductions and straggler
// matchings, 1: forwarding of finished chunks).  The blocks of a rank are then
// split between the lanes and every lane walks its own ops in round order, so
// that forwarding overlaps the matchings instead of queueing behind them in
// the same blocks.  With a single block (or a one-lane table) there is one
// lane that walks every op.
// `lane1_eighths` is the share of the blocks that lane 1 gets, in eighths (0 or 4: half, the
// blocks alternate between the lanes; otherwise lane 0 takes the first blocks and lane 1 the rest,
// at least one block each).
SAR_HD void sar_lane_of_block(uint32_t block, uint32_t nblocks, uint32_t table_lanes, uint32_t lane1_eighths, uint32_t* lanes,
                              uint32_t* lane, uint32_t* lane_block, uint32_t* lane_nblocks) {
  const uint32_t L = (table_lanes >= 2 && nblocks >= 2) ? 2u : 1u;
  *lanes = L;
  if (L == 1 || lane1_eighths == 0 || lane1_eighths == 4) {
    *lane = block % L;
    *lane_block = block / L;
    *lane_nblocks = (nblocks - *lane + L - 1) / L;
    return;
  }
  uint32_t n1 = (nblocks * (lane1_eighths > 7 ? 7u : lane1_eighths) + 4) / 8;
  if (n1 < 1) n1 = 1;
  if (n1 > nblocks - 1) n1 = nblocks - 1;
  const uint32_t n0 = nblocks - n1;
  *lane = block < n0 ? 0u : 1u;
  *lane_block = block < n0 ? block : block - n0;
  *lane_nblocks = block < n0 ? n0 : n1;
}
// wrap-safe "flag has reached target"
SAR_HD bool sar_reached(uint32_t flag, uint32_t target) { return (int32_t)(flag - target) >= 0; }

// Work items of one rank.  The ops of one round (of one lane) are interleaved
// tile by tile: item k of a round with m ops is tile k/m of op k%m (items whose
// op has run out of tiles are skipped), and rounds follow one another.  Block b
// of the G blocks of a lane executes the items b, b+G, b+2G, ... in this order,
// which keeps a rank's blocks on the same round and lets every op of a round
// progress at the same rate.  Items only depend on items of earlier rounds, so
// walking them in this order on co-resident blocks cannot deadlock.
