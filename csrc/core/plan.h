// Collective plans and the schedule compiler.
//
// A Plan is a rank-symmetric description of a collective: a list of steps,
// each in a round, each moving or reducing one chunk.  Plans are produced
// from a synthesized StragglAR schedule (text in the synthesizers' printed
// format) or by the generators for ring, recursive halving-doubling, direct
// and reduce-scatter.  compile() proves a plan correct (every rank ends with
// the full sum, no slot is overwritten while a peer may still read it) and
// lowers it into one SarOp table per physical rank.
//
// The reference has no such component: its schedules are unrolled by hand
// into ncclSend/ncclRecv calls (stragglar/allreduce_8GPU.cu:555-874,
// implementation/custom_backend/src/dummy.cpp:256-658).
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "table.h"

namespace sar {

struct Matching {
  enum Kind { Straggler, OneWay, TwoWay } kind;
  int a, b;        // Straggler: rank a <-> straggler b; OneWay: a -> b; TwoWay: a -> b and b -> a
  int chunk_a;     // chunk sent by a (Straggler: the reduced chunk)
  int chunk_b;     // TwoWay: chunk sent by b
};

struct Schedule {
  int n = 0;
  std::vector<std::vector<Matching>> rounds;
};

// Parses the synthesizers' printed format; only "Round" headers and the
// matching list that follows each are used.
Schedule parse_schedule(const std::string& text);
std::string format_schedule_compact(const Schedule& s);
// Schedules shipped with the library (n = 2, 4, 6, 8, 10, 12, 16); throws for other n.
Schedule builtin_schedule(int n);

enum class StepKind : uint8_t { Copy, Reduce, Exchange };

struct Step {
  int round = 0;
  StepKind kind = StepKind::Copy;
  int chunk = 0;
  int dst = 0;                 // executing rank (Exchange: first side)
  std::vector<int> srcs;       // peers read (Exchange: the second side)
  bool include_local = true;   // Reduce: dst's own slot is an addend
  bool finalize = false;       // result is the final sum: the fused scale applies here
};

enum class Expect : uint8_t { AllReduce, ReduceScatter };

struct Plan {
  std::string name;
  int n = 0;            // ranks (logical)
  int num_chunks = 0;
  std::vector<Step> steps;
  // init[rank][chunk]: bitmask of the ranks whose contribution the slot holds
  // when the collective starts (0 = content is never read)
  std::vector<std::vector<uint32_t>> init;
  std::vector<int> participants;  // ranks whose result is checked
  Expect expect = Expect::AllReduce;
  bool push_copies = false;       // lower Copy steps as SAR_PUSH (executed by the source) instead of SAR_COPY
  int blocks_hint = 0;            // largest block count per rank worth using (0: no preference)
  int stages_hint = 0;            // bulk-copy path: ring stages per block this plan runs best with (0: all)
  bool gate_rounds = false;       // run the rounds one after the other (see SAR_GATE_ALL_DONE in table.h)
  int lane1_eighths = 4;          // two lanes: share of the blocks that forwarding (lane 1) gets, in eighths
  bool two_lanes = false;         // forwarding ops go to lane 1 (their own blocks), the rest to lane 0
  bool split_copies = false;      // forward a chunk as two half-chunk ops, interleaved tile by tile, so that
                                  // forwarding follows both halves of a straggler matching as they are produced
  int num_rounds() const;
};

// StragglAR: optional (n-1)-rank reduce-scatter pre-phase (round 0), then the
// schedule's rounds.  With prephase=false the caller guarantees that rank i
// already holds the partial sum of ranks 0..n-2 in chunk i.
Plan plan_stragglar(const Schedule& s, bool prephase);
// StragglAR on an any-to-any switch: after the pre-phase every rank i reduces
// chunk i with the straggler at the same time (tile-interleaved) and the final
// chunks are all-gathered directly among the n-1 others.
Plan plan_stragglar_a2a(int n, bool prephase);
Plan plan_ring(int n);
Plan plan_rhd(int n);                       // n a power of two
Plan plan_direct(int n, bool prephase);
Plan plan_reduce_scatter(int n);            // rank i ends with the sum of chunk i (n chunks)
Plan plan_rsag(int n);                      // one-shot reduce-scatter + all-gather
Plan plan_by_name(const std::string& alg, int n, bool prephase, const Schedule* sched = nullptr);
// Lowering used for algorithms without a measured preference (STRAGGLAR_COPY / STRAGGLAR_LANES override).
bool default_push_copies();
bool default_two_lanes();

struct RankTable {
  std::vector<SarOp> ops;
  std::vector<uint16_t> round_begin;  // ops [round_begin[i], round_begin[i+1]) form the i-th non-empty round
  std::vector<uint8_t> final_ver;     // per chunk: version of this rank's slot when the collective is done
};

struct Compiled {
  std::string name;
  int n = 0;              // physical ranks of the communicator (tables of non-participants are empty)
  int channel = 0;        // which flag/control set the collective uses
  uint32_t participants = 0;  // bitmask of physical ranks that take part (and must launch)
  int num_chunks = 0;
  int max_version = 0;
  int num_rounds = 0;
  int blocks_hint = 0;    // upper bound of the blocks per rank this table runs best with (0: none)
  int stages_hint = 0;    // bulk-copy path: ring stages per block (0: all); fewer stages keep fewer bytes in flight
  bool gate_rounds = false;   // launch with round gating (every rank of a launch must agree)
  int lane1_eighths = 4;      // share of the blocks of lane 1, in eighths (see sar_lane_of_block)
  std::vector<RankTable> ranks;          // by physical rank
  std::vector<int> logical_to_physical;
  // per-rank traffic in chunks (for rooflines): chunks read from peers, chunks written to peers
  std::vector<double> chunks_in, chunks_out;
};

struct CompileError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// logical_to_physical may be empty (identity); it may also map the plan's
// ranks onto a subset of `n_physical` ranks (a sub-communicator).  Throws
// CompileError when the plan is wrong: bad ranks/chunks, double counting, a
// read of garbage, a slot written twice in a round, a write that is not
// ordered after every read of the value it destroys, or a result that is not
// the expected one.
Compiled compile(const Plan& plan, const std::vector<int>& logical_to_physical = {}, int n_physical = 0);

// Structural check of a rank's table before it is handed to a kernel: op kinds, chunk and peer
// indices in range, no peer named twice or equal to the rank itself, tile ranges well-formed,
// rounds sorted and covered by round_begin, sizes within what the kernels hold in shared memory.
// The data a table came from was hazard-checked by compile(); this catches a table that was
// damaged or built for another communicator on its way to the device.  Returns "" or the reason.
std::string validate_rank_table(const RankTable& t, int rank, int nranks, int num_chunks);

// A collective as the user names it: one or two compiled phases launched back
// to back.  Everything is a single phase except `direct` with its pre-phase,
// where the non-stragglers first all-reduce among themselves on channel 1
// (the straggler takes no part and is not waited for) and all ranks then run
// the exchange and broadcast on channel 0.
struct Program {
  std::string alg;
  int n = 0;
  std::vector<Compiled> phases;
};
// straggler: physical rank that plays logical rank n-1, or -1 for rank n-1.
Program build_program(const std::string& alg, int n, bool prephase, int straggler, const Schedule* sched = nullptr);

// rank map that places `physical_straggler` at logical rank n-1 by swapping it
// with physical rank n-1 (cf. implementation/custom_backend/src/dummy.cpp:157-168,
// where the same swap is done by remapping CUDA devices).
std::vector<int> straggler_rank_map(int n, int physical_straggler);

}  // namespace sar
