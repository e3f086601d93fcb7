// Plan generators, schedule text parser and the schedule compiler.
#include "plan.h"

#include <algorithm>
#include <bitset>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <sstream>

namespace sar {

// ---------------------------------------------------------------- text format
static bool read_int(const std::string& s, size_t& i, int& out) {
  while (i < s.size() && !isdigit((unsigned char)s[i])) ++i;
  if (i >= s.size()) return false;
  long v = 0;
  while (i < s.size() && isdigit((unsigned char)s[i])) v = v * 10 + (s[i++] - '0');
  out = (int)v;
  return true;
}

Schedule parse_schedule(const std::string& text) {
  Schedule sch;
  std::istringstream in(text);
  std::string line;
  bool expect_list = false;
  int max_rank = -1;
  while (std::getline(in, line)) {
    size_t p = line.find_first_not_of(" \t\r");
    if (p == std::string::npos) continue;
    if (line.compare(p, 6, "Round ") == 0) { expect_list = true; continue; }
    if (line.compare(p, 4, "GPU ") == 0) {
      size_t i = p; int g;
      if (read_int(line, i, g)) max_rank = std::max(max_rank, g);
      continue;
    }
    if (!expect_list) continue;
    expect_list = false;
    std::vector<Matching> rnd;
    size_t pos = 0;
    while (true) {
      size_t s = line.find("Matching:", pos);
      if (s == std::string::npos) break;
      // the word before "Matching:" tells the kind
      Matching m{};
      size_t i = s + 9;
      if (s >= 9 && line.compare(s - 9, 9, "Straggler") == 0) {
        m.kind = Matching::Straggler;
        if (!read_int(line, i, m.a) || !read_int(line, i, m.b) || !read_int(line, i, m.chunk_a))
          throw std::runtime_error("bad StragglerMatching: " + line);
        m.chunk_b = m.chunk_a;
      } else if (s >= 6 && line.compare(s - 6, 6, "OneWay") == 0) {
        m.kind = Matching::OneWay;
        if (!read_int(line, i, m.a) || !read_int(line, i, m.b) || !read_int(line, i, m.chunk_a))
          throw std::runtime_error("bad OneWayMatching: " + line);
        m.chunk_b = -1;
      } else if (s >= 6 && line.compare(s - 6, 6, "TwoWay") == 0) {
        m.kind = Matching::TwoWay;
        int b2, a2;
        if (!read_int(line, i, m.a) || !read_int(line, i, m.b) || !read_int(line, i, m.chunk_a) ||
            !read_int(line, i, b2) || !read_int(line, i, a2) || !read_int(line, i, m.chunk_b))
          throw std::runtime_error("bad TwoWayMatching: " + line);
        if (b2 != m.b || a2 != m.a) throw std::runtime_error("TwoWayMatching names four GPUs: " + line);
      } else {
        throw std::runtime_error("unknown matching kind: " + line);
      }
      max_rank = std::max(max_rank, std::max(m.a, m.b));
      rnd.push_back(m);
      pos = i;
    }
    sch.rounds.push_back(rnd);
  }
  sch.n = max_rank + 1;
  return sch;
}

std::string format_schedule_compact(const Schedule& s) {
  std::ostringstream o;
  for (size_t r = 0; r < s.rounds.size(); ++r) {
    o << "R" << r << ":";
    for (const auto& m : s.rounds[r]) {
      if (m.kind == Matching::Straggler) o << " " << m.a << "<->" << m.b << " c" << m.chunk_a << " |";
      else if (m.kind == Matching::OneWay) o << " " << m.a << "->" << m.b << " c" << m.chunk_a << " |";
      else o << " " << m.a << "->" << m.b << " c" << m.chunk_a << ";" << m.b << "->" << m.a << " c" << m.chunk_b << " |";
    }
    o << "\n";
  }
  return o.str();
}

struct BuiltinEntry { int n; const char* text; };
static const BuiltinEntry kBuiltin[] = {
#include "builtin_schedules.inc"
};

Schedule builtin_schedule(int n) {
  if (n == 1) { Schedule s; s.n = 1; return s; }
  for (const auto& e : kBuiltin)
    if (e.n == n) { Schedule s = parse_schedule(e.text); s.n = n; return s; }
  throw std::runtime_error("no built-in StragglAR schedule for n=" + std::to_string(n) +
                           "; synthesize one (python -m stragglar_b200.synth.pow2|nonpow2 <n>) and pass its text");
}

// ------------------------------------------------------------------ generators
int Plan::num_rounds() const {
  int r = 0;
  for (const auto& s : steps) r = std::max(r, s.round + 1);
  return r;
}

static uint32_t full_mask(int n) { return n >= 32 ? 0xffffffffu : ((1u << n) - 1u); }

static Plan blank(const std::string& name, int n, int chunks) {
  if (n < 1 || n > SAR_MAX_RANKS) throw CompileError("rank count out of range: " + std::to_string(n));
  Plan p;
  p.name = name; p.n = n; p.num_chunks = std::max(chunks, 1);
  if (p.num_chunks > SAR_MAX_CHUNKS) throw CompileError("too many chunks");
  p.init.assign(n, std::vector<uint32_t>(p.num_chunks, 0));
  for (int r = 0; r < n; ++r) {
    for (int c = 0; c < p.num_chunks; ++c) p.init[r][c] = 1u << r;
    p.participants.push_back(r);
  }
  if (n == 1) {
    // a single rank has nothing to exchange; one local pass applies the fused scale
    Step s; s.round = 0; s.kind = StepKind::Reduce; s.chunk = 0; s.dst = 0; s.finalize = true;
    p.steps.push_back(s);
  }
  return p;
}

static void add_prephase(Plan& p, int round) {
  // reduce-scatter among ranks 0..n-2: rank i sums chunk i of all of them
  const int n = p.n;
  for (int i = 0; i < n - 1; ++i) {
    if (n - 2 <= 0) break;  // n = 2: the only non-straggler already holds its partial
    Step s; s.round = round; s.kind = StepKind::Reduce; s.chunk = i; s.dst = i;
    for (int k = 1; k < n - 1; ++k) s.srcs.push_back((i + k) % (n - 1));
    p.steps.push_back(s);
  }
}

static void assume_prephase_done(Plan& p) {
  const int n = p.n;
  for (int r = 0; r < n - 1; ++r)
    for (int c = 0; c < p.num_chunks; ++c) p.init[r][c] = (c == r) ? full_mask(n - 1) : 0u;
}

Plan plan_stragglar(const Schedule& s, bool prephase) {
  const int n = s.n;
  Plan p = blank("stragglar", n, n - 1);
  if (n == 1) return p;
  int base = 0;
  if (prephase) { add_prephase(p, 0); base = 1; } else assume_prephase_done(p);
  for (size_t r = 0; r < s.rounds.size(); ++r) {
    for (const auto& m : s.rounds[r]) {
      Step st; st.round = base + (int)r;
      if (m.kind == Matching::Straggler) {
        st.kind = StepKind::Exchange; st.chunk = m.chunk_a; st.dst = m.a; st.srcs = {m.b}; st.finalize = true;
        p.steps.push_back(st);
      } else if (m.kind == Matching::OneWay) {
        st.kind = StepKind::Copy; st.chunk = m.chunk_a; st.dst = m.b; st.srcs = {m.a};
        p.steps.push_back(st);
      } else {
        st.kind = StepKind::Copy; st.chunk = m.chunk_a; st.dst = m.b; st.srcs = {m.a};
        p.steps.push_back(st);
        Step s2 = st; s2.chunk = m.chunk_b; s2.dst = m.a; s2.srcs = {m.b};
        p.steps.push_back(s2);
      }
    }
  }
  return p;
}

Plan plan_stragglar_a2a(int n, bool prephase) {
  Plan p = blank("stragglar_a2a", n, n - 1);
  if (n == 1) return p;
  int base = 0;
  if (prephase) { add_prephase(p, 0); base = 1; } else assume_prephase_done(p);
  for (int i = 0; i < n - 1; ++i) {
    Step st; st.round = base; st.kind = StepKind::Exchange; st.chunk = i; st.dst = i; st.srcs = {n - 1}; st.finalize = true;
    p.steps.push_back(st);
  }
  for (int j = 0; j < n - 1; ++j)
    for (int k = 1; k < n - 1; ++k) {
      int i = (j + k) % (n - 1);
      Step st; st.round = base + 1; st.kind = StepKind::Copy; st.chunk = i; st.dst = j; st.srcs = {i};
      p.steps.push_back(st);
    }
  return p;
}

Plan plan_ring(int n) {
  Plan p = blank("ring", n, n);
  if (n == 1) return p;
  auto md = [n](int x) { return ((x % n) + n) % n; };
  for (int s = 0; s < n - 1; ++s)
    for (int r = 0; r < n; ++r) {
      Step st; st.round = s; st.kind = StepKind::Reduce; st.chunk = md(r - 1 - s); st.dst = r; st.srcs = {md(r - 1)};
      st.finalize = (s == n - 2);
      p.steps.push_back(st);
    }
  for (int s = 0; s < n - 1; ++s)
    for (int r = 0; r < n; ++r) {
      Step st; st.round = n - 1 + s; st.kind = StepKind::Copy; st.chunk = md(r - s); st.dst = r; st.srcs = {md(r - 1)};
      p.steps.push_back(st);
    }
  return p;
}

Plan plan_rhd(int n) {
  if (n & (n - 1)) throw CompileError("recursive halving-doubling needs a power-of-two rank count");
  Plan p = blank("rhd", n, n);
  if (n == 1) return p;
  int L = 0;
  while ((1 << L) < n) ++L;
  // halving: in step k rank r pairs with r ^ 2^k and keeps the half of its
  // current chunk range selected by bit k of r
  std::vector<int> lo(n, 0), hi(n, n);
  for (int k = 0; k < L; ++k) {
    for (int r = 0; r < n; ++r) {
      int partner = r ^ (1 << k);
      int mid = (lo[r] + hi[r]) / 2;
      int klo = (r >> k & 1) ? mid : lo[r], khi = (r >> k & 1) ? hi[r] : mid;
      for (int c = klo; c < khi; ++c) {
        Step st; st.round = k; st.kind = StepKind::Reduce; st.chunk = c; st.dst = r; st.srcs = {partner};
        st.finalize = (k == L - 1);
        p.steps.push_back(st);
      }
    }
    for (int r = 0; r < n; ++r) {
      int mid = (lo[r] + hi[r]) / 2;
      if (r >> k & 1) lo[r] = mid; else hi[r] = mid;
    }
  }
  // doubling: the same pairs in reverse order copy the partner's owned range
  for (int k = L - 1; k >= 0; --k) {
    std::vector<int> nlo = lo, nhi = hi;
    for (int r = 0; r < n; ++r) {
      int partner = r ^ (1 << k);
      for (int c = lo[partner]; c < hi[partner]; ++c) {
        Step st; st.round = L + (L - 1 - k); st.kind = StepKind::Copy; st.chunk = c; st.dst = r; st.srcs = {partner};
        p.steps.push_back(st);
      }
      nlo[r] = std::min(lo[r], lo[partner]);
      nhi[r] = std::max(hi[r], hi[partner]);
    }
    lo = nlo; hi = nhi;
  }
  return p;
}

Plan plan_direct(int n, bool prephase) {
  // The straggler exchanges the whole buffer with rank 0 once the others have
  // all-reduced among themselves; the result is then broadcast down a binary
  // tree from both ends (cf. stragglar/allreduce_8GPU.cu:60-137).
  Plan p = blank("direct", n, std::max(n - 1, 1));
  if (n == 1) return p;
  const int P = p.num_chunks;
  int round = 0;
  // The all-reduce among the non-stragglers cannot share a table with what
  // follows: its all-gather reads slots that the exchange and the broadcast
  // overwrite, and nothing orders those.  It is a phase of its own
  // (build_program), so every rank starts here holding the (n-1)-rank sum.
  (void)prephase;
  for (int r = 0; r < n - 1; ++r)
    for (int c = 0; c < P; ++c) p.init[r][c] = full_mask(n - 1);
  for (int c = 0; c < P; ++c) {
    Step st; st.round = round; st.kind = StepKind::Exchange; st.chunk = c; st.dst = 0; st.srcs = {n - 1}; st.finalize = true;
    p.steps.push_back(st);
  }
  ++round;
  std::vector<int> low = {0}, high = {n - 1};
  int next_low = 1, next_high = n - 2;   // unserved ranks are [next_low, next_high]
  while (next_low <= next_high) {
    std::vector<std::pair<int, int>> moves;  // src -> dst
    std::vector<int> add_low, add_high;
    int remaining = next_high - next_low + 1;
    int take_low = std::min<int>((int)low.size(), (remaining + 1) / 2);
    int take_high = std::min<int>((int)high.size(), remaining - take_low);
    for (int i = 0; i < take_low; ++i) { moves.push_back({low[i], next_low + i}); add_low.push_back(next_low + i); }
    std::sort(high.begin(), high.end());
    for (int i = 0; i < take_high; ++i) {
      int dst = next_high - take_high + 1 + i;
      moves.push_back({high[(int)high.size() - take_high + i], dst});
      add_high.push_back(dst);
    }
    next_low += take_low; next_high -= take_high;
    for (auto& mv : moves)
      for (int c = 0; c < P; ++c) {
        Step st; st.round = round; st.kind = StepKind::Copy; st.chunk = c; st.dst = mv.second; st.srcs = {mv.first};
        p.steps.push_back(st);
      }
    low.insert(low.end(), add_low.begin(), add_low.end());
    high.insert(high.end(), add_high.begin(), add_high.end());
    ++round;
  }
  return p;
}

Plan plan_reduce_scatter(int n) {
  Plan p = blank("reducescatter", n, n);
  p.expect = Expect::ReduceScatter;
  if (n == 1) return p;
  for (int i = 0; i < n && n > 1; ++i) {
    Step s; s.round = 0; s.kind = StepKind::Reduce; s.chunk = i; s.dst = i; s.finalize = true;
    for (int k = 1; k < n; ++k) s.srcs.push_back((i + k) % n);
    p.steps.push_back(s);
  }
  return p;
}

Plan plan_rsag(int n) {
  Plan p = plan_reduce_scatter(n);
  p.name = "rsag";
  p.expect = Expect::AllReduce;
  for (int j = 0; j < n; ++j)
    for (int k = 1; k < n; ++k) {
      int i = (j + k) % n;
      Step st; st.round = 1; st.kind = StepKind::Copy; st.chunk = i; st.dst = j; st.srcs = {i};
      p.steps.push_back(st);
    }
  return p;
}

// Lowering defaults, from measurements on 8 x B200 (1 GiB, fp32, after the straggler's arrival):
//   stragglar      pulled copies, one lane     2.67 ms   (pushed 3.23, pushed + forwarding lane 3.42)
//   stragglar_a2a  pushed copies, two lanes    2.00 ms   (one lane 2.93, pulled 3.01)
//   ring / rsag    pushed copies               2.78 / 2.86 ms (pulled 2.94 / 2.90)
//   direct         pulled copies, one lane     4.42 ms   (pushed 4.53)
// STRAGGLAR_COPY=pull|push and STRAGGLAR_LANES=1|2 override them.
static bool push_default_for(const std::string& alg) {
  const char* v = getenv("STRAGGLAR_COPY");
  if (v && *v) return std::string(v) != "pull";
  return !(alg == "stragglar" || alg == "direct");
}
static bool two_lanes_default_for(const std::string& alg) {
  const char* v = getenv("STRAGGLAR_LANES");
  if (v && *v) return atoi(v) >= 2;
  return alg == "stragglar_a2a";
}
bool default_push_copies() { return push_default_for(""); }
bool default_two_lanes() { return two_lanes_default_for(""); }

static Plan plan_by_name_impl(const std::string& alg, int n, bool prephase, const Schedule* sched);
Plan plan_by_name(const std::string& alg, int n, bool prephase, const Schedule* sched) {
  Plan p = plan_by_name_impl(alg, n, prephase, sched);
  p.push_copies = push_default_for(alg);
  bool has_exchange = false;
  for (const auto& s : p.steps) has_exchange |= s.kind == StepKind::Exchange;
  p.two_lanes = has_exchange && two_lanes_default_for(alg);
  p.split_copies = has_exchange;
  // Blocks per rank beyond which the collective gets slower (8 x B200, 1 GiB, after the arrival):
  //   stragglar, free-running rounds   32: 2.72 ms, 48: 2.72, 64: 2.46-2.56, 128: 2.60
  //   stragglar, gated rounds          32: 2.32, 48: 2.21, 64: 2.17-2.25, 96: 2.17, 128: 2.22
  //   stragglar_a2a                    24: 1.89, 32: 1.81, 48: 1.83, 64: 2.00, 128: 2.64; 48 blocks with three of
  //                                    the six ring stages (fewer bytes in flight per block): 1.74
  // (more concurrent flows per link only add contention once the link is saturated);
  // ring / rhd / rsag keep improving up to 128.
  // With one or two ranks there is a single flow per link and more blocks keep helping.
  if (alg == "stragglar" && n >= 4) p.blocks_hint = 64;
  if (alg == "stragglar_a2a" && n >= 4) { p.blocks_hint = 48; p.stages_hint = 3; }
  // Round gating (see SAR_GATE_ALL_DONE in table.h) pays for the synthesized schedule, whose rounds are matchings:
  // one round at a time every port carries one flow in and one out.  8 x B200, 1 GiB after the arrival: 2.17-2.25 ms
  // against 2.46-2.56 free-running; 256 MiB 0.71 against 0.77; 64 MiB 0.33 against 0.28, hence the size threshold
  // (gate_min_bytes).  The other algorithms lose to the hand-shake per round (ring 3.19 against 2.87 ms).
  // STRAGGLAR_GATE=0 switches it off, STRAGGLAR_GATE=all gates every algorithm.
  p.gate_rounds = alg == "stragglar" && n >= 4;
  const char* gate = getenv("STRAGGLAR_GATE");
  if (gate && *gate) p.gate_rounds = !strcmp(gate, "all") || (atoi(gate) != 0 && alg == "stragglar" && n >= 4);
  // share of the blocks given to the forwarding lane (eighths); half unless STRAGGLAR_LANE1_EIGHTHS says otherwise
  // (forwarding moves n-2 chunks per chunk matched: the model of the executor prefers 5/8 at 32 blocks)
  const char* l1 = getenv("STRAGGLAR_LANE1_EIGHTHS");
  if (l1 && *l1 && atoi(l1) >= 1 && atoi(l1) <= 7) p.lane1_eighths = atoi(l1);
  return p;
}

static Plan plan_by_name_impl(const std::string& alg, int n, bool prephase, const Schedule* sched) {
  if (alg == "stragglar") {
    Schedule s = sched ? *sched : builtin_schedule(n);
    if (s.n != n) throw CompileError("schedule is for n=" + std::to_string(s.n) + ", not " + std::to_string(n));
    return plan_stragglar(s, prephase);
  }
  if (alg == "stragglar_a2a") return plan_stragglar_a2a(n, prephase);
  if (alg == "ring") return plan_ring(n);
  if (alg == "rhd") return plan_rhd(n);
  if (alg == "direct") return plan_direct(n, prephase);
  if (alg == "rsag") return plan_rsag(n);
  if (alg == "reducescatter") return plan_reduce_scatter(n);
  throw CompileError("Invalid algorithm: " + alg);
}

std::vector<int> straggler_rank_map(int n, int physical_straggler) {
  if (physical_straggler < 0 || physical_straggler >= n) throw CompileError("straggler rank out of range");
  std::vector<int> m(n);
  for (int i = 0; i < n; ++i) m[i] = i;
  std::swap(m[n - 1], m[physical_straggler]);
  return m;
}

// -------------------------------------------------------------------- compiler
namespace {
constexpr int kMaxSteps = 4096;
using StepSet = std::bitset<kMaxSteps>;
struct Slot {
  int ver = 0;
  int writer = -1;            // step that wrote the current version (-1: input)
  std::vector<int> readers;   // steps that read the current version
  uint32_t content = 0;       // contributions summed into the slot
};
}  // namespace

Compiled compile(const Plan& plan, const std::vector<int>& l2p_in, int n_physical) {
  const int n = plan.n, P = plan.num_chunks;
  const int np = n_physical > 0 ? n_physical : n;
  if (n < 1 || n > SAR_MAX_RANKS) throw CompileError("rank count out of range");
  if ((int)plan.steps.size() > kMaxSteps) throw CompileError("plan has too many steps");
  std::vector<int> l2p = l2p_in;
  if (l2p.empty()) { l2p.resize(n); for (int i = 0; i < n; ++i) l2p[i] = i; }
  if ((int)l2p.size() != n) throw CompileError("rank map has the wrong length");
  {
    if (np < n || np > SAR_MAX_RANKS) throw CompileError("bad physical rank count");
    std::vector<int> seen(np, 0);
    for (int v : l2p) { if (v < 0 || v >= np || seen[v]++) throw CompileError("rank map is not injective"); }
  }
  // order steps by round, keeping the generator's order inside a round
  std::vector<int> order(plan.steps.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = (int)i;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return plan.steps[a].round < plan.steps[b].round; });

  std::vector<std::vector<Slot>> slot(n, std::vector<Slot>(P));
  for (int r = 0; r < n; ++r)
    for (int c = 0; c < P; ++c) slot[r][c].content = plan.init[r][c];
  std::vector<StepSet> anc(plan.steps.size());

  Compiled out;
  out.name = plan.name; out.n = np; out.num_chunks = P; out.logical_to_physical = l2p;
  out.ranks.assign(np, RankTable{});
  for (int v : l2p) out.participants |= 1u << v;
  out.chunks_in.assign(np, 0.0); out.chunks_out.assign(np, 0.0);
  out.num_rounds = plan.num_rounds();
  std::vector<std::vector<SarOp>> ops(n);  // by logical rank

  auto fail = [&](const Step& s, const std::string& why) {
    throw CompileError(plan.name + " round " + std::to_string(s.round) + " chunk " + std::to_string(s.chunk) +
                       " dst " + std::to_string(s.dst) + ": " + why);
  };

  size_t i = 0;
  while (i < order.size()) {
    size_t j = i;
    const int round = plan.steps[order[i]].round;
    while (j < order.size() && plan.steps[order[j]].round == round) ++j;
    // pass 1: checks against the pre-round state, dependencies, op emission
    std::map<std::pair<int, int>, int> written_by, read_by_other;
    for (size_t k = i; k < j; ++k) {
      const int si = order[k];
      const Step& s = plan.steps[si];
      if (s.chunk < 0 || s.chunk >= P) fail(s, "chunk out of range");
      if (s.dst < 0 || s.dst >= n) fail(s, "rank out of range");
      const bool self_only = s.kind == StepKind::Reduce && s.include_local && s.srcs.empty();
      if ((s.srcs.empty() && !self_only) || (int)s.srcs.size() >= SAR_MAX_RANKS) fail(s, "bad source list");
      if (s.kind != StepKind::Reduce && s.srcs.size() != 1) fail(s, "exactly one source expected");
      for (int src : s.srcs) if (src < 0 || src >= n || src == s.dst) fail(s, "bad source rank");
      std::vector<std::pair<int, int>> reads, writes;
      for (int src : s.srcs) reads.push_back({src, s.chunk});
      const bool reads_local = s.kind == StepKind::Exchange || (s.kind == StepKind::Reduce && s.include_local);
      if (reads_local) reads.push_back({s.dst, s.chunk});
      writes.push_back({s.dst, s.chunk});
      if (s.kind == StepKind::Exchange) writes.push_back({s.srcs[0], s.chunk});
      for (auto& w : writes) {
        if (written_by.count(w)) fail(s, "slot written twice in one round");
        written_by[w] = si;
        // every op waits for the current version of a slot it writes (its own
        // through local_ver, a pushed-to peer slot through src_ver), so the
        // previous writer is always an ancestor
        Slot& sl = slot[w.first][w.second];
        if (sl.writer >= 0) { anc[si] |= anc[sl.writer]; anc[si].set(sl.writer); }
      }
      for (auto& rd : reads) {
        Slot& sl = slot[rd.first][rd.second];
        if (sl.content == 0) fail(s, "reads a slot whose content is undefined");
        if (sl.writer >= 0) { anc[si] |= anc[sl.writer]; anc[si].set(sl.writer); }
        if (std::find(writes.begin(), writes.end(), rd) == writes.end()) read_by_other[rd] = si;
      }
    }
    for (auto& w : written_by) {
      auto it = read_by_other.find(w.first);
      if (it != read_by_other.end() && it->second != w.second)
        fail(plan.steps[w.second], "slot is read by another step of the same round");
    }
    // hazards: every earlier reader (and the previous writer) of a slot must
    // be an ancestor of the step that overwrites it
    for (size_t k = i; k < j; ++k) {
      const int si = order[k];
      const Step& s = plan.steps[si];
      std::vector<std::pair<int, int>> writes = {{s.dst, s.chunk}};
      if (s.kind == StepKind::Exchange) writes.push_back({s.srcs[0], s.chunk});
      for (auto& w : writes) {
        Slot& sl = slot[w.first][w.second];
        for (int rd : sl.readers)
          if (rd != si && !anc[si].test(rd))
            fail(s, "overwrites rank " + std::to_string(w.first) + "'s slot while step of round " +
                        std::to_string(plan.steps[rd].round) + " (dst " + std::to_string(plan.steps[rd].dst) +
                        ") may still read it");
        if (sl.writer >= 0 && sl.writer != si && !anc[si].test(sl.writer))
          fail(s, "is not ordered after the previous write of rank " + std::to_string(w.first) + "'s slot");
      }
    }
    // emit ops from the pre-round versions
    for (size_t k = i; k < j; ++k) {
      const Step& s = plan.steps[order[k]];
      auto ver = [&](int r) { return slot[r][s.chunk].ver; };
      SarOp op{};
      op.round = (uint8_t)round; op.chunk = (uint8_t)s.chunk; op.part = 0; op.parts = 1;
      op.flags = s.finalize ? SAR_F_SCALE : 0;
      op.nsrc = (uint8_t)s.srcs.size();
      for (size_t q = 0; q < s.srcs.size(); ++q) {
        op.src[q] = (uint8_t)l2p[s.srcs[q]];
        op.src_ver[q] = (uint8_t)ver(s.srcs[q]);
      }
      op.local_ver = (uint8_t)ver(s.dst);
      op.post_ver = (uint8_t)(ver(s.dst) + 1);
      if (s.kind == StepKind::Copy) {
        const int nparts = plan.split_copies ? 2 : 1;
        for (int part = 0; part < nparts; ++part) {
          SarOp co = op;
          co.part = (uint8_t)part; co.parts = (uint8_t)nparts;
          co.lane = plan.two_lanes ? 1 : 0;
          if (plan.push_copies) {
            // executed by the source: it waits for its own slot (local_ver), for the destination
            // slot's current version (src_ver) and stores into the destination
            co.kind = SAR_PUSH;
            co.src[0] = (uint8_t)l2p[s.dst];
            co.src_ver[0] = (uint8_t)ver(s.dst);
            co.local_ver = (uint8_t)ver(s.srcs[0]);
            co.post_ver = 0;
            co.push_ver = (uint8_t)(ver(s.dst) + 1);
            ops[s.srcs[0]].push_back(co);
          } else {
            co.kind = SAR_COPY;
            ops[s.dst].push_back(co);
          }
        }
        out.chunks_in[l2p[s.dst]] += 1; out.chunks_out[l2p[s.srcs[0]]] += 1;
      } else if (s.kind == StepKind::Reduce) {
        op.kind = SAR_REDUCE;
        if (s.include_local) op.flags |= SAR_F_LOCAL;
        ops[s.dst].push_back(op);
        for (int src : s.srcs) { out.chunks_in[l2p[s.dst]] += 1; out.chunks_out[l2p[src]] += 1; }
      } else {
        const int a = s.dst, b = s.srcs[0];
        op.kind = SAR_REDUCE_PUSH; op.parts = 2; op.part = 0;
        op.push_ver = (uint8_t)(ver(b) + 1);
        ops[a].push_back(op);
        SarOp ob = op;
        ob.part = 1; ob.src[0] = (uint8_t)l2p[a]; ob.src_ver[0] = (uint8_t)ver(a);
        ob.local_ver = (uint8_t)ver(b); ob.post_ver = (uint8_t)(ver(b) + 1); ob.push_ver = (uint8_t)(ver(a) + 1);
        ops[b].push_back(ob);
        // each side pulls half a chunk and pushes half a chunk
        out.chunks_in[l2p[a]] += 1; out.chunks_out[l2p[a]] += 1;
        out.chunks_in[l2p[b]] += 1; out.chunks_out[l2p[b]] += 1;
      }
    }
    // pass 2: apply the round
    std::vector<std::tuple<int, int, uint32_t>> new_content;
    for (size_t k = i; k < j; ++k) {
      const int si = order[k];
      const Step& s = plan.steps[si];
      uint32_t acc = 0;
      auto add = [&](int r) {
        uint32_t c = slot[r][s.chunk].content;
        if (acc & c) fail(s, "adds a contribution twice");
        acc |= c;
      };
      if (s.kind == StepKind::Copy) acc = slot[s.srcs[0]][s.chunk].content;
      else {
        for (int src : s.srcs) add(src);
        if (s.kind == StepKind::Exchange || s.include_local) add(s.dst);
      }
      new_content.push_back({s.dst, s.chunk, acc});
      if (s.kind == StepKind::Exchange) new_content.push_back({s.srcs[0], s.chunk, acc});
    }
    for (size_t k = i; k < j; ++k) {
      const int si = order[k];
      const Step& s = plan.steps[si];
      for (int src : s.srcs)
        if (s.kind != StepKind::Exchange) slot[src][s.chunk].readers.push_back(si);
      auto wr = [&](int r) {
        Slot& sl = slot[r][s.chunk];
        sl.ver += 1; sl.writer = si; sl.readers.clear();
        out.max_version = std::max(out.max_version, sl.ver);
      };
      wr(s.dst);
      if (s.kind == StepKind::Exchange) wr(s.srcs[0]);
    }
    for (auto& t : new_content) slot[std::get<0>(t)][std::get<1>(t)].content = std::get<2>(t);
    i = j;
  }
  if (out.max_version >= (int)SAR_VER_STRIDE) throw CompileError("too many versions of one slot");
  out.blocks_hint = plan.blocks_hint;
  out.stages_hint = plan.stages_hint;
  out.lane1_eighths = plan.lane1_eighths;
  for (int r = 0; r < (int)out.ranks.size(); ++r) {
    const std::string why = validate_rank_table(out.ranks[r], r, np, P);
    if (!why.empty()) throw CompileError(plan.name + ": table of rank " + std::to_string(r) + " is malformed: " + why);
  }
  out.gate_rounds = plan.gate_rounds;
  for (const RankTable& rt : out.ranks)
    for (const SarOp& op : rt.ops)
      if (op.round >= SAR_GATE_ALL_DONE) out.gate_rounds = false;   // does not fit the announcement word
  // result check
  const uint32_t want = full_mask(n);
  for (int r : plan.participants) {
    for (int c = 0; c < P; ++c) {
      if (plan.expect == Expect::ReduceScatter && c != r) continue;
      if (slot[r][c].content != want)
        throw CompileError(plan.name + ": rank " + std::to_string(r) + " ends without the full sum of chunk " +
                           std::to_string(c));
    }
  }
  // A rank that pushes the same tiles of one chunk to several peers in one round loads them
  // once: merge those pushes into one op with several destinations.
  for (int lr = 0; lr < n; ++lr) {
    std::vector<SarOp> merged;
    for (const SarOp& op : ops[lr]) {
      bool done = false;
      if (op.kind == SAR_PUSH) {
        for (SarOp& m : merged) {
          if (m.kind == SAR_PUSH && m.round == op.round && m.chunk == op.chunk && m.part == op.part &&
              m.parts == op.parts && m.local_ver == op.local_ver && m.push_ver == op.push_ver &&
              m.nsrc < SAR_MAX_RANKS - 1) {
            m.src[m.nsrc] = op.src[0];
            m.src_ver[m.nsrc] = op.src_ver[0];
            ++m.nsrc;
            done = true;
            break;
          }
        }
      }
      if (!done) merged.push_back(op);
    }
    // within a round, lane 0 ops first: every (round, lane) is one contiguous range
    std::stable_sort(merged.begin(), merged.end(), [](const SarOp& a, const SarOp& b) {
      return a.round != b.round ? a.round < b.round : a.lane < b.lane;
    });
    ops[lr] = merged;
  }
  for (int pr = 0; pr < np; ++pr) out.ranks[pr].round_begin.assign(1, 0);
  for (int lr = 0; lr < n; ++lr) {
    RankTable& t = out.ranks[l2p[lr]];
    t.round_begin.clear();
    t.ops = ops[lr];
    if (t.ops.size() > SAR_MAX_OPS) throw CompileError("too many ops for one rank");
    int last = -1;
    for (size_t q = 0; q < t.ops.size(); ++q)
      if (t.ops[q].round != last) { t.round_begin.push_back((uint16_t)q); last = t.ops[q].round; }
    t.round_begin.push_back((uint16_t)t.ops.size());
    t.final_ver.assign(P, 0);
    for (int c = 0; c < P; ++c) t.final_ver[c] = (uint8_t)slot[lr][c].ver;
  }
  return out;
}


std::string validate_rank_table(const RankTable& t, int rank, int nranks, int num_chunks) {
  auto bad = [&](size_t o, const std::string& what) { return "op " + std::to_string(o) + ": " + what; };
  if (t.ops.size() > SAR_MAX_OPS) return "more than " + std::to_string(SAR_MAX_OPS) + " ops";
  if (t.ops.empty()) return t.round_begin.size() <= 1 ? "" : "round list of an empty table";
  if (t.round_begin.size() < 2 || t.round_begin.front() != 0 || t.round_begin.back() != t.ops.size())
    return "round list does not cover the ops";
  if (t.round_begin.size() - 1 > SAR_MAX_ROUNDS) return "more than " + std::to_string(SAR_MAX_ROUNDS) + " rounds";
  for (size_t i = 0; i + 1 < t.round_begin.size(); ++i) {
    if (t.round_begin[i] >= t.round_begin[i + 1]) return "empty or unsorted round " + std::to_string(i);
    for (size_t o = t.round_begin[i]; o < t.round_begin[i + 1]; ++o) {
      if (t.ops[o].round != t.ops[t.round_begin[i]].round) return bad(o, "round differs inside a round");
      if (o > t.round_begin[i] && t.ops[o].lane < t.ops[o - 1].lane) return bad(o, "lanes unsorted inside a round");
    }
    if (i > 0 && t.ops[t.round_begin[i]].round <= t.ops[t.round_begin[i - 1]].round) return "rounds not increasing";
  }
  for (size_t o = 0; o < t.ops.size(); ++o) {
    const SarOp& op = t.ops[o];
    if (op.kind > SAR_PUSH) return bad(o, "unknown kind");
    if ((int)op.chunk >= num_chunks) return bad(o, "chunk out of range");
    if (op.parts == 0 || op.part >= op.parts) return bad(o, "bad tile range");
    if (op.lane > 1) return bad(o, "bad lane");
    if (op.nsrc > SAR_MAX_RANKS || (int)op.nsrc >= std::max(nranks, 2)) return bad(o, "too many peers");
    if ((op.kind == SAR_COPY || op.kind == SAR_REDUCE_PUSH) && op.nsrc != 1) return bad(o, "needs exactly one peer");
    if (op.kind == SAR_PUSH && op.nsrc == 0) return bad(o, "push without a destination");
    uint32_t seen = 0;
    for (int q = 0; q < op.nsrc; ++q) {
      if ((int)op.src[q] >= nranks) return bad(o, "peer out of range");
      if ((int)op.src[q] == rank) return bad(o, "names the rank itself as a peer");
      if (seen >> op.src[q] & 1) return bad(o, "names a peer twice");
      seen |= 1u << op.src[q];
      if (op.src_ver[q] >= SAR_VER_STRIDE) return bad(o, "version out of range");
    }
    if (op.local_ver >= SAR_VER_STRIDE || op.post_ver >= SAR_VER_STRIDE || op.push_ver >= SAR_VER_STRIDE)
      return bad(o, "version out of range");
  }
  return "";
}

Program build_program(const std::string& alg, int n, bool prephase, int straggler, const Schedule* sched) {
  Program prog;
  prog.alg = alg; prog.n = n;
  std::vector<int> map;
  if (straggler >= 0 && n > 1) map = straggler_rank_map(n, straggler);
  if (alg == "direct" && prephase && n > 2) {
    // phase 1: one-shot all-reduce among the n-1 non-stragglers, channel 1
    Plan sub = plan_rsag(n - 1);
    sub.push_copies = default_push_copies();
    std::vector<int> submap(n - 1);
    for (int i = 0; i < n - 1; ++i) submap[i] = map.empty() ? i : map[i];
    Compiled c1 = compile(sub, submap, n);
    c1.channel = 1;
    c1.name = "direct.pre";
    for (auto& t : c1.ranks)
      for (auto& op : t.ops) op.flags &= (uint8_t)~SAR_F_SCALE;  // the scale applies once, in the last phase
    prog.phases.push_back(c1);
  }
  Compiled c = compile(plan_by_name(alg, n, prephase, sched), map, n);
  c.channel = 0;
  prog.phases.push_back(c);
  return prog;
}

}  // namespace sar
