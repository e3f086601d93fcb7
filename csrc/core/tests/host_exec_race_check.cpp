// Race check of the table protocol under ThreadSanitizer.
//
// Builds every algorithm for several rank counts (all lowerings), runs it with
// the host executor -- several threads per rank, the same item order, flags,
// arrival and exit words as the CUDA kernels -- and checks the sums.  Compiled
// with -fsanitize=thread, every unordered pair of accesses to a buffer element
// (a read of a slot that may still be overwritten, a write that is not ordered
// after the reads of the value it destroys) is reported as a data race: this
// is the dynamic counterpart of the compiler's static hazard check, and stands
// in for compute-sanitizer's racecheck, which is not available for the GPU runs.
//
//   g++ -std=c++17 -O1 -g -fsanitize=thread -pthread host_exec_race_check.cpp ../plan.cpp ../host_exec.cpp -o race_check && ./race_check
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "../host_exec.h"
#include "../plan.h"

static float uniform(uint64_t seed, uint64_t i) {
  uint64_t x = (i + 1) * 0x9E3779B97F4A7C15ull + seed * 0xD1B54A32D192ED03ull;
  x ^= x >> 32; x *= 0xD6E8FEB86659FD93ull; x ^= x >> 32;
  return (float)(uint32_t)(x >> 40) * (2.0f / 16777216.0f) - 1.0f;
}

// validate_rank_table accepts what the compiler makes and names what is wrong with a damaged table
static int check_validation() {
  int failures = 0;
  const sar::Program prog = sar::build_program("stragglar", 8, true, -1, nullptr);
  const sar::Compiled& c = prog.phases.back();
  for (int r = 0; r < 8; ++r)
    if (!sar::validate_rank_table(c.ranks[r], r, 8, c.num_chunks).empty()) { printf("intact table of rank %d refused\n", r); ++failures; }
  struct Case { const char* what; void (*damage)(sar::RankTable&); };
  const Case cases[] = {
      {"chunk", [](sar::RankTable& t) { t.ops[1].chunk = 200; }},
      {"peer", [](sar::RankTable& t) { t.ops[0].src[0] = 9; }},
      {"self", [](sar::RankTable& t) { t.ops[0].src[0] = 3; }},
      {"kind", [](sar::RankTable& t) { t.ops[2].kind = 7; }},
      {"parts", [](sar::RankTable& t) { t.ops[0].part = t.ops[0].parts; }},
      {"rounds", [](sar::RankTable& t) { t.round_begin.back() += 1; }},
      {"order", [](sar::RankTable& t) { std::swap(t.ops.front(), t.ops.back()); }},
      {"version", [](sar::RankTable& t) { t.ops[0].post_ver = 40; }},
  };
  for (const Case& k : cases) {
    sar::RankTable t = c.ranks[3];
    k.damage(t);
    if (sar::validate_rank_table(t, 3, 8, c.num_chunks).empty()) { printf("damaged table accepted (%s)\n", k.what); ++failures; }
  }
  if (sar::validate_rank_table(c.ranks[3], 3, 4, c.num_chunks).empty()) { printf("table for 8 ranks accepted for 4\n"); ++failures; }
  return failures;
}

int main() {
  int failures = check_validation(), runs = 0;
  const char* algs[] = {"stragglar", "stragglar_a2a", "ring", "rhd", "direct", "rsag"};
  // round gating (rounds one after the other) is run for every algorithm too, on the lowerings that ship
  // gated twice: with the default slack (a round opens early, items wait for their flags) and with the full barrier
  // (slack 0: gated items skip their flag waits, the barrier alone orders them)
  for (const char* mode : {"0", "all", "all/barrier"})
  for (const char* copy : {"pull", "push"})
    for (const char* lanes : {"1", "2"}) {
      const bool barrier = std::string(mode) == "all/barrier";
      const char* gate = barrier ? "all" : mode;
      if (barrier) setenv("STRAGGLAR_GATE_SLACK", "0", 1); else unsetenv("STRAGGLAR_GATE_SLACK");
      if (std::string(gate) == "all" && std::string(copy) == "push" && std::string(lanes) == "2") continue;   // keeps the run short
      setenv("STRAGGLAR_GATE", gate, 1);
      setenv("STRAGGLAR_COPY", copy, 1);
      setenv("STRAGGLAR_LANES", lanes, 1);
      for (const char* alg : algs)
        for (int n : {2, 4, 6, 8})
          for (int straggler : {-1, 1}) {
            if (std::string(gate) == "all" && (n == 2 || straggler >= 0)) continue;   // the gated pass: 4, 6 and 8 ranks
            if (std::string(alg) == "rhd" && (n & (n - 1))) continue;
            if (straggler >= n) continue;
            sar::Program prog;
            try {
              prog = sar::build_program(alg, n, true, straggler, nullptr);
            } catch (const std::exception& e) {
              printf("compile failed: %s n=%d: %s\n", alg, n, e.what());
              ++failures;
              continue;
            }
            const uint64_t count = 997 * n + 3;
            std::vector<std::vector<float>> buf(n, std::vector<float>(count));
            std::vector<double> want(count, 0.0);
            for (int r = 0; r < n; ++r)
              for (uint64_t i = 0; i < count; ++i) { buf[r][i] = uniform(r, i); want[i] += buf[r][i]; }
            std::vector<void*> ptrs(n);
            for (int r = 0; r < n; ++r) ptrs[r] = buf[r].data();
            std::vector<double> delay(n, 0.0);
            delay[straggler < 0 ? n - 1 : straggler] = 2.0;   // the straggler is 2 ms late
            const uint32_t st = sar::host_execute_program(prog, ptrs.data(), count, SAR_F32, 32, 0.5f, 4, delay.data(), 20.0);
            ++runs;
            if (st) { printf("status %u: %s n=%d copy=%s lanes=%s gate=%s\n", st, alg, n, copy, lanes, mode); ++failures; continue; }
            for (int r = 0; r < n; ++r)
              for (uint64_t i = 0; i < count; ++i)
                if (std::fabs(buf[r][i] - 0.5 * want[i]) > 1e-5) {
                  printf("wrong value: %s n=%d copy=%s lanes=%s gate=%s rank %d elem %llu\n", alg, n, copy, lanes, mode, r, (unsigned long long)i);
                  ++failures;
                  r = n;
                  break;
                }
          }
    }
  printf("%d runs, %d failures\n", runs, failures);
  return failures ? 1 : 0;
}
