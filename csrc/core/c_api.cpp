#include "c_api.h"

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "host_exec.h"
#include "plan.h"

struct sar_table {
  sar::Compiled c;
};

struct sar_program {
  sar::Program prog;
  std::vector<sar_table> tables;
};

static void set_err(char* err, int errlen, const std::string& s) {
  if (err && errlen > 0) { snprintf(err, (size_t)errlen, "%s", s.c_str()); }
}

extern "C" {

sar_table* sar_compile(const char* alg, int n, int prephase, int straggler, const char* schedule_text, char* err,
                       int errlen) {
  try {
    sar::Schedule sched;
    const sar::Schedule* sp = nullptr;
    if (schedule_text && *schedule_text) { sched = sar::parse_schedule(schedule_text); sp = &sched; }
    sar::Plan p = sar::plan_by_name(alg ? alg : "", n, prephase != 0, sp);
    std::vector<int> map;
    if (straggler >= 0) map = sar::straggler_rank_map(n, straggler);
    auto* t = new sar_table{sar::compile(p, map)};
    return t;
  } catch (const std::exception& e) {
    set_err(err, errlen, e.what());
    return nullptr;
  }
}
void sar_table_free(sar_table* t) { delete t; }

sar_program* sar_program_build(const char* alg, int n, int prephase, int straggler, const char* schedule_text,
                               char* err, int errlen) {
  try {
    sar::Schedule sched;
    const sar::Schedule* sp = nullptr;
    if (schedule_text && *schedule_text) { sched = sar::parse_schedule(schedule_text); sp = &sched; }
    auto* p = new sar_program{sar::build_program(alg ? alg : "", n, prephase != 0, straggler, sp), {}};
    for (auto& c : p->prog.phases) p->tables.push_back(sar_table{c});
    return p;
  } catch (const std::exception& e) {
    set_err(err, errlen, e.what());
    return nullptr;
  }
}
void sar_program_free(sar_program* p) { delete p; }
int sar_program_num_phases(const sar_program* p) { return (int)p->tables.size(); }
const sar_table* sar_program_phase(const sar_program* p, int i) { return &p->tables[i]; }
int sar_table_channel(const sar_table* t) { return t->c.channel; }
int sar_table_blocks_hint(const sar_table* t) { return t->c.blocks_hint; }
int sar_table_stages_hint(const sar_table* t) { return t->c.stages_hint; }
void sar_table_final_ver(const sar_table* t, int rank, uint8_t* out) {
  for (int c = 0; c < SAR_MAX_CHUNKS; ++c) out[c] = 0;
  if (rank < 0 || rank >= (int)t->c.ranks.size()) return;
  const auto& fv = t->c.ranks[rank].final_ver;
  for (size_t c = 0; c < fv.size() && c < SAR_MAX_CHUNKS; ++c) out[c] = fv[c];
}
int sar_table_gate_rounds(const sar_table* t) { return t->c.gate_rounds ? 1 : 0; }
uint64_t sar_gate_min_bytes(void) { return sar::gate_min_bytes(); }
int sar_table_lane1_eighths(const sar_table* t) { return t->c.lane1_eighths; }
int sar_table_validate(const sar_table* t, int rank, int nranks, char* err, int errlen) {
  if (rank < 0 || rank >= (int)t->c.ranks.size()) { if (err && errlen > 0) snprintf(err, (size_t)errlen, "no table for rank %d", rank); return 1; }
  const std::string why = sar::validate_rank_table(t->c.ranks[rank], rank, nranks, t->c.num_chunks);
  if (why.empty()) return 0;
  if (err && errlen > 0) snprintf(err, (size_t)errlen, "%s", why.c_str());
  return 1;
}
uint32_t sar_table_participants(const sar_table* t) { return t->c.participants; }
uint32_t sar_host_execute_program(const sar_program* p, void* const* bufs, uint64_t count, int dtype,
                                  uint32_t tile_elems, float scale, int blocks, const double* delay_ms,
                                  double timeout_s) {
  return sar::host_execute_program(p->prog, bufs, count, (SarDtype)dtype, tile_elems, scale, blocks, delay_ms, timeout_s);
}
int sar_table_nranks(const sar_table* t) { return t->c.n; }
int sar_table_num_chunks(const sar_table* t) { return t->c.num_chunks; }
int sar_table_num_rounds(const sar_table* t) { return t->c.num_rounds; }
int sar_table_max_version(const sar_table* t) { return t->c.max_version; }
int sar_table_num_ops(const sar_table* t, int rank) { return (int)t->c.ranks[rank].ops.size(); }
const SarOp* sar_table_ops(const sar_table* t, int rank) { return t->c.ranks[rank].ops.data(); }
int sar_table_num_round_begin(const sar_table* t, int rank) { return (int)t->c.ranks[rank].round_begin.size(); }
const uint16_t* sar_table_round_begin(const sar_table* t, int rank) { return t->c.ranks[rank].round_begin.data(); }
double sar_table_chunks_in(const sar_table* t, int rank) { return t->c.chunks_in[rank]; }
double sar_table_chunks_out(const sar_table* t, int rank) { return t->c.chunks_out[rank]; }

uint32_t sar_pick_tile_elems(uint64_t count, uint32_t esize, uint32_t num_chunks, uint32_t blocks, uint32_t min_bytes,
                             uint32_t max_bytes) {
  return sar::pick_tile_elems(count, esize, num_chunks, blocks, min_bytes, max_bytes);
}

uint32_t sar_host_execute(const sar_table* t, void* const* bufs, uint64_t count, int dtype, uint32_t tile_elems,
                          float scale, int blocks, const double* delay_ms, double timeout_s, int repeats) {
  return sar::host_execute(t->c, bufs, count, (SarDtype)dtype, tile_elems, scale, blocks, delay_ms, timeout_s, repeats);
}

const char* sar_status_string(uint32_t s) {
  switch (s) {
    case SAR_OK: return "ok";
    case SAR_TIMEOUT_ARRIVAL: return "timeout: a peer never entered the collective";
    case SAR_TIMEOUT_FLAG: return "timeout: a tile this rank depends on never became ready";
    case SAR_TIMEOUT_EXIT: return "timeout: a peer never left the collective";
    case SAR_TIMEOUT_PIPE: return "timeout: an on-chip pipeline barrier never completed";
    case SAR_BAD_TABLE: return "bad table";
    case SAR_ABORTED: return "aborted: another block of this rank gave up";
    default: return "unknown status";
  }
}

int sar_schedule_compact(int n, const char* schedule_text, char* out, int outlen) {
  try {
    sar::Schedule s = (schedule_text && *schedule_text) ? sar::parse_schedule(schedule_text) : sar::builtin_schedule(n);
    std::string c = sar::format_schedule_compact(s);
    if (out && outlen > 0) snprintf(out, (size_t)outlen, "%s", c.c_str());
    return (int)c.size();
  } catch (const std::exception&) {
    return -1;
  }
}
}
