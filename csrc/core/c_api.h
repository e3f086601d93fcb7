// C interface of the schedule compiler and the host executor (no CUDA needed).
#pragma once
#include <stdint.h>

#include "table.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct sar_table sar_table;      // one compiled phase
typedef struct sar_program sar_program;  // a collective: one or two phases launched back to back

// alg: stragglar | stragglar_a2a | ring | rhd | direct | rsag | reducescatter.
// prephase: 1 = the (n-1)-rank pre-phase is part of the collective, 0 = the
// caller has done it (the bench's DELAY = -1 mode).  straggler: physical rank
// to place at logical rank n-1, or -1 for none.  schedule_text: a schedule in
// the synthesizers' printed format, or NULL for the built-in one.
// Returns NULL and fills err on failure.
sar_table* sar_compile(const char* alg, int n, int prephase, int straggler, const char* schedule_text, char* err,
                       int errlen);
void sar_table_free(sar_table* t);
// The collective as launched: `direct` with its pre-phase has two phases (the
// non-stragglers' all-reduce on channel 1, then everybody on channel 0);
// everything else has one.  Phases are owned by the program.
sar_program* sar_program_build(const char* alg, int n, int prephase, int straggler, const char* schedule_text,
                               char* err, int errlen);
void sar_program_free(sar_program* p);
int sar_program_num_phases(const sar_program* p);
const sar_table* sar_program_phase(const sar_program* p, int i);
int sar_table_channel(const sar_table* t);
int sar_table_gate_rounds(const sar_table* t);   // 1: launch with round gating (for buffers of sar_gate_min_bytes() or more)
uint64_t sar_gate_min_bytes(void);
// 0 when rank's table is well-formed for a communicator of nranks (see validate_rank_table); else 1 and the reason
int sar_table_validate(const sar_table* t, int rank, int nranks, char* err, int errlen);
int sar_table_lane1_eighths(const sar_table* t);   // share of the blocks of lane 1, in eighths (4: half)
// out[c] (SAR_MAX_CHUNKS entries): the version rank `rank`'s slot of chunk c has when the collective is done
void sar_table_final_ver(const sar_table* t, int rank, uint8_t* out);
int sar_table_stages_hint(const sar_table* t);   // 0, or the ring stages per block the bulk-copy path should use
int sar_table_blocks_hint(const sar_table* t);   // 0, or the largest block count per rank worth using
uint32_t sar_table_participants(const sar_table* t);
int sar_table_nranks(const sar_table* t);
int sar_table_num_chunks(const sar_table* t);
int sar_table_num_rounds(const sar_table* t);
int sar_table_max_version(const sar_table* t);
int sar_table_num_ops(const sar_table* t, int rank);
const SarOp* sar_table_ops(const sar_table* t, int rank);
int sar_table_num_round_begin(const sar_table* t, int rank);
const uint16_t* sar_table_round_begin(const sar_table* t, int rank);
double sar_table_chunks_in(const sar_table* t, int rank);
double sar_table_chunks_out(const sar_table* t, int rank);

uint32_t sar_pick_tile_elems(uint64_t count, uint32_t esize, uint32_t num_chunks, uint32_t blocks, uint32_t min_bytes,
                             uint32_t max_bytes);
// Runs the table with host threads: bufs[r] = rank r's buffer of count
// elements, delay_ms[r] = sleep before rank r arrives (may be NULL).
// Returns a SarStatus.
uint32_t sar_host_execute_program(const sar_program* p, void* const* bufs, uint64_t count, int dtype,
                                  uint32_t tile_elems, float scale, int blocks, const double* delay_ms,
                                  double timeout_s);
uint32_t sar_host_execute(const sar_table* t, void* const* bufs, uint64_t count, int dtype, uint32_t tile_elems,
                          float scale, int blocks, const double* delay_ms, double timeout_s, int repeats);
const char* sar_status_string(uint32_t status);
// the compact text of a built-in or parsed schedule (for tooling); returns bytes written
int sar_schedule_compact(int n, const char* schedule_text, char* out, int outlen);

#ifdef __cplusplus
}
#endif
