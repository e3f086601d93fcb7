// Persistent table-executing collective kernel for sm_100a.
//
// One launch per rank and collective: G resident thread blocks walk the rank's
// op table (csrc/core/table.h) and move data with loads from and stores to
// peer memory over NVLink / NVSwitch.  There is no NCCL call and no host round
// trip between rounds: per-tile flags in the slot owner's memory order the
// rounds, so a tile is forwarded as soon as it is final and the rounds of the
// schedule pipeline into one another.  The reduction is fused into the
// transfer: a reduce op loads the peers' tiles and the own tile, adds in fp32
// and stores the rounded sum once (and, for a straggler matching, also into
// the peer).  Replaces the ncclSend/ncclRecv + reduce_add sequence of the
// reference (stragglar/allreduce_8GPU.cu:29-34,555-874).
//
// Two data paths execute the same table:
//   * simt: every thread moves 16-byte vectors with ld.relaxed.sys / st;
//   * tma:  a producer thread streams tiles from peer memory into a shared
//           memory ring with bulk async copies (cp.async.bulk + mbarrier
//           complete_tx), consumer warps add in place, bulk stores write the
//           result to local and peer memory, and a signal thread announces
//           finished tiles, keeping the system-scope fence off the issue path.
//           Few threads keep hundreds of KB in flight per block.
//
// Every wait (peer arrival, tile flag, pipeline barrier, exit) is bounded by a
// %globaltimer deadline.  On expiry the block records a SarStatus, raises the
// rank's abort word so that its other blocks stop too, waits for its own bulk
// copies in flight and returns; nothing traps and nothing spins forever.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../core/table.h"
#include "sar_params.h"

namespace sar_dev {

// ------------------------------------------------------------------ primitives
__device__ __forceinline__ uint64_t globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
// 16-byte load that is coherent at system scope (never served from a stale L1 line)
__device__ __forceinline__ uint4 ld_vec_sys(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_vec(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// NVLink multicast (NVLS): the switch adds the 16-byte vectors of all members of the multicast
// object, or stores one vector into all of them.
__device__ __forceinline__ void mc_st_vec(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// ----------------------------------------------------------- element handling
template <typename T> struct Vec;  // 16 bytes of T <-> floats
template <> struct Vec<float> {
  static constexpr int N = 4;
  __device__ static uint4 mc_ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  __device__ static void unpack(uint4 v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  __device__ static uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  __device__ static float load1(const void* p) { return __uint_as_float(ld_relaxed_sys((const uint32_t*)p)); }
  __device__ static void store1(void* p, float v) { *(volatile float*)p = v; }
};
template <> struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static uint4 mc_ld_reduce(const void* p) {   // the switch accumulates in fp32 and rounds once
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  __device__ static void unpack(uint4 v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
  __device__ static uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ static float load1(const void* p) {
    unsigned short h;
    asm volatile("ld.relaxed.sys.global.u16 %0, [%1];" : "=h"(h) : "l"(p) : "memory");
    return __uint_as_float((uint32_t)h << 16);
  }
  __device__ static void store1(void* p, float v) {
    __nv_bfloat16 h = __float2bfloat16_rn(v);
    *(volatile unsigned short*)p = *reinterpret_cast<unsigned short*>(&h);
  }
};
template <> struct Vec<__half> {
  static constexpr int N = 8;
  __device__ static uint4 mc_ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  __device__ static void unpack(uint4 v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
  __device__ static uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ static float load1(const void* p) {
    unsigned short h;
    asm volatile("ld.relaxed.sys.global.u16 %0, [%1];" : "=h"(h) : "l"(p) : "memory");
    return __half2float(*reinterpret_cast<__half*>(&h));
  }
  __device__ static void store1(void* p, float v) {
    __half h = __float2half_rn(v);
    *(volatile unsigned short*)p = *reinterpret_cast<unsigned short*>(&h);
  }
};

// --------------------------------------------------------------- bounded waits
struct WaitCtx {
  uint64_t deadline;        // %globaltimer value after which waits give up
  uint32_t* abort_flag;     // this rank's abort word (local memory)
  uint32_t* status;
};
__device__ __forceinline__ void record_failure(const WaitCtx& w, uint32_t code) {
  if (w.status) atomicCAS(w.status, 0u, code);
  atomicExch(w.abort_flag, 1u);
  __threadfence_system();
}
// Spin until *p reaches target; false on abort or deadline (failure recorded).
__device__ __noinline__ bool wait_word(const uint32_t* p, uint32_t target, const WaitCtx& w, uint32_t fail_code) {
  if (sar_reached(ld_acquire_sys(p), target)) return true;
  uint32_t ns = 20;
  for (uint64_t it = 0;; ++it) {
    if (sar_reached(ld_acquire_sys(p), target)) return true;
    if ((it & 15) == 15) {
      if (*(volatile uint32_t*)w.abort_flag) return false;
      if (globaltimer() > w.deadline) { record_failure(w, fail_code); return false; }
    }
    __nanosleep(ns);
    if (ns < 400) ns += ns >> 1;
  }
}

// Waits until the mirror word of every rank in `mask` (arrival_m or exited_m in this rank's own memory) has
// reached `target`.  All words are read at once, so a wait for seven peers costs one local round trip, not seven
// trips over the link.  Returns the ranks that have not got there (0 = all there); failure recorded.
__device__ __noinline__ uint32_t wait_mirrors(const uint32_t* words, uint32_t mask, int nranks, uint32_t target, const WaitCtx& w,
                                              uint32_t fail_code) {
  uint32_t ns = 20;
  for (uint64_t it = 0;; ++it) {
    uint32_t v[SAR_MAX_RANKS];
#pragma unroll
    for (int r = 0; r < SAR_MAX_RANKS; ++r) v[r] = (r < nranks && (mask >> r & 1)) ? ld_relaxed_sys(words + r) : target;
    uint32_t missing = 0;
#pragma unroll
    for (int r = 0; r < SAR_MAX_RANKS; ++r) if (!sar_reached(v[r], target)) missing |= 1u << r;
    if (!missing) { fence_sys(); return 0; }   // acquire: what the announcers wrote before is visible now
    if ((it & 15) == 15) {
      if (*(volatile uint32_t*)w.abort_flag) return missing;
      if (globaltimer() > w.deadline) { record_failure(w, fail_code); return missing; }
    }
    __nanosleep(ns);
    if (ns < 400) ns += ns >> 1;
  }
}

// An item of the rank's work list, resolved against the geometry.
struct Item {
  const SarOp* op;
  uint32_t tile;        // tile index within the chunk
  uint32_t fidx;        // flag index
  uint64_t elem0;       // first element
  uint32_t nelem;       // elements in the tile
  uint32_t need_ver;    // SAR_STAGE_OUT: version the own slot must have reached
};

// Geometry of the table resolved once per launch into shared memory, so that
// walking the items needs no 64-bit division.
struct OpGeom {
  uint64_t elem0;      // first element of the op's first tile
  uint64_t elem_end;   // end of the op's chunk
  uint32_t ntiles;     // tiles the op covers
  uint32_t tile0;      // its first tile within the chunk
};
struct RoundGeom { uint32_t op_begin, m, max_tiles, pad; };
struct TableGeom {
  OpGeom op[SAR_MAX_OPS];
  RoundGeom round[2][SAR_MAX_ROUNDS];   // per lane
  SarOp stage_op[2];                    // pseudo ops of staged mode: [0] SAR_STAGE_IN, [1] SAR_STAGE_OUT
  uint32_t num_rounds;
  uint32_t lanes;                       // lanes in effect for this launch (1 or 2)
  // round gating: round_prefix[R] = this rank's items in the schedule rounds before R (all lanes);
  // round_prefix[SAR_GATE_ALL_DONE] is the total
  uint32_t round_prefix[SAR_GATE_ALL_DONE + 1];
};

// Staged mode: the last blocks of the rank only stage (every tile in, then every tile out as it becomes final) and
// the others only walk the table, so that copying in, reducing and copying out overlap tile by tile instead of
// following one another in every block.  The launch says how many blocks stage (a block moves about 30 GB/s through
// its ring whatever the distance, so local copies at memory speed take many blocks: the backend adds up to 64 to
// the blocks that walk the table); by default a quarter of the blocks.  With a single block there is nobody to
// share with and the block does everything in turn (returns 0).
__device__ __forceinline__ uint32_t staging_blocks(const SarLaunchParams& P, uint32_t nblocks) {
  if (!P.user_in || nblocks < 2) return 0;
  if (P.staging_blocks) return P.staging_blocks < nblocks ? P.staging_blocks : nblocks - 1;
  return nblocks >= 8 ? nblocks / 4 : 1u;
}

// All threads of the block; ends with a block barrier.
__device__ void resolve_table(const SarLaunchParams& P, TableGeom& G, uint32_t nblocks) {
  const uint32_t nrounds = P.num_rounds < SAR_MAX_ROUNDS ? P.num_rounds : SAR_MAX_ROUNDS;
  const uint32_t nops = nrounds ? P.round_begin[nrounds] : 0;
  for (uint32_t o = threadIdx.x; o < nops && o < SAR_MAX_OPS; o += blockDim.x) {
    const SarOp op = P.ops[o];
    uint32_t t0, t1;
    sar_part_range(sar_chunk_tiles(P.geom, op.chunk), op.part, op.parts, &t0, &t1);
    const uint64_t cb = sar_chunk_begin(P.geom, op.chunk);
    G.op[o].elem0 = cb + (uint64_t)t0 * P.geom.tile_elems;
    G.op[o].elem_end = cb + sar_chunk_len(P.geom, op.chunk);
    G.op[o].ntiles = t1 - t0;
    G.op[o].tile0 = t0;
  }
  if (threadIdx.x == 0 && P.gate_rounds) {
    uint32_t items[SAR_GATE_ALL_DONE];
    for (uint32_t r = 0; r < SAR_GATE_ALL_DONE; ++r) items[r] = 0;
    for (uint32_t o = 0; o < nops && o < SAR_MAX_OPS; ++o) {
      const SarOp op = P.ops[o];
      if (op.round < SAR_GATE_ALL_DONE) items[op.round] += sar_op_tiles(P.geom, op);
    }
    G.round_prefix[0] = 0;
    for (uint32_t r = 0; r < SAR_GATE_ALL_DONE; ++r) G.round_prefix[r + 1] = G.round_prefix[r] + items[r];
  }
  if (threadIdx.x == 0) {
    uint32_t table_lanes = 1;
    for (uint32_t o = 0; o < nops && o < SAR_MAX_OPS; ++o) if (P.ops[o].lane) table_lanes = 2;
    uint32_t lanes, lane, lb, lnb;
    sar_lane_of_block(0, nblocks - staging_blocks(P, nblocks), table_lanes, P.lane1_eighths, &lanes, &lane, &lb, &lnb);
    G.lanes = lanes;
    G.num_rounds = nrounds;
    for (int k = 0; k < 2; ++k) {
      SarOp z{};
      z.kind = k == 0 ? SAR_STAGE_IN : SAR_STAGE_OUT;
      z.round = 255; z.parts = 1;       // outside every schedule round: neither traced nor counted by the round gate
      G.stage_op[k] = z;
    }
  }
  __syncthreads();
  for (uint32_t r = threadIdx.x; r < nrounds; r += blockDim.x) {
    const uint32_t ob = P.round_begin[r], oe = P.round_begin[r + 1];
    uint32_t split = oe;                  // one lane: every op of the round
    if (G.lanes == 2) { split = ob; while (split < oe && P.ops[split].lane == 0) ++split; }
    for (uint32_t l = 0; l < 2; ++l) {
      const uint32_t b = l == 0 ? ob : split, e = l == 0 ? split : oe;
      uint32_t mx = 0;
      for (uint32_t o = b; o < e; ++o) mx = G.op[o].ntiles > mx ? G.op[o].ntiles : mx;
      G.round[l][r].op_begin = b; G.round[l][r].m = e - b; G.round[l][r].max_tiles = mx;
    }
  }
  __syncthreads();
}

// Iterates the items of block `block` of `nblocks` in table order.  In staged mode the table's items are
// preceded by one stage-in item per tile of the buffer and followed by one stage-out item per tile (chunks
// interleaved tile by tile, dealt to all blocks of the rank whatever their lane).
struct ItemWalker {
  const SarLaunchParams* P;
  const TableGeom* G;
  uint32_t block_all, nblocks_all;   // position and size among all blocks of the rank
  uint32_t block, nblocks;   // position and size inside the block's lane
  uint32_t lane;
  uint32_t ri;            // current round index
  uint32_t ob, m, items, k, base_mod;
  uint32_t phase;         // 0: stage-in, 1: the table, 2: stage-out, 3: done
  uint32_t sk;            // next staging item of this block
  bool stager, table_only;   // staged mode with several blocks: this block only stages / only walks the table
  __device__ void init(const SarLaunchParams* p, const TableGeom* g, uint32_t b, uint32_t nb) {
    P = p; G = g; ri = 0; base_mod = 0;
    block_all = b; nblocks_all = nb;
    stager = false; table_only = false;
    const uint32_t ns = staging_blocks(*p, nb);
    uint32_t lanes;
    if (ns && b >= nb - ns) {
      // a staging block: its share of the staging items, no table items
      stager = true;
      block_all = b - (nb - ns); nblocks_all = ns;
      lane = 0; block = 0; nblocks = 1; ri = g->num_rounds;
    } else {
      table_only = ns != 0;
      sar_lane_of_block(b, nb - ns, g->lanes, p->lane1_eighths, &lanes, &lane, &block, &nblocks);
    }
    phase = (p->user_in && !table_only) ? 0u : 1u;
    sk = block_all;
    if (!stager) load_round();
  }
  __device__ void load_round() {
    while (ri < G->num_rounds) {
      ob = G->round[lane][ri].op_begin;
      m = G->round[lane][ri].m;
      items = G->round[lane][ri].max_tiles * m;
      k = (block + nblocks - base_mod) % nblocks;
      if (k < items) return;
      base_mod = (base_mod + items) % nblocks;
      ++ri;
    }
  }
  // staging item sk: tile sk / num_chunks of chunk sk % num_chunks
  __device__ bool next_staging(Item* it, uint32_t which) {
    const uint32_t nch = P->geom.num_chunks;
    const uint32_t total = P->geom.tiles_per_chunk * nch;
    while (sk < total) {
      const uint32_t c = sk % nch, lt = sk / nch;
      sk += nblocks_all;
      if (lt >= sar_chunk_tiles(P->geom, c)) continue;
      const uint64_t cb = sar_chunk_begin(P->geom, c);
      const uint64_t ce = cb + sar_chunk_len(P->geom, c);
      const uint64_t e0 = cb + (uint64_t)lt * P->geom.tile_elems;
      const uint64_t e1 = e0 + P->geom.tile_elems < ce ? e0 + P->geom.tile_elems : ce;
      it->op = &G->stage_op[which]; it->tile = lt; it->fidx = sar_flag_index(P->geom, c, lt);
      it->elem0 = e0; it->nelem = (uint32_t)(e1 - e0); it->need_ver = P->final_ver[c];
      return true;
    }
    return false;
  }
  // false when the work list is exhausted
  __device__ bool next(Item* it) {
    if (phase == 0) {
      if (next_staging(it, 0)) return true;
      phase = 1;
    }
    if (phase == 1) {
      while (ri < G->num_rounds) {
        while (k < items) {
          const uint32_t o = ob + k % m;
          const uint32_t lt = k / m;
          k += nblocks;
          const OpGeom& og = G->op[o];
          if (lt >= og.ntiles) continue;
          const SarOp* op = P->ops + o;
          const uint64_t e0 = og.elem0 + (uint64_t)lt * P->geom.tile_elems;
          uint64_t e1 = e0 + P->geom.tile_elems;
          if (e1 > og.elem_end) e1 = og.elem_end;
          it->op = op; it->tile = og.tile0 + lt; it->fidx = sar_flag_index(P->geom, op->chunk, og.tile0 + lt);
          it->elem0 = e0; it->nelem = (uint32_t)(e1 - e0); it->need_ver = 0;
          return true;
        }
        base_mod = (base_mod + items) % nblocks;
        ++ri;
        load_round();
      }
      phase = (P->user_out && !table_only) ? 2u : 3u;
      sk = block_all;
    }
    if (phase == 2) {
      if (next_staging(it, 1)) return true;
      phase = 3;
    }
    return false;
  }
};

__device__ __forceinline__ bool op_reads_local(const SarOp* op) {
  return op->kind == SAR_REDUCE_PUSH || (op->kind == SAR_REDUCE && (op->flags & SAR_F_LOCAL));
}

// Per-round statistics (optional): when the first item of a round had its operands and could start,
// how long the items of the round waited for their operands, when the last one was announced.
__device__ __forceinline__ void trace_item_start(const SarLaunchParams& P, const SarOp* op, uint64_t t_begin, uint64_t t_ready) {
  if (!P.trace_rounds || op->round >= SAR_MAX_ROUNDS) return;
  atomicMin((unsigned long long*)&P.trace[2 + op->round], (unsigned long long)t_ready);
  atomicAdd((unsigned long long*)&P.trace[2 + 2 * SAR_MAX_ROUNDS + op->round], (unsigned long long)(t_ready - t_begin));
}
__device__ __forceinline__ void trace_item_end(const SarLaunchParams& P, const SarOp* op) {
  if (!P.trace_rounds || op->round >= SAR_MAX_ROUNDS) return;
  atomicMax((unsigned long long*)&P.trace[2 + SAR_MAX_ROUNDS + op->round], (unsigned long long)globaltimer());
}

// ---- round gating (see SAR_GATE_ALL_DONE in table.h)
__device__ __forceinline__ uint64_t ld_relaxed_sys_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_max_sys_u64(uint64_t* p, uint64_t v) {
  asm volatile("red.relaxed.sys.global.max.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// The newest round this rank may announce once `done` of its items are finished: the largest R such
// that all but `slack` of its items of the rounds before R are done (rounds without items are skipped).
__device__ __forceinline__ uint32_t gate_round_for(const TableGeom& G, uint32_t done, uint32_t slack) {
  uint32_t R = 0;
  while (R < SAR_GATE_ALL_DONE && G.round_prefix[R + 1] <= done + slack) ++R;
  return R;
}
// Raises this rank's announcement to R in every participant's memory (its own included).  The caller has
// ordered the data of the finished items before this call (fence at system scope).
__device__ __forceinline__ void gate_announce(const SarLaunchParams& P, uint32_t R) {
  SarCtrl* me = P.comm.ctrl[P.rank];
  if (atomicMax(&me->announced, R + 1u) >= R + 1u) return;   // somebody has announced R (or more) already
  for (int q = 0; q < P.nranks; ++q)
    if (P.participants >> q & 1) red_max_sys_u64(&P.comm.ctrl[q]->gate[P.rank], P.gate_base + R);
}
// One thread of the rank's block 0, after resolve_table: the rounds before the first one with items are done.
__device__ __forceinline__ void gate_announce_first(const SarLaunchParams& P, const TableGeom& G) {
  fence_sys();
  gate_announce(P, gate_round_for(G, 0, 0));
}
// The thread that has just announced an item: counts it, and announces the rounds that this completes.
__device__ __forceinline__ void gate_item_done(const SarLaunchParams& P, const TableGeom& G, const SarOp* op) {
  if (!P.gate_rounds || op->round >= SAR_GATE_ALL_DONE) return;
  SarCtrl* me = P.comm.ctrl[P.rank];
  const uint32_t done = atomicAdd(&me->items_done, 1u) + 1u;
  const uint32_t R = gate_round_for(G, done, P.gate_slack);
  if (R == 0 || *(volatile uint32_t*)&me->announced >= R + 1u) return;
  fence_sys();   // the items counted so far (by any thread of this rank) are visible before the announcement
  gate_announce(P, R);
}
// Bounded wait until every participant has announced round `round` (the words are in this rank's memory).
__device__ __noinline__ bool wait_gate(const SarLaunchParams& P, uint32_t round, const WaitCtx& w) {
  const uint64_t target = P.gate_base + round;
  const uint64_t* g = P.comm.ctrl[P.rank]->gate;
  uint32_t ns = 20;
  for (uint64_t it = 0;; ++it) {
    bool all = true;
    for (int r = 0; r < P.nranks; ++r)
      if ((P.participants >> r & 1) && ld_relaxed_sys_u64(g + r) < target) all = false;
    if (all) { fence_sys(); return true; }   // acquire: what the announcers ordered before is visible now
    if ((it & 15) == 15) {
      if (*(volatile uint32_t*)w.abort_flag) return false;
      if (globaltimer() > w.deadline) { record_failure(w, SAR_TIMEOUT_FLAG); return false; }
    }
    __nanosleep(ns);
    if (ns < 200) ns += ns >> 1;
  }
}

// Waits (one thread) until every operand of the item is ready.  `gate_passed`: the newest schedule
// round this thread has seen open (round gating).
__device__ bool wait_item_ready(const SarLaunchParams& P, const Item& it, const WaitCtx& w, uint32_t* arrived_mask,
                                uint32_t* gate_passed) {
  const SarOp* op = it.op;
  if (op->kind == SAR_STAGE_IN) return true;   // the previous collective's exit barrier has released the slot
  if (op->kind == SAR_STAGE_OUT)
    return wait_word(P.comm.flags[P.rank] + it.fidx, P.epoch_base + it.need_ver, w, SAR_TIMEOUT_FLAG);
  // staged mode: version 0 of a tile exists once its owner has copied it in, which the tile's flag tells
  const bool staged = P.user_in != nullptr;
  if (P.gate_rounds && op->round >= 1 && op->round < SAR_GATE_ALL_DONE) {
    if (op->round > *gate_passed) {
      if (!wait_gate(P, op->round, w)) return false;
      *gate_passed = op->round;
    }
    // a full barrier between rounds: every participant has arrived and every operand is complete
    if (P.gate_slack == 0 && !staged) { *arrived_mask = P.participants; return true; }
  }
  {
    uint32_t need = 0;
    for (int q = 0; q < op->nsrc; ++q) need |= 1u << op->src[q];
    need &= ~*arrived_mask;
    if (need) {
      if (wait_mirrors(P.comm.ctrl[P.rank]->arrival_m, need, P.nranks, P.epoch_base, w, SAR_TIMEOUT_ARRIVAL)) return false;
      *arrived_mask |= need;
    }
  }
  // every flag the item depends on, polled together: the loads of one turn are independent, so waiting for seven
  // peers' tiles costs one trip over the link per turn, not seven
  const uint32_t* ptr[SAR_MAX_RANKS + 1];
  uint32_t want[SAR_MAX_RANKS + 1];
  int nf = 0;
  // (A push names the version it replaces in the destination.  Version 0 there, in staged mode, is the
  // destination's own copy-in of that tile, and whatever is pushed into a slot contains that rank's contribution to
  // the chunk or follows a read of it, both of which waited for that copy-in: the push is ordered after it already.)
  for (int q = 0; q < op->nsrc; ++q)
    if (op->src_ver[q] || (staged && op->kind != SAR_PUSH)) {
      ptr[nf] = P.comm.flags[op->src[q]] + it.fidx; want[nf] = P.epoch_base + op->src_ver[q]; ++nf;
    }
  if (op->local_ver || staged) { ptr[nf] = P.comm.flags[P.rank] + it.fidx; want[nf] = P.epoch_base + op->local_ver; ++nf; }
  if (nf == 0) return true;
  if (nf == 1) return wait_word(ptr[0], want[0], w, SAR_TIMEOUT_FLAG);
  uint32_t ns = 20;
  for (uint64_t turn = 0;; ++turn) {
    uint32_t v[SAR_MAX_RANKS + 1];
    for (int i = 0; i < nf; ++i) v[i] = ld_relaxed_sys(ptr[i]);
    bool all = true;
    for (int i = 0; i < nf; ++i) all = all && sar_reached(v[i], want[i]);
    if (all) { fence_sys(); return true; }   // acquire
    if ((turn & 15) == 15) {
      if (*(volatile uint32_t*)w.abort_flag) return false;
      if (globaltimer() > w.deadline) { record_failure(w, SAR_TIMEOUT_FLAG); return false; }
    }
    __nanosleep(ns);
    if (ns < 400) ns += ns >> 1;
  }
}

// Announces a finished tile.  The caller has ordered the tile's stores before
// this call at system scope (fence_sys after the block barrier); the flags are
// plain system-scope stores after that fence (release pattern).
__device__ __forceinline__ void publish_item(const SarLaunchParams& P, const SarOp* op, uint32_t fidx) {
  if (op->kind == SAR_STAGE_OUT) return;
  if (op->kind == SAR_STAGE_IN) { st_relaxed_sys(P.comm.flags[P.rank] + fidx, P.epoch_base); return; }   // version 0
  if (op->kind != SAR_PUSH) st_relaxed_sys(P.comm.flags[P.rank] + fidx, P.epoch_base + op->post_ver);
  if (op->kind == SAR_REDUCE_PUSH) st_relaxed_sys(P.comm.flags[op->src[0]] + fidx, P.epoch_base + op->push_ver);
  if (op->kind == SAR_PUSH)
    for (int q = 0; q < op->nsrc; ++q) st_relaxed_sys(P.comm.flags[op->src[q]] + fidx, P.epoch_base + op->push_ver);
}

// Sub-vector tail (fewer than 16 bytes) of a tile, element by element.
template <typename T>
__device__ void scalar_elems(const SarLaunchParams& P, const SarOp* op, uint64_t e0, uint32_t n) {
  char* own = (char*)P.comm.buf[P.rank];
  const bool local = op_reads_local(op);
  const float scale = (op->flags & SAR_F_SCALE) ? P.scale : 1.0f;
  for (uint32_t i = 0; i < n; ++i) {
    const uint64_t off = (e0 + i) * sizeof(T);
    float acc;
    if (op->kind == SAR_PUSH) {
      const float v = Vec<T>::load1(own + off);
      for (int q = 0; q < op->nsrc; ++q) Vec<T>::store1((char*)P.comm.buf[op->src[q]] + off, v);
      continue;
    }
    if (op->kind == SAR_COPY) acc = Vec<T>::load1((char*)P.comm.buf[op->src[0]] + off);
    else {
      acc = local ? Vec<T>::load1(own + off) : 0.0f;
      for (int q = 0; q < op->nsrc; ++q) acc += Vec<T>::load1((char*)P.comm.buf[op->src[q]] + off);
      acc *= scale;
    }
    Vec<T>::store1(own + off, acc);
    if (op->kind == SAR_REDUCE_PUSH) Vec<T>::store1((char*)P.comm.buf[op->src[0]] + off, acc);
  }
}

// The multicast view that serves this op in one instruction, or nullptr: a reduction over the own
// slot and exactly the other members of a group (the switch adds all members' values), or a push
// to exactly the other members (one multimem.st; it also rewrites the own slot with the value it
// already holds).
__device__ __forceinline__ char* mc_view_for(const SarLaunchParams& P, const SarOp* op) {
  const bool reduce = op->kind == SAR_REDUCE && (op->flags & SAR_F_LOCAL);
  if (!reduce && op->kind != SAR_PUSH) return nullptr;
  if (!P.mc[0].base && !P.mc[1].base) return nullptr;
  uint32_t mask = 1u << P.rank;
  for (int q = 0; q < op->nsrc; ++q) mask |= 1u << op->src[q];
  for (int g = 0; g < 2; ++g)
    if (P.mc[g].base && P.mc[g].members == mask) return (char*)P.mc[g].base;
  return nullptr;
}

// --------------------------------------------------------- staging (all paths)
// Elements [e0, e0 + n) of a buffer of element type `dtype` as floats, and back.
__device__ __forceinline__ float load_as_float(const void* base, uint64_t e, int dtype) {
  // volatile: never served from a stale L1 line (the slot may have been written by a peer or by a bulk copy)
  if (dtype == SAR_F32) return ((const volatile float*)base)[e];
  const unsigned short h = ((const volatile unsigned short*)base)[e];
  if (dtype == SAR_BF16) return __uint_as_float((uint32_t)h << 16);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
__device__ __forceinline__ void store_from_float(void* base, uint64_t e, int dtype, float v) {
  if (dtype == SAR_F32) { ((float*)base)[e] = v; return; }
  unsigned short h;
  if (dtype == SAR_BF16) { __nv_bfloat16 b = __float2bfloat16_rn(v); h = *reinterpret_cast<unsigned short*>(&b); }
  else { __half b = __float2half_rn(v); h = *reinterpret_cast<unsigned short*>(&b); }
  ((unsigned short*)base)[e] = h;
}
// A staging tile: SAR_STAGE_IN copies the caller's elements into the own slot (wire type T), SAR_STAGE_OUT copies
// the own slot into the caller's output.  Same element type and 16-byte aligned on both sides: vector copies;
// otherwise the elements are converted one wire vector at a time.  `tid` of `nth` threads work together.
template <typename T>
__device__ void stage_tile(const SarLaunchParams& P, const Item& it, const uint32_t tid, const uint32_t nth) {
  constexpr int N = Vec<T>::N;
  const bool in = it.op->kind == SAR_STAGE_IN;
  char* own = (char*)P.comm.buf[P.rank];
  const int udt = P.user_dtype;
  const bool same = udt == P.dtype;
  const uint32_t nvec = it.nelem / N;
  if (same) {
    const char* src = in ? (const char*)P.user_in : own;
    char* dst = in ? own : (char*)P.user_out;
    const uint64_t b0 = it.elem0 * sizeof(T);
    if ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
      uint32_t v = tid;
      for (; v + 3 * nth < nvec; v += 4 * nth) {
        uint4 r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) r[u] = ld_vec_sys(src + b0 + (size_t)(v + u * nth) * 16);
#pragma unroll
        for (int u = 0; u < 4; ++u) st_vec(dst + b0 + (size_t)(v + u * nth) * 16, r[u]);
      }
      for (; v < nvec; v += nth) st_vec(dst + b0 + (size_t)v * 16, ld_vec_sys(src + b0 + (size_t)v * 16));
      for (uint32_t i = nvec * N + tid; i < it.nelem; i += nth)
        store_from_float(dst, it.elem0 + i, udt, load_as_float(src, it.elem0 + i, udt));
      return;
    }
  }
  // converting (or unaligned) copy: a thread handles the N elements of one wire vector
  const void* src = in ? P.user_in : (const void*)own;
  void* dst = in ? (void*)own : P.user_out;
  const int sdt = in ? udt : P.dtype, ddt = in ? P.dtype : udt;
  for (uint32_t v = tid; v < nvec; v += nth) {
    float f[N];
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = load_as_float(src, it.elem0 + (uint64_t)v * N + i, sdt);
    if (in) st_vec(own + (it.elem0 + (uint64_t)v * N) * sizeof(T), Vec<T>::pack(f));
    else {
#pragma unroll
      for (int i = 0; i < N; ++i) store_from_float(dst, it.elem0 + (uint64_t)v * N + i, ddt, f[i]);
    }
  }
  for (uint32_t i = nvec * N + tid; i < it.nelem; i += nth)
    store_from_float(dst, it.elem0 + i, ddt, load_as_float(src, it.elem0 + i, sdt));
}

// ------------------------------------------------------------------- simt path
// `tid` of `nth` threads work on the tile together.
template <typename T, int UNROLL>
__device__ void simt_tile(const SarLaunchParams& P, const Item& it, const uint32_t tid, const uint32_t nth) {
  constexpr int N = Vec<T>::N;
  const SarOp* op = it.op;
  if (op->kind >= SAR_STAGE_IN) { stage_tile<T>(P, it, tid, nth); return; }
  const uint32_t nvec = it.nelem / N;
  const uint64_t byte0 = it.elem0 * sizeof(T);
  char* own = (char*)P.comm.buf[P.rank] + byte0;
  char* mcv = mc_view_for(P, op);
  if (mcv) {
    mcv += byte0;
    if (op->kind == SAR_PUSH) {
      // all destinations in one store through the switch
      uint32_t v = tid;
      for (; v + (UNROLL - 1) * nth < nvec; v += UNROLL * nth) {
        uint4 r[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) r[u] = ld_vec_sys(own + (size_t)(v + u * nth) * 16);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) mc_st_vec(mcv + (size_t)(v + u * nth) * 16, r[u]);
      }
      for (; v < nvec; v += nth) mc_st_vec(mcv + (size_t)v * 16, ld_vec_sys(own + (size_t)v * 16));
    } else {
      // the switch loads every member's vector (the own one included) and returns the sum
      const bool scaled = (op->flags & SAR_F_SCALE) != 0;
      const float scale = P.scale;
      uint32_t v = tid;
      for (; v + (UNROLL - 1) * nth < nvec; v += UNROLL * nth) {
        uint4 r[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) r[u] = Vec<T>::mc_ld_reduce(mcv + (size_t)(v + u * nth) * 16);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          if (scaled) {
            float f[N];
            Vec<T>::unpack(r[u], f);
#pragma unroll
            for (int i = 0; i < N; ++i) f[i] *= scale;
            r[u] = Vec<T>::pack(f);
          }
          st_vec(own + (size_t)(v + u * nth) * 16, r[u]);
        }
      }
      for (; v < nvec; v += nth) {
        uint4 r = Vec<T>::mc_ld_reduce(mcv + (size_t)v * 16);
        if (scaled) {
          float f[N];
          Vec<T>::unpack(r, f);
#pragma unroll
          for (int i = 0; i < N; ++i) f[i] *= scale;
          r = Vec<T>::pack(f);
        }
        st_vec(own + (size_t)v * 16, r);
      }
    }
  } else if (op->kind == SAR_COPY || op->kind == SAR_PUSH) {
    const bool push = op->kind == SAR_PUSH;
    const char* src = push ? own : (const char*)P.comm.buf[op->src[0]] + byte0;
    const int ndst = push ? op->nsrc : 1;
    uint32_t v = tid;
    for (; v + (UNROLL - 1) * nth < nvec; v += UNROLL * nth) {
      uint4 r[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) r[u] = ld_vec_sys(src + (size_t)(v + u * nth) * 16);
      for (int q = 0; q < ndst; ++q) {
        char* dst = push ? (char*)P.comm.buf[op->src[q]] + byte0 : own;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) st_vec(dst + (size_t)(v + u * nth) * 16, r[u]);
      }
    }
    for (; v < nvec; v += nth) {
      const uint4 r = ld_vec_sys(src + (size_t)v * 16);
      for (int q = 0; q < ndst; ++q) st_vec((push ? (char*)P.comm.buf[op->src[q]] + byte0 : own) + (size_t)v * 16, r);
    }
  } else {
    const bool local = op_reads_local(op);
    const float scale = (op->flags & SAR_F_SCALE) ? P.scale : 1.0f;
    const int nsrc = op->nsrc;
    char* push = op->kind == SAR_REDUCE_PUSH ? (char*)P.comm.buf[op->src[0]] + byte0 : nullptr;
    if (nsrc == 1) {
      // pairwise: own (+) one peer, unrolled over vectors
      const char* src = (const char*)P.comm.buf[op->src[0]] + byte0;
      uint32_t v = tid;
      for (; v + (UNROLL - 1) * nth < nvec; v += UNROLL * nth) {
        uint4 a[UNROLL], b[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) a[u] = ld_vec_sys(src + (size_t)(v + u * nth) * 16);
        if (local) {
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) b[u] = ld_vec_sys(own + (size_t)(v + u * nth) * 16);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          float fa[N], fb[N];
          Vec<T>::unpack(a[u], fa);
          if (local) {
            Vec<T>::unpack(b[u], fb);
#pragma unroll
            for (int i = 0; i < N; ++i) fa[i] += fb[i];
          }
#pragma unroll
          for (int i = 0; i < N; ++i) fa[i] *= scale;
          const uint4 o = Vec<T>::pack(fa);
          st_vec(own + (size_t)(v + u * nth) * 16, o);
          if (push) st_vec(push + (size_t)(v + u * nth) * 16, o);
        }
      }
      for (; v < nvec; v += nth) {
        float fa[N], fb[N];
        Vec<T>::unpack(ld_vec_sys(src + (size_t)v * 16), fa);
        if (local) {
          Vec<T>::unpack(ld_vec_sys(own + (size_t)v * 16), fb);
#pragma unroll
          for (int i = 0; i < N; ++i) fa[i] += fb[i];
        }
#pragma unroll
        for (int i = 0; i < N; ++i) fa[i] *= scale;
        const uint4 o = Vec<T>::pack(fa);
        st_vec(own + (size_t)v * 16, o);
        if (push) st_vec(push + (size_t)v * 16, o);
      }
    } else {
      // several peers (reduce-scatter stage): all sources of a vector in flight at once
      for (uint32_t v = tid; v < nvec; v += nth) {
        float acc[N];
        if (local) Vec<T>::unpack(ld_vec_sys(own + (size_t)v * 16), acc);
        else {
#pragma unroll
          for (int i = 0; i < N; ++i) acc[i] = 0.0f;
        }
        int q = 0;
        for (; q + 4 <= nsrc; q += 4) {
          uint4 r[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) r[u] = ld_vec_sys((const char*)P.comm.buf[op->src[q + u]] + byte0 + (size_t)v * 16);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float f[N];
            Vec<T>::unpack(r[u], f);
#pragma unroll
            for (int i = 0; i < N; ++i) acc[i] += f[i];
          }
        }
        for (; q < nsrc; ++q) {
          float f[N];
          Vec<T>::unpack(ld_vec_sys((const char*)P.comm.buf[op->src[q]] + byte0 + (size_t)v * 16), f);
#pragma unroll
          for (int i = 0; i < N; ++i) acc[i] += f[i];
        }
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] *= scale;
        st_vec(own + (size_t)v * 16, Vec<T>::pack(acc));
      }
    }
  }
  if (tid == 0 && (it.nelem % N)) scalar_elems<T>(P, op, it.elem0 + (uint64_t)nvec * N, it.nelem % N);
}

// Entry and exit protocol shared by both paths.  Returns the wait context.
__device__ __forceinline__ WaitCtx enter_collective(const SarLaunchParams& P, uint32_t block) {
  WaitCtx w;
  if (P.delay_ns) {
    if (threadIdx.x == 0) {
      const uint64_t t0 = globaltimer();
      const uint64_t d = P.delay_ns < 10000000000ull ? P.delay_ns : 10000000000ull;
      while (globaltimer() - t0 < d) __nanosleep(200);
    }
    __syncthreads();
  }
  w.deadline = globaltimer() + P.timeout_ns;
  w.abort_flag = &P.comm.ctrl[P.rank]->abort_flag;
  w.status = P.status;
  if (block == 0 && threadIdx.x == 0) {
    if (P.trace) P.trace[0] = globaltimer();
    st_release_sys(&P.comm.ctrl[P.rank]->arrival, P.epoch_base);
    // the same word into every participant's memory, where its waits look for it
    for (int q = 0; q < P.nranks; ++q)
      if (q != P.rank && (P.participants >> q & 1)) st_relaxed_sys(&P.comm.ctrl[q]->arrival_m[P.rank], P.epoch_base);
  }
  return w;
}

// Called by one thread per block after all of the block's stores are ordered
// before it (bar.sync).  The last block to finish announces the rank's exit and
// waits until every participant has left: only then may the caller's next
// kernel overwrite memory that peers were reading.
__device__ void leave_collective(const SarLaunchParams& P, const WaitCtx& w, uint32_t nblocks) {
  __threadfence();
  SarCtrl* me = P.comm.ctrl[P.rank];
  const uint32_t done = atomicAdd(&me->blocks_done, 1u) + 1u;
  if (done != nblocks) return;
  me->blocks_done = 0;
  me->items_done = 0;
  me->announced = 0;
  __threadfence();
  if (*(volatile uint32_t*)w.abort_flag == 0) {
    fence_sys();
    st_release_sys(&me->exited, P.epoch_base);
    for (int q = 0; q < P.nranks; ++q)
      if (q != P.rank && (P.participants >> q & 1)) st_relaxed_sys(&P.comm.ctrl[q]->exited_m[P.rank], P.epoch_base);
    wait_mirrors(me->exited_m, P.participants & ~(1u << P.rank), P.nranks, P.epoch_base, w, SAR_TIMEOUT_EXIT);
  } else if (P.status) {
    atomicCAS(P.status, 0u, (uint32_t)SAR_ABORTED);
  }
  if (P.trace) P.trace[1] = globaltimer();
}

template <typename T>
__device__ void run_rank_simt(const SarLaunchParams& P, uint32_t block, uint32_t nblocks) {
  __shared__ TableGeom G;
  __shared__ Item s_item;
  __shared__ int s_state;   // 1: item ready, 0: table exhausted, -1: a wait failed
  WaitCtx w = enter_collective(P, block);
  resolve_table(P, G, nblocks);
  ItemWalker walk;
  uint32_t arrived = 1u << P.rank, gate_passed = 0;
  if (threadIdx.x == 0) {
    if (P.gate_rounds && block == 0) gate_announce_first(P, G);
    walk.init(&P, &G, block, nblocks);
  }
  while (true) {
    if (threadIdx.x == 0) {
      Item it;
      if (!walk.next(&it)) s_state = 0;
      else {
        const uint64_t t_begin = P.trace_rounds ? globaltimer() : 0;
        if (!wait_item_ready(P, it, w, &arrived, &gate_passed)) s_state = -1;
        else {
          if (P.trace_rounds) trace_item_start(P, it.op, t_begin, globaltimer());
          s_item = it; s_state = 1;
        }
      }
    }
    __syncthreads();
    if (s_state != 1) break;
    const Item it = s_item;
    simt_tile<T, 4>(P, it, threadIdx.x, blockDim.x);
    __syncthreads();   // every store of the tile is issued; s_item may be rewritten
    if (threadIdx.x == 0) {
      fence_sys();
      publish_item(P, it.op, it.fidx);
      trace_item_end(P, it.op);
      gate_item_done(P, G, it.op);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) leave_collective(P, w, nblocks);
}

// -------------------------------------------------------------------- tma path
namespace tma {
constexpr int kStages = 6;
constexpr int kStageBytes = 32768;
constexpr int kConsumerWarps = 4;
constexpr int kThreads = 32 * (2 + kConsumerWarps);   // producer warp, consumer warps, signal warp
constexpr int kPendRing = 32;

struct StageDesc {
  const SarOp* op;      // nullptr: no more work
  uint64_t byte_off;    // offset of this piece in the buffers
  uint32_t bytes;       // bytes per source in this piece (multiple of 16)
  uint32_t slot_bytes;  // distance between sources inside the stage
  uint32_t nsrc_total;  // buffers loaded into the stage (peers, then the own one if read)
  uint32_t last;        // last piece of its item
  uint32_t fidx;
  uint32_t tail_elems;  // sub-vector tail of the item (handled with plain loads), last piece only
  uint64_t tail_elem0;
  // staging pieces: bulk-loaded from the caller's tensor (stage-in) or the own slot (stage-out), converted in
  // shared memory when the element types differ, bulk-stored to the other side.  item_elems != 0: the unaligned
  // fallback, the consumer threads move the whole item with plain loads and stores.
  uint64_t item_elem0;
  uint32_t item_elems;
  uint32_t dst_bytes;   // bytes stored (differs from `bytes` when the piece is converted)
  uint64_t dst_off;     // byte offset on the destination side
  uint32_t piece_elems; // elements in this piece
};
struct PendEntry { const SarOp* op; uint32_t fidx; uint32_t seq; };

struct Shared {
  alignas(128) unsigned char ring[kStages][kStageBytes];
  alignas(8) uint64_t full[kStages];
  alignas(8) uint64_t empty[kStages];
  StageDesc desc[kStages];
  TableGeom geom;
  // finished items on their way to the signal warp
  PendEntry pend[kPendRing];
  uint32_t pend_tail;   // written by the storing thread
  uint32_t pend_head;   // written by the signal thread
  uint32_t landed;      // store groups with seq < landed have completed
  uint32_t consumers_done;
  int abort_seen;
  uint32_t issued;      // pieces the producer has issued (written when it stops)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(b)), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait on a pipeline barrier
__device__ __noinline__ bool mbar_wait(uint64_t* b, uint32_t parity, const WaitCtx& w) {
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(b, parity)) return true;
    if ((it & 63) == 63) {
      if (*(volatile uint32_t*)w.abort_flag) return false;
      if (globaltimer() > w.deadline) { record_failure(w, SAR_TIMEOUT_PIPE); return false; }
    }
  }
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(32 * kConsumerWarps) : "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_cta(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_cta(uint32_t* p, uint32_t v) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t pow2_ceil(uint32_t x) {
  uint32_t p = 1;
  while (p < x) p <<= 1;
  return p;
}
}  // namespace tma

// Roles of a block (192 threads):
//   warp 0, one thread   producer: walks the items, waits for their operands
//                        (flags in peer memory), streams the tiles into the ring;
//   warps 1-4            consumers: add the sources of a stage in place; one of
//                        their threads issues the bulk stores and recycles stages;
//   warp 5, one thread   signal: announces finished items (fence + flag stores).
// Announcing costs a system-scope fence; doing it in a thread of its own keeps
// the fence off the path that issues loads and stores.
template <typename T>
__device__ void run_rank_tma(const SarLaunchParams& P, uint32_t block, uint32_t nblocks, tma::Shared& S) {
  using namespace tma;
  constexpr int N = Vec<T>::N;
  const uint32_t tid = threadIdx.x;
  const uint32_t warp = tid >> 5, lane = tid & 31;
  // ring stages in use: fewer stages keep fewer bytes in flight per block
  const uint32_t nst = (P.stages >= 2 && P.stages < (uint32_t)kStages) ? P.stages : (uint32_t)kStages;
  WaitCtx w = enter_collective(P, block);
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], 1); }
    S.abort_seen = 0; S.issued = 0;
    S.pend_tail = 0; S.pend_head = 0; S.landed = 0; S.consumers_done = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  resolve_table(P, S.geom, nblocks);   // ends with a block barrier

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      if (P.gate_rounds && block == 0) gate_announce_first(P, S.geom);
      ItemWalker walk;
      walk.init(&P, &S.geom, block, nblocks);
      uint32_t arrived = 1u << P.rank, gate_passed = 0;
      uint32_t seq = 0;           // pieces issued
      bool ok = true;
      Item it;
      auto acquire_stage = [&](uint32_t s) -> bool {
        // the first pass over the ring finds every stage free
        if (seq >= nst) return mbar_wait(&S.empty[s], ((seq / nst) - 1) & 1, w);
        return true;
      };
      while (ok && walk.next(&it)) {
        const uint64_t t_begin = P.trace_rounds ? globaltimer() : 0;
        if (!wait_item_ready(P, it, w, &arrived, &gate_passed)) { ok = false; break; }
        if (P.trace_rounds) trace_item_start(P, it.op, t_begin, globaltimer());
        fence_proxy_async_global();   // flags were acquired through the generic proxy; the copies use the async one
        const SarOp* op = it.op;
        if (op->kind >= SAR_STAGE_IN) {
          const bool in = op->kind == SAR_STAGE_IN;
          const int sdt = in ? P.user_dtype : P.dtype, ddt = in ? P.dtype : P.user_dtype;
          const uint32_t ssz = sdt == SAR_F32 ? 4u : 2u, dsz = ddt == SAR_F32 ? 4u : 2u;
          const char* src = in ? (const char*)P.user_in : (const char*)P.comm.buf[P.rank];
          if (((((uintptr_t)P.user_in | (uintptr_t)P.user_out) & 15) != 0) || (((it.elem0 * ssz) | (it.elem0 * dsz)) & 15) != 0) {
            // a caller's tensor, or a tile start, that bulk copies cannot address (they need 16-byte alignment on
            // both sides): the consumer threads move (and convert) the tile with plain loads and stores
            const uint32_t s = seq % nst;
            if (!acquire_stage(s)) { ok = false; break; }
            StageDesc& d = S.desc[s];
            d.op = op; d.byte_off = 0; d.bytes = 0; d.slot_bytes = 0; d.nsrc_total = 0; d.fidx = it.fidx; d.last = 1u;
            d.tail_elems = 0; d.tail_elem0 = 0; d.item_elem0 = it.elem0; d.item_elems = it.nelem; d.dst_bytes = 0;
            mbar_arrive(&S.full[s]);
            ++seq;
            continue;
          }
          // pieces of whole 16-byte vectors on both sides (8 elements); a converted piece uses half a stage per side
          const uint32_t big = ssz > dsz ? ssz : dsz;
          const uint32_t piece = sdt == ddt ? (uint32_t)kStageBytes / ssz : (uint32_t)(kStageBytes / 2) / big;
          const uint32_t body = it.nelem & ~7u, tail = it.nelem & 7u;
          uint32_t done = 0;
          do {
            const uint32_t pe = body - done < piece ? body - done : piece;
            const uint32_t s = seq % nst;
            if (!acquire_stage(s)) { ok = false; break; }
            StageDesc& d = S.desc[s];
            d.op = op; d.byte_off = (it.elem0 + done) * ssz; d.bytes = pe * ssz; d.slot_bytes = 0; d.nsrc_total = 1;
            d.dst_off = (it.elem0 + done) * dsz; d.dst_bytes = pe * dsz; d.piece_elems = pe; d.fidx = it.fidx;
            d.item_elems = 0; d.item_elem0 = 0;
            d.last = (done + pe >= body) ? 1u : 0u;
            d.tail_elems = d.last ? tail : 0u;
            d.tail_elem0 = it.elem0 + body;
            if (pe) {
              mbar_arrive_expect_tx(&S.full[s], d.bytes);
              bulk_load(&S.ring[s][0], src + d.byte_off, d.bytes, &S.full[s]);
            } else {
              mbar_arrive(&S.full[s]);
            }
            ++seq;
            done += pe;
          } while (done < body);
          continue;
        }
        const bool push_only = op->kind == SAR_PUSH;            // the only source is the own slot
        const bool local = push_only || op_reads_local(op);
        const uint32_t npeer = push_only ? 0u : op->nsrc;
        const uint32_t nsrc_total = npeer + (local ? 1u : 0u);
        const uint32_t slot_bytes = kStageBytes / pow2_ceil(nsrc_total);
        const uint32_t vec_bytes = (it.nelem / N) * 16u;
        const uint32_t tail = it.nelem % N;
        uint32_t done = 0;
        do {
          const uint32_t bytes = vec_bytes - done < slot_bytes ? vec_bytes - done : slot_bytes;
          const uint32_t s = seq % nst;
          if (!acquire_stage(s)) { ok = false; break; }
          StageDesc& d = S.desc[s];
          d.op = op; d.byte_off = it.elem0 * sizeof(T) + done; d.bytes = bytes; d.slot_bytes = slot_bytes;
          d.nsrc_total = nsrc_total; d.fidx = it.fidx;
          d.last = (done + bytes >= vec_bytes) ? 1u : 0u;
          d.tail_elems = d.last ? tail : 0u;
          d.tail_elem0 = it.elem0 + (uint64_t)(it.nelem / N) * N;
          if (bytes) {
            mbar_arrive_expect_tx(&S.full[s], bytes * nsrc_total);
            for (uint32_t q = 0; q < npeer; ++q)
              bulk_load(&S.ring[s][q * slot_bytes], (const char*)P.comm.buf[op->src[q]] + d.byte_off, bytes, &S.full[s]);
            if (local)
              bulk_load(&S.ring[s][npeer * slot_bytes], (const char*)P.comm.buf[P.rank] + d.byte_off, bytes, &S.full[s]);
          } else {
            mbar_arrive(&S.full[s]);   // an item that is only a sub-vector tail
          }
          ++seq;
          done += bytes;
        } while (done < vec_bytes);
      }
      // end marker (also after a failure, so that the consumers stop)
      {
        const uint32_t s = seq % nst;
        bool got = true;
        if (seq >= nst) {
          // on the failure path the deadline has usually passed: take the stage only if it is free already
          got = ok ? mbar_wait(&S.empty[s], ((seq / nst) - 1) & 1, w) : mbar_try_wait(&S.empty[s], ((seq / nst) - 1) & 1);
        }
        if (got) { S.desc[s].op = nullptr; mbar_arrive(&S.full[s]); }
        else *(volatile int*)&S.abort_seen = 1;
      }
      S.issued = seq;
    }
  } else if (warp <= (uint32_t)kConsumerWarps) {
    // --------------------------------------------------------------- consumers
    const uint32_t ctid = tid - 32;                 // 0 .. 127
    constexpr uint32_t CT = 32 * kConsumerWarps;
    uint32_t seq = 0;
    uint32_t landed = 0, pend_tail = 0;             // private copies of the storing thread (ctid 0)
    const uint32_t win = P.store_window >= 16 ? 16u : (P.store_window >= 8 ? 8u : 3u);
    while (true) {
      const uint32_t s = seq % nst;
      bool ok = true;
      if (lane == 0) {
        if (ctid == 0 && landed < seq && !mbar_try_wait(&S.full[s], (seq / nst) & 1)) {
          // The pipeline has run dry, perhaps because the producer waits for a tile
          // that (through other ranks) depends on an item whose stores have not been
          // reported as landed yet: report everything now.
          bulk_wait_all<0>();
          landed = seq;
          st_release_cta(&S.landed, landed);
        }
        ok = mbar_wait(&S.full[s], (seq / nst) & 1, w);
        if (*(volatile int*)&S.abort_seen) ok = false;
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      const StageDesc d = S.desc[s];
      if (d.op == nullptr) break;
      const SarOp* op = d.op;
      unsigned char* stage = S.ring[s];
      if (op->kind >= SAR_STAGE_IN) {
        if (d.item_elems) {
          Item sit{};
          sit.op = op; sit.elem0 = d.item_elem0; sit.nelem = d.item_elems;
          stage_tile<T>(P, sit, ctid, CT);
        } else if (d.bytes != d.dst_bytes) {
          // convert the piece from the first half of the stage into the second, eight elements per thread and turn
          const bool in = op->kind == SAR_STAGE_IN;
          const int sdt = in ? P.user_dtype : P.dtype, ddt = in ? P.dtype : P.user_dtype;
          unsigned char* out = stage + kStageBytes / 2;
          for (uint32_t g = ctid; g < d.piece_elems / 8; g += CT) {
            float f[8];
            if (sdt == SAR_F32) {
              const float4 a = *reinterpret_cast<const float4*>(stage + (size_t)g * 32), b = *reinterpret_cast<const float4*>(stage + (size_t)g * 32 + 16);
              f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
            } else {
              const uint4 v = *reinterpret_cast<const uint4*>(stage + (size_t)g * 16);
              if (sdt == SAR_BF16) Vec<__nv_bfloat16>::unpack(v, f); else Vec<__half>::unpack(v, f);
            }
            if (ddt == SAR_F32) {
              *reinterpret_cast<float4*>(out + (size_t)g * 32) = make_float4(f[0], f[1], f[2], f[3]);
              *reinterpret_cast<float4*>(out + (size_t)g * 32 + 16) = make_float4(f[4], f[5], f[6], f[7]);
            } else {
              *reinterpret_cast<uint4*>(out + (size_t)g * 16) = ddt == SAR_BF16 ? Vec<__nv_bfloat16>::pack(f) : Vec<__half>::pack(f);
            }
          }
          fence_proxy_async_smem();
        }
      } else if (op->kind != SAR_COPY && op->kind != SAR_PUSH && d.bytes) {
        const float scale = (op->flags & SAR_F_SCALE) ? P.scale : 1.0f;
        const uint32_t nvec = d.bytes / 16;
        const uint32_t nsrc = d.nsrc_total;
        uint32_t v = ctid;
        for (; v + 3 * CT < nvec; v += 4 * CT) {     // four independent vectors per thread
          float acc[4][N];
#pragma unroll
          for (int u = 0; u < 4; ++u) Vec<T>::unpack(*reinterpret_cast<const uint4*>(stage + (size_t)(v + u * CT) * 16), acc[u]);
          for (uint32_t q = 1; q < nsrc; ++q) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              float f[N];
              Vec<T>::unpack(*reinterpret_cast<const uint4*>(stage + (size_t)q * d.slot_bytes + (size_t)(v + u * CT) * 16), f);
#pragma unroll
              for (int i = 0; i < N; ++i) acc[u][i] += f[i];
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
#pragma unroll
            for (int i = 0; i < N; ++i) acc[u][i] *= scale;
            *reinterpret_cast<uint4*>(stage + (size_t)(v + u * CT) * 16) = Vec<T>::pack(acc[u]);
          }
        }
        for (; v < nvec; v += CT) {
          float acc[N];
          Vec<T>::unpack(*reinterpret_cast<const uint4*>(stage + (size_t)v * 16), acc);
          for (uint32_t q = 1; q < nsrc; ++q) {
            float f[N];
            Vec<T>::unpack(*reinterpret_cast<const uint4*>(stage + (size_t)q * d.slot_bytes + (size_t)v * 16), f);
#pragma unroll
            for (int i = 0; i < N; ++i) acc[i] += f[i];
          }
#pragma unroll
          for (int i = 0; i < N; ++i) acc[i] *= scale;
          *reinterpret_cast<uint4*>(stage + (size_t)v * 16) = Vec<T>::pack(acc);
        }
        fence_proxy_async_smem();   // make the sums visible to the bulk store engine
      }
      // Every consumer warp is done with this piece's descriptor and data, and
      // (a fortiori) with the previous piece's stage, which is released below.
      consumer_bar();
      if (ctid == 0) {
        if (op->kind >= SAR_STAGE_IN) {
          if (d.dst_bytes) {
            char* dst = op->kind == SAR_STAGE_IN ? (char*)P.comm.buf[P.rank] : (char*)P.user_out;
            bulk_store(dst + d.dst_off, d.bytes != d.dst_bytes ? stage + kStageBytes / 2 : stage, d.dst_bytes);
          }
        } else if (d.bytes) {
          if (op->kind != SAR_PUSH) bulk_store((char*)P.comm.buf[P.rank] + d.byte_off, stage, d.bytes);
          if (op->kind == SAR_REDUCE_PUSH) bulk_store((char*)P.comm.buf[op->src[0]] + d.byte_off, stage, d.bytes);
          if (op->kind == SAR_PUSH)
            for (int q = 0; q < op->nsrc; ++q) bulk_store((char*)P.comm.buf[op->src[q]] + d.byte_off, stage, d.bytes);
        }
        bulk_commit();          // one group per piece (possibly empty), so group numbers follow seq
        if (d.last) {
          if (d.tail_elems && op->kind >= SAR_STAGE_IN) {
            const bool in = op->kind == SAR_STAGE_IN;
            const void* tsrc = in ? P.user_in : (const void*)P.comm.buf[P.rank];
            void* tdst = in ? (void*)P.comm.buf[P.rank] : P.user_out;
            for (uint32_t i = 0; i < d.tail_elems; ++i)
              store_from_float(tdst, d.tail_elem0 + i, in ? P.dtype : P.user_dtype, load_as_float(tsrc, d.tail_elem0 + i, in ? P.user_dtype : P.dtype));
            __threadfence_system();
          } else if (d.tail_elems) { scalar_elems<T>(P, op, d.tail_elem0, d.tail_elems); __threadfence_system(); }
          // hand the item to the signal thread; wait (bounded) if its ring is full
          if (pend_tail - ld_acquire_cta(&S.pend_head) >= (uint32_t)kPendRing) {
            bulk_wait_all<0>();
            landed = seq + 1;
            st_release_cta(&S.landed, landed);
            while (pend_tail - ld_acquire_cta(&S.pend_head) >= (uint32_t)kPendRing) {
              if (*(volatile uint32_t*)w.abort_flag || globaltimer() > w.deadline) break;
            }
          }
          PendEntry& e = S.pend[pend_tail % kPendRing];
          e.op = op; e.fidx = d.fidx; e.seq = seq;
          ++pend_tail;
          st_release_cta(&S.pend_tail, pend_tail);
        }
        // the previous piece's stores have read their stage: hand it back
        bulk_wait_read<1>();
        if (seq >= 1) mbar_arrive(&S.empty[(seq - 1) % nst]);
        // at most `win` store groups stay in flight; older ones have landed.  Stores to peer memory are
        // posted: a deep window keeps a block's pushes from being paced by the link's round trip.
        if (win >= 16) bulk_wait_all<16>();
        else if (win >= 8) bulk_wait_all<8>();
        else bulk_wait_all<3>();
        if (seq >= win && landed < seq - (win - 1)) { landed = seq - (win - 1); st_release_cta(&S.landed, landed); }
      }
      ++seq;
    }
    if (ctid == 0) {
      bulk_wait_all<0>();
      st_release_cta(&S.landed, 0xffffffffu);
      st_release_cta(&S.consumers_done, 1u);
    }
  } else if (lane == 0) {
    // ------------------------------------------------------------------ signal
    uint32_t head = 0;
    while (true) {
      const uint32_t done = ld_acquire_cta(&S.consumers_done);
      const uint32_t tail = ld_acquire_cta(&S.pend_tail);
      const uint32_t landed = ld_acquire_cta(&S.landed);
      uint32_t n = 0;
      while (head + n != tail && S.pend[(head + n) % kPendRing].seq < landed) ++n;
      if (n) {
        fence_proxy_async_global();   // the tiles were written by bulk copies
        fence_sys();
        for (uint32_t i = 0; i < n; ++i) {
          const PendEntry& e = S.pend[(head + i) % kPendRing];
          publish_item(P, e.op, e.fidx);
          trace_item_end(P, e.op);
          gate_item_done(P, S.geom, e.op);
        }
        head += n;
        st_release_cta(&S.pend_head, head);
        continue;
      }
      if (done && head == tail) break;
      if (*(volatile uint32_t*)w.abort_flag && done) break;
      if (globaltimer() > w.deadline + 1000000000ull) break;   // the other roles have given up long ago
      __nanosleep(64);
    }
  }
  __syncthreads();
  // Bulk loads still in flight would write into shared memory after the block
  // has gone.  On the failure path the consumers may not have waited for every
  // issued piece: wait here (at most 2 ms) for the newest use of every stage.
  if (tid == 0 && *(volatile uint32_t*)w.abort_flag) {
    const uint32_t issued = S.issued;
    const uint64_t limit = globaltimer() + 2000000ull;
    for (uint32_t s = 0; s < nst; ++s) {
      if (issued <= s) continue;
      const uint32_t use = (issued - 1 - s) / nst;   // newest use of stage s
      while (!mbar_try_wait(&S.full[s], use & 1) && globaltimer() < limit) {}
    }
  }
  __syncthreads();
  if (tid == 0) leave_collective(P, w, nblocks);
}

// ------------------------------------------------------- simt path, decoupled
// The simt data path with the control work taken off the threads that move data (512 threads):
//   warps 0-13           workers: move the tile with 16-byte loads and stores (simt_tile);
//   warp 14, one thread  control: walks the items and waits for their operands (flags in
//                        peer memory) one item ahead of the workers;
//   warp 15, one thread  signal: announces finished items (system-scope fence + flag stores).
// In run_rank_simt every tile pays, on all 512 threads, the flag wait before it and the fence
// after it; here both overlap the workers' copying.  This is also the path on which
// reductions over, and pushes to, a whole multicast group go through the switch.
namespace simta {
constexpr int kThreads = 512;
constexpr int kWorkerWarps = 14;
constexpr int kWorkers = 32 * kWorkerWarps;
constexpr int kSlots = 2;
constexpr int kPendRing = 16;

struct Shared {
  TableGeom geom;
  Item slot[kSlots];
  int state[kSlots];          // 1: item ready, 0: table exhausted, -1: a wait failed
  int decision;               // the state the workers act on (written by worker thread 0)
  alignas(8) uint64_t full[kSlots];
  alignas(8) uint64_t empty[kSlots];
  tma::PendEntry pend[kPendRing];
  uint32_t pend_tail;         // written by worker thread 0
  uint32_t pend_head;         // written by the signal thread
  uint32_t workers_done;
};
__device__ __forceinline__ void worker_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kWorkers) : "memory"); }
}  // namespace simta

template <typename T>
__device__ void run_rank_simta(const SarLaunchParams& P, uint32_t block, uint32_t nblocks, simta::Shared& S) {
  using namespace simta;
  using tma::ld_acquire_cta;
  using tma::mbar_arrive;
  using tma::mbar_init;
  using tma::mbar_wait;
  using tma::st_release_cta;
  const uint32_t tid = threadIdx.x;
  const uint32_t warp = tid >> 5, lane = tid & 31;
  WaitCtx w = enter_collective(P, block);
  if (tid == 0) {
    for (int s = 0; s < kSlots; ++s) { mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], 1); }
    S.pend_tail = 0; S.pend_head = 0; S.workers_done = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  resolve_table(P, S.geom, nblocks);   // ends with a block barrier

  if (warp < (uint32_t)kWorkerWarps) {
    // ----------------------------------------------------------------- workers
    uint32_t pend_tail = 0;            // private copy of worker thread 0
    for (uint32_t seq = 0;; ++seq) {
      const uint32_t s = seq % kSlots;
      // One thread waits for the control thread and decides for all workers, so that they
      // leave the loop together even when a wait runs out for some and not for others.
      if (tid == 0) {
        const bool ok = mbar_wait(&S.full[s], (seq / kSlots) & 1, w);
        *(volatile int*)&S.decision = ok ? *(volatile int*)&S.state[s] : -1;
      }
      worker_bar();
      if (*(volatile int*)&S.decision != 1) break;
      const Item it = S.slot[s];
      simt_tile<T, 4>(P, it, tid, kWorkers);
      worker_bar();                    // every store of the tile is issued; every worker has read the slot and the decision
      if (tid == 0) {
        // hand the item to the signal thread (bounded wait if its ring is full), free the slot
        while (pend_tail - ld_acquire_cta(&S.pend_head) >= (uint32_t)kPendRing) {
          if (*(volatile uint32_t*)w.abort_flag || globaltimer() > w.deadline) break;
        }
        tma::PendEntry& e = S.pend[pend_tail % kPendRing];
        e.op = it.op; e.fidx = it.fidx; e.seq = seq;
        ++pend_tail;
        st_release_cta(&S.pend_tail, pend_tail);
        mbar_arrive(&S.empty[s]);
      }
    }
    if (tid == 0) st_release_cta(&S.workers_done, 1u);
  } else if (warp == (uint32_t)kWorkerWarps) {
    // ----------------------------------------------------------------- control
    if (lane == 0) {
      if (P.gate_rounds && block == 0) gate_announce_first(P, S.geom);
      ItemWalker walk;
      walk.init(&P, &S.geom, block, nblocks);
      uint32_t arrived = 1u << P.rank, gate_passed = 0;
      for (uint32_t seq = 0;; ++seq) {
        const uint32_t s = seq % kSlots;
        // the slot is free once the workers are done with the item that used it last
        if (seq >= (uint32_t)kSlots && !mbar_wait(&S.empty[s], ((seq / kSlots) - 1) & 1, w)) {
          // the workers have stopped or the deadline has passed; they see the abort word themselves
          break;
        }
        Item it;
        int state = 1;
        if (!walk.next(&it)) state = 0;
        else {
          const uint64_t t_begin = P.trace_rounds ? globaltimer() : 0;
          if (!wait_item_ready(P, it, w, &arrived, &gate_passed)) state = -1;
          else if (P.trace_rounds) trace_item_start(P, it.op, t_begin, globaltimer());
        }
        if (state == 1) S.slot[s] = it;
        *(volatile int*)&S.state[s] = state;
        mbar_arrive(&S.full[s]);       // release: the workers' wait acquires the slot contents
        if (state != 1) break;
      }
    }
  } else if (lane == 0) {
    // ------------------------------------------------------------------ signal
    uint32_t head = 0;
    while (true) {
      const uint32_t done = ld_acquire_cta(&S.workers_done);
      const uint32_t tail = ld_acquire_cta(&S.pend_tail);
      if (head != tail) {
        fence_sys();                   // the tiles' stores (ordered before the hand-off) become visible first
        for (; head != tail; ++head) {
          const tma::PendEntry& e = S.pend[head % kPendRing];
          publish_item(P, e.op, e.fidx);
          trace_item_end(P, e.op);
          gate_item_done(P, S.geom, e.op);
        }
        st_release_cta(&S.pend_head, head);
        continue;
      }
      if (done) break;
      if (globaltimer() > w.deadline + 1000000000ull) break;   // the other roles have given up long ago
      __nanosleep(64);
    }
  }
  __syncthreads();
  if (tid == 0) leave_collective(P, w, nblocks);
}

}  // namespace sar_dev
