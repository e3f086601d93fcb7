#include "host_exec.h"

#include <chrono>
#include <cmath>
#include <cstddef>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <thread>
#include <vector>

namespace sar {

static inline float bf16_to_f(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }
static inline uint16_t f_to_bf16(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static inline float f16_to_f(uint16_t h) {
  uint32_t s = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023, u;
  if (e == 0) {
    if (m == 0) u = s << 31;
    else { int k = 0; while (!(m & 1024)) { m <<= 1; ++k; } m &= 1023; u = (s << 31) | ((uint32_t)(113 - k) << 23) | (m << 13); }
  } else if (e == 31) u = (s << 31) | 0x7f800000u | (m << 13);
  else u = (s << 31) | ((e + 112) << 23) | (m << 13);
  float f; memcpy(&f, &u, 4); return f;
}
static inline uint16_t f_to_f16(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  uint32_t s = (u >> 16) & 0x8000u; int32_t e = (int32_t)((u >> 23) & 255) - 112; uint32_t m = u & 0x7fffffu;
  if (((u >> 23) & 255) == 255) return (uint16_t)(s | 0x7c00u | (m ? 0x200u : 0));
  if (e >= 31) return (uint16_t)(s | 0x7c00u);
  if (e <= 0) {
    if (e < -10) return (uint16_t)s;
    m |= 0x800000u; uint32_t shift = (uint32_t)(14 - e);
    uint32_t half = m >> shift, rem = m & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return (uint16_t)(s | half);
  }
  uint32_t half = ((uint32_t)e << 10) | (m >> 13), rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return (uint16_t)(s | half);
}

static inline float load_elem(const void* p, uint64_t i, SarDtype d) {
  if (d == SAR_F32) return ((const float*)p)[i];
  uint16_t h = ((const uint16_t*)p)[i];
  return d == SAR_BF16 ? bf16_to_f(h) : f16_to_f(h);
}
static inline void store_elem(void* p, uint64_t i, SarDtype d, float v) {
  if (d == SAR_F32) ((float*)p)[i] = v;
  else ((uint16_t*)p)[i] = d == SAR_BF16 ? f_to_bf16(v) : f_to_f16(v);
}

uint64_t gate_min_bytes() {
  const char* v = getenv("STRAGGLAR_GATE_MIN_BYTES");
  return (v && *v) ? strtoull(v, nullptr, 10) : (128ull << 20);
}

uint32_t gate_slack(uint32_t tiles_per_chunk) {
  const char* v = getenv("STRAGGLAR_GATE_SLACK");
  if (v && *v) return (uint32_t)strtoul(v, nullptr, 10);
  return (uint32_t)(((uint64_t)tiles_per_chunk * 3 + 5) / 10);
}

uint32_t pick_tile_elems(uint64_t count, uint32_t esize, uint32_t num_chunks, uint32_t blocks, uint32_t min_bytes,
                         uint32_t max_bytes) {
  const uint64_t vw = SAR_VEC_BYTES / esize;
  uint64_t chunk_bytes = (count * esize + num_chunks - 1) / num_chunks;
  uint64_t want = (chunk_bytes + blocks - 1) / (blocks ? blocks : 1);
  if (want < min_bytes) want = min_bytes;
  if (want > max_bytes) want = max_bytes;
  // keep the flag array within capacity
  while (((chunk_bytes + want - 1) / want + 1) * num_chunks > SAR_FLAG_CAPACITY) want *= 2;
  uint64_t granule = 512;  // bytes
  want = (want + granule - 1) / granule * granule;
  uint64_t elems = want / esize;
  elems = (elems + vw - 1) / vw * vw;
  return (uint32_t)elems;
}

SarGeom make_geom(uint64_t count, uint32_t esize, uint32_t num_chunks, uint32_t tile_elems) {
  SarGeom g{};
  g.count = count; g.esize = esize; g.num_chunks = num_chunks; g.tile_elems = tile_elems;
  uint32_t mx = 0;
  for (uint32_t c = 0; c < num_chunks; ++c) { uint32_t t = sar_chunk_tiles(g, c); if (t > mx) mx = t; }
  g.tiles_per_chunk = mx ? mx : 1;
  return g;
}

namespace {
using clk = std::chrono::steady_clock;

struct Waiter {
  clk::time_point deadline;
  std::atomic<uint32_t>* abort_flag;
  bool wait(std::atomic<uint32_t>* w, uint32_t target) const {
    unsigned spins = 0;
    while (!sar_reached(w->load(std::memory_order_acquire), target)) {
      if ((++spins & 63) == 0) {
        if (abort_flag->load(std::memory_order_relaxed)) return false;
        if (clk::now() > deadline) return false;
        std::this_thread::yield();
      }
    }
    return true;
  }
  bool wait64(std::atomic<uint64_t>* w, uint64_t target) const {
    unsigned spins = 0;
    while (w->load(std::memory_order_acquire) < target) {
      if ((++spins & 63) == 0) {
        if (abort_flag->load(std::memory_order_relaxed)) return false;
        if (clk::now() > deadline) return false;
        std::this_thread::yield();
      }
    }
    return true;
  }
};
}  // namespace

uint32_t host_run_block(const HostRankView& v, const RankTable& t, const HostLaunch& l, int block, int nblocks) {
  const SarGeom& g = l.geom;
  const int me = v.rank;
  SarCtrl* my_ctrl_raw = reinterpret_cast<SarCtrl*>(v.ctrl[me]);
  (void)my_ctrl_raw;
  // 0 arrival, 1 exited, 2 abort, 3 blocks_done, 4 items_done, 5 announced (the words of SarCtrl);
  // the 64-bit gate words follow at word 32
  auto ctrl_word = [&](int r, int idx) { return v.ctrl[r] + idx; };
  Waiter w{clk::now() + std::chrono::duration_cast<clk::duration>(std::chrono::duration<double>(l.timeout_s + l.delay_ms * 1e-3)),
           ctrl_word(me, 2)};
  uint32_t status = SAR_OK;
  auto give_up = [&](uint32_t code) { status = code; ctrl_word(me, 2)->store(1, std::memory_order_relaxed); };

  // an injected delay stands for a late launch: no block of the rank runs before it is over
  if (l.delay_ms > 0) std::this_thread::sleep_for(std::chrono::duration<double, std::milli>(l.delay_ms));
  if (block == 0) ctrl_word(me, 0)->store(l.epoch_base, std::memory_order_release);
  uint32_t arrived_mask = 1u << me;
  auto need_arrival = [&](int r) -> bool {
    if (arrived_mask >> r & 1) return true;
    if (!w.wait(ctrl_word(r, 0), l.epoch_base)) { give_up(SAR_TIMEOUT_ARRIVAL); return false; }
    arrived_mask |= 1u << r;
    return true;
  };

  const size_t nrounds = t.round_begin.empty() ? 0 : t.round_begin.size() - 1;
  // round gating: round_prefix[R] = items this rank has in the schedule rounds before R (all lanes);
  // the table's round list is compact, so the schedule round is taken from the ops
  uint32_t round_prefix[SAR_GATE_ALL_DONE + 1] = {};
  if (l.gate_rounds) {
    uint32_t items[SAR_GATE_ALL_DONE] = {};
    for (const SarOp& op : t.ops)
      if (op.round < SAR_GATE_ALL_DONE) items[op.round] += sar_op_tiles(g, op);
    for (uint32_t rd = 0; rd < SAR_GATE_ALL_DONE; ++rd) round_prefix[rd + 1] = round_prefix[rd] + items[rd];
  }
  auto gate_word = [&](int owner, int about) {
    return reinterpret_cast<std::atomic<uint64_t>*>(v.ctrl[owner] + offsetof(SarCtrl, gate) / 4) + about;
  };
  auto gate_round_for = [&](uint32_t done) -> uint32_t {
    uint32_t R = 0;
    while (R < SAR_GATE_ALL_DONE && round_prefix[R + 1] <= done + l.gate_slack) ++R;
    return R;
  };
  // raises this rank's announcement to R in every participant's memory (max: announcements may overtake one another)
  auto gate_announce = [&](uint32_t R) {
    uint32_t seen = ctrl_word(me, 5)->load(std::memory_order_relaxed);
    while (seen < R + 1u && !ctrl_word(me, 5)->compare_exchange_weak(seen, R + 1u, std::memory_order_acq_rel)) {}
    if (seen >= R + 1u) return;
    for (int q = 0; q < v.nranks; ++q) {
      if (!(l.participants >> q & 1)) continue;
      std::atomic<uint64_t>* gw = gate_word(q, me);
      uint64_t cur = gw->load(std::memory_order_relaxed);
      while (cur < l.gate_base + R && !gw->compare_exchange_weak(cur, l.gate_base + R, std::memory_order_acq_rel)) {}
    }
  };
  if (l.gate_rounds && block == 0) gate_announce(gate_round_for(0));
  uint32_t gate_passed = 0;   // schedule rounds up to this one may start
  uint32_t table_lanes = 1;
  for (const SarOp& op : t.ops) if (op.lane) table_lanes = 2;
  uint32_t lanes, lane, lblock, lnblocks;
  sar_lane_of_block((uint32_t)block, (uint32_t)nblocks, table_lanes, l.lane1_eighths, &lanes, &lane, &lblock, &lnblocks);
  const int block_all = block, nblocks_all = nblocks;
  block = (int)lblock; nblocks = (int)lnblocks;   // from here on: position inside the lane
  uint64_t item_base = 0;
  for (size_t ri = 0; ri < nrounds && status == SAR_OK; ++ri) {
    uint32_t ob = t.round_begin[ri], oe = t.round_begin[ri + 1];
    if (lanes == 2) {
      // the round's ops are sorted by lane: lane 0 is a prefix, lane 1 the rest
      uint32_t split = ob;
      while (split < oe && t.ops[split].lane == 0) ++split;
      if (lane == 0) oe = split; else ob = split;
    }
    const uint32_t m = oe - ob;
    if (m == 0) continue;
    uint32_t max_tiles = 0;
    for (uint32_t o = ob; o < oe; ++o) max_tiles = std::max(max_tiles, sar_op_tiles(g, t.ops[o]));
    const uint64_t items = (uint64_t)max_tiles * m;
    // first item of this round that belongs to this block
    uint64_t k = ((uint64_t)block + nblocks - (item_base % nblocks)) % nblocks;
    for (; k < items && status == SAR_OK; k += nblocks) {
      const SarOp& op = t.ops[ob + (uint32_t)(k % m)];
      const uint32_t local_tile = (uint32_t)(k / m);
      uint32_t t0, t1;
      sar_part_range(sar_chunk_tiles(g, op.chunk), op.part, op.parts, &t0, &t1);
      if (local_tile >= t1 - t0) continue;
      const uint32_t tile = t0 + local_tile;
      const uint32_t fidx = sar_flag_index(g, op.chunk, tile);
      bool ok = true;
      // round gate (not for the first round): every participant has announced this round in this rank's memory
      bool operands_known = false;
      if (l.gate_rounds && op.round >= 1 && op.round < SAR_GATE_ALL_DONE) {
        if (op.round > gate_passed) {
          for (int r = 0; r < v.nranks && ok; ++r)
            if ((l.participants >> r & 1) && !w.wait64(gate_word(me, r), l.gate_base + op.round)) { give_up(SAR_TIMEOUT_FLAG); ok = false; }
          if (!ok) break;
          gate_passed = op.round;
        }
        operands_known = l.gate_slack == 0;   // a full barrier: nothing left to wait for
      }
      // wait for the operands
      for (int q = 0; q < op.nsrc && ok && !operands_known; ++q) {
        const int src = op.src[q];
        if (!need_arrival(src)) { ok = false; break; }
        if (op.src_ver[q] && !w.wait(v.flags[src] + fidx, l.epoch_base + op.src_ver[q])) { give_up(SAR_TIMEOUT_FLAG); ok = false; }
      }
      const bool reads_local = op.kind == SAR_REDUCE_PUSH || (op.kind == SAR_REDUCE && (op.flags & SAR_F_LOCAL));
      // the own slot must hold the version this op reads or replaces
      if (ok && !operands_known && op.local_ver && !w.wait(v.flags[me] + fidx, l.epoch_base + op.local_ver)) {
        give_up(SAR_TIMEOUT_FLAG); ok = false;
      }
      if (!ok) break;
      const uint64_t cb = sar_chunk_begin(g, op.chunk), cl = sar_chunk_len(g, op.chunk);
      const uint64_t e0 = cb + (uint64_t)tile * g.tile_elems;
      const uint64_t e1 = std::min<uint64_t>(cb + cl, e0 + g.tile_elems);
      const float scale = (op.flags & SAR_F_SCALE) ? l.scale : 1.0f;
      if (op.kind == SAR_COPY) {
        memcpy((char*)v.buf[me] + e0 * g.esize, (const char*)v.buf[op.src[0]] + e0 * g.esize, (e1 - e0) * g.esize);
      } else if (op.kind == SAR_PUSH) {
        for (int q = 0; q < op.nsrc; ++q)
          memcpy((char*)v.buf[op.src[q]] + e0 * g.esize, (const char*)v.buf[me] + e0 * g.esize, (e1 - e0) * g.esize);
      } else {
        for (uint64_t e = e0; e < e1; ++e) {
          float acc = reads_local ? load_elem(v.buf[me], e, l.dtype) : 0.0f;
          for (int q = 0; q < op.nsrc; ++q) acc += load_elem(v.buf[op.src[q]], e, l.dtype);
          acc *= scale;
          store_elem(v.buf[me], e, l.dtype, acc);
          if (op.kind == SAR_REDUCE_PUSH) store_elem(v.buf[op.src[0]], e, l.dtype, acc);
        }
      }
      if (op.kind != SAR_PUSH) v.flags[me][fidx].store(l.epoch_base + op.post_ver, std::memory_order_release);
      if (op.kind == SAR_REDUCE_PUSH)
        v.flags[op.src[0]][fidx].store(l.epoch_base + op.push_ver, std::memory_order_release);
      if (op.kind == SAR_PUSH)
        for (int q = 0; q < op.nsrc; ++q)
          v.flags[op.src[q]][fidx].store(l.epoch_base + op.push_ver, std::memory_order_release);
      // round gate: whoever finishes the rank's last item of the round announces the next round
      if (l.gate_rounds && op.round < SAR_GATE_ALL_DONE) {
        const uint32_t R = gate_round_for(ctrl_word(me, 4)->fetch_add(1, std::memory_order_acq_rel) + 1);
        if (R) gate_announce(R);
      }
    }
    item_base += items;
  }
  // the last block of this rank to finish announces the exit and waits for every peer's
  (void)block_all;
  uint32_t done = ctrl_word(me, 3)->fetch_add(1, std::memory_order_acq_rel) + 1;
  if (done == (uint32_t)nblocks_all) {
    ctrl_word(me, 3)->store(0, std::memory_order_relaxed);
    ctrl_word(me, 4)->store(0, std::memory_order_relaxed);
    ctrl_word(me, 5)->store(0, std::memory_order_relaxed);
    if (status == SAR_OK && !ctrl_word(me, 2)->load(std::memory_order_relaxed)) {
      ctrl_word(me, 1)->store(l.epoch_base, std::memory_order_release);
      for (int r = 0; r < v.nranks; ++r)
        if (r != me && (l.participants >> r & 1) && !w.wait(ctrl_word(r, 1), l.epoch_base)) { status = SAR_TIMEOUT_EXIT; break; }
    }
  }
  if (status == SAR_OK && ctrl_word(me, 2)->load(std::memory_order_relaxed)) status = SAR_ABORTED;
  return status;
}

namespace {
struct HostArena {
  int n;
  size_t nflags;
  std::vector<std::unique_ptr<std::atomic<uint32_t>[]>> flags, ctrl;  // [rank] -> all channels
  explicit HostArena(int n_) : n(n_), nflags((size_t)SAR_NUM_CHANNELS * SAR_FLAG_CAPACITY), flags(n_), ctrl(n_) {
    for (int r = 0; r < n; ++r) {
      flags[r].reset(new std::atomic<uint32_t>[nflags]);
      for (size_t i = 0; i < nflags; ++i) flags[r][i].store(0, std::memory_order_relaxed);
      ctrl[r].reset(new std::atomic<uint32_t>[SAR_CTRL_WORDS * SAR_NUM_CHANNELS]);
      for (int i = 0; i < (int)(SAR_CTRL_WORDS * SAR_NUM_CHANNELS); ++i) ctrl[r][i].store(0, std::memory_order_relaxed);
    }
  }
};

// a reusable barrier for the blocks of one rank (stream order between phases)
struct RankBarrier {
  std::atomic<int> count{0}, gen{0};
  void wait(int parties) {
    int g = gen.load();
    if (count.fetch_add(1) + 1 == parties) { count.store(0); gen.fetch_add(1); }
    else while (gen.load() == g) std::this_thread::yield();
  }
};
}  // namespace

static uint32_t run_phases(const std::vector<const Compiled*>& phases, void* const* bufs, uint64_t count,
                           SarDtype dtype, uint32_t tile_elems, float scale, int blocks, const double* delay_ms,
                           double timeout_s, int repeats) {
  const int n = phases[0]->n;
  const uint32_t esize = dtype == SAR_F32 ? 4 : 2;
  HostArena arena(n);
  std::vector<RankBarrier> bar(n);
  std::atomic<uint32_t> worst{0};
  std::vector<std::thread> th;
  for (int r = 0; r < n; ++r)
    for (int b = 0; b < blocks; ++b)
      th.emplace_back([&, r, b]() {
        bool delayed = false;
        for (int rep = 0; rep < repeats; ++rep)
          for (size_t ph = 0; ph < phases.size(); ++ph) {
            const Compiled& c = *phases[ph];
            if (c.participants >> r & 1) {
              HostRankView v; v.rank = r; v.nranks = n;
              for (int q = 0; q < n; ++q) {
                v.buf[q] = bufs[q];
                v.flags[q] = arena.flags[q].get() + (size_t)c.channel * SAR_FLAG_CAPACITY;
                v.ctrl[q] = arena.ctrl[q].get() + SAR_CTRL_WORDS * c.channel;
              }
              HostLaunch l;
              uint32_t te = tile_elems ? tile_elems : pick_tile_elems(count, esize, c.num_chunks, blocks, 256, 1 << 16);
              l.geom = make_geom(count, esize, c.num_chunks, te);
              l.dtype = dtype; l.scale = scale; l.timeout_s = timeout_s; l.participants = c.participants;
              l.gate_rounds = c.gate_rounds;
              l.gate_slack = gate_slack(l.geom.tiles_per_chunk);
              l.gate_base = (uint64_t)(rep + 1) * SAR_VER_STRIDE;
              l.lane1_eighths = (uint32_t)c.lane1_eighths;
              l.epoch_base = (uint32_t)(rep + 1) * SAR_VER_STRIDE;
              l.delay_ms = (!delayed && delay_ms) ? delay_ms[r] : 0.0;
              delayed = true;
              uint32_t s = host_run_block(v, c.ranks[r], l, b, blocks);
              uint32_t prev = worst.load();
              while (s > prev && !worst.compare_exchange_weak(prev, s)) {}
            }
            bar[r].wait(blocks);
          }
      });
  for (auto& t : th) t.join();
  return worst.load();
}

uint32_t host_execute(const Compiled& c, void* const* bufs, uint64_t count, SarDtype dtype, uint32_t tile_elems,
                      float scale, int blocks, const double* delay_ms, double timeout_s, int repeats) {
  return run_phases({&c}, bufs, count, dtype, tile_elems, scale, blocks, delay_ms, timeout_s, repeats);
}

uint32_t host_execute_program(const Program& p, void* const* bufs, uint64_t count, SarDtype dtype, uint32_t tile_elems,
                              float scale, int blocks, const double* delay_ms, double timeout_s) {
  std::vector<const Compiled*> ph;
  for (auto& c : p.phases) ph.push_back(&c);
  return run_phases(ph, bufs, count, dtype, tile_elems, scale, blocks, delay_ms, timeout_s, 1);
}

}  // namespace sar
