#include "local_comm.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../core/host_exec.h"
#include "../kernels/sar_params.h"
#include "../kernels/sar_cuda.h"
#include "symm_alloc.h"

namespace {
struct DevTable { SarOp* ops = nullptr; uint16_t* round_begin = nullptr; uint32_t num_rounds = 0; };
struct Rank {
  int dev = 0;
  cudaStream_t stream = nullptr;
  uint32_t* flags = nullptr;   // SAR_NUM_CHANNELS * SAR_FLAG_CAPACITY
  SarCtrl* ctrl = nullptr;     // SAR_NUM_CHANNELS
  uint32_t* status = nullptr;  // 1 word
  uint64_t* trace = nullptr;   // SAR_TRACE_WORDS words
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  bool timed = false;
  std::map<std::pair<uint64_t, int>, DevTable> tables;   // keyed by the table's contents, not its address
};
}  // namespace

struct sar_local_comm {
  int n = 0;
  bool emulate = false;
  std::vector<Rank> ranks;
  uint64_t epoch[SAR_NUM_CHANNELS] = {};   // 64-bit: the low word is the flag epoch, the whole value the gate base
  SarLaunchParams* d_params = nullptr;   // emulate: n entries on devices[0]
  std::vector<sar::SymmAlloc*> allocs;   // symmetric buffers handed out by sar_local_alloc
};

// The symmetric allocation that holds bufs[r] for every rank at one common offset, or nullptr.
static const sar::SymmAlloc* find_alloc(const sar_local_comm* c, void* const* bufs, size_t bytes, size_t* offset) {
  for (const sar::SymmAlloc* a : c->allocs) {
    const char* b0 = (const char*)a->uc[0];
    const char* p0 = (const char*)bufs[0];
    if (p0 < b0 || p0 + bytes > b0 + a->mapped) continue;
    const size_t off = (size_t)(p0 - b0);
    bool same = true;
    for (int r = 1; r < c->n && same; ++r) same = (const char*)bufs[r] == (const char*)a->uc[r] + off;
    if (!same) continue;
    *offset = off;
    return a;
  }
  return nullptr;
}

#define CK(x)                                                                          \
  do {                                                                                 \
    cudaError_t e_ = (x);                                                              \
    if (e_ != cudaSuccess) {                                                           \
      if (err && errlen > 0) snprintf(err, errlen, "%s: %s", #x, cudaGetErrorString(e_)); \
      return fail_value;                                                               \
    }                                                                                  \
  } while (0)

static uint64_t fnv1a(uint64_t h, const void* p, size_t n) {
  const unsigned char* c = (const unsigned char*)p;
  for (size_t i = 0; i < n; ++i) { h ^= c[i]; h *= 0x100000001b3ull; }
  return h;
}

// Device copy of a rank's table.  The cache is keyed by a hash of the table's
// contents: programs come and go on the host, and a new one may live at the
// address of one that was freed.
static DevTable* upload(Rank& rk, const sar_table* t, int rank, char* err, int errlen) {
  const int nops = sar_table_num_ops(t, rank);
  const int nrb = sar_table_num_round_begin(t, rank);
  uint64_t h = 0xcbf29ce484222325ull;
  if (nops) h = fnv1a(h, sar_table_ops(t, rank), sizeof(SarOp) * nops);
  if (nrb) h = fnv1a(h, sar_table_round_begin(t, rank), sizeof(uint16_t) * nrb);
  h = fnv1a(h, &nops, sizeof nops);
  auto key = std::make_pair(h, rank);
  auto it = rk.tables.find(key);
  if (it != rk.tables.end()) return &it->second;
  DevTable* fail_value = nullptr;
  {
    char why[200] = "";
    if (sar_table_validate(t, rank, sar_table_nranks(t), why, sizeof why)) {
      if (err && errlen > 0) snprintf(err, errlen, "refusing to launch a malformed table (%s): %s", sar_status_string(SAR_BAD_TABLE), why);
      return nullptr;
    }
  }
  DevTable d;
  CK(cudaMalloc(&d.ops, sizeof(SarOp) * (nops > 0 ? nops : 1)));
  CK(cudaMalloc(&d.round_begin, sizeof(uint16_t) * (nrb > 0 ? nrb : 1)));
  if (nops) CK(cudaMemcpy(d.ops, sar_table_ops(t, rank), sizeof(SarOp) * nops, cudaMemcpyHostToDevice));
  if (nrb) CK(cudaMemcpy(d.round_begin, sar_table_round_begin(t, rank), sizeof(uint16_t) * nrb, cudaMemcpyHostToDevice));
  d.num_rounds = nrb > 0 ? (uint32_t)(nrb - 1) : 0;
  return &(rk.tables[key] = d);
}

extern "C" {

sar_local_comm* sar_local_create(int n, const int* devices, int emulate, char* err, int errlen) {
  sar_local_comm* fail_value = nullptr;
  if (n < 1 || n > SAR_MAX_RANKS) {
    if (err) snprintf(err, errlen, "rank count %d out of range", n);
    return nullptr;
  }
  auto* c = new sar_local_comm;
  c->n = n; c->emulate = emulate != 0;
  c->ranks.resize(n);
  for (int r = 0; r < n; ++r) {
    Rank& rk = c->ranks[r];
    rk.dev = emulate ? devices[0] : devices[r];
    CK(cudaSetDevice(rk.dev));
    if (emulate && r > 0) rk.stream = c->ranks[0].stream;
    else CK(cudaStreamCreateWithFlags(&rk.stream, cudaStreamNonBlocking));
    const size_t fbytes = sizeof(uint32_t) * SAR_NUM_CHANNELS * (size_t)SAR_FLAG_CAPACITY;
    CK(cudaMalloc(&rk.flags, fbytes));
    CK(cudaMemset(rk.flags, 0, fbytes));
    CK(cudaMalloc(&rk.ctrl, sizeof(SarCtrl) * SAR_NUM_CHANNELS));
    CK(cudaMemset(rk.ctrl, 0, sizeof(SarCtrl) * SAR_NUM_CHANNELS));
    CK(cudaMalloc(&rk.status, 16));
    CK(cudaMemset(rk.status, 0, 16));
    CK(cudaMalloc(&rk.trace, sizeof(uint64_t) * SAR_TRACE_WORDS));
    CK(cudaMemset(rk.trace, 0, sizeof(uint64_t) * SAR_TRACE_WORDS));
    CK(cudaEventCreate(&rk.ev0));
    CK(cudaEventCreate(&rk.ev1));
  }
  if (emulate) {
    CK(cudaSetDevice(devices[0]));
    CK(cudaMalloc(&c->d_params, sizeof(SarLaunchParams) * n));
  } else {
    for (int a = 0; a < n; ++a) {
      CK(cudaSetDevice(c->ranks[a].dev));
      for (int b = 0; b < n; ++b) {
        if (a == b || c->ranks[a].dev == c->ranks[b].dev) continue;
        int can = 0;
        CK(cudaDeviceCanAccessPeer(&can, c->ranks[a].dev, c->ranks[b].dev));
        if (!can) {
          if (err) snprintf(err, errlen, "device %d cannot access device %d", c->ranks[a].dev, c->ranks[b].dev);
          return nullptr;
        }
        cudaError_t e = cudaDeviceEnablePeerAccess(c->ranks[b].dev, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
        else CK(e);
      }
    }
  }
  for (int r = 0; r < n; ++r) { CK(cudaSetDevice(c->ranks[r].dev)); CK(cudaDeviceSynchronize()); }
  return c;
}

void sar_local_destroy(sar_local_comm* c) {
  if (!c) return;
  for (int r = 0; r < c->n; ++r) {
    Rank& rk = c->ranks[r];
    cudaSetDevice(rk.dev);
    cudaDeviceSynchronize();
    for (auto& kv : rk.tables) { cudaFree(kv.second.ops); cudaFree(kv.second.round_begin); }
    cudaFree(rk.flags); cudaFree(rk.ctrl); cudaFree(rk.status); cudaFree(rk.trace);
    cudaEventDestroy(rk.ev0); cudaEventDestroy(rk.ev1);
    if (!(c->emulate && r > 0)) cudaStreamDestroy(rk.stream);
  }
  if (c->d_params) { cudaSetDevice(c->ranks[0].dev); cudaFree(c->d_params); }
  for (sar::SymmAlloc* a : c->allocs) { sar::symm_free(a); delete a; }
  delete c;
}

int sar_local_nranks(const sar_local_comm* c) { return c->n; }
void* sar_local_stream(sar_local_comm* c, int rank) { return c->ranks[rank].stream; }

int sar_local_run(sar_local_comm* c, const sar_program* prog, void* const* bufs, uint64_t count, int dtype,
                  const sar_run_opts* o, const uint64_t* delay_ns, char* err, int errlen) {
  int fail_value = 1;
  const int n = c->n;
  const int nph = sar_program_num_phases(prog);
  if (nph < 1 || sar_table_nranks(sar_program_phase(prog, 0)) != n) {
    if (err) snprintf(err, errlen, "program is for %d ranks, communicator has %d", nph ? sar_table_nranks(sar_program_phase(prog, 0)) : 0, n);
    return 1;
  }
  if (o->user_in && o->user_out && nph != 1) {
    if (err) snprintf(err, errlen, "staged mode serves single-phase programs");
    return 1;
  }
  for (int r = 0; r < n; ++r)
    if (((uintptr_t)bufs[r]) & 15) { if (err) snprintf(err, errlen, "buffer of rank %d is not 16-byte aligned", r); return 1; }
  const uint32_t esize = dtype == SAR_F32 ? 4 : 2;
  const int path = o->path;
  int blocks = o->blocks > 0 ? o->blocks : sar_cuda_pick_blocks(path, count * esize);
  if (c->emulate && o->blocks <= 0) blocks = 4;   // all ranks share one device
  if (n == 1 && o->blocks <= 0 && blocks == 128) blocks = 148;   // a lone rank streams its own memory: one block per SM
  const double timeout_s = o->timeout_s > 0 ? o->timeout_s : 10.0;
  const uint32_t tile_max = o->tile_bytes ? o->tile_bytes : sar_cuda_default_tile_bytes(path);
  std::vector<bool> delayed(n, false);

  for (int r = 0; r < n; ++r) c->ranks[r].timed = o->timed != 0;

  // multicast views of the buffers, when they come from sar_local_alloc (simt path only: multimem
  // instructions are issued by threads, not by the bulk-copy engine)
  size_t mc_off = 0;
  const sar::SymmAlloc* mc_alloc = nullptr;
  if (!c->emulate && path != SAR_PATH_TMA && !c->allocs.empty()) {
    mc_alloc = find_alloc(c, bufs, (size_t)count * esize, &mc_off);
    if (mc_alloc && !mc_alloc->mc_handle[0]) mc_alloc = nullptr;
  }

  // ---- prepare every phase: geometry, device tables (uploaded on first use), launch parameters
  struct PhaseLaunch { std::vector<SarLaunchParams> hp; int blocks; uint32_t parts; };
  std::vector<PhaseLaunch> launches(nph);
  for (int ph = 0; ph < nph; ++ph) {
    const sar_table* t = sar_program_phase(prog, ph);
    const int ch = sar_table_channel(t);
    const uint32_t parts = sar_table_participants(t);
    const uint32_t nch = (uint32_t)sar_table_num_chunks(t);
    c->epoch[ch] += SAR_VER_STRIDE;
    int pblocks = blocks;   // this phase's block count: the table may ask for fewer
    const int hint = sar_table_blocks_hint(t);
    if (o->blocks <= 0 && !c->emulate && hint > 0 && hint < pblocks) pblocks = hint;
    const bool gated = sar_table_gate_rounds(t) && count * esize >= sar_gate_min_bytes();
    const uint32_t ptile_max = (gated && !o->tile_bytes && !c->emulate) ? sar::gate_tile_bytes() : tile_max;
    const uint32_t tile_elems = sar_pick_tile_elems(count, esize, nch, (uint32_t)pblocks, 2048, ptile_max);
    SarGeom g = sar::make_geom(count, esize, nch, tile_elems);
    if ((uint64_t)g.tiles_per_chunk * g.num_chunks > SAR_FLAG_CAPACITY) {
      if (err) snprintf(err, errlen, "buffer too large for the flag array");
      return 1;
    }
    PhaseLaunch& L = launches[ph];
    L.hp.resize(n); L.blocks = pblocks; L.parts = parts;
    for (int r = 0; r < n; ++r) {
      Rank& rk = c->ranks[r];
      SarLaunchParams& P = L.hp[r];
      memset(&P, 0, sizeof(P));
      for (int q = 0; q < n; ++q) {
        P.comm.flags[q] = c->ranks[q].flags + (size_t)ch * SAR_FLAG_CAPACITY;
        P.comm.ctrl[q] = c->ranks[q].ctrl + ch;
        P.comm.buf[q] = bufs[q];
      }
      CK(cudaSetDevice(rk.dev));
      DevTable* dt = upload(rk, t, r, err, errlen);
      if (!dt) return 1;
      P.ops = dt->ops; P.round_begin = dt->round_begin; P.num_rounds = dt->num_rounds;
      P.geom = g; P.rank = r; P.nranks = n; P.participants = parts;
      P.epoch_base = (uint32_t)c->epoch[ch]; P.gate_base = c->epoch[ch]; P.scale = o->scale; P.dtype = dtype;
      P.timeout_ns = (uint64_t)(timeout_s * 1e9);
      P.status = rk.status; P.trace = rk.trace; P.trace_rounds = o->trace_rounds ? 1u : 0u;
      P.gate_rounds = gated ? 1u : 0u;
      P.gate_slack = sar::gate_slack(g.tiles_per_chunk);
      P.stages = o->stages > 0 ? (uint32_t)o->stages : (uint32_t)sar_table_stages_hint(t);
      P.store_window = o->store_window > 0 ? (uint32_t)o->store_window : 0u;
      P.lane1_eighths = (uint32_t)sar_table_lane1_eighths(t);
      if (mc_alloc) {
        for (int grp = 0; grp < 2; ++grp) {
          if (!mc_alloc->mc[grp][r]) continue;
          P.mc[grp].base = (char*)mc_alloc->mc[grp][r] + mc_off;
          P.mc[grp].members = mc_alloc->members[grp];
        }
      }
      if (o->user_in && o->user_out) {
        P.user_in = o->user_in[r]; P.user_out = o->user_out[r]; P.user_dtype = o->user_dtype;
        sar_table_final_ver(t, r, P.final_ver);
      }
      P.delay_ns = 0;
      if (c->emulate && delay_ns && delay_ns[r] && !delayed[r] && (parts >> r & 1)) { P.delay_ns = delay_ns[r]; delayed[r] = true; }
    }
  }

  if (o->trace_rounds) {
    // start stamps begin at the maximum (they are lowered with atomicMin), the rest at zero
    for (int r = 0; r < n; ++r) {
      Rank& rk = c->ranks[r];
      CK(cudaSetDevice(rk.dev));
      CK(cudaMemsetAsync(rk.trace + 2, 0xff, sizeof(uint64_t) * SAR_MAX_ROUNDS, rk.stream));
      CK(cudaMemsetAsync(rk.trace + 2 + SAR_MAX_ROUNDS, 0, sizeof(uint64_t) * 2 * SAR_MAX_ROUNDS, rk.stream));
    }
  }

  if (c->emulate) {
    // every rank on one device: one cooperative launch per phase on one stream
    Rank& r0 = c->ranks[0];
    CK(cudaSetDevice(r0.dev));
    if (o->timed) CK(cudaEventRecord(r0.ev0, r0.stream));
    for (int ph = 0; ph < nph; ++ph) {
      CK(cudaMemcpyAsync(c->d_params, launches[ph].hp.data(), sizeof(SarLaunchParams) * n, cudaMemcpyHostToDevice, r0.stream));
      // the copy is from pageable memory: it has completed with respect to the host buffer on return
      cudaError_t e = (cudaError_t)sar_cuda_launch_emulated(c->d_params, n, dtype, path, launches[ph].blocks, o->threads, r0.stream);
      if (e != cudaSuccess) {
        if (err) snprintf(err, errlen, "emulated launch (%d ranks x %d blocks): %s", n, launches[ph].blocks, cudaGetErrorString(e));
        return (int)e;
      }
    }
    if (o->timed) CK(cudaEventRecord(r0.ev1, r0.stream));
    return 0;
  }

  // ---- one rank per device.  Everything of a rank is enqueued before the next rank is touched:
  // [start barrier, start event,] [delay,] its phases [, stop event].  The start barrier holds
  // every stream until the last rank's barrier kernel runs, by which time the work of all
  // other ranks is already queued behind theirs, so the host's launch order stays out of the
  // timed window.
  uint32_t barrier_epoch = 0;
  SarCtrl* bctrl[SAR_MAX_RANKS] = {};
  if (o->timed) {
    barrier_epoch = (uint32_t)++c->epoch[SAR_NUM_CHANNELS - 1];
    for (int r = 0; r < n; ++r) bctrl[r] = c->ranks[r].ctrl + (SAR_NUM_CHANNELS - 1);
  }
  for (int r = 0; r < n; ++r) {
    Rank& rk = c->ranks[r];
    CK(cudaSetDevice(rk.dev));
    if (o->timed) {
      CK((cudaError_t)sar_cuda_barrier(bctrl, r, n, (1u << n) - 1u, barrier_epoch, (uint64_t)(timeout_s * 1e9), rk.status, rk.stream));
      CK(cudaEventRecord(rk.ev0, rk.stream));
    }
    for (int ph = 0; ph < nph; ++ph) {
      if (!(launches[ph].parts >> r & 1)) continue;
      if (delay_ns && delay_ns[r] && !delayed[r]) { CK((cudaError_t)sar_cuda_delay(delay_ns[r], rk.stream)); delayed[r] = true; }
      CK((cudaError_t)sar_cuda_launch(&launches[ph].hp[r], path, launches[ph].blocks, o->threads, rk.stream));
    }
    if (o->timed) CK(cudaEventRecord(rk.ev1, rk.stream));
  }
  return 0;
}

int sar_local_round_trace(sar_local_comm* c, uint64_t* out) {
  for (int r = 0; r < c->n; ++r) {
    cudaSetDevice(c->ranks[r].dev);
    cudaError_t e = cudaMemcpy(out + (size_t)r * 3 * SAR_MAX_ROUNDS, c->ranks[r].trace + 2, sizeof(uint64_t) * 3 * SAR_MAX_ROUNDS,
                               cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

int sar_local_alloc(sar_local_comm* c, size_t bytes, int mode, uint32_t sub_members, void** bufs, char* err, int errlen) {
  int devs[SAR_MAX_RANKS];
  for (int r = 0; r < c->n; ++r) devs[r] = c->ranks[r].dev;
  if (c->emulate) {
    if (mode == sar::SYMM_MULTICAST) {
      if (err) snprintf(err, errlen, "multicast needs one device per rank (the ranks are emulated on one device)");
      return 1;
    }
    mode = sar::SYMM_PLAIN;
  }
  auto* a = new sar::SymmAlloc;
  if (sar::symm_alloc(a, c->n, devs, bytes, mode, sub_members, err, errlen) != 0) { delete a; return 1; }
  for (int r = 0; r < c->n; ++r) bufs[r] = a->uc[r];
  c->allocs.push_back(a);
  return 0;
}

int sar_local_free(sar_local_comm* c, void* buf0) {
  for (size_t i = 0; i < c->allocs.size(); ++i) {
    if (c->allocs[i]->uc[0] != buf0) continue;
    sar::symm_free(c->allocs[i]);
    delete c->allocs[i];
    c->allocs.erase(c->allocs.begin() + (long)i);
    return 0;
  }
  return 1;
}

int sar_local_multicast_groups(sar_local_comm* c, const void* buf0) {
  for (const sar::SymmAlloc* a : c->allocs) {
    const char* b0 = (const char*)a->uc[0];
    if ((const char*)buf0 < b0 || (const char*)buf0 >= b0 + a->mapped) continue;
    return (a->mc_handle[0] ? 1 : 0) | (a->mc_handle[1] ? 2 : 0);
  }
  return 0;
}

int sar_local_multicast_supported(sar_local_comm* c) {
  if (c->emulate) return 0;
  int devs[SAR_MAX_RANKS];
  for (int r = 0; r < c->n; ++r) {
    devs[r] = c->ranks[r].dev;
    for (int q = 0; q < r; ++q) if (devs[q] == devs[r]) return 0;
  }
  return sar::multicast_supported(c->n, devs) ? 1 : 0;
}

uint32_t sar_local_sync(sar_local_comm* c, float* ms) {
  uint32_t worst = 0;
  for (int r = 0; r < c->n; ++r) {
    Rank& rk = c->ranks[r];
    cudaSetDevice(rk.dev);
    cudaError_t e = cudaStreamSynchronize(rk.stream);
    if (e != cudaSuccess) { worst = 0x1000u + (uint32_t)e; continue; }
    uint32_t st = 0;
    cudaMemcpy(&st, rk.status, 4, cudaMemcpyDeviceToHost);
    if (st) {
      worst = worst > st ? worst : st;
      cudaMemset(rk.status, 0, 4);
      for (int ch = 0; ch < SAR_NUM_CHANNELS; ++ch) {
        cudaMemset(&rk.ctrl[ch].abort_flag, 0, 4);
        cudaMemset(&rk.ctrl[ch].blocks_done, 0, 4);
      }
    }
    if (ms) {
      ms[r] = 0.f;
      const Rank& ev = c->emulate ? c->ranks[0] : rk;
      if (rk.timed) cudaEventElapsedTime(&ms[r], ev.ev0, ev.ev1);
    }
  }
  return worst;
}

int sar_local_trace(sar_local_comm* c, uint64_t* out) {
  for (int r = 0; r < c->n; ++r) {
    cudaSetDevice(c->ranks[r].dev);
    cudaError_t e = cudaMemcpy(out + 2 * r, c->ranks[r].trace, 16, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}
}
