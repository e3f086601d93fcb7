// Shared pieces of the benchmark programs: environment options, buffers,
// seeded fill, per-iteration on-device verification.
#pragma once
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../core/c_api.h"
#include "../core/table.h"
#include "../kernels/sar_cuda.h"
#include "../runtime/local_comm.h"

#define CHECK_CUDA(cmd)                                                                      \
  do {                                                                                       \
    cudaError_t e_ = (cmd);                                                                  \
    if (e_ != cudaSuccess) {                                                                 \
      fprintf(stderr, "CUDA error %s:%d: '%s'\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
      exit(EXIT_FAILURE);                                                                    \
    }                                                                                        \
  } while (0)

namespace bench {

inline const char* env_str(const char* name, const char* dflt) {
  const char* v = getenv(name);
  return (v && *v) ? v : dflt;
}
inline long env_int(const char* name, long dflt) {
  const char* v = getenv(name);
  return (v && *v) ? strtol(v, nullptr, 10) : dflt;
}

struct Options {
  int ngpus = 0;           // STRAGGLAR_NGPUS (default: all visible, at most 8)
  int dtype = SAR_F32;     // STRAGGLAR_DTYPE = float32 | bfloat16 | float16
  int straggler = -1;      // STRAGGLAR_STRAGGLER: physical rank that is late (default n-1)
  int path = SAR_PATH_SIMT;// STRAGGLAR_PATH = simt | tma | simta
  int blocks = 0, threads = 0;
  int store_window = 0;    // STRAGGLAR_STORE_WINDOW: store groups a block keeps in flight on the bulk-copy path (3, 8, 16)
  int stages = 0;          // STRAGGLAR_STAGES: ring stages per block on the bulk-copy path (0: all)
  uint32_t tile_bytes = 0;
  double timeout_s = 10.0; // STRAGGLAR_TIMEOUT_MS
  int warmup = 10;         // STRAGGLAR_WARMUP
  bool emulate = false;    // STRAGGLAR_EMULATE=1: every rank on device 0, one cooperative launch
  bool const_fill = false; // STRAGGLAR_FILL=const: rank r holds r+1 everywhere (the reference's inputs)
  int verify = 2;          // STRAGGLAR_VERIFY = each (2) | last (1) | none (0)
  bool trace = false;      // STRAGGLAR_TRACE=1: per-round statistics of the last timed iteration on stderr
  int nvls = 0;            // STRAGGLAR_NVLS = 0 | 1 (buffers bound to NVLink multicast objects, required) | try
  std::string schedule_text;  // STRAGGLAR_SCHEDULE=<file with a synthesizer printout>
};

inline int dtype_from(const char* s) {
  if (!strcmp(s, "float32") || !strcmp(s, "fp32") || !strcmp(s, "float")) return SAR_F32;
  if (!strcmp(s, "bfloat16") || !strcmp(s, "bf16")) return SAR_BF16;
  if (!strcmp(s, "float16") || !strcmp(s, "fp16") || !strcmp(s, "half")) return SAR_F16;
  fprintf(stderr, "Invalid dtype: %s\n", s);
  exit(EXIT_FAILURE);
}
inline int path_from(const char* s) {
  if (!strcmp(s, "tma")) return SAR_PATH_TMA;
  if (!strcmp(s, "simt")) return SAR_PATH_SIMT;
  if (!strcmp(s, "simta")) return SAR_PATH_SIMTA;
  fprintf(stderr, "Invalid path: %s (simt, tma or simta)\n", s);
  exit(EXIT_FAILURE);
}
// path column of the CSV; "+nvls" when multicast views serve the buffers
inline const char* path_label(int path, int mc_groups) {
  if (path == SAR_PATH_TMA) return "tma";
  if (path == SAR_PATH_SIMTA) return mc_groups ? "simta+nvls" : "simta";
  return mc_groups ? "simt+nvls" : "simt";
}
inline const char* dtype_name(int d) { return d == SAR_F32 ? "float32" : d == SAR_BF16 ? "bfloat16" : "float16"; }
inline uint32_t dtype_size(int d) { return d == SAR_F32 ? 4 : 2; }

inline Options read_options() {
  Options o;
  int visible = 0;
  CHECK_CUDA(cudaGetDeviceCount(&visible));
  o.emulate = env_int("STRAGGLAR_EMULATE", 0) != 0;
  o.ngpus = (int)env_int("STRAGGLAR_NGPUS", o.emulate ? 8 : (visible > 8 ? 8 : visible));
  if (!o.emulate && o.ngpus > visible) {
    printf("Need at least %d GPUs\n", o.ngpus);
    exit(EXIT_FAILURE);
  }
  o.dtype = dtype_from(env_str("STRAGGLAR_DTYPE", "float32"));
  o.straggler = (int)env_int("STRAGGLAR_STRAGGLER", -1);
  {
    const char* nv = env_str("STRAGGLAR_NVLS", "0");
    o.nvls = !strcmp(nv, "try") ? 2 : (atoi(nv) != 0 ? 1 : 0);
  }
  // multimem instructions are issued by threads: with multicast buffers the simt path is the default
  o.path = path_from(env_str("STRAGGLAR_PATH", o.nvls ? "simt" : "tma"));
  o.blocks = (int)env_int("STRAGGLAR_BLOCKS", 0);
  o.threads = (int)env_int("STRAGGLAR_THREADS", 0);
  o.stages = (int)env_int("STRAGGLAR_STAGES", 0);
  o.store_window = (int)env_int("STRAGGLAR_STORE_WINDOW", 0);
  o.tile_bytes = (uint32_t)env_int("STRAGGLAR_TILE_BYTES", 0);
  o.timeout_s = env_int("STRAGGLAR_TIMEOUT_MS", 10000) / 1000.0;
  o.warmup = (int)env_int("STRAGGLAR_WARMUP", 10);
  o.trace = env_int("STRAGGLAR_TRACE", 0) != 0;
  o.const_fill = !strcmp(env_str("STRAGGLAR_FILL", "uniform"), "const");
  const char* v = env_str("STRAGGLAR_VERIFY", "each");
  o.verify = !strcmp(v, "none") ? 0 : !strcmp(v, "last") ? 1 : 2;
  const char* sf = getenv("STRAGGLAR_SCHEDULE");
  if (sf && *sf) {
    FILE* f = fopen(sf, "r");
    if (!f) { fprintf(stderr, "cannot open schedule file %s\n", sf); exit(EXIT_FAILURE); }
    char buf[4096];
    size_t k;
    while ((k = fread(buf, 1, sizeof buf, f)) > 0) o.schedule_text.append(buf, k);
    fclose(f);
  }
  return o;
}

// element range of chunk c when `count` elements are cut in `chunks` (the library's rule)
inline void chunk_range(uint64_t count, uint32_t esize, uint32_t chunks, uint32_t c, uint64_t* b, uint64_t* e) {
  SarGeom g{};
  g.count = count; g.esize = esize; g.num_chunks = chunks; g.tile_elems = 16 / esize; g.tiles_per_chunk = 1;
  *b = sar_chunk_begin(g, c);
  *e = sar_chunk_begin(g, c + 1);
}

struct Buffers {
  int n = 0;
  std::vector<int> dev;
  std::vector<void*> ptr;
  std::vector<uint32_t*> result;  // per rank: 2 words for the verifier
  sar_local_comm* owner = nullptr;
  int mc_groups = 0;              // bit g: multicast group g serves the buffers
  // mode: 0 plain device memory, 1 multicast required, 2 multicast when available (see sar_local_alloc)
  void alloc(sar_local_comm* comm, int n_, const std::vector<int>& devs, size_t bytes, int mode = 0, uint32_t sub_members = 0) {
    n = n_; dev = devs; ptr.assign(n, nullptr); result.assign(n, nullptr); owner = comm;
    char err[512] = {0};
    if (sar_local_alloc(comm, bytes, mode, sub_members, ptr.data(), err, sizeof err)) {
      fprintf(stderr, "buffer allocation failed: %s\n", err);
      exit(EXIT_FAILURE);
    }
    mc_groups = sar_local_multicast_groups(comm, ptr[0]);
    for (int r = 0; r < n; ++r) {
      CHECK_CUDA(cudaSetDevice(dev[r]));
      CHECK_CUDA(cudaMalloc(&result[r], 8));
    }
  }
  void release() {
    for (int r = 0; r < n; ++r) { cudaSetDevice(dev[r]); cudaFree(result[r]); }
    if (owner && n) sar_local_free(owner, ptr[0]);
  }
};

}  // namespace bench
