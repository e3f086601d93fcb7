// allreduce <NUM_BYTES> <ALG> <ITERS> <DELAY>
//
// AllReduce benchmark over the GPUs of one box, one host process driving all of
// them.  ALG is stragglar, ring, rhd or direct (also: stragglar_a2a, rsag).
// DELAY is the straggler's delay in ms; -1 means "the pre-phase (ReduceScatter
// for stragglar, sub-AllReduce for direct) has already happened": it is
// emulated by pre-filling the buffers and only the post-arrival rounds are
// timed; 0 times the pre-phase too, without a delay.  Same command line, same
// first six CSV columns and same semantics as the reference programs
// (stragglar/allreduce_8GPU.cu:907-1093, README.md:32-33), for any GPU count
// with a schedule (1, 2, 4, 6, 8, ...), fp32/bf16/fp16, seeded uniform inputs
// verified on the device after every iteration.
//
// What differs from the reference, on purpose: the collectives are the
// library's own peer-memory kernels (no NCCL); runtime_ms is the maximum over
// ranks of the device time between per-rank events placed after a device-side
// start barrier (the reference times device 0 only); the delay is spun on
// %globaltimer, so it lasts DELAY ms at any SM clock; extra columns follow the
// reference's six.  Options come from STRAGGLAR_* environment variables (see
// bench_common.h).  Each of <NUM_BYTES>, <ALG> and <DELAY> may be a
// comma-separated list; the matrix then runs in one process.  An ALG entry may carry
// options of its own, "name:key=value:...", which override the environment for that entry:
// blocks, stages, win (store groups in flight), tile (bytes), path (run options) and copy, lanes, lane1, gate, slack, gatemin
// (the STRAGGLAR_COPY / _LANES / _LANE1_EIGHTHS / _GATE / _GATE_SLACK / _GATE_MIN_BYTES lowering switches).
#include <algorithm>
#include <cmath>

#include "bench_common.h"

using namespace bench;

static std::vector<std::string> split_list(const char* s) {
  std::vector<std::string> out;
  std::string cur;
  for (const char* p = s;; ++p) {
    if (*p == ',' || *p == 0) { if (!cur.empty()) out.push_back(cur); cur.clear(); if (!*p) break; }
    else cur.push_back(*p);
  }
  return out;
}

// One (size, algorithm, delay) configuration on an existing communicator.
// Per rank: when each schedule round started and ended on it (microseconds after the first start of
// any rank) and how long its items waited for their operands (summed over the items of the round).
static void print_round_trace(sar_local_comm* comm, int n, const char* alg, size_t bytes, float delay) {
  std::vector<uint64_t> tr((size_t)n * 3 * SAR_MAX_ROUNDS);
  if (sar_local_round_trace(comm, tr.data())) return;
  uint64_t t0 = UINT64_MAX;
  for (int r = 0; r < n; ++r)
    for (int k = 0; k < SAR_MAX_ROUNDS; ++k) t0 = std::min(t0, tr[((size_t)r * 3 + 0) * SAR_MAX_ROUNDS + k]);
  fprintf(stderr, "round trace: %s, %zu bytes, delay %.1f ms; per round: [start .. end] us after the first start, (wait us summed over items)\n",
          alg, bytes, delay);
  for (int r = 0; r < n; ++r) {
    fprintf(stderr, "  rank %d:", r);
    for (int k = 0; k < SAR_MAX_ROUNDS; ++k) {
      const uint64_t s = tr[((size_t)r * 3 + 0) * SAR_MAX_ROUNDS + k];
      if (s == UINT64_MAX) continue;
      const uint64_t e = tr[((size_t)r * 3 + 1) * SAR_MAX_ROUNDS + k], w = tr[((size_t)r * 3 + 2) * SAR_MAX_ROUNDS + k];
      fprintf(stderr, " r%d [%.0f .. %.0f] (%.0f)", k, (s - t0) / 1e3, (e - t0) / 1e3, w / 1e3);
    }
    fprintf(stderr, "\n");
  }
}

static std::vector<std::string> split_on(const std::string& s, char sep) {
  std::vector<std::string> out;
  std::string cur;
  for (char ch : s) { if (ch == sep) { out.push_back(cur); cur.clear(); } else cur.push_back(ch); }
  out.push_back(cur);
  return out;
}

// "name:key=value:..." -> name; run options go to `o`, lowering switches to the environment (names returned in `set`)
static std::string apply_variant(const std::string& label, Options& o, std::vector<std::string>& set) {
  static const struct { const char* key; const char* env; } kEnv[] = {
      {"copy", "STRAGGLAR_COPY"}, {"lanes", "STRAGGLAR_LANES"}, {"lane1", "STRAGGLAR_LANE1_EIGHTHS"},
      {"gate", "STRAGGLAR_GATE"}, {"slack", "STRAGGLAR_GATE_SLACK"}, {"gatemin", "STRAGGLAR_GATE_MIN_BYTES"}};
  const std::vector<std::string> parts = split_on(label, ':');
  for (size_t i = 1; i < parts.size(); ++i) {
    const size_t eq = parts[i].find('=');
    if (eq == std::string::npos) { fprintf(stderr, "bad option '%s' in %s\n", parts[i].c_str(), label.c_str()); exit(EXIT_FAILURE); }
    const std::string k = parts[i].substr(0, eq), v = parts[i].substr(eq + 1);
    if (k == "blocks") o.blocks = atoi(v.c_str());
    else if (k == "stages") o.stages = atoi(v.c_str());
    else if (k == "win") o.store_window = atoi(v.c_str());
    else if (k == "tile") o.tile_bytes = (uint32_t)strtoul(v.c_str(), nullptr, 10);
    else if (k == "path") o.path = path_from(v.c_str());
    else {
      bool known = false;
      for (const auto& e : kEnv)
        if (k == e.key) { setenv(e.env, v.c_str(), 1); set.push_back(e.env); known = true; }
      if (!known) { fprintf(stderr, "unknown option '%s' in %s\n", k.c_str(), label.c_str()); exit(EXIT_FAILURE); }
    }
  }
  return parts[0];
}

static int run_config(sar_local_comm* comm, Buffers& B, const Options& o_in, const std::vector<int>& devs, size_t bytes,
                      const char* label, int numIters, float sleepTime, bool header) {
  Options o = o_in;
  std::vector<std::string> env_set;
  const std::string alg_name = apply_variant(label, o, env_set);
  const char* alg = alg_name.c_str();
  const int n = o.ngpus;
  const uint32_t esize = dtype_size(o.dtype);
  const uint64_t count = bytes / esize;
  const int straggler = o.straggler >= 0 ? o.straggler : n - 1;
  const bool prephase = sleepTime >= 0;
  char err[512] = {0};
  const char* sched = o.schedule_text.empty() ? nullptr : o.schedule_text.c_str();
  sar_program* prog = sar_program_build(alg, n, prephase ? 1 : 0, o.straggler, sched, err, sizeof err);
  if (!prog) { fprintf(stderr, "%s\n", err); return 1; }
  // roofline input: bytes the busiest rank moves in one direction after the straggler arrived
  sar_program* post = sar_program_build(alg, n, sleepTime == 0 ? 1 : 0, o.straggler, sched, err, sizeof err);
  double link_bytes = 0;
  for (int ph = 0; post && ph < sar_program_num_phases(post); ++ph) {
    const sar_table* t = sar_program_phase(post, ph);
    double mx = 0;
    for (int r = 0; r < n; ++r) mx = std::max(mx, std::max(sar_table_chunks_in(t, r), sar_table_chunks_out(t, r)));
    link_bytes += mx * (double)bytes / sar_table_num_chunks(t);
  }
  const double link_gbs = atof(env_str("STRAGGLAR_LINK_GBS", "770"));

  // the delay as the device really serves it
  double real_delay_ms = 0;
  if (sleepTime > 0) {
    CHECK_CUDA(cudaSetDevice(devs[straggler]));
    cudaEvent_t a, b;
    CHECK_CUDA(cudaEventCreate(&a)); CHECK_CUDA(cudaEventCreate(&b));
    cudaStream_t st = (cudaStream_t)sar_local_stream(comm, straggler);
    CHECK_CUDA((cudaError_t)sar_cuda_delay(1000, st));   // first launch loads the module: keep it out of the measurement
    float best = 1e30f;
    for (int k = 0; k < 3; ++k) {
      CHECK_CUDA(cudaEventRecord(a, st));
      CHECK_CUDA((cudaError_t)sar_cuda_delay((uint64_t)(sleepTime * 1e6), st));
      CHECK_CUDA(cudaEventRecord(b, st));
      CHECK_CUDA(cudaEventSynchronize(b));
      float ms = 0; CHECK_CUDA(cudaEventElapsedTime(&ms, a, b));
      best = ms < best ? ms : best;
    }
    real_delay_ms = best;
    CHECK_CUDA(cudaEventDestroy(a)); CHECK_CUDA(cudaEventDestroy(b));
    if (header) printf("Sleep: requested %.3f ms, measured %.3f ms on device %d\n", sleepTime, real_delay_ms, devs[straggler]);
  }

  std::vector<uint64_t> seeds(n), delay_ns(n, 0);
  if (sleepTime > 0) delay_ns[straggler] = (uint64_t)(sleepTime * 1e6);
  sar_run_opts ro{};
  ro.path = o.path; ro.blocks = o.blocks; ro.threads = o.threads; ro.tile_bytes = o.tile_bytes; ro.stages = o.stages; ro.store_window = o.store_window;
  ro.timeout_s = o.timeout_s + (sleepTime > 0 ? sleepTime / 1e3 : 0); ro.scale = 1.0f; ro.timed = 1;
  const float atol = o.dtype == SAR_F32 ? 2e-5f : o.dtype == SAR_BF16 ? 0.07f : 0.01f;
  const float rtol = o.dtype == SAR_F32 ? 1e-6f : o.dtype == SAR_BF16 ? 0.02f : 0.004f;
  const bool is_sar = !strncmp(alg, "stragglar", 9);

  if (header)
    printf("algorithm,buffer_size_bytes,iteration,delay,runtime_ms,BW(GB/s),n,dtype,path,time_us_max,algbw_GBps,busbw_GBps,roofline_frac,real_delay_ms,kernel_us_max\n");
  int failures = 0;
  std::vector<float> ms(n);
  for (int iter = -o.warmup; iter < numIters; ++iter) {
    for (int r = 0; r < n; ++r) {
      seeds[r] = (uint64_t)r + 131ull * (uint64_t)(iter + o.warmup);
      CHECK_CUDA(cudaSetDevice(devs[r]));
      cudaStream_t st = (cudaStream_t)sar_local_stream(comm, r);
      if (o.const_fill) CHECK_CUDA((cudaError_t)sar_cuda_fill_const(B.ptr[r], count, o.dtype, (float)(r + 1), st));
      else CHECK_CUDA((cudaError_t)sar_cuda_fill_uniform(B.ptr[r], count, o.dtype, seeds[r], st));
    }
    if (!prephase && n > 1 && (is_sar || !strcmp(alg, "direct"))) {
      // emulate the finished pre-phase (cf. stragglar/allreduce_8GPU.cu:1013-1020)
      std::vector<uint64_t> non;
      float csum = 0;
      for (int r = 0; r < n; ++r) if (r != straggler) { non.push_back(seeds[r]); csum += (float)(r + 1); }
      std::vector<int> l2p(n);
      for (int i = 0; i < n; ++i) l2p[i] = i;
      std::swap(l2p[n - 1], l2p[straggler]);
      for (int i = 0; i < n - 1; ++i) {
        const int r = l2p[i];
        uint64_t b = 0, e = count;
        if (is_sar) chunk_range(count, esize, n - 1, i, &b, &e);
        CHECK_CUDA(cudaSetDevice(devs[r]));
        cudaStream_t st = (cudaStream_t)sar_local_stream(comm, r);
        if (o.const_fill) CHECK_CUDA((cudaError_t)sar_cuda_fill_const((char*)B.ptr[r] + b * esize, e - b, o.dtype, csum, st));
        else CHECK_CUDA((cudaError_t)sar_cuda_fill_uniform_sum(B.ptr[r], b, e, o.dtype, non.data(), (int)non.size(), st));
      }
    }
    for (int r = 0; r < n; ++r) { CHECK_CUDA(cudaSetDevice(devs[r])); CHECK_CUDA(cudaStreamSynchronize((cudaStream_t)sar_local_stream(comm, r))); }

    ro.trace_rounds = (o.trace && iter == numIters - 1) ? 1 : 0;
    if (sar_local_run(comm, prog, B.ptr.data(), count, o.dtype, &ro, sleepTime > 0 ? delay_ns.data() : nullptr, err, sizeof err)) {
      fprintf(stderr, "launch failed: %s\n", err);
      exit(EXIT_FAILURE);
    }
    const uint32_t status = sar_local_sync(comm, ms.data());
    if (status) {
      fprintf(stderr, "collective failed in iteration %d: %s\n", iter, status < 0x1000 ? sar_status_string(status) : cudaGetErrorString((cudaError_t)(status - 0x1000)));
      exit(2);
    }
    if (ro.trace_rounds) print_round_trace(comm, n, label, bytes, sleepTime);
    if (o.verify == 2 || (o.verify == 1 && iter == numIters - 1)) {
      for (int r = 0; r < n; ++r) {
        CHECK_CUDA(cudaSetDevice(devs[r]));
        uint32_t res[2] = {0, 0};
        if (o.const_fill) {
          // constant inputs: every element must be n(n+1)/2 (the reference's check, on a 1 MiB sample)
          std::vector<char> h(std::min<size_t>(count * esize, 1 << 20));
          CHECK_CUDA(cudaMemcpy(h.data(), B.ptr[r], h.size(), cudaMemcpyDeviceToHost));
          const float want = n * (n + 1) / 2.0f;
          for (size_t i = 0; i < h.size() / esize; ++i) {
            float v;
            if (o.dtype == SAR_F32) v = ((float*)h.data())[i];
            else { uint16_t u = ((uint16_t*)h.data())[i]; uint32_t w = (uint32_t)u << 16; if (o.dtype == SAR_BF16) memcpy(&v, &w, 4); else v = want; }
            if (v != want) ++res[0];
          }
        } else {
          CHECK_CUDA((cudaError_t)sar_cuda_verify_uniform_sum(B.ptr[r], 0, count, o.dtype, seeds.data(), n, 1.0f, atol, rtol, B.result[r], nullptr));
          CHECK_CUDA(cudaMemcpy(res, B.result[r], 8, cudaMemcpyDeviceToHost));
        }
        if (res[0]) {
          float worst; memcpy(&worst, &res[1], 4);
          fprintf(stderr, "VERIFY FAILED: %s %zu B delay %.1f iteration %d rank %d: %u wrong elements (max abs error %g)\n", label, bytes, sleepTime, iter, r, res[0], worst);
          ++failures;
        }
      }
    }
    if (iter < 0) continue;
    const float t = *std::max_element(ms.begin(), ms.end());
    float bw;   // the reference's column: GiB/s with the nominal delay taken off
    if (sleepTime > 0) bw = (float)bytes / 1024.0f / 1024.0f / 1024.0f * 1000.0f / (t - sleepTime);
    else bw = (float)bytes / 1024.0f / 1024.0f / 1024.0f * 1000.0f / t;
    const double net_ms = t - real_delay_ms;
    const double algbw = (double)bytes / 1e9 / (net_ms / 1e3);
    const double busbw = algbw * 2.0 * (n - 1) / std::max(n, 1);
    const double roof_ms = link_bytes / (link_gbs * 1e9) * 1e3;
    // inside the kernels: from a rank's arrival to its exit (its last phase), longest over the ranks
    double kernel_us = 0;
    {
      std::vector<uint64_t> tr(2 * (size_t)n);
      if (!sar_local_trace(comm, tr.data()))
        for (int r = 0; r < n; ++r) if (tr[2 * r + 1] > tr[2 * r]) kernel_us = std::max(kernel_us, (tr[2 * r + 1] - tr[2 * r]) / 1e3);
    }
    printf("%s,%zu,%d,%.3f,%.3f,%.3f,%d,%s,%s,%.1f,%.2f,%.2f,%.3f,%.3f,%.1f\n", label, (size_t)count * esize, iter + 1, sleepTime, t, bw, n,
           dtype_name(o.dtype), path_label(o.path, B.mc_groups), t * 1e3, algbw, busbw, net_ms > 0 ? roof_ms / net_ms : 0.0, real_delay_ms, kernel_us);
  }
  sar_program_free(prog);
  if (post) sar_program_free(post);
  for (const std::string& e : env_set) unsetenv(e.c_str());
  return failures;
}

int main(int argc, char* argv[]) {
  if (argc != 5) {
    fprintf(stderr, "Usage: %s <bufferSize> <algorithm> <numIters> <sleepTimeMs>\n", argv[0]);
    exit(EXIT_FAILURE);
  }
  // every positional argument may be a comma-separated list: the whole matrix then runs in one
  // process on one communicator (sizes outermost), which saves the start-up cost per configuration
  const std::vector<std::string> sizes = split_list(argv[1]), algs = split_list(argv[2]), delays = split_list(argv[4]);
  const int numIters = atoi(argv[3]);
  static const char* kAlgs[] = {"ring", "rhd", "direct", "stragglar", "stragglar_a2a", "rsag"};
  for (const auto& a : algs)
    if (std::none_of(std::begin(kAlgs), std::end(kAlgs), [&](const char* k) { return a.substr(0, a.find(':')) == k; })) {
      fprintf(stderr, "Invalid algorithm: %s\n", a.c_str());
      exit(EXIT_FAILURE);
    }
  if (sizes.empty() || algs.empty() || delays.empty()) { fprintf(stderr, "empty argument\n"); exit(EXIT_FAILURE); }
  Options o = read_options();
  const int n = o.ngpus;
  size_t max_bytes = 0;
  for (const auto& s : sizes) max_bytes = std::max(max_bytes, (size_t)strtoull(s.c_str(), NULL, 10));
  char err[512] = {0};
  std::vector<int> devs(n);
  for (int i = 0; i < n; ++i) devs[i] = o.emulate ? 0 : i;
  sar_local_comm* comm = sar_local_create(n, devs.data(), o.emulate ? 1 : 0, err, sizeof err);
  if (!comm) { fprintf(stderr, "%s\n", err); exit(EXIT_FAILURE); }
  Buffers B;
  {
    // second multicast group: the non-stragglers (the ranks of the pre-phase)
    const int straggler = (o.straggler >= 0 && o.straggler < n) ? o.straggler : n - 1;
    const uint32_t all = (n >= 32) ? 0xffffffffu : ((1u << n) - 1u);
    B.alloc(comm, n, devs, max_bytes, o.nvls, all & ~(1u << straggler));
    if (o.nvls) fprintf(stderr, "multicast groups serving the buffers: %s%s%s\n", B.mc_groups & 1 ? "all ranks" : "none",
                        B.mc_groups & 2 ? ", non-stragglers" : "", o.path != SAR_PATH_TMA ? "" : " (unused: the bulk-copy path does not issue multimem instructions)");
  }
  int failures = 0;
  bool header = true;
  for (const auto& s : sizes)
    for (const auto& a : algs)
      for (const auto& d : delays) {
        if (a.substr(0, a.find(':')) == "rhd" && (n & (n - 1))) { fprintf(stderr, "rhd needs a power-of-two GPU count; skipped\n"); continue; }
        failures += run_config(comm, B, o, devs, (size_t)strtoull(s.c_str(), NULL, 10), a.c_str(), numIters, (float)atof(d.c_str()), header);
        header = false;
        fflush(stdout);
      }
  B.release();
  sar_local_destroy(comm);
  for (int i = 0; i < n; ++i) printf("Rank %d, done\n", i);
  if (failures) { fprintf(stderr, "%d verification failures\n", failures); return 3; }
  return 0;
}
