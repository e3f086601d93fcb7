// reducescatter <bufferSize> <numIters>
//
// Stand-alone ReduceScatter among the non-straggler GPUs (all visible GPUs but
// one, as in the reference program which uses 7 of 8: stragglar/reducescatter.cu:66-73).
// Rank r ends with the sum of chunk r in place.  The collective is the
// library's own kernel: every rank pulls its chunk from all peers at once over
// NVSwitch, adds in fp32 and rounds once.  Output: the reference's headerless
// CSV `bytes,iter,ms,GiB/s` (stragglar/reducescatter.cu:116-121), with the time
// taken as the maximum over ranks; unlike the reference, every iteration's
// result is verified on the device.  STRAGGLAR_RS_RANKS overrides the rank count.
#include <algorithm>

#include "bench_common.h"

using namespace bench;

int main(int argc, char* argv[]) {
  if (argc != 3) {
    fprintf(stderr, "Usage: %s <bufferSize> <numIters>\n", argv[0]);
    exit(EXIT_FAILURE);
  }
  const size_t bytes = (size_t)strtoull(argv[1], NULL, 10);
  const int numIters = atoi(argv[2]);
  Options o = read_options();
  const int n = (int)env_int("STRAGGLAR_RS_RANKS", std::max(o.ngpus - 1, 1));
  const uint32_t esize = dtype_size(o.dtype);
  const uint64_t count = bytes / esize;
  char err[512] = {0};
  sar_program* prog = sar_program_build("reducescatter", n, 1, -1, nullptr, err, sizeof err);
  if (!prog) { fprintf(stderr, "%s\n", err); exit(EXIT_FAILURE); }
  std::vector<int> devs(n);
  for (int i = 0; i < n; ++i) devs[i] = o.emulate ? 0 : i;
  sar_local_comm* comm = sar_local_create(n, devs.data(), o.emulate ? 1 : 0, err, sizeof err);
  if (!comm) { fprintf(stderr, "%s\n", err); exit(EXIT_FAILURE); }
  Buffers B;
  B.alloc(comm, n, devs, count * esize, o.nvls, 0);
  if (o.nvls) fprintf(stderr, "multicast groups serving the buffers: %s\n", B.mc_groups & 1 ? "all ranks" : "none");
  sar_run_opts ro{};
  ro.path = o.path; ro.blocks = o.blocks; ro.threads = o.threads; ro.tile_bytes = o.tile_bytes;
  ro.timeout_s = o.timeout_s; ro.scale = 1.0f; ro.timed = 1;
  const float atol = o.dtype == SAR_F32 ? 2e-5f : o.dtype == SAR_BF16 ? 0.07f : 0.01f;
  const float rtol = o.dtype == SAR_F32 ? 1e-6f : o.dtype == SAR_BF16 ? 0.02f : 0.004f;
  std::vector<uint64_t> seeds(n);
  std::vector<float> ms(n);
  int failures = 0;
  for (int iter = -o.warmup; iter < numIters; ++iter) {
    for (int r = 0; r < n; ++r) {
      seeds[r] = (uint64_t)r + 977ull * (uint64_t)(iter + o.warmup);
      CHECK_CUDA(cudaSetDevice(devs[r]));
      CHECK_CUDA((cudaError_t)sar_cuda_fill_uniform(B.ptr[r], count, o.dtype, seeds[r], (cudaStream_t)sar_local_stream(comm, r)));
    }
    for (int r = 0; r < n; ++r) { CHECK_CUDA(cudaSetDevice(devs[r])); CHECK_CUDA(cudaStreamSynchronize((cudaStream_t)sar_local_stream(comm, r))); }
    if (sar_local_run(comm, prog, B.ptr.data(), count, o.dtype, &ro, nullptr, err, sizeof err)) { fprintf(stderr, "launch failed: %s\n", err); exit(EXIT_FAILURE); }
    const uint32_t status = sar_local_sync(comm, ms.data());
    if (status) { fprintf(stderr, "collective failed: %s\n", status < 0x1000 ? sar_status_string(status) : "CUDA error"); exit(2); }
    if (o.verify) {
      for (int r = 0; r < n; ++r) {
        uint64_t b, e;
        chunk_range(count, esize, n, r, &b, &e);
        CHECK_CUDA(cudaSetDevice(devs[r]));
        uint32_t res[2];
        CHECK_CUDA((cudaError_t)sar_cuda_verify_uniform_sum(B.ptr[r], b, e, o.dtype, seeds.data(), n, 1.0f, atol, rtol, B.result[r], nullptr));
        CHECK_CUDA(cudaMemcpy(res, B.result[r], 8, cudaMemcpyDeviceToHost));
        if (res[0]) { fprintf(stderr, "VERIFY FAILED: iteration %d rank %d: %u wrong elements\n", iter, r, res[0]); ++failures; }
      }
    }
    if (iter < 0) continue;
    const float t = *std::max_element(ms.begin(), ms.end());
    printf("%zu,%d,%.3f,%.3f\n", (size_t)count * esize, iter + 1, t, (double)bytes / 1024.0 / 1024.0 / 1024.0 * 1000.0 / t);
  }
  B.release();
  sar_local_destroy(comm);
  sar_program_free(prog);
  return failures ? 3 : 0;
}
