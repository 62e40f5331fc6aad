// NVLink / NCCL latency-bandwidth benchmark on the GPUs of one box (single process).
//
//   nvcc -O2 -std=c++17 benchmarks/nvlink_bench.cpp -lnccl -o nvlink_bench
//   ./nvlink_bench [--gpus N] [--min-bytes 8] [--max-bytes 1073741824] [--iters 200]
//
// For every message size (powers of four) it reports
//   * ncclAllReduce(float, sum) over N GPUs: latency, algorithm and bus bandwidth
//     (the reference's benchmark, benchmarks/bench.cpp:21-103 there, fixed to devices {0, 6},
//      1 MiB at most and 10000 iterations);
//   * cudaMemcpyPeerAsync GPU0 -> GPU1: the per-direction peer-copy bandwidth a fused kernel's
//     NVLink roofline is quoted against.
// Times are CUDA-event device times on GPU 0's stream after warm-up.
#include <cuda_runtime.h>
#include <nccl.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#define CHECK_CUDA(x) do { cudaError_t e = (x); if (e != cudaSuccess) { std::fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__); std::exit(1); } } while (0)
#define CHECK_NCCL(x) do { ncclResult_t r = (x); if (r != ncclSuccess) { std::fprintf(stderr, "NCCL error %s at %s:%d\n", ncclGetErrorString(r), __FILE__, __LINE__); std::exit(1); } } while (0)

int main(int argc, char** argv) {
  int want = 0, iters = 200;
  size_t min_bytes = 8, max_bytes = 1ull << 30;
  for (int i = 1; i + 1 < argc; i += 2) {
    if (!std::strcmp(argv[i], "--gpus")) want = std::atoi(argv[i + 1]);
    else if (!std::strcmp(argv[i], "--iters")) iters = std::atoi(argv[i + 1]);
    else if (!std::strcmp(argv[i], "--min-bytes")) min_bytes = std::strtoull(argv[i + 1], nullptr, 10);
    else if (!std::strcmp(argv[i], "--max-bytes")) max_bytes = std::strtoull(argv[i + 1], nullptr, 10);
  }
  int n = 0;
  CHECK_CUDA(cudaGetDeviceCount(&n));
  if (want > 0 && want < n) n = want;
  if (n < 1) { std::fprintf(stderr, "no GPU\n"); return 1; }

  std::vector<int> devs(n);
  std::vector<ncclComm_t> comms(n);
  std::vector<cudaStream_t> streams(n);
  std::vector<float*> send(n), recv(n);
  for (int i = 0; i < n; ++i) devs[i] = i;
  for (int i = 0; i < n; ++i) {
    CHECK_CUDA(cudaSetDevice(i));
    CHECK_CUDA(cudaStreamCreate(&streams[i]));
    CHECK_CUDA(cudaMalloc(&send[i], max_bytes));
    CHECK_CUDA(cudaMalloc(&recv[i], max_bytes));
    CHECK_CUDA(cudaMemset(send[i], 0, max_bytes));
  }
  if (n > 1) CHECK_NCCL(ncclCommInitAll(comms.data(), n, devs.data()));
  cudaEvent_t t0, t1;
  CHECK_CUDA(cudaSetDevice(0));
  CHECK_CUDA(cudaEventCreate(&t0));
  CHECK_CUDA(cudaEventCreate(&t1));

  std::printf("%14s %12s %12s %12s %14s\n", "bytes", "ar_lat_us", "ar_alg_GB/s", "ar_bus_GB/s", "peer_copy_GB/s");
  for (size_t bytes = min_bytes; bytes <= max_bytes; bytes *= 4) {
    const size_t count = bytes / sizeof(float);
    const int reps = bytes >= (64u << 20) ? std::max(5, iters / 20) : iters;
    double ar_us = 0.0;
    if (n > 1 && count > 0) {
      auto all_reduce = [&] {
        CHECK_NCCL(ncclGroupStart());
        for (int i = 0; i < n; ++i) CHECK_NCCL(ncclAllReduce(send[i], recv[i], count, ncclFloat, ncclSum, comms[i], streams[i]));
        CHECK_NCCL(ncclGroupEnd());
      };
      for (int w = 0; w < 5; ++w) all_reduce();
      for (int i = 0; i < n; ++i) { CHECK_CUDA(cudaSetDevice(i)); CHECK_CUDA(cudaStreamSynchronize(streams[i])); }
      CHECK_CUDA(cudaSetDevice(0));
      CHECK_CUDA(cudaEventRecord(t0, streams[0]));
      for (int r = 0; r < reps; ++r) all_reduce();
      CHECK_CUDA(cudaEventRecord(t1, streams[0]));
      for (int i = 0; i < n; ++i) { CHECK_CUDA(cudaSetDevice(i)); CHECK_CUDA(cudaStreamSynchronize(streams[i])); }
      float ms = 0.f;
      CHECK_CUDA(cudaEventElapsedTime(&ms, t0, t1));
      ar_us = 1e3 * ms / reps;
    }
    double copy_gbs = 0.0;
    if (n > 1) {
      CHECK_CUDA(cudaSetDevice(0));
      int can = 0;
      CHECK_CUDA(cudaDeviceCanAccessPeer(&can, 0, 1));
      if (can) { cudaError_t e = cudaDeviceEnablePeerAccess(1, 0); if (e != cudaSuccess) cudaGetLastError(); }
      for (int w = 0; w < 3; ++w) CHECK_CUDA(cudaMemcpyPeerAsync(recv[1], 1, send[0], 0, bytes, streams[0]));
      CHECK_CUDA(cudaEventRecord(t0, streams[0]));
      for (int r = 0; r < reps; ++r) CHECK_CUDA(cudaMemcpyPeerAsync(recv[1], 1, send[0], 0, bytes, streams[0]));
      CHECK_CUDA(cudaEventRecord(t1, streams[0]));
      CHECK_CUDA(cudaStreamSynchronize(streams[0]));
      float ms = 0.f;
      CHECK_CUDA(cudaEventElapsedTime(&ms, t0, t1));
      copy_gbs = bytes / (1e6 * ms / reps);
    }
    const double alg = ar_us > 0 ? bytes / (1e3 * ar_us) : 0.0;
    std::printf("%14zu %12.2f %12.2f %12.2f %14.2f\n", bytes, ar_us, alg, alg * 2.0 * (n - 1) / n, copy_gbs);
  }
  for (int i = 0; i < n; ++i) {
    CHECK_CUDA(cudaSetDevice(i));
    if (n > 1) ncclCommDestroy(comms[i]);
    cudaFree(send[i]);
    cudaFree(recv[i]);
    cudaStreamDestroy(streams[i]);
  }
  return 0;
}
