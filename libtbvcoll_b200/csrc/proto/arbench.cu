// arbench.cu — standalone native all-reduce microbenchmark (no Python, no torch).
//
// Role of the reference's prototype executables (step4/allreduce2.cpp:17-19,188-215 and
// step4/allreduce_mr.cpp:18-20): one process per rank, fp32 buffers filled with rank+1,
// 20 warm-ups, then two timed modes — "host-sync" (the host waits for every call) and
// "stream-ordered" (calls queued back to back, one wait at the end) — latency in us, algorithm
// bandwidth, and verify=OK/BAD on the first 1024 floats.
//
//   tbv_arbench <rank> <world> <cuda-dev> <bytes> <iters> [peer_ip=127.0.0.1] [port=18990]
//   env: TBV_ALGO, TBV_NCHAN, TBV_NSLOT, TBV_WDOG ... as for the library;
//        HOSTBUF=1 puts the user buffers in pinned, device-mapped HOST memory — the control experiment of
//        step4/allreduce_mr.cpp:81-93,113-116 (how much of the latency is where the payload lives)
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <vector>

#include "../tbvcoll.h"

static double now_us() {
  return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv) {
  if (argc < 6) {
    fprintf(stderr, "usage: %s <rank> <world> <cuda-dev> <bytes> <iters> [peer_ip] [port]\n", argv[0]);
    return 2;
  }
  const int rank = atoi(argv[1]), world = atoi(argv[2]), dev = atoi(argv[3]);
  const size_t bytes = strtoull(argv[4], nullptr, 0) & ~size_t(3);
  const int iters = atoi(argv[5]);
  const char* ip = argc > 6 ? argv[6] : "127.0.0.1";
  const int port = argc > 7 ? atoi(argv[7]) : 18990;
  if (cudaSetDevice(dev) != cudaSuccess) { fprintf(stderr, "cudaSetDevice(%d) failed\n", dev); return 1; }
  tbv_comm* c = nullptr;
  if (tbv_comm_create(&c, rank, world, dev, ip, port, bytes) != TBV_OK) { fprintf(stderr, "init failed\n"); return 1; }
  const size_t n = bytes / 4;
  std::vector<float> h(n, float(rank + 1));
  float *in = nullptr, *out = nullptr;
  const bool hostbuf = getenv("HOSTBUF") && atoi(getenv("HOSTBUF")) != 0;
  if (hostbuf) {
    float *hin = nullptr, *hout = nullptr;
    if (cudaHostAlloc(&hin, bytes, cudaHostAllocMapped) != cudaSuccess || cudaHostAlloc(&hout, bytes, cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(&in, hin, 0) != cudaSuccess || cudaHostGetDevicePointer(&out, hout, 0) != cudaSuccess) {
      fprintf(stderr, "HOSTBUF: pinned allocation failed\n");
      return 1;
    }
    memcpy(hin, h.data(), bytes);
    if (rank == 0) printf("# HOSTBUF=1: user buffers in pinned host memory\n");
  } else {
    cudaMalloc(&in, bytes);
    cudaMalloc(&out, bytes);
    cudaMemcpy(in, h.data(), bytes, cudaMemcpyHostToDevice);
  }
  cudaStream_t st;
  cudaStreamCreate(&st);
  for (int i = 0; i < 20; i++)
    if (tbv_comm_allreduce(c, in, out, bytes, TBV_F32, st) != TBV_OK) { fprintf(stderr, "all-reduce failed\n"); return 1; }
  cudaStreamSynchronize(st);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  const char* modes[2] = {"host-sync", "stream-ordered"};
  for (int mode = 0; mode < 2; mode++) {
    double t0 = now_us();
    cudaEventRecord(e0, st);
    for (int i = 0; i < iters; i++) {
      tbv_comm_allreduce(c, in, out, bytes, TBV_F32, st);
      if (mode == 0) cudaStreamSynchronize(st);
    }
    cudaEventRecord(e1, st);
    cudaStreamSynchronize(st);
    double wall = (now_us() - t0) / iters;
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    double pre, xfer, post, enq, drain;
    unsigned long long cnt;
    tbv_comm_stats5(c, &pre, &xfer, &post, &enq, &drain, &cnt);
    if (rank == 0)
      printf("%-14s bytes=%zu  lat=%.2f us (device %.2f us)  algbw=%.2f GB/s  [enqueue %.2f | wait-for-peers %.2f | reduce %.2f] us\n",
             modes[mode], bytes, wall, ms * 1e3 / iters, bytes / wall / 1e3, enq, xfer, post);
  }
  cudaMemcpy(h.data(), out, bytes < 4096 ? bytes : 4096, cudaMemcpyDeviceToHost);
  const float want = world * (world + 1) / 2.0f;
  bool ok = true;
  for (size_t i = 0; i < (n < 1024 ? n : 1024); i++) ok &= (h[i] > want - 0.01f && h[i] < want + 0.01f);
  printf("rank %d verify=%s (expect %.1f, got %.3f) err=%d\n", rank, ok ? "OK" : "BAD", want, h[0], tbv_comm_err(c));
  if (getenv("RAILS") && atoi(getenv("RAILS")) != 0) { tbv_comm_rails(c); tbv_comm_hist(c); }
  tbv_comm_destroy(c);
  return ok ? 0 : 1;
}
