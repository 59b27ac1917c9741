// cpu_backend.h — the collective protocol on host memory (no GPU).
//
// N processes of one host share a POSIX shared-memory segment that plays the role
// of the peer-mapped slot memory: a slot ring, per-(slot, source) sequence flags,
// push-then-flag, bounded wait, rank-ordered fp32 reduction.  One progress thread
// per rank drains a FIFO of calls so that `allreduce` returns at once (async mode),
// which is the shape of the reference's host side — SPSC queue, 30 us spin then a
// 2 ms timed wait, back-pressure when NSLOT calls are in flight, a watchdog that
// makes the call complete with an error instead of hanging, and a sticky error
// (step4/libtbvcoll.cpp:226-277, 441-455) — but here it is the test/plumbing
// backend, never the production path.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <atomic>
#include <condition_variable>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "bootstrap.h"
#include "stats.h"

namespace tbv {

enum CpuOp : int { kOpAllReduce = 0, kOpReduceScatter = 1, kOpAllGather = 2 };

struct CpuItem {
  unsigned long long seq;
  const void* in;
  void* out;
  size_t nbytes;  // all-reduce: tensor bytes; reduce-scatter: output bytes; all-gather: input bytes
  int dtype, op;
  double t_queued;
};

class CpuBackend {
 public:
  CpuBackend(int rank, int world, size_t cap, int nslot, bool async, double wdog_s, int pin_cpu,
             Stats* stats);
  ~CpuBackend();
  int init(Bootstrap* bs, int port);
  int submit(const void* in, void* out, size_t nbytes, int dtype, int op);
  int sync();
  bool err() const { return err_.load(std::memory_order_acquire) != 0; }
  void set_wdog(double s) { wdog_s_ = s; }
  void last_error(unsigned long long out[4]) const;
  const std::string& error() const { return errmsg_; }

 private:
  void run();                       // progress thread
  void execute(const CpuItem& it);  // one collective, on whichever thread
  std::atomic<uint64_t>* flag(int owner, int slot, int src);
  char* region(int owner, int slot, int src);

  int rank_, world_, nslot_;
  size_t cap_;
  bool async_;
  double wdog_s_;
  int pin_cpu_;
  Stats* stats_;
  std::string shm_name_, errmsg_;
  char* base_ = nullptr;
  size_t total_ = 0, per_rank_ = 0, flag_bytes_ = 0;
  bool owner_ = false;

  std::vector<CpuItem> q_;
  std::atomic<unsigned long long> q_head_{0}, q_tail_{0};  // head: produced, tail: consumed
  unsigned long long seq_ = 0;
  std::mutex mu_;
  std::condition_variable cv_item_, cv_room_;
  std::atomic<int> err_{0};
  std::atomic<bool> run_{false};
  std::thread th_;
  unsigned long long err_seq_ = 0, err_peer_ = 0;
};

// bf16 / fp16 <-> fp32 on the host, round-to-nearest-even (used by the CPU
// backend and by nothing on the GPU path).
float bf16_to_f32(uint16_t h);
uint16_t f32_to_bf16(float f);
float f16_to_f32(uint16_t h);
uint16_t f32_to_f16(float f);

}  // namespace tbv
