// cpu_backend.cpp — see cpu_backend.h.
#include "cpu_backend.h"

#include <errno.h>
#include <fcntl.h>
#include <pthread.h>
#include <sched.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "tbvcoll.h"

namespace tbv {

// ---- scalar conversions -----------------------------------------------------------
float bf16_to_f32(uint16_t h) {  // small enough to inline in the loops below
  uint32_t u = uint32_t(h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);  // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return uint16_t(u >> 16);
}
float f16_to_f32(uint16_t h) {
  uint32_t s = uint32_t(h & 0x8000u) << 16, e = (h >> 10) & 0x1fu, m = h & 0x3ffu, u;
  if (e == 0) {
    if (m == 0) {
      u = s;
    } else {  // subnormal: normalise
      int sh = 0;
      while (!(m & 0x400u)) { m <<= 1; sh++; }
      m &= 0x3ffu;
      u = s | (uint32_t(127 - 15 - sh + 1) << 23) | (m << 13);
    }
  } else if (e == 31) {
    u = s | 0x7f800000u | (m << 13);
  } else {
    u = s | ((e + 112u) << 23) | (m << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}
uint16_t f32_to_f16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint32_t s = (u >> 16) & 0x8000u, a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return uint16_t(s | 0x7e00u);   // NaN
  if (a >= 0x47800000u) {                              // >= 65536: overflow or inf
    return uint16_t(s | 0x7c00u);
  }
  if (a >= 0x38800000u) {  // normal half range
    uint32_t m = a - 0x38000000u;                      // rebias exponent 127 -> 15
    uint32_t r = m + 0xfffu + ((m >> 13) & 1u);        // round to nearest even at bit 13
    uint32_t h = r >> 13;
    if (h >= 0x7c00u) h = 0x7c00u;                     // rounded up to inf (>= 65520)
    return uint16_t(s | h);
  }
  if (a < 0x33000000u) return uint16_t(s);             // below half of the smallest subnormal
  // subnormal half: value = mant * 2^(e-150); want units of 2^-24
  uint32_t e = a >> 23, mant = (a & 0x7fffffu) | 0x800000u;
  int shift = int(126 - e);                            // 14..24 -> shift mant right by shift
  uint32_t h = mant >> shift, rem = mant & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (h & 1u))) h++;
  return uint16_t(s | h);
}

static inline float load_elem(const void* p, size_t i, int dtype) {
  switch (dtype) {
    case TBV_F32: return static_cast<const float*>(p)[i];
    case TBV_F16: return f16_to_f32(static_cast<const uint16_t*>(p)[i]);
    default: return bf16_to_f32(static_cast<const uint16_t*>(p)[i]);
  }
}
static inline void store_elem(void* p, size_t i, int dtype, float v) {
  switch (dtype) {
    case TBV_F32: static_cast<float*>(p)[i] = v; break;
    case TBV_F16: static_cast<uint16_t*>(p)[i] = f32_to_f16(v); break;
    default: static_cast<uint16_t*>(p)[i] = f32_to_bf16(v); break;
  }
}

// ---- backend ------------------------------------------------------------------------
CpuBackend::CpuBackend(int rank, int world, size_t cap, int nslot, bool async, double wdog_s,
                       int pin_cpu, Stats* stats)
    : rank_(rank), world_(world), nslot_(nslot), cap_(cap), async_(async), wdog_s_(wdog_s),
      pin_cpu_(pin_cpu), stats_(stats) {
  q_.resize(TBV_MAXSLOT);
}

CpuBackend::~CpuBackend() {
  if (run_.load()) {
    run_.store(false);
    { std::lock_guard<std::mutex> g(mu_); }
    cv_item_.notify_all();
    if (th_.joinable()) th_.join();
  }
  if (base_) munmap(base_, total_);
  if (owner_) shm_unlink(shm_name_.c_str());
}

std::atomic<uint64_t>* CpuBackend::flag(int owner, int slot, int src) {
  return reinterpret_cast<std::atomic<uint64_t>*>(base_ + size_t(owner) * per_rank_ +
                                                   (size_t(slot) * world_ + src) * 64);
}
char* CpuBackend::region(int owner, int slot, int src) {
  return base_ + size_t(owner) * per_rank_ + flag_bytes_ + (size_t(slot) * world_ + src) * cap_;
}

int CpuBackend::init(Bootstrap* bs, int port) {
  flag_bytes_ = (size_t(nslot_) * world_ * 64 + 4095) & ~size_t(4095);
  per_rank_ = flag_bytes_ + size_t(nslot_) * world_ * cap_;
  total_ = per_rank_ * world_;
  char name[64];
  snprintf(name, sizeof(name), "/tbvcoll.%d.%d", port, int(getuid()));
  shm_name_ = name;
  int fd = -1;
  if (rank_ == 0) {
    shm_unlink(name);  // a stale segment of a crashed run
    fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0 || ftruncate(fd, off_t(total_)) != 0) {
      errmsg_ = std::string("shm_open/ftruncate: ") + strerror(errno);
      if (fd >= 0) close(fd);
      fd = -1;
    } else {
      owner_ = true;
    }
  }
  // Everyone learns whether rank 0 has the segment before opening it.
  int ok = (rank_ != 0) || (fd >= 0);
  std::vector<int> oks(world_);
  if (bs->allgather(&ok, oks.data(), sizeof(int)) != 0) { errmsg_ = bs->error(); return -1; }
  if (!oks[0]) return -1;
  if (rank_ != 0) {
    fd = shm_open(name, O_RDWR, 0600);
    if (fd < 0) { errmsg_ = std::string("shm_open (peer): ") + strerror(errno); }
  }
  void* p = fd >= 0 ? mmap(nullptr, total_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0) : MAP_FAILED;
  if (fd >= 0) close(fd);
  ok = (p != MAP_FAILED);
  if (bs->allgather(&ok, oks.data(), sizeof(int)) != 0) { errmsg_ = bs->error(); return -1; }
  for (int r = 0; r < world_; r++)
    if (!oks[r]) { if (p != MAP_FAILED) munmap(p, total_); return -1; }
  base_ = static_cast<char*>(p);  // fresh segment: zero-filled, all flags 0
  // Once everybody has it mapped the name can go: no leak if a rank dies later.
  if (bs->barrier() != 0) return -1;
  if (owner_) { shm_unlink(name); owner_ = false; }
  if (async_) {
    run_.store(true);
    th_ = std::thread([this] { run(); });
  }
  return 0;
}

int CpuBackend::submit(const void* in, void* out, size_t nbytes, int dtype, int op) {
  if (err()) return TBV_FAIL;
  size_t need = nbytes;
  if (need > cap_) return TBV_FALLBACK;
  CpuItem it{++seq_, in, out, nbytes, dtype, op, now_us()};
  if (!async_) {
    execute(it);
    return err() ? TBV_FAIL : TBV_OK;
  }
  // back-pressure: at most nslot calls in flight
  double t0 = now_us();
  while (q_head_.load(std::memory_order_relaxed) - q_tail_.load(std::memory_order_acquire) >=
         (unsigned long long)nslot_) {
    if (err()) return TBV_FAIL;
    if (now_us() - t0 < 30.0) continue;  // short spin first
    std::unique_lock<std::mutex> lk(mu_);
    cv_room_.wait_for(lk, std::chrono::milliseconds(2));
  }
  unsigned long long h = q_head_.load(std::memory_order_relaxed);
  q_[h % TBV_MAXSLOT] = it;
  q_head_.store(h + 1, std::memory_order_release);
  { std::lock_guard<std::mutex> g(mu_); }
  cv_item_.notify_one();
  return TBV_OK;
}

int CpuBackend::sync() {
  double t0 = now_us();
  while (q_tail_.load(std::memory_order_acquire) != q_head_.load(std::memory_order_relaxed)) {
    if (now_us() - t0 < 30.0) continue;
    std::unique_lock<std::mutex> lk(mu_);
    cv_room_.wait_for(lk, std::chrono::milliseconds(2));
  }
  return err() ? TBV_FAIL : TBV_OK;
}

void CpuBackend::run() {
  if (pin_cpu_ >= 0) {
    cpu_set_t cs;
    CPU_ZERO(&cs);
    CPU_SET(pin_cpu_, &cs);
    pthread_setaffinity_np(pthread_self(), sizeof(cs), &cs);
  }
  while (run_.load(std::memory_order_relaxed)) {
    unsigned long long t = q_tail_.load(std::memory_order_relaxed);
    double t0 = now_us();
    bool have = false;
    while (run_.load(std::memory_order_relaxed)) {
      if (q_head_.load(std::memory_order_acquire) != t) { have = true; break; }
      if (now_us() - t0 < 30.0) continue;
      std::unique_lock<std::mutex> lk(mu_);
      if (q_head_.load(std::memory_order_acquire) != t) { have = true; break; }
      cv_item_.wait_for(lk, std::chrono::milliseconds(2));
    }
    if (!have) break;
    CpuItem it = q_[t % TBV_MAXSLOT];
    execute(it);  // completes even on error, so the queue always drains
    q_tail_.store(t + 1, std::memory_order_release);
    { std::lock_guard<std::mutex> g(mu_); }
    cv_room_.notify_all();
  }
}

void CpuBackend::execute(const CpuItem& it) {
  const int slot = int(it.seq % (unsigned long long)nslot_);
  const double t_start = now_us();
  const size_t esz = it.dtype == TBV_F32 ? 4 : 2;
  // push
  for (int d = 1; d < world_; d++) {
    int p = (rank_ + d) % world_;
    const char* src = static_cast<const char*>(it.in);
    if (it.op == kOpReduceScatter) src += size_t(p) * it.nbytes;
    memcpy(region(p, slot, rank_), src, it.nbytes);
    flag(p, slot, rank_)->store(it.seq, std::memory_order_release);
  }
  // bounded wait for every peer
  bool ok = !err();
  for (int d = 1; d < world_ && ok; d++) {
    int p = (rank_ + d) % world_;
    double w0 = now_us();
    while (flag(rank_, slot, p)->load(std::memory_order_acquire) < it.seq) {
      double el = now_us() - w0;
      if (el > wdog_s_ * 1e6) {
        fprintf(stderr, "[tbvcoll] rank %d: watchdog %.2fs: seq %llu, no data from rank %d\n", rank_, wdog_s_,
                it.seq, p);
        err_seq_ = it.seq;
        err_peer_ = (unsigned long long)p;
        err_.store(1, std::memory_order_release);
        ok = false;
        break;
      }
      if (el > 50.0) sched_yield();
    }
    if (ok) {
      std::lock_guard<std::mutex> g(stats_->mu);
      stats_->peer_wait_us[p] += now_us() - w0;
      stats_->peer_n[p]++;
    }
  }
  const double t_ready = now_us();
  if (ok) {
    if (it.op == kOpAllGather) {
      for (int r = 0; r < world_; r++)
        memcpy(static_cast<char*>(it.out) + size_t(r) * it.nbytes,
               r == rank_ ? static_cast<const char*>(it.in) : region(rank_, slot, r), it.nbytes);
    } else {
      const size_t n = it.nbytes / esz;
      const char* mine = static_cast<const char*>(it.in);
      if (it.op == kOpReduceScatter) mine += size_t(rank_) * it.nbytes;
      // rank order 0..N-1 in fp32, one rounding: identical bits on every rank
      const void* srcs[TBV_MAXRANK];
      for (int r = 0; r < world_; r++) srcs[r] = (r == rank_) ? static_cast<const void*>(mine) : region(rank_, slot, r);
      if (it.dtype == TBV_F32) {
        float* o = static_cast<float*>(it.out);
        for (size_t i = 0; i < n; i++) {
          float acc = static_cast<const float*>(srcs[0])[i];
          for (int r = 1; r < world_; r++) acc += static_cast<const float*>(srcs[r])[i];
          o[i] = acc;
        }
      } else if (it.dtype == TBV_BF16) {
        uint16_t* o = static_cast<uint16_t*>(it.out);
        for (size_t i = 0; i < n; i++) {
          float acc = bf16_to_f32(static_cast<const uint16_t*>(srcs[0])[i]);
          for (int r = 1; r < world_; r++) acc += bf16_to_f32(static_cast<const uint16_t*>(srcs[r])[i]);
          o[i] = f32_to_bf16(acc);
        }
      } else {
        for (size_t i = 0; i < n; i++) {
          float acc = load_elem(srcs[0], i, it.dtype);
          for (int r = 1; r < world_; r++) acc += load_elem(srcs[r], i, it.dtype);
          store_elem(it.out, i, it.dtype, acc);
        }
      }
    }
  }
  const double t_done = now_us();
  stats_->add_xfer(it.nbytes, t_start - it.t_queued, t_ready - t_start, t_done - t_ready, 0.0, 1, TBV_ALGO_ONESHOT);
}

void CpuBackend::last_error(unsigned long long out[4]) const {
  out[0] = (unsigned long long)err_.load();
  out[1] = err_seq_;
  out[2] = 1;
  out[3] = err_peer_;
}

}  // namespace tbv
