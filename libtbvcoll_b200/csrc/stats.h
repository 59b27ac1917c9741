// stats.h — read-and-reset phase accumulators and the log2-size histogram.
//
// Same observable quantities as the reference's accumulators and getters
// (step4/libtbvcoll.cpp:114-116, 205-209, 510-561): pre / xfer / post / enq / drain in
// microseconds, a 32-bucket log2(bytes) histogram with count, mean transfer time and
// mean channel count, plus the algorithm chosen per bucket, and per-channel/per-peer
// arrival numbers for the `rails` dump.
#pragma once
#include <stdio.h>
#include <string.h>
#include <time.h>

#include <mutex>

namespace tbv {

inline double now_us() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec * 1e6 + ts.tv_nsec * 1e-3;
}

struct Stats {
  std::mutex mu;
  double t_pre = 0, t_acc = 0, t_post = 0, t_enq = 0, t_drain = 0;
  unsigned long long n_acc = 0, n_enq = 0;
  double hb_us[32] = {0}, hb_chan[32] = {0};
  unsigned long long hb_n[32] = {0};
  unsigned long long hb_algo[32][8] = {{0}};
  double peer_wait_us[8] = {0};
  unsigned long long peer_n[8] = {0};
  unsigned long long stream_switches = 0, streams_seen = 0, fallbacks = 0;

  static int bucket(size_t nbytes) {
    int b = 0;
    while ((size_t(1) << (b + 1)) <= nbytes && b < 31) b++;
    return b;
  }
  void add_enq(double us) { std::lock_guard<std::mutex> g(mu); t_enq += us; n_enq++; }
  void add_xfer(size_t nbytes, double pre, double xfer, double post, double drain, int nchan, int algo) {
    std::lock_guard<std::mutex> g(mu);
    t_pre += pre; t_acc += xfer; t_post += post; t_drain += drain; n_acc++;
    int b = bucket(nbytes);
    hb_us[b] += xfer; hb_chan[b] += nchan; hb_n[b]++;
    hb_algo[b][algo & 7]++;
  }
  // averages, then reset (reference: libtbvcoll.cpp:522-536)
  void read5(double* pre, double* xfer, double* post, double* enq, double* drain, unsigned long long* n) {
    std::lock_guard<std::mutex> g(mu);
    unsigned long long k = n_acc ? n_acc : 1, ke = n_enq ? n_enq : 1;
    if (pre) *pre = t_pre / k;
    if (xfer) *xfer = t_acc / k;
    if (post) *post = t_post / k;
    if (enq) *enq = t_enq / ke;
    if (drain) *drain = t_drain / k;
    if (n) *n = n_acc;
    t_pre = t_acc = t_post = t_enq = t_drain = 0;
    n_acc = n_enq = 0;
  }
  void dump_hist(int rank, unsigned long long tag_bad, unsigned long long tag_checked = 0) {
    std::lock_guard<std::mutex> g(mu);
    static const char* an[8] = {"auto", "oneshot", "twoshot", "nvls", "ll", "ce", "?", "?"};
    fprintf(stderr, "[tbvcoll] rank %d hist: streams=%llu switches=%llu fallbacks=%llu tag_checked=%llu tag_bad=%llu\n", rank,
            streams_seen, stream_switches, fallbacks, tag_checked, tag_bad);
    for (int b = 0; b < 32; b++) {
      if (!hb_n[b]) continue;
      int best = 1;
      for (int a = 1; a < 8; a++) if (hb_algo[b][a] > hb_algo[b][best]) best = a;
      fprintf(stderr, "[tbvcoll]   2^%-2d B  n=%-8llu xfer=%8.2f us  chan=%5.1f  algo=%s\n", b, hb_n[b],
              hb_us[b] / hb_n[b], hb_chan[b] / hb_n[b], an[best]);
    }
    memset(hb_us, 0, sizeof(hb_us)); memset(hb_chan, 0, sizeof(hb_chan));
    memset(hb_n, 0, sizeof(hb_n)); memset(hb_algo, 0, sizeof(hb_algo));
  }
  void dump_rails(int rank, int world) {
    std::lock_guard<std::mutex> g(mu);
    for (int p = 0; p < world; p++) {
      if (p == rank) continue;
      fprintf(stderr, "[tbvcoll] rank %d peer %d: n=%llu mean wait-for-arrival %.2f us\n", rank, p, peer_n[p],
              peer_n[p] ? peer_wait_us[p] / peer_n[p] : 0.0);
      peer_wait_us[p] = 0; peer_n[p] = 0;
    }
  }
};

}  // namespace tbv
