// comm.h — the communicator object behind the C ABI (internal).
//
// The reference keeps one process-global state block `G` (step4/libtbvcoll.cpp:82-117).
// Here it is an object, so several worlds (and emulated worlds) can coexist in one
// process; the `tbv_ar_*` functions operate on one default instance.
#pragma once
#include <atomic>
#include <map>
#include <tuple>
#include <memory>
#include <string>
#include <vector>

#include "ar_device.cuh"
#include "bootstrap.h"
#include "cpu_backend.h"
#include "nvtx_range.h"
#include "stats.h"
#include "tbvcoll.h"

namespace tbv {

struct Knobs {
  int async = 1;          // TBV_ASYNC: 0 = host waits for each collective (attribution/debug)
  int nslot = 4;          // TBV_NSLOT (2..32)
  double wdog_s = 10.0;   // TBV_WDOG seconds
  int tag = 0;            // TBV_TAG: seq stamp behind the payload, checked by the receiver
  long oneshot_max = -1;  // TBV_RAIL1MAX: largest message that uses the one-shot kernel (-1 = table)
  long chunk = 0;         // TBV_CHUNK: bytes per channel (0 = table)
  int cpu = -1;           // TBV_CPU: pin the CPU backend's progress thread
  int algo = TBV_ALGO_AUTO;  // TBV_ALGO
  int nchan = 0;          // TBV_NCHAN (0 = table)
  int ce = 0;             // TBV_CE: 1 = reserve one more slot for the copy-engine two-shot path (TBV_ALGO=ce / set_algo)
  int nvls = 0;           // TBV_NVLS: 1 = set up a multicast object and allow the NVLS kernels
  int mem = 0;            // TBV_MEM: 0 = VMM with IPC fallback, 1 = VMM only, 2 = cudaIpc only
  double init_timeout_s = 60.0;  // TBV_INIT_TIMEOUT
  long ll_max = -1;              // TBV_LL_MAX: largest message that uses flag-in-payload (LL) packets (-1: by world size)
  int ll_wide = 1;               // TBV_LL_WIDE: LL packets as one 32-byte store / load per unit (0 = two 16-byte ones)
  int streamwait = 0;            // TBV_STREAMWAIT: 1 = host-driven debug mode, the stream waits for the peers' flags (wait-value operations)
  int ll_spread = 0;             // TBV_LL_SPREAD: CTAs (a cluster) that share one row in the LL all-reduce + norm (0 or 1 = one CTA per row, the default)
  int ll_threads = 0;            // TBV_LL_THREADS: threads per CTA of the plain LL all-reduce (fewer threads = more SMs pushing; 0 = from world size)
  long nvls_min = 0x7fffffffffffffffl;  // TBV_NVLS_MIN: smallest message for the switch-reduced kernel in auto mode
  long nvls_direct_max = 1l << 20;      // TBV_NVLS_DIRECT_MAX: up to here the switch-reduced kernel has every rank reduce the whole tensor (one pass)
  static Knobs from_env();
};

struct GpuRank {  // one (real or emulated) rank's device resources
  int device = 0;
  char* base = nullptr;        // flags + data, this rank's own allocation
  size_t alloc_bytes = 0;
  DevState* st = nullptr;
  DevMirror* dm = nullptr;     // device memory: breadcrumbs + timing ring
  HostMirror* hm = nullptr;    // host pointer
  HostMirror* hm_dev = nullptr;
  RankCtx ctx{};
};

}  // namespace tbv

struct tbv_comm {
  int rank = 0, world = 1, device = -1;
  bool local = false;  // emulated world in one process
  size_t cap = 0;
  tbv::Knobs knobs;
  tbv::Stats stats;
  tbv::Bootstrap bs;
  std::unique_ptr<tbv::CpuBackend> cpu;
  // GPU backend
  std::vector<tbv::GpuRank> ranks;       // size 1 (real) or world (emulated)
  tbv::RankCtx* ctxs_dev = nullptr;      // emulated: device array of contexts
  size_t flag_bytes = 0, data_bytes = 0, ll_bytes = 0, ll_cap = 0;
  size_t tag_off = 0;                    // byte offset of the sequence-stamp words inside the flag area
  bool vmm = false, nvls = false;
  std::vector<void*> peer_maps;          // mapped peer bases (to unmap at teardown)
  std::vector<unsigned long long> vmm_handles;  // CUmemGenericAllocationHandle per rank (imported + own)
  unsigned long long mc_handle = 0;
  char* mc_base = nullptr;
  size_t mc_bytes = 0;
  int sm_count = 148;
  std::atomic<int> skip{0};
  int mute_rank = -1;                    // emulated world: rank that sits out the next `mute_left` launches
  std::atomic<int> mute_left{0};
  // device arrays of TMA tensor maps over this communicator's gather buffers, keyed by
  // (emulated rank, rows per rank, K, tile rows); freed in tbv_comm_destroy
  std::map<std::tuple<int, int, int, int>, void*> gather_maps;
  std::atomic<int> sticky_err{0};
  unsigned long long host_seq = 0, trace_read = 0;
  cudaStream_t side_stream = nullptr;      // stream-wait debug mode: the host looks at (and releases) flag words beside a blocked stream
  std::vector<tbv::TraceRec> trace_host;   // staging for the timing ring
  void* last_stream = nullptr;
  std::vector<void*> streams_seen;
  std::string errmsg;
};
