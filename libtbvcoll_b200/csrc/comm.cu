// comm.cu — communicator bring-up, kernel launch and the C ABI.
//
// Bring-up replaces the reference's tbv_ar_init (step4/libtbvcoll.cpp:279-414): instead
// of dmabuf memory regions registered with ibverbs queue pairs, each rank creates one
// CUDA VMM allocation (slot ring + flag arrays), exports it as a POSIX fd, passes the fd
// to its peers over unix sockets, maps every peer's allocation into its own address
// space and, optionally, binds all of them to one NVLink multicast object (NVLS).
// cudaIpc handles are the fallback when VMM export is not possible.
//
// A call replaces tbv_ar_allreduce (:417-508): ONE kernel on the caller's stream.
#include <cuda.h>
#include <cuda_runtime.h>
#include <limits.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <algorithm>
#include <mutex>

#include "comm.h"
#include "ops/ops.h"
#include "pdl.cuh"

using namespace tbv;

#define LOG(...)                      \
  do {                                \
    fprintf(stderr, "[tbvcoll] ");    \
    fprintf(stderr, __VA_ARGS__);     \
    fprintf(stderr, "\n");            \
  } while (0)

#define CUDA_TRY(c, expr)                                                       \
  do {                                                                          \
    cudaError_t e__ = (expr);                                                   \
    if (e__ != cudaSuccess) {                                                   \
      (c)->errmsg = std::string(#expr) + ": " + cudaGetErrorString(e__);        \
      LOG("%s", (c)->errmsg.c_str());                                           \
      return TBV_FAIL;                                                          \
    }                                                                           \
  } while (0)

// ---- knobs --------------------------------------------------------------------------
static long env_long(const char* k, long d) {
  const char* v = getenv(k);
  return (v && *v) ? strtol(v, nullptr, 0) : d;
}
static double env_double(const char* k, double d) {
  const char* v = getenv(k);
  return (v && *v) ? strtod(v, nullptr) : d;
}
Knobs Knobs::from_env() {
  Knobs k;
  k.async = int(env_long("TBV_ASYNC", 1));
  k.nslot = int(std::min(long(TBV_MAXSLOT), std::max(2l, env_long("TBV_NSLOT", 4))));
  k.wdog_s = env_double("TBV_WDOG", 10.0);
  k.tag = int(env_long("TBV_TAG", 0));
  k.oneshot_max = env_long("TBV_RAIL1MAX", -1);
  k.chunk = env_long("TBV_CHUNK", 0);
  k.cpu = int(env_long("TBV_CPU", -1));
  k.nchan = int(env_long("TBV_NCHAN", 0));
  k.nvls = int(env_long("TBV_NVLS", 0));
  k.init_timeout_s = env_double("TBV_INIT_TIMEOUT", 60.0);
  k.ll_max = env_long("TBV_LL_MAX", -1);  // -1: chosen from the world size when the communicator is created
  k.nvls_min = env_long("TBV_NVLS_MIN", LONG_MAX);  // auto never picks the switch-reduced kernel unless asked
  k.nvls_direct_max = env_long("TBV_NVLS_DIRECT_MAX", 1l << 20);
  k.ce = int(env_long("TBV_CE", 0));
  k.ll_wide = int(env_long("TBV_LL_WIDE", 1)) != 0;
  k.streamwait = int(env_long("TBV_STREAMWAIT", 0)) != 0;
  k.ll_spread = int(env_long("TBV_LL_SPREAD", 0));
  k.ll_threads = int(env_long("TBV_LL_THREADS", 0));
  const char* a = getenv("TBV_ALGO");
  if (a) {
    if (!strcmp(a, "oneshot")) k.algo = TBV_ALGO_ONESHOT;
    else if (!strcmp(a, "twoshot")) k.algo = TBV_ALGO_TWOSHOT;
    else if (!strcmp(a, "nvls")) k.algo = TBV_ALGO_NVLS;
    else if (!strcmp(a, "ll")) k.algo = TBV_ALGO_LL;
    else if (!strcmp(a, "ce")) k.algo = TBV_ALGO_CE;
  }
  const char* m = getenv("TBV_MEM");
  if (m) k.mem = !strcmp(m, "vmm") ? 1 : (!strcmp(m, "ipc") ? 2 : 0);
  // Knobs of the reference that have no meaning without its transport: accepted, ignored.
  static bool once = false;
  if (!once) {
    once = true;
    for (const char* n : {"TBV_GPUSIG", "TBV_UNCACHED", "TBV_KWAIT"})
      if (getenv(n)) LOG("%s is accepted and ignored (in-kernel signalling is the only mode)", n);
  }
  return k;
}

// ---- driver API through the runtime (no link-time dependency on libcuda) ----------------
namespace {
struct Drv {
  bool ok = false;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*GetErrorString)(CUresult, const char**);
  CUresult (*StreamWaitValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);   // optional (stream-wait debug mode)
};
Drv g_drv;
std::once_flag g_drv_once;

template <typename F>
bool drv_sym(const char* name, F* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
    return false;
  *out = reinterpret_cast<F>(p);
  return true;
}
const Drv& drv() {
  std::call_once(g_drv_once, [] {
    Drv& d = g_drv;
    bool ok = true;
    ok &= drv_sym("cuMemGetAllocationGranularity", &d.MemGetAllocationGranularity);
    ok &= drv_sym("cuMemCreate", &d.MemCreate);
    ok &= drv_sym("cuMemRelease", &d.MemRelease);
    ok &= drv_sym("cuMemExportToShareableHandle", &d.MemExportToShareableHandle);
    ok &= drv_sym("cuMemImportFromShareableHandle", &d.MemImportFromShareableHandle);
    ok &= drv_sym("cuMemAddressReserve", &d.MemAddressReserve);
    ok &= drv_sym("cuMemAddressFree", &d.MemAddressFree);
    ok &= drv_sym("cuMemMap", &d.MemMap);
    ok &= drv_sym("cuMemUnmap", &d.MemUnmap);
    ok &= drv_sym("cuMemSetAccess", &d.MemSetAccess);
    ok &= drv_sym("cuDeviceGetAttribute", &d.DeviceGetAttribute);
    ok &= drv_sym("cuGetErrorString", &d.GetErrorString);
    // multicast is optional
    bool mc = drv_sym("cuMulticastCreate", &d.MulticastCreate);
    mc &= drv_sym("cuMulticastAddDevice", &d.MulticastAddDevice);
    mc &= drv_sym("cuMulticastBindMem", &d.MulticastBindMem);
    mc &= drv_sym("cuMulticastUnbind", &d.MulticastUnbind);
    mc &= drv_sym("cuMulticastGetGranularity", &d.MulticastGetGranularity);
    if (!mc) d.MulticastCreate = nullptr;
    if (!drv_sym("cuStreamWaitValue32", &d.StreamWaitValue32)) d.StreamWaitValue32 = nullptr;
    d.ok = ok;
  });
  return g_drv;
}
const char* cu_err(CUresult r) {
  const char* s = nullptr;
  if (g_drv.GetErrorString) g_drv.GetErrorString(r, &s);
  return s ? s : "unknown";
}
}  // namespace

// ---- kernels ------------------------------------------------------------------------------
struct LocalPtrs {
  const void* in[TBV_MAXRANK];
  void* out[TBV_MAXRANK];
  const void* aux[TBV_MAXRANK];   // residual
  void* aux_out[TBV_MAXRANK];     // residual_out
  int io;                          // kInAligned | kOutAligned, over all emulated ranks
  int mute;                        // emulated rank whose CTAs leave at once (a rank that never makes the call), or -1
};

template <typename T, bool VEC>
__global__ void __launch_bounds__(512) k_ar_oneshot(const __grid_constant__ RankCtx c, const T* in, T* out, size_t nbytes, int io) {
  __shared__ unsigned long long sh_seq;
  pdl::launch_dependents();
  pdl::grid_dependency_wait();  // before the device sequence number or any input is read
  ar_oneshot_body<T, VEC>(c, in, out, nbytes, gridDim.x, blockIdx.x, io, &sh_seq);
}
template <typename T, bool VEC>
__global__ void __launch_bounds__(512) k_ar_oneshot_local(const RankCtx* ctxs, const __grid_constant__ LocalPtrs p, size_t nbytes) {
  __shared__ unsigned long long sh_seq;
  pdl::launch_dependents();
  pdl::grid_dependency_wait();  // before the device sequence number or any input is read
  if (int(blockIdx.y) == p.mute) return;
  ar_oneshot_body<T, VEC>(ctxs[blockIdx.y], static_cast<const T*>(p.in[blockIdx.y]), static_cast<T*>(p.out[blockIdx.y]),
                          nbytes, gridDim.x, blockIdx.x, p.io, &sh_seq);
}
// One-shot all-reduce split around stream wait-value operations (TBV_STREAMWAIT=1): `part` = push half or reduce half.
// Plain launches: nothing in them waits for another rank, so the emulated ranks need no co-residency either.
template <typename T, bool VEC>
__global__ void __launch_bounds__(512) k_ar_oneshot_half(const __grid_constant__ RankCtx c, const T* in, T* out, size_t nbytes, int io, int part) {
  __shared__ unsigned long long sh_seq;
  ar_oneshot_body<T, VEC>(c, in, out, nbytes, gridDim.x, blockIdx.x, io, &sh_seq, part);
}
template <typename T, bool VEC>
__global__ void __launch_bounds__(512) k_ar_oneshot_half_local(const RankCtx* ctxs, const __grid_constant__ LocalPtrs p, size_t nbytes, int part) {
  __shared__ unsigned long long sh_seq;
  if (int(blockIdx.y) == p.mute && part == kPushHalf) return;   // a rank that never publishes
  ar_oneshot_body<T, VEC>(ctxs[blockIdx.y], static_cast<const T*>(p.in[blockIdx.y]), static_cast<T*>(p.out[blockIdx.y]),
                          nbytes, gridDim.x, blockIdx.x, p.io, &sh_seq, part);
}
template <typename T, bool VEC>
__global__ void __launch_bounds__(512) k_ar_twoshot(const __grid_constant__ RankCtx c, const T* in, T* out, size_t nbytes, int mode, int io) {
  __shared__ unsigned long long sh_seq;
  pdl::launch_dependents();
  pdl::grid_dependency_wait();  // before the device sequence number or any input is read
  ar_twoshot_body<T, VEC>(c, in, out, nbytes, gridDim.x, blockIdx.x, mode, io, &sh_seq);
}
template <typename T, bool VEC>
__global__ void __launch_bounds__(512) k_ar_twoshot_local(const RankCtx* ctxs, const __grid_constant__ LocalPtrs p, size_t nbytes, int mode) {
  __shared__ unsigned long long sh_seq;
  pdl::launch_dependents();
  pdl::grid_dependency_wait();  // before the device sequence number or any input is read
  if (int(blockIdx.y) == p.mute) return;
  ar_twoshot_body<T, VEC>(ctxs[blockIdx.y], static_cast<const T*>(p.in[blockIdx.y]), static_cast<T*>(p.out[blockIdx.y]),
                          nbytes, gridDim.x, blockIdx.x, mode, p.io, &sh_seq);
}
template <typename T>
__global__ void __launch_bounds__(512) k_ar_ll(const __grid_constant__ RankCtx c, const T* in, T* out, size_t nbytes, int io) {
  __shared__ unsigned long long sh_seq;
  pdl::launch_dependents();
  pdl::grid_dependency_wait();
  ar_oneshot_ll_body<T>(c, in, out, nbytes, gridDim.x, blockIdx.x, io, &sh_seq);
}
template <typename T>
__global__ void __launch_bounds__(512) k_ar_ll_local(const RankCtx* ctxs, const __grid_constant__ LocalPtrs p, size_t nbytes) {
  __shared__ unsigned long long sh_seq;
  if (int(blockIdx.y) == p.mute) return;
  ar_oneshot_ll_body<T>(ctxs[blockIdx.y], static_cast<const T*>(p.in[blockIdx.y]), static_cast<T*>(p.out[blockIdx.y]), nbytes,
                        gridDim.x, blockIdx.x, p.io, &sh_seq);
}
template <typename T>
__global__ void __launch_bounds__(512) k_ar_nvls(const __grid_constant__ RankCtx c, const T* in, T* out, size_t nbytes, int io, bool direct) {
  __shared__ unsigned long long sh_seq;
  pdl::launch_dependents();
  pdl::grid_dependency_wait();  // before the device sequence number or any input is read
  ar_nvls_body<T>(c, in, out, nbytes, gridDim.x, blockIdx.x, io, direct, &sh_seq);
}
__global__ void __launch_bounds__(1024) k_ar_rmsnorm(const __grid_constant__ RankCtx c, const __nv_bfloat16* x,
                                                     const __nv_bfloat16* residual, const __nv_bfloat16* gamma,
                                                     __nv_bfloat16* residual_out, __nv_bfloat16* y, int tokens, int hidden,
                                                     float eps) {
  __shared__ unsigned long long sh_seq;
  pdl::launch_dependents();
  pdl::grid_dependency_wait();  // before the device sequence number or any input is read
  __shared__ float sh_red[32];
  ar_rmsnorm_body(c, x, residual, gamma, residual_out, y, tokens, hidden, eps, gridDim.x, blockIdx.x, &sh_seq, sh_red);
}
__global__ void __launch_bounds__(1024) k_ar_rmsnorm_local(const RankCtx* ctxs, const __grid_constant__ LocalPtrs p,
                                                           const __nv_bfloat16* gamma, int tokens, int hidden, float eps) {
  __shared__ unsigned long long sh_seq;
  pdl::launch_dependents();
  pdl::grid_dependency_wait();  // before the device sequence number or any input is read
  __shared__ float sh_red[32];
  const int r = blockIdx.y;
  if (r == p.mute) return;
  ar_rmsnorm_body(ctxs[r], static_cast<const __nv_bfloat16*>(p.in[r]), static_cast<const __nv_bfloat16*>(p.aux[r]), gamma,
                  static_cast<__nv_bfloat16*>(p.aux_out[r]), static_cast<__nv_bfloat16*>(p.out[r]), tokens, hidden, eps,
                  gridDim.x, blockIdx.x, &sh_seq, sh_red);
}
// grid (row channels, 1 or emulated ranks, parts); the parts of a row form a cluster along z
template <int VPT>
__global__ void __launch_bounds__(512) k_ar_rmsnorm_ll(const __grid_constant__ RankCtx c, const __nv_bfloat16* x,
                                                       const __nv_bfloat16* residual, const __nv_bfloat16* gamma,
                                                       __nv_bfloat16* residual_out, __nv_bfloat16* y, int tokens, int hidden,
                                                       float eps, int norm_threads) {
  __shared__ unsigned long long sh_seq;
  pdl::launch_dependents();
  pdl::grid_dependency_wait();  // before the device sequence number or any input is read
  __shared__ float sh_red[64];
  ar_rmsnorm_ll_body<VPT>(c, x, residual, gamma, residual_out, y, tokens, hidden, eps, gridDim.x, blockIdx.x, blockIdx.z, gridDim.z,
                          norm_threads, &sh_seq, sh_red);
}
template <int VPT>
__global__ void __launch_bounds__(512) k_ar_rmsnorm_ll_local(const RankCtx* ctxs, const __grid_constant__ LocalPtrs p,
                                                             const __nv_bfloat16* gamma, int tokens, int hidden, float eps,
                                                             int norm_threads) {
  __shared__ unsigned long long sh_seq;
  pdl::launch_dependents();
  pdl::grid_dependency_wait();  // before the device sequence number or any input is read
  __shared__ float sh_red[64];
  const int r = blockIdx.y;
  if (r == p.mute) return;      // a whole emulated rank, i.e. whole clusters
  ar_rmsnorm_ll_body<VPT>(ctxs[r], static_cast<const __nv_bfloat16*>(p.in[r]), static_cast<const __nv_bfloat16*>(p.aux[r]), gamma,
                          static_cast<__nv_bfloat16*>(p.aux_out[r]), static_cast<__nv_bfloat16*>(p.out[r]), tokens, hidden, eps,
                          gridDim.x, blockIdx.x, blockIdx.z, gridDim.z, norm_threads, &sh_seq, sh_red);
}

template <typename T>
__global__ void __launch_bounds__(512) k_ar_ce_a(const __grid_constant__ RankCtx c, const T* in, T* out, size_t nbytes) {
  __shared__ unsigned long long sh_seq;
  ar_ce_phase_a<T>(c, in, out, nbytes, gridDim.x, blockIdx.x, &sh_seq);
}
template <typename T>
__global__ void __launch_bounds__(512) k_ar_ce_b(const __grid_constant__ RankCtx c, T* out, size_t nbytes) {
  __shared__ unsigned long long sh_seq;
  ar_ce_phase_b<T>(c, out, nbytes, gridDim.x, blockIdx.x, &sh_seq);
}

// ---- sizing tables --------------------------------------------------------------------------
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Which kernel runs is a function of (bytes, world, knobs) only — never of a pointer — and the
// knobs that enter it are checked for agreement between the ranks when the communicator is
// created: ranks that picked different kernels would wait on flags nobody raises.
static int pick_algo(const tbv_comm* c, size_t nbytes, bool vec) {
  int a = c->knobs.algo;
  if (a == TBV_ALGO_NVLS && !(c->nvls && vec)) a = TBV_ALGO_AUTO;
  if (a == TBV_ALGO_CE && !(c->knobs.ce && !c->local && nbytes % (size_t(16) * c->world) == 0)) a = TBV_ALGO_AUTO;
  const bool ll_ok = vec && nbytes * 2 <= c->ll_cap;
  if (a == TBV_ALGO_LL && !ll_ok) a = TBV_ALGO_AUTO;
  if (a != TBV_ALGO_AUTO) return a;
  if (ll_ok && long(nbytes) <= c->knobs.ll_max) return TBV_ALGO_LL;
  if (c->nvls && vec && long(nbytes) >= c->knobs.nvls_min) return TBV_ALGO_NVLS;
  long lim = c->knobs.oneshot_max;
  // measured crossovers (graph-timed, B200 NVSwitch, one build): 2 ranks one-shot wins up to 2 MiB (17.6 vs 19.9 us) and
  // loses at 4 MiB; 4 ranks up to 1 MiB (18.4 vs 20.2) and loses at 2 MiB (29.5 vs 23.2); 8 ranks up to 512 KiB (19.9 vs 25.8)
  if (lim < 0) lim = c->world <= 2 ? (2l << 20) : (c->world <= 4 ? (1l << 20) : (512l << 10));
  return long(nbytes) <= lim ? TBV_ALGO_ONESHOT : TBV_ALGO_TWOSHOT;
}
// Channels (CTAs).  The rule must be a pure function of (bytes, world, knobs): every
// rank has to launch the same grid because flags are per channel.
static int pick_nchan(const tbv_comm* c, int algo, size_t units_per_rankchunk, int threads) {
  int maxchan = c->local ? std::max(1, std::min(TBV_MAXCHAN, c->sm_count / c->world)) : TBV_MAXCHAN;
  if (c->knobs.nchan > 0) return std::min(c->knobs.nchan, maxchan);
  size_t per_chan_units = c->knobs.chunk > 0 ? std::max<size_t>(1, size_t(c->knobs.chunk) / 16)
                                             : size_t(threads);  // one 16-byte unit per thread and pass (measured: fatter channels leave two-shot latency-bound at 8 ranks)
  size_t n = (units_per_rankchunk + per_chan_units - 1) / per_chan_units;
  // two-shot: 64 channels keep the latency of mid-size messages low; from 4096 units (64 KiB) per channel on,
  // bandwidth is what counts and more CTAs put more bytes in flight
  int cap = algo == TBV_ALGO_LL ? 64 : (algo == TBV_ALGO_ONESHOT ? 32 : (units_per_rankchunk >= size_t(64) * 4096 ? 128 : 64));
  return int(std::max<size_t>(1, std::min<size_t>(n, size_t(std::min(cap, maxchan)))));
}

// ---- bring-up ---------------------------------------------------------------------------------
static void fill_ctx(tbv_comm* c, GpuRank& g, int rank) {
  RankCtx& x = g.ctx;
  x.rank = rank;
  x.world = c->world;
  x.nslot = c->knobs.nslot;
  x.debug_tag = c->knobs.tag;
  x.ll_wide = c->knobs.ll_wide;
  x.cap = c->cap;
  x.slot_stride = size_t(c->world + 1) * c->cap;
  x.ll_cap = c->ll_cap;
  // TBV_DEBUG_CAP (meant for the bounds-checked build): the extent the device-side guards compare with, smaller than
  // what is really reserved, so that a test can trip a guard with a call that stays inside real memory
  const long dbg_cap = env_long("TBV_DEBUG_CAP", 0);
  x.guard_cap = dbg_cap > 0 ? (unsigned long long)dbg_cap : c->cap;
  x.guard_ll_cap = dbg_cap > 0 ? (unsigned long long)dbg_cap * 2 : c->ll_cap;
  x.wdog_ns = (unsigned long long)(c->knobs.wdog_s * 1e9);
  x.st = g.st;
  x.dm = g.dm;
  x.hm = g.hm_dev;
  x.mc_data = c->mc_base ? c->mc_base + c->flag_bytes : nullptr;
}

static int alloc_rank_state(tbv_comm* c, GpuRank& g) {
  CUDA_TRY(c, cudaMalloc(&g.st, sizeof(DevState)));
  CUDA_TRY(c, cudaMemset(g.st, 0, sizeof(DevState)));
  CUDA_TRY(c, cudaMalloc(&g.dm, sizeof(DevMirror)));
  CUDA_TRY(c, cudaMemset(g.dm, 0, sizeof(DevMirror)));
  CUDA_TRY(c, cudaHostAlloc(&g.hm, sizeof(HostMirror), cudaHostAllocMapped | cudaHostAllocPortable));
  memset(g.hm, 0, sizeof(HostMirror));
  CUDA_TRY(c, cudaHostGetDevicePointer(&g.hm_dev, g.hm, 0));
  return TBV_OK;
}

static void compute_sizes(tbv_comm* c) {
  // LL packets double the bytes and every rank writes to every peer, so the size up to which they win
  // shrinks with the world.  The receiver fetches the packets of all sources with one batch of loads,
  // so the cost of a call no longer grows with one memory round trip per peer.
  // Measured with 32-byte packets: 2 ranks, LL 6.1 / 8.1 / 13.4 us at 512 KB / 1 MB / 2 MB against 10.8 / 13.1 / 18.9 for the
  // flag form; 8 ranks, 7.6 / 8.5 us at 64 / 128 KB against 12.3 / 13.0.  With more ranks every rank sends (world - 1) x 2 x the
  // bytes, so the limit comes down; 256 KB at 4 and 8 ranks continues the measured slope (+0.9 us per doubling at 8 ranks,
  // one-shot 14.9 us at 256 KB) and has not been timed itself.
  if (c->knobs.ll_max < 0) c->knobs.ll_max = c->world <= 2 ? (2048 << 10) : (256 << 10);
  c->knobs.ll_max = std::min<long>(c->knobs.ll_max, long(c->cap));   // no packet area beyond what a call may carry
  const size_t nflag = size_t(c->knobs.nslot + 1) * 2 * c->world * TBV_MAXCHAN;   // + the fixed slot of the copy-engine path
  c->tag_off = (nflag * sizeof(unsigned) + 255) & ~size_t(255);
  // flags, then one 8-byte sequence stamp per flag (TBV_TAG diagnostic; its own words, never inside a payload region)
  c->flag_bytes = (c->tag_off + nflag * sizeof(unsigned long long) + 4095) & ~size_t(4095);
  c->data_bytes = size_t(c->knobs.nslot + (c->knobs.ce ? 1 : 0)) * size_t(c->world + 1) * c->cap;   // TBV_CE=1: one more slot, outside the ring
  // LL area: two bytes on the wire per payload byte, one region per (slot, source)
  c->ll_cap = (size_t(std::max(0l, c->knobs.ll_max)) * 2 + 4095) & ~size_t(4095);
  c->ll_bytes = size_t(c->knobs.nslot) * c->world * c->ll_cap;
}

// VMM path: returns TBV_OK, or TBV_FALLBACK if VMM cannot be used here (caller tries IPC).
static int setup_vmm(tbv_comm* c) {
  const Drv& d = drv();
  if (!d.ok) return TBV_FALLBACK;
  GpuRank& g = c->ranks[0];
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = c->device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  if (d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || !gran)
    return TBV_FALLBACK;
  bool want_mc = c->knobs.nvls && d.MulticastCreate && c->world > 1;
  CUmulticastObjectProp mprop{};
  if (want_mc) {
    int sup = 0;
    d.DeviceGetAttribute(&sup, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, c->device);
    if (!sup) want_mc = false;
  }
  size_t total = c->flag_bytes + c->data_bytes + c->ll_bytes;
  if (want_mc) {
    mprop.numDevices = unsigned(c->world);
    mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mprop.size = total;
    size_t mg = 0;
    if (d.MulticastGetGranularity(&mg, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg)
      gran = std::max(gran, mg);
    else
      want_mc = false;
  }
  total = (total + gran - 1) / gran * gran;
  mprop.size = total;
  g.alloc_bytes = total;

  // Everything that can fail locally is followed by an agreement round, so that no rank
  // is left alone in a rendezvous.
  CUmemGenericAllocationHandle h = 0;
  int fd = -1;
  CUresult r = d.MemCreate(&h, total, &prop, 0);
  if (r == CUDA_SUCCESS) r = d.MemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  int ok = (r == CUDA_SUCCESS);
  std::vector<int> oks(c->world);
  if (c->bs.allgather(&ok, oks.data(), sizeof(int)) != 0) return TBV_FAIL;
  bool all_ok = true;
  for (int v : oks) all_ok &= (v != 0);
  if (!all_ok) {
    if (!ok) LOG("rank %d: VMM create/export failed (%s); trying cudaIpc", c->rank, cu_err(r));
    if (fd >= 0) close(fd);
    if (h) d.MemRelease(h);
    return TBV_FALLBACK;
  }
  std::vector<int> fds;
  if (c->bs.allgather_fd(fd, &fds) != 0) { c->errmsg = c->bs.error(); return TBV_FAIL; }

  c->vmm_handles.assign(c->world, 0);
  c->peer_maps.assign(c->world, nullptr);
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = c->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  ok = 1;
  for (int p = 0; p < c->world && ok; p++) {
    CUmemGenericAllocationHandle ph = h;
    if (p != c->rank) {
      r = d.MemImportFromShareableHandle(&ph, (void*)(uintptr_t)fds[p], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      if (r != CUDA_SUCCESS) { ok = 0; break; }
    }
    c->vmm_handles[p] = ph;
    CUdeviceptr va = 0;
    r = d.MemAddressReserve(&va, total, gran, 0, 0);
    if (r == CUDA_SUCCESS) r = d.MemMap(va, total, 0, ph, 0);
    if (r == CUDA_SUCCESS) r = d.MemSetAccess(va, total, &acc, 1);
    if (r != CUDA_SUCCESS) { ok = 0; break; }
    c->peer_maps[p] = reinterpret_cast<void*>(va);
  }
  for (int p = 0; p < c->world; p++)
    if (fds[p] >= 0) close(fds[p]);
  if (!ok) LOG("rank %d: VMM import/map failed: %s", c->rank, cu_err(r));
  if (c->bs.allgather(&ok, oks.data(), sizeof(int)) != 0) return TBV_FAIL;
  for (int v : oks)
    if (!v) { c->errmsg = "VMM mapping failed on some rank"; return TBV_FAIL; }
  g.base = static_cast<char*>(c->peer_maps[c->rank]);
  c->vmm = true;

  // NVLS: one multicast object over all ranks' allocations.
  if (want_mc) {
    CUmemGenericAllocationHandle mc = 0;
    int mfd = -1;
    ok = 1;
    if (c->rank == 0) {
      r = d.MulticastCreate(&mc, &mprop);
      if (r == CUDA_SUCCESS) r = d.MemExportToShareableHandle(&mfd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      ok = (r == CUDA_SUCCESS);
      if (!ok) LOG("multicast create/export failed: %s (NVLS off)", cu_err(r));
    }
    if (c->bs.allgather(&ok, oks.data(), sizeof(int)) != 0) return TBV_FAIL;
    if (oks[0]) {
      int got = -1;
      if (c->bs.broadcast_fd(0, mfd, &got) != 0) { c->errmsg = c->bs.error(); return TBV_FAIL; }
      ok = 1;
      if (c->rank != 0) {
        r = d.MemImportFromShareableHandle(&mc, (void*)(uintptr_t)got, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
        ok = (r == CUDA_SUCCESS);
      }
      if (got >= 0) close(got);
      if (ok) { r = d.MulticastAddDevice(mc, c->device); ok = (r == CUDA_SUCCESS); }
      if (c->bs.allgather(&ok, oks.data(), sizeof(int)) != 0) return TBV_FAIL;  // all devices added before any bind
      all_ok = true;
      for (int v : oks) all_ok &= (v != 0);
      if (all_ok) {
        r = d.MulticastBindMem(mc, 0, h, 0, total, 0);
        CUdeviceptr va = 0;
        if (r == CUDA_SUCCESS) r = d.MemAddressReserve(&va, total, gran, 0, 0);
        if (r == CUDA_SUCCESS) r = d.MemMap(va, total, 0, mc, 0);
        if (r == CUDA_SUCCESS) r = d.MemSetAccess(va, total, &acc, 1);
        ok = (r == CUDA_SUCCESS);
        if (!ok) LOG("rank %d: multicast bind/map failed: %s", c->rank, cu_err(r));
        if (c->bs.allgather(&ok, oks.data(), sizeof(int)) != 0) return TBV_FAIL;
        all_ok = true;
        for (int v : oks) all_ok &= (v != 0);
        if (all_ok) {
          c->mc_handle = mc;
          c->mc_base = reinterpret_cast<char*>(va);
          c->mc_bytes = total;
          c->nvls = true;
        } else if (ok) {
          d.MemUnmap(va, total);
          d.MemAddressFree(va, total);
        }
      }
      if (!c->nvls && mc) d.MemRelease(mc);
    }
  }
  return TBV_OK;
}

static int setup_ipc(tbv_comm* c) {
  GpuRank& g = c->ranks[0];
  size_t total = c->flag_bytes + c->data_bytes + c->ll_bytes;
  g.alloc_bytes = total;
  CUDA_TRY(c, cudaMalloc(&g.base, total));
  cudaIpcMemHandle_t mine;
  CUDA_TRY(c, cudaIpcGetMemHandle(&mine, g.base));
  std::vector<cudaIpcMemHandle_t> all(c->world);
  if (c->bs.allgather(&mine, all.data(), sizeof(mine)) != 0) { c->errmsg = c->bs.error(); return TBV_FAIL; }
  c->peer_maps.assign(c->world, nullptr);
  for (int p = 0; p < c->world; p++) {
    if (p == c->rank) { c->peer_maps[p] = g.base; continue; }
    CUDA_TRY(c, cudaIpcOpenMemHandle(&c->peer_maps[p], all[p], cudaIpcMemLazyEnablePeerAccess));
  }
  return TBV_OK;
}

static int gpu_init(tbv_comm* c) {
  CUDA_TRY(c, cudaSetDevice(c->device));
  CUDA_TRY(c, cudaFree(0));
  cudaDeviceProp prop;
  CUDA_TRY(c, cudaGetDeviceProperties(&prop, c->device));
  c->sm_count = prop.multiProcessorCount;
  compute_sizes(c);
  c->ranks.resize(1);
  GpuRank& g = c->ranks[0];
  g.device = c->device;
  if (alloc_rank_state(c, g) != TBV_OK) return TBV_FAIL;

  // agree on the parameters that shape the protocol and on every knob that enters the choice of
  // kernel or of the channel count (ranks that chose differently would wait on flags nobody raises)
  struct Hello {
    int world, nslot, tag, dev, algo, nchan, nvls, ce;
    long long ll_max, oneshot_max, chunk, nvls_min;
    unsigned long long cap;
    char uuid[16];
  } me{}, all[TBV_MAXRANK];
  me.world = c->world; me.nslot = c->knobs.nslot; me.tag = c->knobs.tag; me.dev = c->device; me.cap = c->cap;
  me.algo = c->knobs.algo; me.nchan = c->knobs.nchan; me.nvls = c->knobs.nvls; me.ce = c->knobs.ce; me.ll_max = c->knobs.ll_max;
  me.oneshot_max = c->knobs.oneshot_max; me.chunk = c->knobs.chunk; me.nvls_min = c->knobs.nvls_min;
  memcpy(me.uuid, &prop.uuid, 16);
  if (c->bs.allgather(&me, all, sizeof(Hello)) != 0) { c->errmsg = c->bs.error(); return TBV_FAIL; }
  for (int p = 0; p < c->world; p++) {
    if (all[p].world != me.world || all[p].nslot != me.nslot || all[p].cap != me.cap || all[p].tag != me.tag) {
      c->errmsg = "ranks disagree on world/nslot/cap/tag";
      LOG("rank %d: %s (rank %d has nslot=%d cap=%llu)", c->rank, c->errmsg.c_str(), p, all[p].nslot, all[p].cap);
      return TBV_FAIL;
    }
    if (all[p].algo != me.algo || all[p].nchan != me.nchan || all[p].nvls != me.nvls || all[p].ce != me.ce || all[p].ll_max != me.ll_max ||
        all[p].oneshot_max != me.oneshot_max || all[p].chunk != me.chunk || all[p].nvls_min != me.nvls_min) {
      c->errmsg = "ranks disagree on TBV_ALGO/TBV_NCHAN/TBV_NVLS/TBV_CE/TBV_LL_MAX/TBV_RAIL1MAX/TBV_CHUNK/TBV_NVLS_MIN";
      LOG("rank %d: %s (compared with rank %d)", c->rank, c->errmsg.c_str(), p);
      return TBV_FAIL;
    }
    if (p != c->rank && !memcmp(all[p].uuid, me.uuid, 16)) {
      c->errmsg = "two ranks on the same GPU: kernels that wait on one another must not share a device";
      LOG("rank %d: %s", c->rank, c->errmsg.c_str());
      return TBV_FAIL;
    }
  }

  int rc = TBV_FALLBACK;
  if (c->world == 1) {
    CUDA_TRY(c, cudaMalloc(&g.base, c->flag_bytes + c->data_bytes + c->ll_bytes));
    c->peer_maps.assign(1, g.base);
    rc = TBV_OK;
  } else {
    if (c->knobs.mem != 2) rc = setup_vmm(c);
    if (rc == TBV_FALLBACK) {
      if (c->knobs.mem == 1) { c->errmsg = "TBV_MEM=vmm but VMM export is unavailable"; return TBV_FAIL; }
      rc = setup_ipc(c);
    }
  }
  if (rc != TBV_OK) return TBV_FAIL;
  CUDA_TRY(c, cudaMemset(g.base, 0, c->flag_bytes));
  CUDA_TRY(c, cudaMemset(g.base + c->flag_bytes + c->data_bytes, 0, c->ll_bytes));  // no stale word may look like a packet
  CUDA_TRY(c, cudaDeviceSynchronize());
  fill_ctx(c, g, c->rank);
  for (int p = 0; p < c->world; p++) {
    g.ctx.flags[p] = reinterpret_cast<unsigned*>(c->peer_maps[p]);
    g.ctx.tags[p] = reinterpret_cast<unsigned long long*>(static_cast<char*>(c->peer_maps[p]) + c->tag_off);
    g.ctx.data[p] = static_cast<char*>(c->peer_maps[p]) + c->flag_bytes;
    g.ctx.ll[p] = static_cast<char*>(c->peer_maps[p]) + c->flag_bytes + c->data_bytes;
  }
  CUDA_TRY(c, cudaMalloc(&c->ctxs_dev, sizeof(RankCtx)));
  CUDA_TRY(c, cudaMemcpy(c->ctxs_dev, &g.ctx, sizeof(RankCtx), cudaMemcpyHostToDevice));
  // nobody may push before everybody has cleared its flags
  if (c->bs.barrier() != 0) { c->errmsg = c->bs.error(); return TBV_FAIL; }
  return TBV_OK;
}

static int gpu_init_local(tbv_comm* c) {
  CUDA_TRY(c, cudaSetDevice(c->device));
  cudaDeviceProp prop;
  CUDA_TRY(c, cudaGetDeviceProperties(&prop, c->device));
  c->sm_count = prop.multiProcessorCount;
  compute_sizes(c);
  c->ranks.resize(c->world);
  for (int r = 0; r < c->world; r++) {
    GpuRank& g = c->ranks[r];
    g.device = c->device;
    if (alloc_rank_state(c, g) != TBV_OK) return TBV_FAIL;
    g.alloc_bytes = c->flag_bytes + c->data_bytes + c->ll_bytes;
    CUDA_TRY(c, cudaMalloc(&g.base, g.alloc_bytes));
    CUDA_TRY(c, cudaMemset(g.base, 0, c->flag_bytes));
    CUDA_TRY(c, cudaMemset(g.base + c->flag_bytes + c->data_bytes, 0, c->ll_bytes));
  }
  std::vector<RankCtx> host(c->world);
  for (int r = 0; r < c->world; r++) {
    GpuRank& g = c->ranks[r];
    fill_ctx(c, g, r);
    for (int p = 0; p < c->world; p++) {
      g.ctx.flags[p] = reinterpret_cast<unsigned*>(c->ranks[p].base);
      g.ctx.tags[p] = reinterpret_cast<unsigned long long*>(c->ranks[p].base + c->tag_off);
      g.ctx.data[p] = c->ranks[p].base + c->flag_bytes;
      g.ctx.ll[p] = c->ranks[p].base + c->flag_bytes + c->data_bytes;
    }
    host[r] = g.ctx;
  }
  CUDA_TRY(c, cudaMalloc(&c->ctxs_dev, sizeof(RankCtx) * c->world));
  CUDA_TRY(c, cudaMemcpy(c->ctxs_dev, host.data(), sizeof(RankCtx) * c->world, cudaMemcpyHostToDevice));
  CUDA_TRY(c, cudaDeviceSynchronize());
  return TBV_OK;
}

static void banner(const tbv_comm* c) {
  if (c->rank != 0) return;
  LOG("rank %d/%d %s cap=%zu slots=%d mode=%s mem=%s nvls=%d wdog=%.1fs", c->rank, c->world,
      c->device < 0 ? "cpu(shm)" : (c->local ? "cuda(emulated ranks)" : "cuda"), c->cap, c->knobs.nslot,
      c->knobs.async ? "ASYNC" : "SYNC", c->device < 0 ? "shm" : (c->vmm ? "vmm" : "ipc"), int(c->nvls), c->knobs.wdog_s);
}

// ---- host-side error / stats plumbing ---------------------------------------------------------
static bool check_err(tbv_comm* c) {
  if (c->sticky_err.load(std::memory_order_relaxed)) return true;
  if (c->cpu) {
    if (c->cpu->err()) { c->sticky_err.store(1); return true; }
    return false;
  }
  for (auto& g : c->ranks) {
    if (*(volatile unsigned*)&g.hm->err != 0) {
      c->sticky_err.store(1);
      LOG("rank %d: device watchdog: seq %llu gave up at wait site %u on rank %u (channel %u); breadcrumbs enter=%llu pushed=%llu pass=%llu done=%llu",
          g.ctx.rank, g.hm->err_seq, g.hm->where, g.hm->peer, g.hm->chan, g.hm->bc[0], g.hm->bc[1], g.hm->bc[2], g.hm->bc[3]);
      return true;
    }
  }
  return false;
}

// Fold finished calls' device timestamps into the statistics (lazy: runs in the getters).
static void harvest_trace(tbv_comm* c) {
  if (c->cpu || c->ranks.empty()) return;
  // The device's own count of completed collectives: calls replayed from a CUDA graph never pass through the
  // host, so the host-side counter would miss them.  (Synchronous copy; the getters are off the hot path.)
  unsigned long long upto = c->host_seq;
  DevState ds;
  if (cudaMemcpy(&ds, c->ranks[0].st, sizeof(ds), cudaMemcpyDeviceToHost) == cudaSuccess && ds.seq > upto) upto = ds.seq;
  if (upto == c->trace_read) return;
  c->trace_host.resize(kTraceN);
  // device -> host copy of the ring (the getters are off the hot path)
  if (cudaMemcpy(c->trace_host.data(), c->ranks[0].dm->ring, sizeof(TraceRec) * kTraceN, cudaMemcpyDeviceToHost) != cudaSuccess) return;
  if (upto - c->trace_read > kTraceN) c->trace_read = upto - kTraceN;
  for (unsigned long long s = c->trace_read + 1; s <= upto; s++) {
    const TraceRec& r = c->trace_host[s & (kTraceN - 1)];
    if (r.seq != s) break;  // not finished yet
    double xfer = r.t_ready > r.t_enter ? (r.t_ready - r.t_enter) * 1e-3 : 0.0;
    double post = r.t_done > r.t_ready && r.t_ready ? (r.t_done - r.t_ready) * 1e-3 : 0.0;
    c->stats.add_xfer(size_t(r.nbytes), 0.0, xfer, post, 0.0, int(r.nchan), int(r.algo));
    c->trace_read = s;
  }
}

static void note_stream(tbv_comm* c, void* stream) {
  if (stream == c->last_stream && !c->streams_seen.empty()) return;
  bool seen = std::find(c->streams_seen.begin(), c->streams_seen.end(), stream) != c->streams_seen.end();
  if (!seen && c->streams_seen.size() < 16) {
    c->streams_seen.push_back(stream);
    c->stats.streams_seen++;
  }
  if (c->last_stream != stream && c->host_seq > 0) {
    // Calls on different streams are not ordered against each other by this library:
    // the slot ring assumes stream order.  Count them so that a user can see it.
    if (++c->stats.stream_switches <= 20 && getenv("TBV_VERBOSE")) LOG("stream switch #%llu", c->stats.stream_switches);
  }
  c->last_stream = stream;
}

// ---- launch -----------------------------------------------------------------------------------
template <typename T>
static cudaError_t launch_ar_t(tbv_comm* c, int algo, bool vec, int nchan, int threads, const void* in, void* out,
                               size_t nbytes, cudaStream_t st, int mode, int io) {
  const RankCtx& x = c->ranks[0].ctx;
  const T* i = static_cast<const T*>(in);
  T* o = static_cast<T*>(out);
  const dim3 g(nchan), b(threads);
  // switch-reduced kernel: below TBV_NVLS_DIRECT_MAX every rank reduces the whole tensor itself (one pass)
  if (algo == TBV_ALGO_NVLS) return pdl::launch(k_ar_nvls<T>, g, b, 0, st, 1, x, i, o, nbytes, io, long(nbytes) <= c->knobs.nvls_direct_max);
  if (algo == TBV_ALGO_LL) return pdl::launch(k_ar_ll<T>, g, b, 0, st, 1, x, i, o, nbytes, io);
  if (algo == TBV_ALGO_ONESHOT)
    return vec ? pdl::launch(k_ar_oneshot<T, true>, g, b, 0, st, 1, x, i, o, nbytes, io)
               : pdl::launch(k_ar_oneshot<T, false>, g, b, 0, st, 1, x, i, o, nbytes, io);
  return vec ? pdl::launch(k_ar_twoshot<T, true>, g, b, 0, st, 1, x, i, o, nbytes, mode, io)
             : pdl::launch(k_ar_twoshot<T, false>, g, b, 0, st, 1, x, i, o, nbytes, mode, io);
}

template <typename T>
static cudaError_t launch_ar_local_t(tbv_comm* c, int algo, bool vec, int nchan, int threads, const LocalPtrs& p,
                                     size_t nbytes, cudaStream_t st, int mode) {
  dim3 grid(nchan, c->world);
  const RankCtx* ctxs = c->ctxs_dev;
  void* fn;
  if (algo == TBV_ALGO_LL) {
    fn = (void*)k_ar_ll_local<T>;
    void* args[] = {(void*)&ctxs, (void*)&p, (void*)&nbytes};
    return cudaLaunchCooperativeKernel(fn, grid, dim3(threads), args, 0, st);
  }
  if (algo == TBV_ALGO_ONESHOT) {
    fn = vec ? (void*)k_ar_oneshot_local<T, true> : (void*)k_ar_oneshot_local<T, false>;
    void* args[] = {(void*)&ctxs, (void*)&p, (void*)&nbytes};
    return cudaLaunchCooperativeKernel(fn, grid, dim3(threads), args, 0, st);
  }
  fn = vec ? (void*)k_ar_twoshot_local<T, true> : (void*)k_ar_twoshot_local<T, false>;
  void* args[] = {(void*)&ctxs, (void*)&p, (void*)&nbytes, (void*)&mode};
  return cudaLaunchCooperativeKernel(fn, grid, dim3(threads), args, 0, st);
}

// Copy-engine two-shot: copies, kernel A, copies, kernel B on the caller's stream (see ar_device.cuh).
template <typename T>
static cudaError_t launch_ar_ce_t(tbv_comm* c, const void* in, void* out, size_t nbytes, cudaStream_t st) {
  const RankCtx& x = c->ranks[0].ctx;
  const int W = c->world, me = c->rank;
  const size_t chunk = nbytes / W;
  char* const ce0 = nullptr;
  (void)ce0;
  const size_t ce_off = size_t(x.nslot) * x.slot_stride;
  int nchan = int(std::min<size_t>(64, std::max<size_t>(1, chunk / 16 / 512)));
  if (c->knobs.nchan > 0) nchan = std::min(c->knobs.nchan, TBV_MAXCHAN);
  cudaError_t e = cudaSuccess;
  for (int d = 1; d < W && e == cudaSuccess; d++) {
    const int p = (me + d) % W;
    e = cudaMemcpyAsync(x.data[p] + ce_off + size_t(me) * x.cap, static_cast<const char*>(in) + chunk * p, chunk, cudaMemcpyDeviceToDevice, st);
  }
  if (e != cudaSuccess) return e;
  k_ar_ce_a<T><<<nchan, 512, 0, st>>>(x, static_cast<const T*>(in), static_cast<T*>(out), nbytes);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  for (int d = 1; d < W && e == cudaSuccess; d++) {
    const int p = (me + d) % W;
    e = cudaMemcpyAsync(x.data[p] + ce_off + size_t(W) * x.cap + chunk * me, static_cast<const char*>(out) + chunk * me, chunk,
                        cudaMemcpyDeviceToDevice, st);
  }
  if (e != cudaSuccess) return e;
  k_ar_ce_b<T><<<nchan, 512, 0, st>>>(x, static_cast<T*>(out), nbytes);
  return cudaGetLastError();
}

// Emulated world only: the rank named by tbv_comm_mute_rank sits out this launch.
static int take_mute(tbv_comm* c) {
  if (!c->local || c->mute_left.load() <= 0) return -1;
  c->mute_left.fetch_sub(1);
  return c->mute_rank;
}

static size_t dtype_size(int dtype) { return dtype == TBV_F32 ? 4 : 2; }

// ---- host-driven debug mode: the stream, not a kernel, waits for the peers (TBV_STREAMWAIT=1) ----------------
// The reference's default wait was a stream memory operation (hipStreamWaitValue64 on the slot's flag,
// step4/libtbvcoll.cpp:479-480); here the in-kernel bounded spin is the product path and this is the optional
// counterpart for attribution and for looking at a stuck exchange from the host: push half (payload stores, fence,
// flags), one cuStreamWaitValue32 per (source rank, channel) on this rank's own flag words, reduce half.  A stream
// wait has no deadline of its own, so the HOST bounds it: the call polls the stream until TBV_WDOG expires, then
// reads the flag words on a side stream, records which source never published (same error record as the device
// watchdog), stores the awaited value into the missing words itself so that the stream drains, and fails the
// communicator.  The call is therefore synchronous and reads the device's sequence number first: not for graphs.
template <typename T>
static cudaError_t launch_half_t(tbv_comm* c, bool vec, int nchan, int threads, const void* const* ins, void* const* outs, size_t nbytes,
                                 int io, int part, int mute, cudaStream_t st) {
  if (c->local) {
    LocalPtrs p{};
    for (int r = 0; r < c->world; r++) { p.in[r] = ins[r]; p.out[r] = outs[r]; }
    p.io = io;
    p.mute = mute;
    if (vec) k_ar_oneshot_half_local<T, true><<<dim3(nchan, c->world), threads, 0, st>>>(c->ctxs_dev, p, nbytes, part);
    else k_ar_oneshot_half_local<T, false><<<dim3(nchan, c->world), threads, 0, st>>>(c->ctxs_dev, p, nbytes, part);
  } else {
    const RankCtx& x = c->ranks[0].ctx;
    if (vec) k_ar_oneshot_half<T, true><<<nchan, threads, 0, st>>>(x, static_cast<const T*>(ins[0]), static_cast<T*>(outs[0]), nbytes, io, part);
    else k_ar_oneshot_half<T, false><<<nchan, threads, 0, st>>>(x, static_cast<const T*>(ins[0]), static_cast<T*>(outs[0]), nbytes, io, part);
  }
  return cudaGetLastError();
}
static cudaError_t launch_half(tbv_comm* c, int dtype, bool vec, int nchan, int threads, const void* const* ins, void* const* outs,
                               size_t nbytes, int io, int part, int mute, cudaStream_t st) {
  switch (dtype) {
    case TBV_F32: return launch_half_t<float>(c, vec, nchan, threads, ins, outs, nbytes, io, part, mute, st);
    case TBV_F16: return launch_half_t<__half>(c, vec, nchan, threads, ins, outs, nbytes, io, part, mute, st);
    default: return launch_half_t<__nv_bfloat16>(c, vec, nchan, threads, ins, outs, nbytes, io, part, mute, st);
  }
}

static int stream_wait_allreduce(tbv_comm* c, const void* const* ins, void* const* outs, size_t nbytes, int dtype, bool vec, int io,
                                 cudaStream_t st) {
  const Drv& d = drv();
  if (!d.StreamWaitValue32) { c->stats.fallbacks++; return TBV_FALLBACK; }
  const double t0 = now_us();
  // the device's own sequence number (replayed graphs advance it without the host)
  DevState ds;
  if (cudaStreamSynchronize(st) != cudaSuccess || cudaMemcpy(&ds, c->ranks[0].st, sizeof(ds), cudaMemcpyDeviceToHost) != cudaSuccess) {
    c->sticky_err.store(1);
    return TBV_FAIL;
  }
  const unsigned long long seq = ds.seq + 1;
  const unsigned want = unsigned(seq);
  const int slot = int(seq % (unsigned long long)c->knobs.nslot), W = c->world, nr = c->local ? W : 1;
  const size_t units = nbytes / (vec ? 16 : dtype_size(dtype));
  const int threads = units < 512 ? int(std::max<size_t>(32, (units + 31) / 32 * 32)) : 512;
  const int nchan = int(std::max<size_t>(1, std::min<size_t>(4, units / 512)));
  const int mute = take_mute(c);
  auto flag_word = [&](int r, int src, int chan) {
    return c->ranks[r].ctx.flags[c->ranks[r].ctx.rank] + ((size_t(slot) * 2 + 0) * W + src) * TBV_MAXCHAN + chan;   // flag_index(slot, phase 0, src, chan)
  };
  cudaError_t e = launch_half(c, dtype, vec, nchan, threads, ins, outs, nbytes, io, kPushHalf, mute, st);
  for (int r = 0; r < nr && e == cudaSuccess; r++)
    for (int src = 0; src < W; src++) {
      if (src == c->ranks[r].ctx.rank) continue;
      for (int ch = 0; ch < nchan; ch++)
        if (d.StreamWaitValue32(st, CUdeviceptr(uintptr_t(flag_word(r, src, ch))), want, CU_STREAM_WAIT_VALUE_EQ) != CUDA_SUCCESS) e = cudaErrorUnknown;
    }
  if (e == cudaSuccess) e = launch_half(c, dtype, vec, nchan, threads, ins, outs, nbytes, io, kReduceHalf, -1, st);
  if (e != cudaSuccess) {
    c->errmsg = std::string("stream-wait mode: ") + cudaGetErrorString(e);
    LOG("%s", c->errmsg.c_str());
    c->sticky_err.store(1);
    return TBV_FAIL;
  }
  c->host_seq++;
  // the host's bound on the stream's wait
  const double deadline = now_us() + c->knobs.wdog_s * 1e6;
  cudaError_t q;
  while ((q = cudaStreamQuery(st)) == cudaErrorNotReady && now_us() < deadline) usleep(20);
  if (q == cudaErrorNotReady) {
    if (!c->side_stream) cudaStreamCreateWithFlags(&c->side_stream, cudaStreamNonBlocking);
    bool named = false;
    for (int r = 0; r < nr; r++)
      for (int src = 0; src < W; src++) {
        if (src == c->ranks[r].ctx.rank) continue;
        for (int ch = 0; ch < nchan; ch++) {
          unsigned v = 0;
          cudaMemcpyAsync(&v, flag_word(r, src, ch), sizeof(v), cudaMemcpyDeviceToHost, c->side_stream);
          cudaStreamSynchronize(c->side_stream);
          if (v == want) continue;
          if (!named) {
            named = true;
            HostMirror* hm = c->ranks[r].hm;
            hm->err_seq = seq; hm->where = kWhereStreamWait; hm->peer = unsigned(src); hm->chan = unsigned(ch);
            hm->err = kErrTimeout;
          }
          cudaMemcpyAsync(flag_word(r, src, ch), &want, sizeof(want), cudaMemcpyHostToDevice, c->side_stream);   // let the stream drain
          cudaStreamSynchronize(c->side_stream);
        }
      }
    cudaStreamSynchronize(st);
    c->sticky_err.store(1);
    check_err(c);       // logs the record
    return TBV_FAIL;
  }
  if (q != cudaSuccess) { c->sticky_err.store(1); return TBV_FAIL; }
  if (check_err(c)) return TBV_FAIL;
  c->stats.add_enq(now_us() - t0);
  return TBV_OK;
}

// mode: 0 all-reduce (nbytes = tensor), 1 reduce-scatter (nbytes = output), 2 all-gather (nbytes = input)
static int gpu_collective(tbv_comm* c, const void* const* ins, void* const* outs, size_t nbytes, int dtype, void* stream,
                          int mode) {
  NvtxRange nvtx(mode == 0 ? "tbv.allreduce" : (mode == 1 ? "tbv.reduce_scatter" : "tbv.all_gather"), nbytes);
  const double t0 = now_us();
  if (check_err(c)) { LOG("previous collective failed: unrecoverable"); return TBV_FAIL; }
  if (dtype < 0 || dtype > 2) return TBV_FALLBACK;
  const size_t full = mode == 0 ? nbytes : nbytes * c->world;  // bytes of the gathered tensor
  if (full > c->cap || nbytes % dtype_size(dtype)) { c->stats.fallbacks++; return TBV_FALLBACK; }
  if (nbytes == 0) return TBV_OK;
  if (c->skip.load() > 0) { c->skip.fetch_sub(1); return TBV_OK; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  note_stream(c, stream);
  const int nr = c->local ? c->world : 1;
  if (c->world == 1) {
    if (outs[0] != ins[0]) CUDA_TRY(c, cudaMemcpyAsync(outs[0], ins[0], nbytes, cudaMemcpyDeviceToDevice, st));
    return TBV_OK;
  }
  // 16-byte units whenever the byte count allows: the partition into channels and the choice of kernel
  // must not depend on where a rank's tensor sits (ranks would disagree); a tensor that is not 16-byte
  // aligned is only accessed element by element inside the same kernel
  const bool vec = (nbytes % 16 == 0);
  int io = kInAligned | kOutAligned;
  for (int r = 0; r < nr; r++) {
    if (!aligned16(ins[r])) io &= ~kInAligned;
    if (!aligned16(outs[r])) io &= ~kOutAligned;
  }
  if (c->knobs.streamwait && mode == 0) return stream_wait_allreduce(c, ins, outs, nbytes, dtype, vec, io, st);
  int algo = mode == 0 ? pick_algo(c, nbytes, vec) : TBV_ALGO_TWOSHOT;
  if (mode != 0 && !vec && (nbytes % dtype_size(dtype))) return TBV_FALLBACK;
  if (c->local && algo == TBV_ALGO_NVLS) algo = TBV_ALGO_TWOSHOT;
  const size_t unit = vec ? 16 : dtype_size(dtype);
  size_t units = full / unit;
  if (mode != 0 && (nbytes % unit)) return TBV_FALLBACK;
  const bool oneshot_like = algo == TBV_ALGO_ONESHOT || algo == TBV_ALGO_LL;
  size_t per_rank_units = oneshot_like ? units : (units + c->world - 1) / c->world;
  if (mode != 0 && per_rank_units * unit != nbytes) return TBV_FALLBACK;  // chunks must be exactly the blocks
  int threads = 512;
  if (algo == TBV_ALGO_LL) {
    // An SM hands one 32-byte sector per clock to the fabric: keep what one CTA pushes (threads x 32 bytes x peers)
    // near 28 KB and let more SMs push instead (measured on 8 GPUs: 512 threads spend 2 us in the push, growing with the peers)
    const int fit = int(28672 / (32 * size_t(c->world - 1)));
    threads = c->knobs.ll_threads > 0 ? c->knobs.ll_threads : (fit >= 512 ? 512 : (fit >= 256 ? 256 : 128));
    threads = std::max(32, std::min(512, threads / 32 * 32));
  }
  if (per_rank_units < size_t(threads)) threads = int(std::max<size_t>(32, (per_rank_units + 31) / 32 * 32));
  int nchan = pick_nchan(c, algo, per_rank_units, threads);
  cudaError_t e;
  if (c->local) {
    LocalPtrs p{};
    for (int r = 0; r < nr; r++) { p.in[r] = ins[r]; p.out[r] = outs[r]; }
    p.io = io;
    p.mute = take_mute(c);
    switch (dtype) {
      case TBV_F32: e = launch_ar_local_t<float>(c, algo, vec, nchan, threads, p, full, st, mode); break;
      case TBV_F16: e = launch_ar_local_t<__half>(c, algo, vec, nchan, threads, p, full, st, mode); break;
      default: e = launch_ar_local_t<__nv_bfloat16>(c, algo, vec, nchan, threads, p, full, st, mode); break;
    }
  } else if (algo == TBV_ALGO_CE && mode == 0 && io == (kInAligned | kOutAligned)) {
    switch (dtype) {
      case TBV_F32: e = launch_ar_ce_t<float>(c, ins[0], outs[0], full, st); break;
      case TBV_F16: e = launch_ar_ce_t<__half>(c, ins[0], outs[0], full, st); break;
      default: e = launch_ar_ce_t<__nv_bfloat16>(c, ins[0], outs[0], full, st); break;
    }
  } else {
    if (algo == TBV_ALGO_CE) algo = TBV_ALGO_TWOSHOT;   // a tensor that cannot be copied 16 bytes at a time
    switch (dtype) {
      case TBV_F32: e = launch_ar_t<float>(c, algo, vec, nchan, threads, ins[0], outs[0], full, st, mode, io); break;
      case TBV_F16: e = launch_ar_t<__half>(c, algo, vec, nchan, threads, ins[0], outs[0], full, st, mode, io); break;
      default: e = launch_ar_t<__nv_bfloat16>(c, algo, vec, nchan, threads, ins[0], outs[0], full, st, mode, io); break;
    }
  }
  if (e != cudaSuccess) {
    c->errmsg = std::string("kernel launch: ") + cudaGetErrorString(e);
    LOG("%s", c->errmsg.c_str());
    c->sticky_err.store(1);
    return TBV_FAIL;
  }
  c->host_seq++;
  if (!c->knobs.async) {
    // SYNC mode: the host waits for the collective (attribution/debugging, like TBV_ASYNC=0
    // in the reference, libtbvcoll.cpp:483-492).
    double ts = now_us();
    cudaError_t se = cudaStreamSynchronize(st);
    std::lock_guard<std::mutex> g(c->stats.mu);
    c->stats.t_pre += now_us() - ts;
    if (se != cudaSuccess) { c->sticky_err.store(1); return TBV_FAIL; }
    if (check_err(c)) return TBV_FAIL;
  }
  c->stats.add_enq(now_us() - t0);
  return TBV_OK;
}

static int gpu_ar_rmsnorm(tbv_comm* c, const void* const* xs, const void* const* residuals, const void* gamma,
                          void* const* residual_outs, void* const* ys, int tokens, int hidden, float eps, void* stream) {
  NvtxRange nvtx("tbv.allreduce_rmsnorm", size_t(tokens) * hidden * 2);
  const double t0 = now_us();
  if (check_err(c)) return TBV_FAIL;
  const size_t nbytes = size_t(tokens) * hidden * 2;
  if (hidden % 8 || hidden > 8 * 4 * 1024 || nbytes > c->cap || tokens <= 0) { c->stats.fallbacks++; return TBV_FALLBACK; }
  const int nr = c->local ? c->world : 1;
  for (int r = 0; r < nr; r++)
    if (!aligned16(xs[r]) || !aligned16(residuals[r]) || !aligned16(residual_outs[r]) || !aligned16(ys[r]) || !aligned16(gamma))
      return TBV_FALLBACK;
  if (c->skip.load() > 0) { c->skip.fetch_sub(1); return TBV_OK; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  note_stream(c, stream);
  const int nt = tbvops::norm_threads(hidden);  // same mapping as the plain norm op: identical bits
  int maxchan = c->local ? std::max(1, std::min(TBV_MAXCHAN, c->sm_count / c->world)) : TBV_MAXCHAN;
  int nchan = std::min(tokens, c->knobs.nchan > 0 ? std::min(c->knobs.nchan, maxchan) : maxchan);
  cudaError_t e;
  const bool ll = (c->knobs.algo == TBV_ALGO_AUTO || c->knobs.algo == TBV_ALGO_LL) && nbytes * 2 <= c->ll_cap &&
                  long(nbytes) <= c->knobs.ll_max && hidden <= 8 * kLLNormVPT * 512;
  // LL form: the CTAs of a cluster can share a row (TBV_LL_SPREAD = 2, 4, 8) so that no SM pushes or pulls a whole row's packets.
  // Measured on 8 GPUs in the engine with 4 CTAs per row: the push takes 1.85 instead of 2.95 us, the cluster barrier of the norm
  // costs 0.7 us, and the step is the same (1.700 vs 1.690 ms); so one CTA per row stays the default.
  int parts = 1;
  if (ll) {
    const int upr = hidden / 8;
    int want = c->knobs.ll_spread > 0 ? c->knobs.ll_spread : 1;
    if (c->local) want = std::min(want, std::max(1, maxchan));
    while (parts * 2 <= 8 && parts < want && upr % (parts * 2 * 32) == 0) parts *= 2;
    if (c->local) nchan = std::max(1, std::min(tokens, maxchan / parts));
  }
  const int per = hidden / 8 / parts;
  const int threads = ll ? std::min((per + 31) / 32 * 32, 512) : nt;
  const bool one_unit = ll && per <= threads;     // one 16-byte unit per thread where the part fits
  const __nv_bfloat16* g = static_cast<const __nv_bfloat16*>(gamma);
  if (c->local) {
    LocalPtrs p{};
    for (int r = 0; r < nr; r++) { p.in[r] = xs[r]; p.out[r] = ys[r]; p.aux[r] = residuals[r]; p.aux_out[r] = residual_outs[r]; }
    p.io = kInAligned | kOutAligned;
    p.mute = take_mute(c);
    const RankCtx* ctxs = c->ctxs_dev;
    int ntv = nt;
    void* args[] = {(void*)&ctxs, (void*)&p, (void*)&g, (void*)&tokens, (void*)&hidden, (void*)&eps, (void*)&ntv};
    void* fn = !ll ? (void*)k_ar_rmsnorm_local : (one_unit ? (void*)k_ar_rmsnorm_ll_local<1> : (void*)k_ar_rmsnorm_ll_local<2>);
    // cooperative: the emulated ranks wait for one another, so every CTA has to be resident
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(nchan, c->world, parts);
    cfg.blockDim = dim3(threads);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = unsigned(parts);
    cfg.attrs = attr;
    cfg.numAttrs = parts > 1 ? 2 : 1;
    e = cudaLaunchKernelExC(&cfg, fn, args);
  } else if (c->world == 1) {
    return TBV_FALLBACK;  // nothing to reduce: the caller uses the plain fused add+norm op
  } else if (ll) {
    auto kern = one_unit ? k_ar_rmsnorm_ll<1> : k_ar_rmsnorm_ll<2>;
    e = pdl::launch(kern, dim3(nchan, 1, parts), dim3(threads), 0, st, parts, c->ranks[0].ctx,
                    static_cast<const __nv_bfloat16*>(xs[0]), static_cast<const __nv_bfloat16*>(residuals[0]), g,
                    static_cast<__nv_bfloat16*>(residual_outs[0]), static_cast<__nv_bfloat16*>(ys[0]), tokens, hidden, eps, nt);
  } else {
    e = pdl::launch(k_ar_rmsnorm, dim3(nchan), dim3(threads), 0, st, 1, c->ranks[0].ctx,
                    static_cast<const __nv_bfloat16*>(xs[0]), static_cast<const __nv_bfloat16*>(residuals[0]), g,
                    static_cast<__nv_bfloat16*>(residual_outs[0]), static_cast<__nv_bfloat16*>(ys[0]), tokens, hidden, eps);
  }
  if (e != cudaSuccess) {
    c->errmsg = std::string("kernel launch: ") + cudaGetErrorString(e);
    LOG("%s", c->errmsg.c_str());
    c->sticky_err.store(1);
    return TBV_FAIL;
  }
  c->host_seq++;
  if (!c->knobs.async) {
    if (cudaStreamSynchronize(st) != cudaSuccess) { c->sticky_err.store(1); return TBV_FAIL; }
    if (check_err(c)) return TBV_FAIL;
  }
  c->stats.add_enq(now_us() - t0);
  return TBV_OK;
}

// ---- C ABI: explicit communicator ---------------------------------------------------------------
extern "C" {

int tbv_comm_create(tbv_comm** out, int rank, int world, int device, const char* peer_ip, int port, size_t cap_bytes) {
  if (!out || world < 1 || world > TBV_MAXRANK || rank < 0 || rank >= world) return TBV_FAIL;
  std::unique_ptr<tbv_comm> c(new tbv_comm);
  c->rank = rank;
  c->world = world;
  c->device = device;
  c->knobs = Knobs::from_env();
  long cap_env = env_long("TBV_CAP", 0);
  if (cap_env > 0) cap_bytes = size_t(cap_env);
  c->cap = (cap_bytes + 4095) & ~size_t(4095);  // reference rounds to 4 KiB too (libtbvcoll.cpp:281)
  if (c->cap == 0) c->cap = 4096;
  if (c->bs.init(rank, world, peer_ip, port, c->knobs.init_timeout_s) != 0) {
    LOG("rank %d: bootstrap failed: %s", rank, c->bs.error().c_str());
    return TBV_FAIL;
  }
  int rc;
  if (device < 0) {
    c->cpu.reset(new CpuBackend(rank, world, c->cap, c->knobs.nslot, c->knobs.async != 0, c->knobs.wdog_s, c->knobs.cpu, &c->stats));
    rc = c->cpu->init(&c->bs, port);
    if (rc != 0) LOG("rank %d: cpu backend init failed: %s", rank, c->cpu->error().c_str());
  } else {
    rc = gpu_init(c.get());
  }
  // final agreement: either everybody is up or everybody fails
  int ok = (rc == 0);
  std::vector<int> oks(world);
  if (c->bs.allgather(&ok, oks.data(), sizeof(int)) != 0) return TBV_FAIL;
  for (int v : oks)
    if (!v) return TBV_FAIL;
  banner(c.get());
  *out = c.release();
  return TBV_OK;
}

int tbv_comm_create_local(tbv_comm** out, int world, int device, size_t cap_bytes) {
  if (!out || world < 1 || world > TBV_MAXRANK || device < 0) return TBV_FAIL;
  std::unique_ptr<tbv_comm> c(new tbv_comm);
  c->rank = 0;
  c->world = world;
  c->device = device;
  c->local = true;
  c->knobs = Knobs::from_env();
  c->cap = (cap_bytes + 4095) & ~size_t(4095);
  if (gpu_init_local(c.get()) != TBV_OK) return TBV_FAIL;
  banner(c.get());
  *out = c.release();
  return TBV_OK;
}

int tbv_comm_destroy(tbv_comm* c) {
  if (!c) return TBV_OK;
  if (c->device >= 0) {
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    // Peers must stop touching my memory before it goes away (and all ranks must leave a
    // multicast object together).
    if (!c->local && c->world > 1) c->bs.barrier();
    const Drv& d = drv();
    if (c->nvls) {
      d.MemUnmap(CUdeviceptr(c->mc_base), c->mc_bytes);
      d.MemAddressFree(CUdeviceptr(c->mc_base), c->mc_bytes);
      d.MulticastUnbind(c->mc_handle, c->device, 0, c->mc_bytes);
      d.MemRelease(c->mc_handle);
    }
    if (c->vmm) {
      for (int p = 0; p < c->world; p++) {
        if (c->peer_maps[p]) {
          d.MemUnmap(CUdeviceptr(c->peer_maps[p]), c->ranks[0].alloc_bytes);
          d.MemAddressFree(CUdeviceptr(c->peer_maps[p]), c->ranks[0].alloc_bytes);
        }
        if (c->vmm_handles[p]) d.MemRelease(c->vmm_handles[p]);
      }
    } else if (!c->local) {
      for (int p = 0; p < c->world; p++)
        if (p != c->rank && p < int(c->peer_maps.size()) && c->peer_maps[p]) cudaIpcCloseMemHandle(c->peer_maps[p]);
      if (!c->ranks.empty() && c->ranks[0].base) {
        if (c->world > 1) c->bs.barrier();  // peers have closed their mappings
        cudaFree(c->ranks[0].base);
      }
    }
    for (auto& g : c->ranks) {
      if (c->local && g.base) cudaFree(g.base);
      if (g.st) cudaFree(g.st);
      if (g.dm) cudaFree(g.dm);
      if (g.hm) cudaFreeHost(g.hm);
    }
    if (c->ctxs_dev) cudaFree(c->ctxs_dev);
    if (c->side_stream) cudaStreamDestroy(c->side_stream);
    for (auto& kv : c->gather_maps) cudaFree(kv.second);   // tensor maps over this communicator's slot memory die with it
    c->gather_maps.clear();
  }
  c->cpu.reset();
  c->bs.close_all();
  delete c;
  return TBV_OK;
}

int tbv_comm_allreduce(tbv_comm* c, const void* in, void* out, size_t nbytes, int dtype, void* stream) {
  if (!c) return TBV_FAIL;
  if (!in && nbytes) return TBV_FALLBACK;  // not a materialised tensor (e.g. a tracing placeholder): never launch on it
  if (!out) out = const_cast<void*>(in);
  if (c->cpu) {
    const double t0 = now_us();
    if (dtype < 0 || dtype > 2) return TBV_FALLBACK;
    if (nbytes == 0) return TBV_OK;
    if (c->skip.load() > 0) { c->skip.fetch_sub(1); return TBV_OK; }
    int rc = c->world == 1 ? (out != in ? (memcpy(out, in, nbytes), TBV_OK) : TBV_OK) : c->cpu->submit(in, out, nbytes, dtype, kOpAllReduce);
    if (rc == TBV_FALLBACK) c->stats.fallbacks++;
    c->stats.add_enq(now_us() - t0);
    return rc;
  }
  if (c->local) return TBV_FAIL;
  return gpu_collective(c, &in, &out, nbytes, dtype, stream, 0);
}

int tbv_comm_allreduce_local(tbv_comm* c, const void* const* ins, void* const* outs, size_t nbytes, int dtype, void* stream) {
  if (!c || !c->local) return TBV_FAIL;
  return gpu_collective(c, ins, outs, nbytes, dtype, stream, 0);
}

int tbv_comm_allreduce_rmsnorm(tbv_comm* c, const void* x, const void* residual, const void* gamma, void* residual_out,
                               void* y, int tokens, int hidden, float eps, void* stream) {
  if (!c) return TBV_FAIL;
  if (c->cpu || c->local) return TBV_FALLBACK;
  return gpu_ar_rmsnorm(c, &x, &residual, gamma, &residual_out, &y, tokens, hidden, eps, stream);
}

int tbv_comm_allreduce_rmsnorm_local(tbv_comm* c, const void* const* xs, const void* const* residuals, const void* gamma,
                                     void* const* residual_outs, void* const* ys, int tokens, int hidden, float eps,
                                     void* stream) {
  if (!c || !c->local) return TBV_FAIL;
  return gpu_ar_rmsnorm(c, xs, residuals, gamma, residual_outs, ys, tokens, hidden, eps, stream);
}

int tbv_comm_reduce_scatter(tbv_comm* c, const void* in, void* out, size_t out_bytes, int dtype, void* stream) {
  if (!c) return TBV_FAIL;
  if (c->cpu) {
    if (out_bytes == 0) return TBV_OK;
    if (c->skip.load() > 0) { c->skip.fetch_sub(1); return TBV_OK; }
    if (c->world == 1) { if (out != in) memcpy(out, in, out_bytes); return TBV_OK; }
    return c->cpu->submit(in, out, out_bytes, dtype, kOpReduceScatter);
  }
  if (c->local) return TBV_FAIL;
  return gpu_collective(c, &in, &out, out_bytes, dtype, stream, 1);
}

int tbv_comm_all_gather(tbv_comm* c, const void* in, void* out, size_t in_bytes, void* stream) {
  if (!c) return TBV_FAIL;
  if (c->cpu) {
    if (in_bytes == 0) return TBV_OK;
    if (c->skip.load() > 0) { c->skip.fetch_sub(1); return TBV_OK; }
    if (c->world == 1) { if (out != in) memcpy(out, in, in_bytes); return TBV_OK; }
    return c->cpu->submit(in, out, in_bytes, TBV_BF16, kOpAllGather);
  }
  if (c->local) return TBV_FAIL;
  return gpu_collective(c, &in, &out, in_bytes, TBV_BF16, stream, 2);
}

int tbv_comm_sync(tbv_comm* c) {
  if (!c) return TBV_FAIL;
  if (c->cpu) return c->cpu->sync();
  return check_err(c) ? TBV_FAIL : TBV_OK;
}

int tbv_comm_rank(tbv_comm* c) { return c ? c->rank : -1; }
int tbv_comm_world(tbv_comm* c) { return c ? c->world : 0; }
size_t tbv_comm_cap(tbv_comm* c) { return c ? c->cap : 0; }
int tbv_comm_nslot(tbv_comm* c) { return c ? c->knobs.nslot : 0; }
int tbv_comm_is_async(tbv_comm* c) { return c ? c->knobs.async : 0; }
int tbv_comm_err(tbv_comm* c) { return c ? int(check_err(c)) : 1; }
int tbv_comm_has_nvls(tbv_comm* c) { return c ? int(c->nvls) : 0; }
// 1 if this library was compiled with the device-side bounds guards (-DTBV_BOUNDS_CHECK)
int tbv_bounds_checked_build(void) {
#ifdef TBV_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}
// Sequence stamps (TBV_TAG=1) compared and found wrong since the communicator was created, summed over (emulated) ranks.
int tbv_comm_tag_counts(tbv_comm* c, unsigned long long* checked, unsigned long long* bad) {
  if (!c || c->cpu) return TBV_FAIL;
  unsigned long long b = 0, k = 0;
  for (auto& g : c->ranks) {
    unsigned long long v[2] = {0, 0};
    if (!g.dm || cudaMemcpy(v, &g.dm->tag_bad, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return TBV_FAIL;
    b += v[0]; k += v[1];
  }
  if (checked) *checked = k;
  if (bad) *bad = b;
  return TBV_OK;
}
int tbv_comm_set_algo(tbv_comm* c, int algo) {
  if (!c || algo < 0 || algo > 5) return TBV_FAIL;
  c->knobs.algo = algo;
  return TBV_OK;
}
int tbv_comm_set_nchan(tbv_comm* c, int nchan) {
  if (!c || nchan < 0 || nchan > TBV_MAXCHAN) return TBV_FAIL;
  c->knobs.nchan = nchan;
  return TBV_OK;
}
int tbv_comm_set_wdog(tbv_comm* c, double seconds) {
  if (!c || seconds <= 0) return TBV_FAIL;
  c->knobs.wdog_s = seconds;
  if (c->cpu) c->cpu->set_wdog(seconds);
  for (auto& g : c->ranks) g.ctx.wdog_ns = (unsigned long long)(seconds * 1e9);
  if (c->ctxs_dev) {
    std::vector<RankCtx> host(c->ranks.size());
    for (size_t r = 0; r < c->ranks.size(); r++) host[r] = c->ranks[r].ctx;
    cudaMemcpy(c->ctxs_dev, host.data(), sizeof(RankCtx) * host.size(), cudaMemcpyHostToDevice);
  }
  return TBV_OK;
}
int tbv_comm_skip_next(tbv_comm* c, int n) {
  if (!c) return TBV_FAIL;
  c->skip.store(n);
  return TBV_OK;
}
// Emulated world only, host-side fault injection: for the next n collective launches the CTAs of
// emulated rank r return before they push anything, like a rank that never makes the call.  The other
// ranks' bounded waits run out and report it; nothing faults.
int tbv_comm_mute_rank(tbv_comm* c, int r, int n) {
  if (!c || !c->local || r < 0 || r >= c->world || n < 0) return TBV_FAIL;
  c->mute_rank = r;
  c->mute_left.store(n);
  return TBV_OK;
}
int tbv_comm_ctx(tbv_comm* c, void* ctx_out, size_t ctx_bytes) {
  if (!c || c->cpu || c->ranks.empty() || ctx_bytes < sizeof(RankCtx)) return TBV_FAIL;
  memcpy(ctx_out, &c->ranks[0].ctx, sizeof(RankCtx));
  return TBV_OK;
}
void tbv_comm_stats5(tbv_comm* c, double* pre, double* xfer, double* post, double* enq, double* drain, unsigned long long* n) {
  if (!c) return;
  harvest_trace(c);
  c->stats.read5(pre, xfer, post, enq, drain, n);
}
void tbv_comm_rails(tbv_comm* c) {
  if (!c) return;
  harvest_trace(c);
  if (!c->cpu && !c->ranks.empty() && c->ranks[0].dm) {
    // per-peer flag-wait times accumulated on the device (channel 0); read and reset
    unsigned long long buf[2 * TBV_MAXRANK] = {0};
    DevMirror* dm = c->ranks[0].dm;
    if (cudaMemcpy(buf, dm->peer_wait_ns, sizeof(buf), cudaMemcpyDeviceToHost) == cudaSuccess) {
      std::lock_guard<std::mutex> g(c->stats.mu);
      for (int p = 0; p < c->world; p++) { c->stats.peer_wait_us[p] += buf[p] * 1e-3; c->stats.peer_n[p] += buf[TBV_MAXRANK + p]; }
      cudaMemset(dm->peer_wait_ns, 0, sizeof(buf));
    }
  }
  c->stats.dump_rails(c->rank, c->world);
}
void tbv_comm_hist(tbv_comm* c) {
  if (!c) return;
  harvest_trace(c);
  unsigned long long bad = 0, checked = 0;
  for (auto& g : c->ranks) {
    unsigned long long v[2] = {0, 0};   // tag_bad, tag_checked are adjacent in DevMirror
    if (g.dm && cudaMemcpy(v, &g.dm->tag_bad, sizeof(v), cudaMemcpyDeviceToHost) == cudaSuccess) { bad += v[0]; checked += v[1]; }
  }
  c->stats.dump_hist(c->rank, bad, checked);
}
// Device breadcrumbs of (emulated) rank r: bc[0..3] = sequence numbers at enter / pushed /
// wait-pass / done; bc[4..7] = %globaltimer stamps of the last fused GEMM call (accumulator
// ready, flag published, all tiles arrived, kernel entry).  Synchronous copy.
int tbv_comm_breadcrumbs(tbv_comm* c, int r, unsigned long long out[8]) {
  if (!c || c->cpu || r < 0 || r >= int(c->ranks.size())) return TBV_FAIL;
  return cudaMemcpy(out, c->ranks[r].dm->bc, 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) == cudaSuccess ? TBV_OK : TBV_FAIL;
}
// The timing ring of (emulated) rank r as rows of five numbers: sequence number, then %globaltimer stamps (ns)
// of channel 0 / thread 0 at kernel entry, own payload issued, every source's payload seen, kernel done.  Only
// completed calls that are still in the ring are returned, oldest first, at most `max_rows`; returns the row
// count or TBV_FAIL.  A stamp a kernel does not take reads 0.  Synchronous copy; nothing is reset.
int tbv_comm_trace(tbv_comm* c, int r, unsigned long long* out, int max_rows) {
  if (!c || c->cpu || r < 0 || r >= int(c->ranks.size()) || !out || max_rows < 0) return TBV_FAIL;
  std::vector<TraceRec> ring(kTraceN);
  DevState ds;
  if (cudaMemcpy(&ds, c->ranks[r].st, sizeof(ds), cudaMemcpyDeviceToHost) != cudaSuccess) return TBV_FAIL;
  if (cudaMemcpy(ring.data(), c->ranks[r].dm->ring, sizeof(TraceRec) * kTraceN, cudaMemcpyDeviceToHost) != cudaSuccess) return TBV_FAIL;
  const unsigned long long upto = ds.seq;
  unsigned long long from = upto > kTraceN ? upto - kTraceN + 1 : 1;
  if (upto - from + 1 > (unsigned long long)max_rows) from = upto - max_rows + 1;
  int n = 0;
  for (unsigned long long s = from; s <= upto; s++) {
    const TraceRec& t = ring[s & (kTraceN - 1)];
    if (t.seq != s) continue;
    unsigned long long* row = out + size_t(n++) * 5;
    row[0] = s;
    row[1] = t.t_enter;
    row[2] = (t.t_pushed >= t.t_enter && t.t_pushed <= t.t_done) ? t.t_pushed : 0;   // a stale stamp of an older call does not fall inside this one
    row[3] = t.t_ready;
    row[4] = t.t_done;
  }
  return n;
}
// %globaltimer stamps (ns) of the last fused GEMM + all-reduce + norm call on (emulated) rank r:
// [0] = [1] the first tile's CTA is resident, [2] the first finisher starts (all but the last few of this rank's CTAs have
// pushed their tile), [3] its first row's packets of all ranks are pulled, [4] its rows are normalised, [5] the last tile's
// CTA (in launch order) is resident, [6] its accumulator is complete, [7] its packets are issued.  Synchronous copy.
int tbv_comm_timestamps(tbv_comm* c, int r, unsigned long long out[8]) {
  if (!c || c->cpu || r < 0 || r >= int(c->ranks.size())) return TBV_FAIL;
  return cudaMemcpy(out, c->ranks[r].dm->ts, 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) == cudaSuccess ? TBV_OK : TBV_FAIL;
}
void tbv_comm_last_error(tbv_comm* c, unsigned long long out[4]) {
  out[0] = out[1] = out[2] = out[3] = 0;
  if (!c) return;
  if (c->cpu) { c->cpu->last_error(out); return; }
  for (auto& g : c->ranks) {
    if (g.hm && g.hm->err) {
      out[0] = g.hm->err; out[1] = g.hm->err_seq; out[2] = g.hm->where; out[3] = g.hm->peer;
      return;
    }
  }
}

// ---- C ABI: process-global communicator with the reference's names -------------------------------
static tbv_comm* g_comm = nullptr;
static std::mutex g_mu;

tbv_comm* tbv_ar_comm(void) { return g_comm; }

int tbv_ar_init_n(int rank, int world, int device, const char* peer_ip, int port, size_t cap) {
  std::lock_guard<std::mutex> g(g_mu);
  if (g_comm) return TBV_OK;  // idempotent (reference: libtbvcoll.cpp:280)
  return tbv_comm_create(&g_comm, rank, world, device, peer_ip, port, cap);
}

int tbv_ar_init(int rank, const char* devs, const char* peer_ip, int port, size_t cap) {
  int world = int(env_long("TBV_WORLD", 2));
  int device = 0;
  if (devs && !strncmp(devs, "cpu", 3)) {
    device = -1;
  } else if (devs && !strncmp(devs, "cuda:", 5)) {
    device = atoi(devs + 5);
  } else if (devs && *devs && strspn(devs, "0123456789") == strlen(devs)) {
    device = atoi(devs);
  } else {
    if (cudaGetDevice(&device) != cudaSuccess) return TBV_FAIL;
  }
  return tbv_ar_init_n(rank, world, device, peer_ip, port, cap);
}

int tbv_ar_allreduce(const void* in, void* out, size_t nbytes, int dtype, void* stream) {
  if (!g_comm) { LOG("not initialised"); return TBV_FAIL; }
  return tbv_comm_allreduce(g_comm, in, out, nbytes, dtype, stream);
}
void tbv_ar_stats(double* xfer_us, unsigned long long* n) { tbv_comm_stats5(g_comm, nullptr, xfer_us, nullptr, nullptr, nullptr, n); }
void tbv_ar_stats4(double* pre, double* xfer, double* post, double* enq, unsigned long long* n) {
  tbv_comm_stats5(g_comm, pre, xfer, post, enq, nullptr, n);
}
void tbv_ar_stats5(double* pre, double* xfer, double* post, double* enq, double* drain, unsigned long long* n) {
  tbv_comm_stats5(g_comm, pre, xfer, post, enq, drain, n);
}
int tbv_ar_cap(void) { return g_comm ? int(std::min<size_t>(g_comm->cap, size_t(INT_MAX))) : 0; }
size_t tbv_ar_cap64(void) { return g_comm ? g_comm->cap : 0; }
int tbv_ar_async(void) { return g_comm ? g_comm->knobs.async : 0; }
int tbv_ar_err(void) { return g_comm ? tbv_comm_err(g_comm) : 0; }
void tbv_ar_rails(void) { tbv_comm_rails(g_comm); }
void tbv_ar_hist(void) { tbv_comm_hist(g_comm); }
int tbv_ar_sync(void) { return g_comm ? tbv_comm_sync(g_comm) : TBV_FAIL; }
int tbv_ar_fini(void) {
  std::lock_guard<std::mutex> g(g_mu);
  int rc = tbv_comm_destroy(g_comm);
  g_comm = nullptr;
  return rc;
}

}  // extern "C"
