// ar_device.cuh — device side of the collective library (sm_100a).
//
// One stream-ordered kernel per collective.  A rank pushes its data into its
// peers' slot memory with plain 16-byte stores over NVLink, publishes a per-channel
// sequence flag with system-scope release semantics, waits (bounded) for the same
// flag from every peer, and reduces the N copies in rank order 0..N-1 in fp32 with
// one final rounding, so every rank produces identical bits.
//
// This replaces, in one launch, the reference's k_copy_sig + RDMA write + stream
// wait-value + k_acc sequence (step4/libtbvcoll.cpp:126-166, 181-204, 456-503) and
// its diagnostic kernels k_waitflag / k_tagchk / k_mark (:143-161): the wait, the
// tag check and the breadcrumbs live inside the collective kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tbvcoll.h"

namespace tbv {

constexpr int kTraceN = 1024;  // per-call timing ring entries (power of two)

// Device-resident per-rank state.  The sequence number lives here (not in launch
// parameters) so that a captured CUDA graph replays correctly.
struct DevState {
  unsigned long long seq;   // last completed collective on this rank
  unsigned int arrive;      // CTA completion counter of the running kernel
  unsigned int err;         // sticky: first device-side error code
  unsigned int tag_bad;     // seq-stamp mismatches seen (debug mode)
  unsigned int gemm_done;   // fused GEMM + all-reduce: GEMM CTAs of the running call that have pushed their tile
};

struct TraceRec {
  unsigned long long seq, t_enter, t_ready, t_done;
  unsigned long long nbytes;
  unsigned int algo, nchan;
  unsigned long long t_pushed;  // channel 0, thread 0: its own packets / payload stores have been issued (0 where a kernel does not stamp it)
};

// Device-resident diagnostics written on every call: breadcrumbs and the timing ring.  They
// live in device memory on purpose: a store to host memory ahead of a system-scope fence
// would put a PCIe round trip on the critical path of every collective.  The host copies
// them out in the statistics getters; on a watchdog expiry the kernel copies the breadcrumbs
// into the host-mapped record below.
struct DevMirror {
  unsigned long long bc[8];  // breadcrumbs: 0 enter, 1 pushed, 2 wait-pass, 3 done (seq values)
  unsigned long long tag_bad;      // sequence stamps that did not match after their flag had been seen (TBV_TAG=1)
  unsigned long long tag_checked;  // sequence stamps compared
  unsigned long long ts[8];        // %globaltimer stamps of the last fused GEMM + all-reduce call (see tbv_comm_timestamps)
  unsigned long long peer_wait_ns[TBV_MAXRANK];  // channel 0: time spent waiting for each source rank's flag
  unsigned long long peer_n[TBV_MAXRANK];
  TraceRec ring[kTraceN];
};

// Host-mapped error record, written only when a wait gives up; the host reads it without a sync.
struct HostMirror {
  unsigned int err;       // same code as DevState::err
  unsigned int where;     // wait site that gave up (kWhere*)
  unsigned int peer;      // rank that did not arrive
  unsigned int chan;
  unsigned long long err_seq;
  unsigned long long bc[8];  // copy of the breadcrumbs at the time of the error
  unsigned long long tag_bad;
};

enum : unsigned { kErrNone = 0, kErrTimeout = 1, kErrTag = 2, kErrBounds = 3 };
enum : int { kWholeCall = 0, kPushHalf = 1, kReduceHalf = 2 };   // a one-shot call as one kernel, or split around stream wait-value operations
enum : unsigned { kWherePhase0 = 1, kWherePhase1 = 2, kWhereFused = 3, kWhereStreamWait = 4,
                  kGuardSlotBytes = 16, kGuardLLBytes = 17, kGuardChannels = 18 };   // sites of the bounds-checked build

// Everything a kernel needs to talk to the other ranks; passed by value.
struct RankCtx {
  int rank, world, nslot, debug_tag;
  int ll_wide;                     // LL packets move as one 32-byte store / load per unit instead of two 16-byte ones
  unsigned long long cap;          // bytes per (slot, source-rank) region
  unsigned long long slot_stride;  // bytes per slot = (world + 1) * cap
  unsigned long long wdog_ns;      // bound on every device-side wait
  unsigned long long guard_cap, guard_ll_cap;  // what the bounds-checked build compares extents with (= cap, ll_cap)
  char* data[TBV_MAXRANK];         // data[p]: rank p's slot memory as mapped here
  unsigned int* flags[TBV_MAXRANK];
  char* ll[TBV_MAXRANK];           // ll[p]: rank p's LL packet area (only ever holds LL packets)
  unsigned long long ll_cap;       // bytes per (slot, source-rank) LL region
  unsigned long long* tags[TBV_MAXRANK];  // tags[p]: rank p's sequence-stamp area, one word per flag, outside the payload regions
  char* mc_data;                   // multicast (NVLS) mapping of the slot memory, or null
  DevState* st;
  DevMirror* dm;
  HostMirror* hm;
};

__device__ __forceinline__ size_t flag_index(const RankCtx& c, int slot, int phase, int src,
                                             int chan) {
  return ((size_t(slot) * 2 + phase) * c.world + src) * TBV_MAXCHAN + chan;
}
__device__ __forceinline__ char* slot_region(const RankCtx& c, int peer, int slot, int region) {
  return c.data[peer] + size_t(slot) * c.slot_stride + size_t(region) * c.cap;
}

// LL packets live in an area of their own: a region that only ever holds (payload, sequence)
// packets can never show a stale word that equals a future sequence number.
__device__ __forceinline__ char* ll_region(const RankCtx& c, int peer, int slot, int src) {
  return c.ll[peer] + (size_t(slot) * c.world + src) * c.ll_cap;
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(unsigned* p, unsigned v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}
__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__device__ __forceinline__ void report_error(const RankCtx& c, unsigned code, unsigned where,
                                             int peer, int chan, unsigned long long seq) {
  if (atomicCAS(&c.st->err, 0u, code) == 0u) {
    for (int i = 0; i < 8; i++) c.hm->bc[i] = c.dm->bc[i];
    c.hm->where = where;
    c.hm->peer = unsigned(peer);
    c.hm->chan = unsigned(chan);
    c.hm->err_seq = seq;
    __threadfence_system();
    c.hm->err = code;
    __threadfence_system();
  }
}

// Bounded wait for `*f` to reach `want` (wrap-safe).  A few thousand fast polls,
// then timed polls with a short sleep.  On expiry: record the error and return
// false; the caller carries on so that the kernel always terminates.
__device__ __forceinline__ bool wait_flag(const RankCtx& c, const unsigned* f, unsigned want,
                                          unsigned where, int peer, int chan,
                                          unsigned long long seq) {
  unsigned spins = 0;
  unsigned long long t0 = 0;
  while (int(ld_acquire_sys(f) - want) < 0) {
    if (++spins > 4096u) {
      unsigned long long now = globaltimer();
      if (t0 == 0) {
        t0 = now;
        // A sticky error from an earlier call means the peer is gone: do not
        // spend the whole watchdog period again.
        if (*(volatile unsigned*)&c.st->err != 0u) return false;
      } else if (now - t0 > c.wdog_ns) {
        report_error(c, kErrTimeout, where, peer, chan, seq);
        return false;
      }
      __nanosleep(128);
    }
  }
  return true;
}

// ---- bounds-checked build (-DTBV_BOUNDS_CHECK) -------------------------------------------------
// compute-sanitizer's job, done by hand where it is not available: before a collective body touches
// slot or packet memory it compares the extent it is about to use (and its channel count) with what
// the communicator reserved.  A violation is RECORDED (sticky error kErrBounds, the site, the
// offending value in place of the sequence number) and the body then moves no data at all — it still
// raises its flags, so no peer is left waiting.  Compiled out of the normal build.
#ifdef TBV_BOUNDS_CHECK
__device__ __forceinline__ bool guard_extent(const RankCtx& c, unsigned long long need, unsigned long long have, unsigned site,
                                             int chan) {
  if (need <= have) return true;
  report_error(c, kErrBounds, site, 0, chan, need);
  return false;
}
#define TBV_GUARD(c, need, have, site, chan) guard_extent(c, (unsigned long long)(need), (unsigned long long)(have), site, chan)
#else
#define TBV_GUARD(c, need, have, site, chan) (true)
#endif

// ---- element packs ---------------------------------------------------------------
template <typename T> struct Pack;  // 16 bytes of T <-> fp32 lanes
template <> struct Pack<float> {
  static constexpr int N = 4;
  __device__ static void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  __device__ static uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
  }
  __device__ static float to_f(float x) { return x; }
  __device__ static float from_f(float x) { return x; }
};
template <> struct Pack<__half> {
  static constexpr int N = 8;
  __device__ static void unpack(const uint4& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; i++) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  }
  __device__ static uint4 pack(const float* f) {
    uint4 v; __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return v;
  }
  __device__ static float to_f(__half x) { return __half2float(x); }
  __device__ static __half from_f(float x) { return __float2half_rn(x); }
};
template <> struct Pack<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void unpack(const uint4& v, float* f) {
    // bf16 -> fp32 is a 16-bit shift
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
  }
  __device__ static uint4 pack(const float* f) {
    uint4 v; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
  }
  __device__ static float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ static __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};

// ---- per-kernel prologue / epilogue ------------------------------------------------
struct CallInfo {
  unsigned long long seq;
  unsigned want;  // low 32 bits of seq: the flag value of this call
  int slot;
};

// Every CTA reads the device sequence; the kernel that ran before this one on the
// stream left it at "last completed".
__device__ __forceinline__ CallInfo call_begin(const RankCtx& c, unsigned long long* sh_seq) {
  if (threadIdx.x == 0) *sh_seq = *(volatile unsigned long long*)&c.st->seq + 1ull;
  __syncthreads();
  CallInfo ci;
  ci.seq = *sh_seq;
  ci.want = unsigned(ci.seq);
  ci.slot = int(ci.seq % (unsigned long long)c.nslot);
  return ci;
}

// Last CTA to finish publishes the new sequence and the timing record.
__device__ __forceinline__ void call_end(const RankCtx& c, const CallInfo& ci, unsigned nctas,
                                         unsigned long long t_enter, unsigned long long t_ready,
                                         unsigned long long nbytes, unsigned algo) {
  __syncthreads();
  if (threadIdx.x == 0) {
    TraceRec* r = &c.dm->ring[ci.seq & (kTraceN - 1)];
    if (t_enter) { r->t_enter = t_enter; r->nbytes = nbytes; r->algo = algo; r->nchan = nctas; }
    if (t_ready) r->t_ready = t_ready;
    // No fence: the next kernel on the stream starts after this grid has completed (or, with
    // programmatic dependent launch, passes its dependency wait only then), which orders
    // everything written here before it.
    unsigned old = atomicAdd(&c.st->arrive, 1u);
    if (old == nctas - 1) {
      c.st->arrive = 0;
      c.st->gemm_done = 0;   // the next call's GEMM CTAs push only after this grid has completed
      r->t_done = globaltimer();
      r->seq = ci.seq;
      c.dm->bc[3] = ci.seq;
      *(volatile unsigned long long*)&c.st->seq = ci.seq;
    }
  }
}

// ---- 16-byte units of a caller's tensor ---------------------------------------------------------
// Channel ranges and the choice of kernel depend on the byte count only, never on where a
// rank's tensor happens to sit, so every rank launches the same protocol.  A tensor that is
// not 16-byte aligned is read and written element by element; slot memory is always aligned.
template <typename T>
__device__ __forceinline__ uint4 ld_unit(const T* p, size_t u, bool aligned) {
  if (aligned) return reinterpret_cast<const uint4*>(p)[u];
  constexpr int N = 16 / sizeof(T);
  union { uint4 v; T e[N]; } x;
#pragma unroll
  for (int i = 0; i < N; i++) x.e[i] = p[u * N + i];
  return x.v;
}
template <typename T>
__device__ __forceinline__ void st_unit(T* p, size_t u, const uint4& v, bool aligned) {
  if (aligned) { reinterpret_cast<uint4*>(p)[u] = v; return; }
  constexpr int N = 16 / sizeof(T);
  union { uint4 v; T e[N]; } x;
  x.v = v;
#pragma unroll
  for (int i = 0; i < N; i++) p[u * N + i] = x.e[i];
}
enum : int { kInAligned = 1, kOutAligned = 2 };

// publish: all threads' stores are done (caller did __syncthreads); thread 0 fences
// at system scope once and then stores the flag to every peer.  With the sequence-stamp
// diagnostic on (TBV_TAG=1) the same thread first writes the call's sequence number into
// the peer's stamp word of this (slot, phase, source, channel): a plain store issued after
// the payload and before the fence, so a receiver that sees the flag must also see the
// stamp.  The stamp has a word of its own next to the flags and never overlaps a payload.
// (The reference carried the stamp behind the payload in a widened slot stride,
// step4/libtbvcoll.cpp:88-91,296-297, and compared it in k_tagchk, :143-150.)
__device__ __forceinline__ void publish(const RankCtx& c, const CallInfo& ci, int phase, int chan) {
  if (threadIdx.x == 0) {
    if (c.debug_tag) {
      for (int p = 0; p < c.world; p++)
        if (p != c.rank) *(volatile unsigned long long*)(c.tags[p] + flag_index(c, ci.slot, phase, c.rank, chan)) = ci.seq;
    }
    fence_sys();
    for (int p = 0; p < c.world; p++) {
      if (p == c.rank) continue;
      st_relaxed_sys(c.flags[p] + flag_index(c, ci.slot, phase, c.rank, chan), ci.want);
    }
  }
}
// threads 0..world-1 each wait for one source rank; then the CTA synchronises.
__device__ __forceinline__ void wait_all(const RankCtx& c, const CallInfo& ci, int phase, int chan,
                                         unsigned where) {
  if (threadIdx.x < unsigned(c.world) && int(threadIdx.x) != c.rank) {
    const unsigned long long t0 = chan == 0 ? globaltimer() : 0;
    const bool ok = wait_flag(c, c.flags[c.rank] + flag_index(c, ci.slot, phase, threadIdx.x, chan), ci.want,
                              where, threadIdx.x, chan, ci.seq);
    if (chan == 0) {  // arrival skew per peer, for the `rails` dump (one writer per entry: no atomics needed)
      c.dm->peer_wait_ns[threadIdx.x] += globaltimer() - t0;
      c.dm->peer_n[threadIdx.x] += 1;
    }
    if (c.debug_tag && ok) {
      const unsigned long long tag = *(volatile unsigned long long*)(c.tags[c.rank] + flag_index(c, ci.slot, phase, threadIdx.x, chan));
      atomicAdd(&c.dm->tag_checked, 1ull);
      if (tag != ci.seq) { atomicAdd(&c.st->tag_bad, 1u); atomicAdd(&c.dm->tag_bad, 1ull); }
    }
  }
  __syncthreads();
}

// Unit `idx` of the regions that the source ranks in `mask` own in `owner`'s slot memory: every load is issued
// before any value is used (fully unrolled, constant indices), so a reduce step pays one memory round trip and
// not one per source rank.  The sum itself stays in rank order (sum_units_rank_order).
__device__ __forceinline__ void gather_units(const RankCtx& c, int owner, int slot, size_t idx, unsigned mask,
                                             uint4 (&got)[TBV_MAXRANK]) {
#pragma unroll
  for (int r = 0; r < TBV_MAXRANK; r++)
    if ((mask >> r) & 1u) got[r] = ld_volatile_v4(reinterpret_cast<const uint4*>(slot_region(c, owner, slot, r)) + idx);
}
// rank-ordered fp32 sum of one unit: `mine` stands in for every rank below the world size whose bit is not set in `mask`
template <typename T>
__device__ __forceinline__ void sum_units_rank_order(const RankCtx& c, const uint4 (&got)[TBV_MAXRANK], unsigned mask,
                                                     const uint4& mine, float* acc) {
#pragma unroll
  for (int r = 0; r < TBV_MAXRANK; r++) {
    if (r < c.world) {
      const uint4 v = ((mask >> r) & 1u) ? got[r] : mine;
      float f[Pack<T>::N];
      Pack<T>::unpack(v, f);
#pragma unroll
      for (int i = 0; i < Pack<T>::N; i++) acc[i] = (r == 0) ? f[i] : acc[i] + f[i];
    }
  }
}

// ---- one-shot all-reduce ------------------------------------------------------------
// VEC: 16-byte units (nbytes % 16 == 0); otherwise one element per unit.  io: kInAligned /
// kOutAligned say whether the caller's tensors can be accessed 16 bytes at a time.
template <typename T, bool VEC>
__device__ void ar_oneshot_body(const RankCtx& c, const T* __restrict__ in, T* out, size_t nbytes,
                                int nchan, int chan, int io, unsigned long long* sh_seq, int part = kWholeCall) {
  unsigned long long t_enter = (threadIdx.x == 0 && chan == 0) ? globaltimer() : 0;
  CallInfo ci = call_begin(c, sh_seq);   // both halves of a split call read the same number: only call_end advances it
  const size_t unit_bytes = VEC ? 16 : sizeof(T);
  const size_t units = nbytes / unit_bytes;
  const size_t per = (units + nchan - 1) / nchan;
  const size_t u0 = per * chan;
  size_t u1 = (u0 + per < units) ? (u0 + per) : units;
  const bool in_al = io & kInAligned, out_al = io & kOutAligned;
  if (chan == 0 && threadIdx.x == 0) c.dm->bc[0] = ci.seq;
  if (!(TBV_GUARD(c, nbytes, c.guard_cap, kGuardSlotBytes, chan) && TBV_GUARD(c, nchan, TBV_MAXCHAN, kGuardChannels, chan)))
    u1 = u0;   // bounds-checked build: nothing is moved after a violation

  if (part != kReduceHalf) {
    // push my range to every peer's [slot][src = me] region
    for (size_t u = u0 + threadIdx.x; u < u1; u += blockDim.x) {
      if (VEC) {
        uint4 v = ld_unit(in, u, in_al);
        for (int p = 0; p < c.world; p++)
          if (p != c.rank) reinterpret_cast<uint4*>(slot_region(c, p, ci.slot, c.rank))[u] = v;
      } else {
        T v = in[u];
        for (int p = 0; p < c.world; p++)
          if (p != c.rank) reinterpret_cast<T*>(slot_region(c, p, ci.slot, c.rank))[u] = v;
      }
    }
    __syncthreads();
    publish(c, ci, 0, chan);
    if (chan == 0 && threadIdx.x == 0) { c.dm->bc[1] = ci.seq; c.dm->ring[ci.seq & (kTraceN - 1)].t_pushed = globaltimer(); }
    if (part == kPushHalf) {        // the stream waits for the peers' flags (wait-value operations), then the reduce half runs
      if (chan == 0 && threadIdx.x == 0) c.dm->ts[0] = t_enter;
      return;
    }
    wait_all(c, ci, 0, chan, kWherePhase0);
  } else if (chan == 0 && threadIdx.x == 0) {
    t_enter = c.dm->ts[0];
  }
  unsigned long long t_ready = (threadIdx.x == 0 && chan == 0) ? globaltimer() : 0;
  if (chan == 0 && threadIdx.x == 0) c.dm->bc[2] = ci.seq;

  // reduce in rank order, fp32, one rounding
  const unsigned peers = ((1u << c.world) - 1u) & ~(1u << c.rank);
  for (size_t u = u0 + threadIdx.x; u < u1; u += blockDim.x) {
    if (VEC) {
      float acc[Pack<T>::N];
#pragma unroll
      for (int i = 0; i < Pack<T>::N; i++) acc[i] = 0.f;
      uint4 mine = ld_unit(in, u, in_al);
      uint4 got[TBV_MAXRANK];
      gather_units(c, c.rank, ci.slot, u, peers, got);
      sum_units_rank_order<T>(c, got, peers, mine, acc);
      st_unit(out, u, Pack<T>::pack(acc), out_al);
    } else {
      float acc = 0.f;
      for (int r = 0; r < c.world; r++) {
        float f = (r == c.rank)
                      ? Pack<T>::to_f(in[u])
                      : Pack<T>::to_f(*(reinterpret_cast<volatile const T*>(slot_region(c, c.rank, ci.slot, r)) + u));
        acc = (r == 0) ? f : acc + f;
      }
      out[u] = Pack<T>::from_f(acc);
    }
  }
  call_end(c, ci, nchan, t_enter, t_ready, nbytes, TBV_ALGO_ONESHOT);
}

// ---- LL ("low latency") one-shot all-reduce ---------------------------------------------
// Every 8-byte store carries 4 bytes of payload and the 4-byte sequence number of the call, so
// the data announces itself: no fence, no separate flag, no second round trip.  The receiver
// polls the packet until both of its flags show this call's sequence number.  Costs twice the
// bytes, so it is used for small messages only (nbytes * 2 <= slot capacity and <= TBV_LL_MAX).
// 8-byte stores are single transactions on NVLink; a 16-byte store is two self-describing halves.
__device__ __forceinline__ void st_v4(void* p, unsigned a, unsigned b, unsigned c2, unsigned d) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(b), "r"(c2), "r"(d) : "memory");
}
// 256-bit forms (sm_100): one instruction and one fully written 32-byte sector per unit.  Nothing is
// assumed about their atomicity beyond 8 bytes: every 8-byte piece still carries its own flag.
__device__ __forceinline__ void st_v8(void* p, unsigned a, unsigned b, unsigned c2, unsigned d, unsigned e, unsigned f,
                                      unsigned g, unsigned h) {
  asm volatile("st.volatile.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(a), "r"(b), "r"(c2), "r"(d), "r"(e),
               "r"(f), "r"(g), "r"(h)
               : "memory");
}
__device__ __forceinline__ void ld_volatile_v8(const void* p, uint4& lo, uint4& hi) {
  asm volatile("ld.volatile.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
               : "l"(p)
               : "memory");
}
__device__ __forceinline__ void ll_load_unit(const RankCtx& c, const char* p, uint4& lo, uint4& hi) {
  if (c.ll_wide) {
    ld_volatile_v8(p, lo, hi);
  } else {
    lo = ld_volatile_v4(p);
    hi = ld_volatile_v4(p + 16);
  }
}
// push one 16-byte input unit `v` as two LL lines (32 bytes) at line index u of every peer's region
__device__ __forceinline__ void ll_push_unit(const RankCtx& c, int slot, size_t u, const uint4& v, unsigned want) {
  for (int d = 1; d < c.world; d++) {
    const int p = (c.rank + d) % c.world;
    char* dst = ll_region(c, p, slot, c.rank) + u * 32;
    if (c.ll_wide) {
      st_v8(dst, v.x, want, v.y, want, v.z, want, v.w, want);
    } else {
      st_v4(dst, v.x, want, v.y, want);
      st_v4(dst + 16, v.z, want, v.w, want);
    }
  }
}
// Pull unit u (two LL lines) of every source rank in `mask` from this rank's own LL area.  All
// the loads are issued before any flag is looked at, so a call pays one memory round trip once
// the packets have landed instead of one per source; only lines that have not arrived are read
// again.  Bounded like wait_flag: on expiry the error is recorded (naming the first silent
// source) and whatever is there is returned.  Every loop is fully unrolled with constant
// indices so that the lines stay in registers.
__device__ __forceinline__ void ll_pull_all(const RankCtx& c, int slot, size_t u, unsigned want, unsigned mask, int chan,
                                            unsigned long long seq, uint4 (&out)[TBV_MAXRANK]) {
  uint4 lo[TBV_MAXRANK], hi[TBV_MAXRANK];
  const char* base = c.ll[c.rank] + size_t(slot) * c.world * c.ll_cap + u * 32;
#pragma unroll
  for (int r = 0; r < TBV_MAXRANK; r++)
    if ((mask >> r) & 1u) ll_load_unit(c, base + size_t(r) * c.ll_cap, lo[r], hi[r]);
  unsigned pending = mask, spins = 0;
  unsigned long long t0 = 0;
  for (;;) {
    unsigned still = 0;
#pragma unroll
    for (int r = 0; r < TBV_MAXRANK; r++)
      if (((pending >> r) & 1u) && (lo[r].y != want || lo[r].w != want || hi[r].y != want || hi[r].w != want)) still |= 1u << r;
    if (!still) break;
    if (++spins > 4096u) {
      const unsigned long long now = globaltimer();
      if (t0 == 0) {
        t0 = now;
        if (*(volatile unsigned*)&c.st->err != 0u) break;
      } else if (now - t0 > c.wdog_ns) {
        report_error(c, kErrTimeout, kWherePhase0, __ffs(int(still)) - 1, chan, seq);
        break;
      }
      __nanosleep(64);
    }
#pragma unroll
    for (int r = 0; r < TBV_MAXRANK; r++)
      if ((still >> r) & 1u) ll_load_unit(c, base + size_t(r) * c.ll_cap, lo[r], hi[r]);
    pending = still;
  }
#pragma unroll
  for (int r = 0; r < TBV_MAXRANK; r++)
    if ((mask >> r) & 1u) out[r] = make_uint4(lo[r].x, lo[r].z, hi[r].x, hi[r].z);
}
template <typename T>
__device__ __forceinline__ void ll_sum_unit(const RankCtx& c, const uint4 (&got)[TBV_MAXRANK], unsigned mask, const uint4& mine,
                                            float* acc) {
  sum_units_rank_order<T>(c, got, mask, mine, acc);
}

template <typename T>
__device__ void ar_oneshot_ll_body(const RankCtx& c, const T* __restrict__ in, T* out, size_t nbytes, int nchan, int chan,
                                   int io, unsigned long long* sh_seq) {
  unsigned long long t_enter = (threadIdx.x == 0 && chan == 0) ? globaltimer() : 0;
  const size_t units = nbytes / 16;
  const size_t per = (units + nchan - 1) / nchan;
  const size_t u0 = per * chan;
  size_t u1 = (u0 + per < units) ? (u0 + per) : units;
  if (!(TBV_GUARD(c, nbytes * 2, c.guard_ll_cap, kGuardLLBytes, chan) && TBV_GUARD(c, nchan, TBV_MAXCHAN, kGuardChannels, chan))) u1 = u0;
  const bool in_al = io & kInAligned, out_al = io & kOutAligned;
  // the first unit's load is issued before the sequence number is known (they do not depend on each other)
  const size_t uf = u0 + threadIdx.x;
  uint4 first = make_uint4(0, 0, 0, 0);
  if (uf < u1) first = ld_unit(in, uf, in_al);
  CallInfo ci = call_begin(c, sh_seq);
  if (chan == 0 && threadIdx.x == 0) c.dm->bc[0] = ci.seq;
  for (size_t u = uf; u < u1; u += blockDim.x) {
    const uint4 v = (u == uf) ? first : ld_unit(in, u, in_al);
    ll_push_unit(c, ci.slot, u, v, ci.want);
  }
  if (chan == 0 && threadIdx.x == 0) { c.dm->bc[1] = ci.seq; c.dm->ring[ci.seq & (kTraceN - 1)].t_pushed = globaltimer(); }
  const unsigned peers = ((1u << c.world) - 1u) & ~(1u << c.rank);
  unsigned long long t_ready = 0;
  for (size_t u = uf; u < u1; u += blockDim.x) {
    const uint4 mine = (u == uf) ? first : ld_unit(in, u, in_al);
    uint4 got[TBV_MAXRANK];
    ll_pull_all(c, ci.slot, u, ci.want, peers, chan, ci.seq, got);
    float acc[Pack<T>::N];
#pragma unroll
    for (int i = 0; i < Pack<T>::N; i++) acc[i] = 0.f;
    ll_sum_unit<T>(c, got, peers, mine, acc);
    st_unit(out, u, Pack<T>::pack(acc), out_al);
  }
  if (threadIdx.x == 0 && chan == 0) { t_ready = globaltimer(); c.dm->bc[2] = ci.seq; }
  call_end(c, ci, nchan, t_enter, t_ready, nbytes, TBV_ALGO_LL);
}

__device__ __forceinline__ void multimem_st_v4(void* p, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- two-shot all-reduce (reduce-scatter + all-gather over peer stores) --------------
// Rank r owns chunk r.  Phase 0: every rank pushes chunk p of its input to rank p.
// Rank r reduces chunk r (rank order, fp32, one rounding) — a single reducer per
// element, so all ranks end with identical bits by construction — and pushes the
// result into every peer's result region.  Phase 1: copy the gathered result out.
// mode: 0 = all-reduce, 1 = reduce-scatter only (out holds chunk `rank`),
//       2 = all-gather only (in holds this rank's chunk).
template <typename T, bool VEC>
__device__ void ar_twoshot_body(const RankCtx& c, const T* __restrict__ in, T* out, size_t nbytes,
                                int nchan, int chan, int mode, int io, unsigned long long* sh_seq) {
  unsigned long long t_enter = (threadIdx.x == 0 && chan == 0) ? globaltimer() : 0;
  CallInfo ci = call_begin(c, sh_seq);
  const size_t unit_bytes = VEC ? 16 : sizeof(T);
  size_t units = nbytes / unit_bytes;                    // whole (gathered) tensor
  if (!(TBV_GUARD(c, nbytes, c.guard_cap, kGuardSlotBytes, chan) && TBV_GUARD(c, nchan, TBV_MAXCHAN, kGuardChannels, chan))) units = 0;
  const size_t cu = (units + c.world - 1) / c.world;     // units per rank chunk
  const size_t per = (cu + nchan - 1) / nchan;           // units per channel inside a chunk
  const int W = c.world, me = c.rank;
  const bool in_al = io & kInAligned, out_al = io & kOutAligned;
  if (chan == 0 && threadIdx.x == 0) c.dm->bc[0] = ci.seq;
  const int R = W;  // index of the result region inside a slot
  unsigned long long t_ready = 0;

  auto chunk_len = [&](int r) -> size_t {
    size_t b = cu * r;
    return b >= units ? 0 : ((units - b < cu) ? units - b : cu);
  };
  auto sub_begin = [&](size_t len) -> size_t { size_t b = per * chan; return b < len ? b : len; };
  auto sub_end = [&](size_t len) -> size_t { size_t e = per * chan + per; return e < len ? e : len; };

  if (mode != 2) {
    // phase 0 push: chunk p of my input -> rank p, region [src = me], chunk-relative offsets
    for (int d = 1; d < W; d++) {
      int p = (me + d) % W;
      size_t len = chunk_len(p), b = sub_begin(len), e = sub_end(len);
      if (VEC) {
        // four independent 16-byte loads per thread before the stores: large messages need megabytes in flight
        uint4* dst = reinterpret_cast<uint4*>(slot_region(c, p, ci.slot, me));
        for (size_t i = b + threadIdx.x; i < e; i += size_t(4) * blockDim.x) {
          uint4 v[4];
#pragma unroll
          for (int k = 0; k < 4; k++) { const size_t j = i + size_t(k) * blockDim.x; if (j < e) v[k] = ld_unit(in, cu * p + j, in_al); }
#pragma unroll
          for (int k = 0; k < 4; k++) { const size_t j = i + size_t(k) * blockDim.x; if (j < e) dst[j] = v[k]; }
        }
      } else {
        for (size_t i = b + threadIdx.x; i < e; i += blockDim.x) reinterpret_cast<T*>(slot_region(c, p, ci.slot, me))[i] = in[cu * p + i];
      }
    }
    __syncthreads();
    publish(c, ci, 0, chan);
    if (chan == 0 && threadIdx.x == 0) { c.dm->bc[1] = ci.seq; c.dm->ring[ci.seq & (kTraceN - 1)].t_pushed = globaltimer(); }
    wait_all(c, ci, 0, chan, kWherePhase0);
    if (threadIdx.x == 0 && chan == 0) { t_ready = globaltimer(); c.dm->bc[2] = ci.seq; }
  }

  {
    // reduce my chunk; write it out and (all-reduce) push it to every peer's result region
    size_t len = chunk_len(me), b = sub_begin(len), e = sub_end(len);
    const unsigned others = ((1u << W) - 1u) & ~(1u << me);
    for (size_t i = b + threadIdx.x; i < e; i += blockDim.x) {
      if (VEC) {
        uint4 res;
        if (mode == 2) {
          res = ld_unit(in, i, in_al);
        } else {
          float acc[Pack<T>::N];
#pragma unroll
          for (int k = 0; k < Pack<T>::N; k++) acc[k] = 0.f;
          const uint4 mine = ld_unit(in, cu * me + i, in_al);
          uint4 got[TBV_MAXRANK];
          gather_units(c, me, ci.slot, i, others, got);
          sum_units_rank_order<T>(c, got, others, mine, acc);
          res = Pack<T>::pack(acc);
        }
        if (mode == 1) {
          st_unit(out, i, res, out_al);
        } else {
          st_unit(out, cu * me + i, res, out_al);
          if (c.mc_data) {
            // one store through the NVSwitch multicast object lands in every rank's result
            // region (the reduction above stays in rank order: results are still exact)
            multimem_st_v4(c.mc_data + size_t(ci.slot) * c.slot_stride + size_t(R) * c.cap + (cu * me + i) * 16, res);
          } else {
            for (int d = 1; d < W; d++) {
              int p = (me + d) % W;
              reinterpret_cast<uint4*>(slot_region(c, p, ci.slot, R))[cu * me + i] = res;
            }
          }
        }
      } else {
        T res;
        if (mode == 2) {
          res = in[i];
        } else {
          float acc = 0.f;
          for (int r = 0; r < W; r++) {
            float f = (r == me) ? Pack<T>::to_f(in[cu * me + i])
                                : Pack<T>::to_f(*(reinterpret_cast<volatile const T*>(slot_region(c, me, ci.slot, r)) + i));
            acc = (r == 0) ? f : acc + f;
          }
          res = Pack<T>::from_f(acc);
        }
        if (mode == 1) {
          out[i] = res;
        } else {
          out[cu * me + i] = res;
          for (int d = 1; d < W; d++) {
            int p = (me + d) % W;
            reinterpret_cast<T*>(slot_region(c, p, ci.slot, R))[cu * me + i] = res;
          }
        }
      }
    }
  }

  if (mode != 1) {
    __syncthreads();
    publish(c, ci, 1, chan);
    wait_all(c, ci, 1, chan, kWherePhase1);
    if (mode == 2 && threadIdx.x == 0 && chan == 0) t_ready = globaltimer();
    // copy the peers' reduced chunks from my result region to the output
    for (int d = 1; d < W; d++) {
      int p = (me + d) % W;
      size_t len = chunk_len(p), b = sub_begin(len), e = sub_end(len);
      if (VEC) {
        const uint4* src = reinterpret_cast<const uint4*>(slot_region(c, me, ci.slot, R)) + cu * p;
        for (size_t i = b + threadIdx.x; i < e; i += size_t(4) * blockDim.x) {
          uint4 v[4];
#pragma unroll
          for (int k = 0; k < 4; k++) { const size_t j = i + size_t(k) * blockDim.x; if (j < e) v[k] = ld_volatile_v4(src + j); }
#pragma unroll
          for (int k = 0; k < 4; k++) { const size_t j = i + size_t(k) * blockDim.x; if (j < e) st_unit(out, cu * p + j, v[k], out_al); }
        }
      } else {
        for (size_t i = b + threadIdx.x; i < e; i += blockDim.x)
          out[cu * p + i] = *(reinterpret_cast<volatile const T*>(slot_region(c, me, ci.slot, R)) + cu * p + i);
      }
    }
  }
  call_end(c, ci, nchan, t_enter, t_ready, nbytes, TBV_ALGO_TWOSHOT);
}

// ---- copy-engine two-shot (large messages, opt-in) -----------------------------------------------
// The bulk transfers are stream-ordered device-to-device copies issued by the host (the copy
// engines move the bytes, the SMs stay free); two small kernels do the signalling and the arithmetic.
// This is the counterpart of the reference's memcpy + event path (TBV_GPUSIG=0,
// step4/libtbvcoll.cpp:463-464,483).  Stream order per call:
//   copies   chunk p of my input  -> rank p's CE region [src = me]           (W-1 copies)
//   phase A  flag 0 to all, wait for all; reduce my chunk in rank order into out[chunk me]
//   copies   out[chunk me]        -> every peer's CE result region            (W-1 copies)
//   phase B  flag 1 to all, wait for all; copy the peers' chunks out; sequence number + 1
// The CE regions are a fixed extra "slot" (index nslot), not part of the ring, so the copy
// destinations do not depend on the sequence number and a captured graph replays correctly.
// Reuse is safe without a ring: my kernel A of call s+1 passes only after every peer raised flag 0
// of s+1, which each does after finishing its own call s entirely, so nobody still reads the
// regions my next copies overwrite; the same holds for the result regions through flag 1.
template <typename T>
__device__ void ar_ce_phase_a(const RankCtx& c, const T* __restrict__ in, T* out, size_t nbytes, int nchan, int chan,
                              unsigned long long* sh_seq) {
  CallInfo ci = call_begin(c, sh_seq);
  ci.slot = c.nslot;   // the fixed CE slot (flags and regions)
  const size_t units = nbytes / 16, cu = units / c.world;
  const size_t per = (cu + nchan - 1) / nchan;
  const size_t b = per * chan < cu ? per * chan : cu, e = per * chan + per < cu ? per * chan + per : cu;
  const int W = c.world, me = c.rank;
  if (chan == 0 && threadIdx.x == 0) { c.dm->bc[0] = ci.seq; c.dm->ts[0] = globaltimer(); }
  publish(c, ci, 0, chan);          // the copies before this kernel have completed: their bytes are in place
  wait_all(c, ci, 0, chan, kWherePhase0);
  if (chan == 0 && threadIdx.x == 0) { c.dm->bc[2] = ci.seq; c.dm->ts[1] = globaltimer(); }
  const uint4* mine = reinterpret_cast<const uint4*>(in) + cu * me;
  uint4* dst = reinterpret_cast<uint4*>(out) + cu * me;
  const unsigned others = ((1u << W) - 1u) & ~(1u << me);
  for (size_t i = b + threadIdx.x; i < e; i += blockDim.x) {
    float acc[Pack<T>::N];
#pragma unroll
    for (int k = 0; k < Pack<T>::N; k++) acc[k] = 0.f;
    const uint4 own = mine[i];
    uint4 got[TBV_MAXRANK];
    gather_units(c, me, ci.slot, i, others, got);
    sum_units_rank_order<T>(c, got, others, own, acc);
    dst[i] = Pack<T>::pack(acc);
  }
}
template <typename T>
__device__ void ar_ce_phase_b(const RankCtx& c, T* out, size_t nbytes, int nchan, int chan, unsigned long long* sh_seq) {
  CallInfo ci = call_begin(c, sh_seq);
  const unsigned long long seq = ci.seq;
  ci.slot = c.nslot;
  const size_t units = nbytes / 16, cu = units / c.world;
  const size_t per = (cu + nchan - 1) / nchan;
  const size_t b = per * chan < cu ? per * chan : cu, e = per * chan + per < cu ? per * chan + per : cu;
  const int W = c.world, me = c.rank;
  publish(c, ci, 1, chan);
  wait_all(c, ci, 1, chan, kWherePhase1);
  const unsigned long long t_ready = (chan == 0 && threadIdx.x == 0) ? globaltimer() : 0;
  const uint4* res = reinterpret_cast<const uint4*>(slot_region(c, me, ci.slot, W));
  for (int d = 1; d < W; d++) {
    const int p = (me + d) % W;
    for (size_t i = b + threadIdx.x; i < e; i += size_t(4) * blockDim.x) {
      uint4 v[4];
#pragma unroll
      for (int k = 0; k < 4; k++) { const size_t j = i + size_t(k) * blockDim.x; if (j < e) v[k] = ld_volatile_v4(res + cu * p + j); }
#pragma unroll
      for (int k = 0; k < 4; k++) { const size_t j = i + size_t(k) * blockDim.x; if (j < e) reinterpret_cast<uint4*>(out)[cu * p + j] = v[k]; }
    }
  }
  ci.seq = seq;
  ci.slot = int(seq % (unsigned long long)c.nslot);
  call_end(c, ci, nchan, c.dm->ts[0], t_ready, nbytes, TBV_ALGO_CE);
}

// ---- NVLS all-reduce (multimem through the NVSwitch) -----------------------------------
// Measured on B200: for fp32 the in-switch sum matched the oracle at N = 2; for bf16/fp16
// (fp32 accumulate requested) about one element in five differs from round-to-nearest-even of
// the fp32 sum by one unit in the last place.  Every rank gets identical bits and repeated runs
// agree, but it is NOT the fixed-order oracle, so `auto` never selects this kernel; the exact
// use of the multicast object is the broadcast half of the two-shot kernel above.
// Stage the input in this rank's own slot memory (same offset on every rank), flag,
// wait for all; rank r then reduces chunk r with one multimem.ld_reduce per 16 bytes
// (the switch reads all N copies and adds them, fp32 accumulate for 16-bit types) and
// broadcasts it with multimem.st into every rank's result region.  A single reduction
// per element: all ranks get identical bits.  16-byte units only.
template <typename T> struct Multimem;
template <> struct Multimem<float> {
  __device__ static uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
template <> struct Multimem<__half> {
  __device__ static uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
template <> struct Multimem<__nv_bfloat16> {
  __device__ static uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
// `direct` (small and medium messages): after the staging flags every rank reduces the WHOLE
// tensor through the switch straight into its output — one staging pass and one reduction
// pass, no broadcast, no second flag round and no copy-out.
template <typename T>
__device__ void ar_nvls_body(const RankCtx& c, const T* __restrict__ in, T* out, size_t nbytes,
                             int nchan, int chan, int io, bool direct, unsigned long long* sh_seq) {
  unsigned long long t_enter = (threadIdx.x == 0 && chan == 0) ? globaltimer() : 0;
  CallInfo ci = call_begin(c, sh_seq);
  const size_t units = nbytes / 16;
  const size_t cu = (units + c.world - 1) / c.world;
  const size_t per = (cu + nchan - 1) / nchan;
  const int W = c.world, me = c.rank;
  const int R = W;
  const bool in_al = io & kInAligned, out_al = io & kOutAligned;
  if (chan == 0 && threadIdx.x == 0) c.dm->bc[0] = ci.seq;
  // stage: region 0 of my own slot memory; channel `chan` stages its sub-range of EVERY chunk
  uint4* stage = reinterpret_cast<uint4*>(slot_region(c, me, ci.slot, 0));
  for (int r = 0; r < W; r++) {
    size_t base = cu * r;
    size_t len = base >= units ? 0 : ((units - base < cu) ? units - base : cu);
    size_t b = per * chan; if (b > len) b = len;
    size_t e = per * chan + per; if (e > len) e = len;
    for (size_t i = b + threadIdx.x; i < e; i += blockDim.x)
      stage[base + i] = ld_unit(in, base + i, in_al);
  }
  __syncthreads();
  publish(c, ci, 0, chan);
  if (chan == 0 && threadIdx.x == 0) { c.dm->bc[1] = ci.seq; c.dm->ring[ci.seq & (kTraceN - 1)].t_pushed = globaltimer(); }
  wait_all(c, ci, 0, chan, kWherePhase0);
  unsigned long long t_ready = (threadIdx.x == 0 && chan == 0) ? globaltimer() : 0;
  if (direct) {
    const char* mc_stage = c.mc_data + size_t(ci.slot) * c.slot_stride;
    for (int r = 0; r < W; r++) {
      size_t base = cu * r;
      size_t len = base >= units ? 0 : ((units - base < cu) ? units - base : cu);
      size_t b = per * chan; if (b > len) b = len;
      size_t e = per * chan + per; if (e > len) e = len;
      for (size_t i = b + threadIdx.x; i < e; i += blockDim.x)
        st_unit(out, base + i, Multimem<T>::ld_reduce(mc_stage + (base + i) * 16), out_al);
    }
    call_end(c, ci, nchan, t_enter, t_ready, nbytes, TBV_ALGO_NVLS);
    return;
  }
  {
    size_t base = cu * me;
    size_t len = base >= units ? 0 : ((units - base < cu) ? units - base : cu);
    size_t b = per * chan; if (b > len) b = len;
    size_t e = per * chan + per; if (e > len) e = len;
    const char* mc_stage = c.mc_data + size_t(ci.slot) * c.slot_stride;
    char* mc_res = c.mc_data + size_t(ci.slot) * c.slot_stride + size_t(R) * c.cap;
    for (size_t i = b + threadIdx.x; i < e; i += blockDim.x) {
      uint4 v = Multimem<T>::ld_reduce(mc_stage + (base + i) * 16);
      multimem_st_v4(mc_res + (base + i) * 16, v);
    }
  }
  __syncthreads();
  publish(c, ci, 1, chan);
  wait_all(c, ci, 1, chan, kWherePhase1);
  const uint4* res = reinterpret_cast<const uint4*>(slot_region(c, me, ci.slot, R));
  for (int r = 0; r < W; r++) {
    size_t base = cu * r;
    size_t len = base >= units ? 0 : ((units - base < cu) ? units - base : cu);
    size_t b = per * chan; if (b > len) b = len;
    size_t e = per * chan + per; if (e > len) e = len;
    for (size_t i = b + threadIdx.x; i < e; i += blockDim.x)
      st_unit(out, base + i, ld_volatile_v4(res + base + i), out_al);
  }
  call_end(c, ci, nchan, t_enter, t_ready, nbytes, TBV_ALGO_NVLS);
}

// ---- RMSNorm row math shared by the fused collective and the plain op -------------------
// The thread mapping and the reduction tree are the same wherever this is used, so a
// fused and an unfused pipeline produce the same bits.
// Semantics (HF Llama): var = mean(h^2) in fp32 over bf16-rounded h; y = bf16(h * rsqrt(var + eps));
// out = bf16(gamma * y).
constexpr int kNormMaxUnits = 4;  // 16-byte units per thread: hidden <= 8 * 4 * 1024

__device__ __forceinline__ float block_sum_fixed(float v, float* sh /* >= 32 floats */) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();  // protect sh from the previous use
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; i++) t += sh[i];  // every thread adds in the same order
  return t;
}

// h: this thread's values of one row (units u = threadIdx.x + k*blockDim.x), already
// rounded to bf16 precision.  Writes the normalised row.
template <int MAXU = kNormMaxUnits>
__device__ __forceinline__ void rmsnorm_row_store(const float (*h)[8], int nunits_row, int hidden,
                                                  float eps, const uint4* __restrict__ gamma,
                                                  uint4* y_row, float* sh) {
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < MAXU; k++) {
    int u = threadIdx.x + k * blockDim.x;
    if (u < nunits_row) {
#pragma unroll
      for (int i = 0; i < 8; i++) ss += h[k][i] * h[k][i];
    }
  }
  float tot = block_sum_fixed(ss, sh);
  float rs = rsqrtf(tot / float(hidden) + eps);
#pragma unroll
  for (int k = 0; k < MAXU; k++) {
    int u = threadIdx.x + k * blockDim.x;
    if (u < nunits_row) {
      float g[8], o[8];
      Pack<__nv_bfloat16>::unpack(gamma[u], g);
#pragma unroll
      for (int i = 0; i < 8; i++) {
        float n = __bfloat162float(__float2bfloat16_rn(h[k][i] * rs));
        o[i] = g[i] * n;
      }
      y_row[u] = Pack<__nv_bfloat16>::pack(o);
    }
  }
}

// The same row normalisation run by CTAs of a different size, or by the CTAs of a cluster that share one row.
// `nt` is the thread count the plain op uses for this hidden size (one 16-byte unit per thread: hidden <= 8192);
// this CTA is part `part` of `nparts` and owns the units [part * per, (part + 1) * per), per = row units / nparts
// (a multiple of 32, so no 32-unit group is shared by two CTAs); each real thread plays the "virtual" threads
// part * per + threadIdx.x + j * blockDim.x.  Sums are formed in the order of the nt-thread CTA (per unit, 32-lane
// butterfly per virtual warp, warps in order), so the result has the same bits as rmsnorm_row_store with
// blockDim.x == nt.  With nparts > 1 every CTA stores its warps' partial sums into the `sh` array of every CTA of
// the cluster (distributed shared memory) and one cluster barrier orders them before they are read; `sh` holds two
// sets of 32 partials used in turn (`phase` = this call's count within the kernel), which makes that one barrier
// per row enough.  `gpre`: this thread's gamma units already in registers (loaded before a wait so that the load's
// round trip is not paid after it), or null to load them here.  blockDim.x % 32 == 0.
template <int VPT>
__device__ __forceinline__ void rmsnorm_row_store_virtual(const float (*h)[8], int nunits_row, int hidden, float eps,
                                                          const uint4* __restrict__ gamma, uint4* y_row, float* sh, int nt,
                                                          const uint4* gpre = nullptr, int part = 0, int nparts = 1,
                                                          int phase = 0) {
  const int lane = threadIdx.x & 31, nvw = nt >> 5;
  const int per = nunits_row / nparts, u_base = part * per;
  float* buf = sh + (phase & 1) * 32;
  if (nparts == 1) __syncthreads();  // protect sh from the previous use (a cluster alternates between two sets instead)
#pragma unroll
  for (int j = 0; j < VPT; j++) {
    const int li = threadIdx.x + j * blockDim.x, vt = u_base + li;
    float ss = 0.f;
    if (li < per && vt < nunits_row) {
#pragma unroll
      for (int i = 0; i < 8; i++) ss += h[j][i] * h[j][i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const int vw = vt >> 5;
    if (lane == 0 && vw < nvw && li < per) {
      if (nparts == 1) {
        buf[vw] = ss;
      } else {
        const unsigned mine = unsigned(__cvta_generic_to_shared(buf + vw));
        for (int q = 0; q < nparts; q++) {
          unsigned remote;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(mine), "r"(q));
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(ss) : "memory");
        }
      }
    }
  }
  if (nparts == 1) {
    __syncthreads();
  } else {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  float tot = 0.f;
  for (int i = 0; i < nvw; i++) tot += buf[i];
  const float rs = rsqrtf(tot / float(hidden) + eps);
#pragma unroll
  for (int j = 0; j < VPT; j++) {
    const int li = threadIdx.x + j * blockDim.x, u = u_base + li;
    if (li < per && u < nunits_row) {
      float g[8], o[8];
      Pack<__nv_bfloat16>::unpack(gpre ? gpre[j] : gamma[u], g);
#pragma unroll
      for (int i = 0; i < 8; i++) {
        float n = __bfloat162float(__float2bfloat16_rn(h[j][i] * rs));
        o[i] = g[i] * n;
      }
      y_row[u] = Pack<__nv_bfloat16>::pack(o);
    }
  }
}

// ---- fused all-reduce + residual add + RMSNorm (one-shot, bf16) ---------------------------
// Channel c owns rows c, c + nchan, ...  It pushes those rows, flags once, waits once,
// then for each row: s = bf16(sum in rank order); h = bf16(s + residual);
// residual_out = h; y = RMSNorm(h) * gamma.
__device__ inline void ar_rmsnorm_body(const RankCtx& c, const __nv_bfloat16* __restrict__ x,
                                       const __nv_bfloat16* residual,
                                       const __nv_bfloat16* __restrict__ gamma,
                                       __nv_bfloat16* residual_out, __nv_bfloat16* y, int tokens,
                                       int hidden, float eps, int nchan, int chan,
                                       unsigned long long* sh_seq, float* sh_red) {
  unsigned long long t_enter = (threadIdx.x == 0 && chan == 0) ? globaltimer() : 0;
  const int upr = hidden / 8;  // 16-byte units per row
  CallInfo ci = call_begin(c, sh_seq);
  if (chan == 0 && threadIdx.x == 0) c.dm->bc[0] = ci.seq;
  if (!(TBV_GUARD(c, size_t(tokens) * hidden * 2, c.guard_cap, kGuardSlotBytes, chan) && TBV_GUARD(c, nchan, TBV_MAXCHAN, kGuardChannels, chan)))
    tokens = 0;
  for (int row = chan; row < tokens; row += nchan) {
    const uint4* src = reinterpret_cast<const uint4*>(x) + size_t(row) * upr;
    for (int u = threadIdx.x; u < upr; u += blockDim.x) {
      const uint4 v = src[u];
      for (int p = 0; p < c.world; p++)
        if (p != c.rank)
          reinterpret_cast<uint4*>(slot_region(c, p, ci.slot, c.rank))[size_t(row) * upr + u] = v;
    }
  }
  __syncthreads();
  publish(c, ci, 0, chan);
  if (chan == 0 && threadIdx.x == 0) { c.dm->bc[1] = ci.seq; c.dm->ring[ci.seq & (kTraceN - 1)].t_pushed = globaltimer(); }
  wait_all(c, ci, 0, chan, kWhereFused);
  unsigned long long t_ready = (threadIdx.x == 0 && chan == 0) ? globaltimer() : 0;
  for (int row = chan; row < tokens; row += nchan) {
    float h[kNormMaxUnits][8];
#pragma unroll
    for (int k = 0; k < kNormMaxUnits; k++) {
      int u = threadIdx.x + k * blockDim.x;
      if (u < upr) {
        size_t off = size_t(row) * upr + u;
        float acc[8];
        uint4 mine = reinterpret_cast<const uint4*>(x)[off];
        for (int r = 0; r < c.world; r++) {
          uint4 v = (r == c.rank) ? mine
                                  : ld_volatile_v4(reinterpret_cast<const uint4*>(slot_region(c, c.rank, ci.slot, r)) + off);
          float f[8];
          Pack<__nv_bfloat16>::unpack(v, f);
#pragma unroll
          for (int i = 0; i < 8; i++) acc[i] = (r == 0) ? f[i] : acc[i] + f[i];
        }
        float res[8];
        Pack<__nv_bfloat16>::unpack(reinterpret_cast<const uint4*>(residual)[off], res);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          float s = __bfloat162float(__float2bfloat16_rn(acc[i]));
          h[k][i] = __bfloat162float(__float2bfloat16_rn(s + res[i]));
        }
        reinterpret_cast<uint4*>(residual_out)[off] = Pack<__nv_bfloat16>::pack(h[k]);
      }
    }
    rmsnorm_row_store(h, upr, hidden, eps, reinterpret_cast<const uint4*>(gamma),
                      reinterpret_cast<uint4*>(y) + size_t(row) * upr, sh_red);
  }
  call_end(c, ci, nchan, t_enter, t_ready, size_t(tokens) * hidden * 2, TBV_ALGO_ONESHOT);
}

// The same with LL packets: no fence, no flag, no flag wait — a row is pushed as self-announcing
// packets and the packets of all peers are pulled with one batch of loads.  Runs with at most 512
// threads (128 registers each for the batch); a hidden size whose plain norm kernel uses more
// threads is handled by two virtual threads per thread, same bits.  hidden <= 8192.
constexpr int kLLNormVPT = 2;   // the largest VPT instantiated: hidden <= 8 * 2 * 512
// LL form of the fused all-reduce + residual + RMSNorm.  Channel c owns rows c, c + nchan, ...; a row is shared by
// the `nparts` CTAs of a cluster (blockIdx.z = part), each of which pushes, pulls, adds and normalises its own
// 1 / nparts of the row's units and exchanges only the per-warp sums of squares (see rmsnorm_row_store_virtual).
// Why parts: an SM hands one 32-byte sector per clock to the fabric, so a CTA that pushes a whole 8 KB row to seven
// peers (112 KB of packets) spends 2 us on the push alone (measured on 8 GPUs; it grows by 0.3-0.4 us per peer);
// four CTAs on four SMs spend a quarter of that, and pull a quarter of the packets each.
template <int VPT>
__device__ inline void ar_rmsnorm_ll_body(const RankCtx& c, const __nv_bfloat16* __restrict__ x,
                                          const __nv_bfloat16* residual, const __nv_bfloat16* __restrict__ gamma,
                                          __nv_bfloat16* residual_out, __nv_bfloat16* y, int tokens, int hidden, float eps,
                                          int nchan, int chan, int part, int nparts, int norm_threads,
                                          unsigned long long* sh_seq, float* sh_red) {
  const bool lead = threadIdx.x == 0 && chan == 0 && part == 0;
  unsigned long long t_enter = lead ? globaltimer() : 0;
  const int upr = hidden / 8, per = upr / nparts, u_base = part * per;
  if (!TBV_GUARD(c, size_t(tokens) * hidden * 4, c.guard_ll_cap, kGuardLLBytes, chan)) tokens = 0;
  // first row's first unit: loaded before the sequence number is known
  uint4 first = make_uint4(0, 0, 0, 0);
  if (chan < tokens && int(threadIdx.x) < per) first = reinterpret_cast<const uint4*>(x)[size_t(chan) * upr + u_base + threadIdx.x];
  CallInfo ci = call_begin(c, sh_seq);
  if (lead) c.dm->bc[0] = ci.seq;
  for (int row = chan; row < tokens; row += nchan) {
    const uint4* src = reinterpret_cast<const uint4*>(x) + size_t(row) * upr + u_base;
    for (int li = threadIdx.x; li < per; li += blockDim.x) {
      const uint4 v = (row == chan && li == int(threadIdx.x)) ? first : src[li];
      ll_push_unit(c, ci.slot, size_t(row) * upr + u_base + li, v, ci.want);
    }
  }
  if (lead) { c.dm->bc[1] = ci.seq; c.dm->ring[ci.seq & (kTraceN - 1)].t_pushed = globaltimer(); }
  const unsigned peers = ((1u << c.world) - 1u) & ~(1u << c.rank);
  unsigned long long t_ready = 0;
  // gamma does not depend on the row: fetch this thread's units once, while the packets are in flight
  uint4 gpre[VPT];
#pragma unroll
  for (int j = 0; j < VPT; j++) {
    const int li = threadIdx.x + j * blockDim.x;
    gpre[j] = li < per ? reinterpret_cast<const uint4*>(gamma)[u_base + li] : make_uint4(0, 0, 0, 0);
  }
  int iter = 0;
  for (int row = chan; row < tokens; row += nchan, iter++) {
    float h[VPT][8];
    // the residual units of this row too: their round trip overlaps the packets' flight instead of following it
    uint4 rpre[VPT];
#pragma unroll
    for (int j = 0; j < VPT; j++) {
      const int li = threadIdx.x + j * blockDim.x;
      rpre[j] = li < per ? reinterpret_cast<const uint4*>(residual)[size_t(row) * upr + u_base + li] : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < VPT; j++) {
      const int li = threadIdx.x + j * blockDim.x;
      if (li < per) {
        const size_t off = size_t(row) * upr + u_base + li;
        const uint4 mine = (row == chan && j == 0) ? first : reinterpret_cast<const uint4*>(x)[off];
        uint4 got[TBV_MAXRANK];
        ll_pull_all(c, ci.slot, off, ci.want, peers, chan, ci.seq, got);
        float acc[8];
        ll_sum_unit<__nv_bfloat16>(c, got, peers, mine, acc);
        float res[8];
        Pack<__nv_bfloat16>::unpack(rpre[j], res);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          float s = __bfloat162float(__float2bfloat16_rn(acc[i]));
          h[j][i] = __bfloat162float(__float2bfloat16_rn(s + res[i]));
        }
        reinterpret_cast<uint4*>(residual_out)[off] = Pack<__nv_bfloat16>::pack(h[j]);
      }
    }
    if (row == chan && lead) { t_ready = globaltimer(); c.dm->bc[2] = ci.seq; }
    rmsnorm_row_store_virtual<VPT>(h, upr, hidden, eps, reinterpret_cast<const uint4*>(gamma),
                                   reinterpret_cast<uint4*>(y) + size_t(row) * upr, sh_red, norm_threads, gpre, part, nparts, iter);
  }
  call_end(c, ci, nchan * nparts, t_enter, t_ready, size_t(tokens) * hidden * 2, TBV_ALGO_LL);
}

}  // namespace tbv
