// tbvcoll.h — C ABI of libtbvcoll (B200 build).
//
// The `tbv_ar_*` names, argument orders and return codes are the ones the
// reference exports from step4/libtbvcoll.cpp:279-566 so that a ctypes caller
// written against it keeps working.  Everything behind the ABI is different:
// peers are GPUs of one NVSwitch domain reached through mapped peer memory, the
// collective is one stream-ordered kernel, and there is no host progress thread
// on the GPU path.  A second family, `tbv_comm_*`, takes an explicit
// communicator so that several worlds can live in one process.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Return codes (reference: libtbvcoll.cpp:62,420).
#define TBV_OK 0
#define TBV_FAIL (-1)
#define TBV_FALLBACK (-2)  // over capacity / unsupported: caller falls back to NCCL

// dtype codes (reference: tbvcoll.py:10).
#define TBV_F32 0
#define TBV_F16 1
#define TBV_BF16 2

// Algorithm ids (TBV_ALGO / tbv_comm_set_algo).
#define TBV_ALGO_AUTO 0
#define TBV_ALGO_ONESHOT 1
#define TBV_ALGO_TWOSHOT 2
#define TBV_ALGO_NVLS 3
#define TBV_ALGO_LL 4   // one-shot with flag-in-payload packets (small messages)
#define TBV_ALGO_CE 5   // two-shot whose bulk transfers are copy-engine copies (TBV_CE=1 at bring-up; large messages; never picked by auto)

#define TBV_MAXRANK 8
#define TBV_MAXSLOT 32
#define TBV_MAXCHAN 256

typedef struct tbv_comm tbv_comm;

// ---- explicit-communicator API -------------------------------------------------
// device >= 0: CUDA backend on that device.  device == -1: CPU backend (POSIX
// shared memory + one progress thread; the plumbing/test backend).
// Every rank of the world calls this together (SPMD); rank 0 listens on
// peer_ip:port, the others connect to it.
int tbv_comm_create(tbv_comm** out, int rank, int world, int device,
                    const char* peer_ip, int port, size_t cap_bytes);
// N emulated ranks inside ONE process on ONE GPU.  Collectives on such a
// communicator run as a single cooperative launch whose blockIdx.y is the rank;
// this is how the multi-rank protocol is exercised when fewer GPUs than ranks exist.
int tbv_comm_create_local(tbv_comm** out, int world, int device, size_t cap_bytes);
int tbv_comm_destroy(tbv_comm* c);

int tbv_comm_allreduce(tbv_comm* c, const void* in, void* out, size_t nbytes,
                       int dtype, void* stream);
// Local (emulated) world: one pointer per rank.
int tbv_comm_allreduce_local(tbv_comm* c, const void* const* ins, void* const* outs,
                             size_t nbytes, int dtype, void* stream);
// all-reduce(x) -> h = bf16(sum) + residual -> residual_out = h ; y = RMSNorm(h)*gamma.
// x: [tokens, hidden] partial sums of this rank.  bf16 only.  hidden % 8 == 0.
// residual_out may alias residual; y may alias x.
int tbv_comm_allreduce_rmsnorm(tbv_comm* c, const void* x, const void* residual,
                               const void* gamma, void* residual_out, void* y,
                               int tokens, int hidden, float eps, void* stream);
int tbv_comm_allreduce_rmsnorm_local(tbv_comm* c, const void* const* xs,
                                     const void* const* residuals, const void* gamma,
                                     void* const* residual_outs, void* const* ys,
                                     int tokens, int hidden, float eps, void* stream);
// Row-parallel linear fused with its all-reduce, the residual add and RMSNorm in ONE kernel
// (tcgen05 GEMM whose epilogue stores into every rank's slot memory):
//   h = bf16(sum over ranks of bf16(x @ w^T)) + residual; residual_out = h; y = RMSNorm(h) * gamma.
// x: [tokens, k_local] bf16 (row stride ldx), w: [hidden, k_local] bf16.  tokens <= 256.
int tbv_comm_gemm_allreduce_rmsnorm(tbv_comm* c, const void* w, const void* x, const void* residual,
                                    const void* gamma, void* residual_out, void* y, int tokens, int hidden,
                                    int k_local, int ldx, float eps, void* stream);
int tbv_comm_gemm_allreduce_rmsnorm_local(tbv_comm* c, const void* const* ws, const void* const* xs,
                                          const void* const* residuals, const void* gamma,
                                          void* const* residual_outs, void* const* ys, int tokens,
                                          int hidden, int k_local, int ldx, float eps, void* stream);
// Sequence-parallel prefill pairs (tcgen05 GEMM fused with its collective; see ops/gemm_sp.cu).
// GEMM -> reduce-scatter: x [tokens, k_local], w [hidden, k_local]; tokens % world == 0.  This rank
// receives rows [rank*tokens/world, ...) of the rank-ordered sum.  mode 0: out = sum;
// mode 1: h = sum + residual -> residual_out, y = RMSNorm(h) * gamma (all [tokens/world, hidden]).
int tbv_comm_gemm_reduce_scatter(tbv_comm* c, const void* w, const void* x, void* out, const void* residual,
                                 const void* gamma, void* residual_out, void* y, int tokens, int hidden,
                                 int k_local, int ldx, float eps, int mode, void* stream);
int tbv_comm_gemm_reduce_scatter_local(tbv_comm* c, const void* const* ws, const void* const* xs, void* const* outs,
                                       const void* const* residuals, const void* gamma, void* const* residual_outs,
                                       void* const* ys, int tokens, int hidden, int k_local, int ldx, float eps,
                                       int mode, void* stream);
// all-gather -> GEMM: x [rows_per_rank, K] (this rank's token rows), w [M, K]; y [world*rows_per_rank, M].
// The first call for a shape allocates a small table of tensor maps: make it outside stream capture.
int tbv_comm_allgather_gemm(tbv_comm* c, const void* w, const void* x, void* y, int rows_per_rank, int M, int K,
                            int ldx, int ldy, void* stream);
int tbv_comm_allgather_gemm_local(tbv_comm* c, const void* const* ws, const void* const* xs, void* const* ys,
                                  int rows_per_rank, int M, int K, int ldx, int ldy, void* stream);
// reduce-scatter / all-gather over the same slot ring (rows of `row_bytes`).
// reduce_scatter: in [world*rows_per_rank rows] -> out [rows_per_rank rows] (this rank's block).
int tbv_comm_reduce_scatter(tbv_comm* c, const void* in, void* out, size_t out_bytes,
                            int dtype, void* stream);
// all_gather: in [in_bytes] -> out [world*in_bytes], block r from rank r.
int tbv_comm_all_gather(tbv_comm* c, const void* in, void* out, size_t in_bytes,
                        void* stream);
// CPU backend: block until every queued call has completed (GPU backend:
// returns at once; completion is stream-ordered).  Returns TBV_FAIL if any failed.
int tbv_comm_sync(tbv_comm* c);

int tbv_comm_rank(tbv_comm* c);
int tbv_comm_world(tbv_comm* c);
size_t tbv_comm_cap(tbv_comm* c);
int tbv_comm_nslot(tbv_comm* c);
int tbv_comm_is_async(tbv_comm* c);
int tbv_comm_err(tbv_comm* c);
int tbv_comm_has_nvls(tbv_comm* c);
int tbv_comm_set_algo(tbv_comm* c, int algo);        // TBV_ALGO_*
int tbv_comm_set_nchan(tbv_comm* c, int nchan);      // 0 = auto
int tbv_comm_set_wdog(tbv_comm* c, double seconds);  // device + host watchdog
// Fault injection on the HOST: the next `n` collective calls on this rank return
// TBV_OK without launching/queueing anything, so the peers' bounded waits run out.
int tbv_comm_skip_next(tbv_comm* c, int n);
// Emulated world only, also on the host: for the next `n` collective launches the CTAs of
// emulated rank `r` return before they push anything — a rank that never makes the call.  The
// other ranks' bounded waits run out, the kernel ends, tbv_comm_err turns sticky and
// tbv_comm_last_error names `r`.  This is how the device watchdog is exercised on one GPU.
int tbv_comm_mute_rank(tbv_comm* c, int r, int n);
// 1 if the library was built with -DTBV_BOUNDS_CHECK (python -m libtbvcoll_b200._build --bounds): every collective
// body then compares the extent it is about to touch with what the communicator reserved, records a violation
// (sticky error code 3, tbv_comm_last_error) and moves no data instead of making the access.
int tbv_bounds_checked_build(void);
// Device time stamps of the last fused GEMM + all-reduce + norm call on (emulated) rank r (see comm.cu).
int tbv_comm_timestamps(tbv_comm* c, int r, unsigned long long out[8]);
// Per-call device time stamps from the timing ring: rows of {seq, enter, pushed, ready, done} (ns); returns the row count.
int tbv_comm_trace(tbv_comm* c, int r, unsigned long long* out, int max_rows);
// TBV_TAG=1 diagnostic: every flag a rank raises is preceded by a sequence stamp in a word of
// its own next to the flag; the receiver compares it after it has seen the flag.  Totals since
// the communicator was created (synchronous device-to-host copy).
int tbv_comm_tag_counts(tbv_comm* c, unsigned long long* checked, unsigned long long* bad);
// Peer-visible buffers for fused producers (GEMM epilogues push straight into them).
// Fills a device-side context blob (tbv::RankCtx) the fused kernels take by value.
int tbv_comm_ctx(tbv_comm* c, void* ctx_out, size_t ctx_bytes);
// Read-and-reset statistics, all in microseconds (reference: libtbvcoll.cpp:510-536).
void tbv_comm_stats5(tbv_comm* c, double* pre, double* xfer, double* post, double* enq,
                     double* drain, unsigned long long* n);
void tbv_comm_rails(tbv_comm* c);
void tbv_comm_hist(tbv_comm* c);
// Last device breadcrumbs / watchdog record, for tests: out[0]=err code, out[1]=seq,
// out[2]=where, out[3]=peer.
void tbv_comm_last_error(tbv_comm* c, unsigned long long out[4]);
// Device breadcrumbs of (emulated) rank r (see comm.cu); synchronous device-to-host copy.
int tbv_comm_breadcrumbs(tbv_comm* c, int r, unsigned long long out[8]);

// ---- process-global API with the reference's names ------------------------------
// devs: "cpu" selects the CPU backend, "cuda:N" / "N" a device; any other string
// (e.g. the reference's rail list "usb4_rdma0,usb4_rdma5") means "current CUDA
// device" (rails have no meaning here: channels are CTAs, see TBV_NCHAN).  World size
// is 2 unless TBV_WORLD is set.  Idempotent.
int tbv_ar_init(int rank, const char* devs, const char* peer_ip, int port, size_t cap);
int tbv_ar_init_n(int rank, int world, int device, const char* peer_ip, int port, size_t cap);
int tbv_ar_allreduce(const void* in, void* out, size_t nbytes, int dtype, void* stream);
void tbv_ar_stats(double* xfer_us, unsigned long long* n);
void tbv_ar_stats4(double* pre, double* xfer, double* post, double* enq, unsigned long long* n);
void tbv_ar_stats5(double* pre, double* xfer, double* post, double* enq, double* drain,
                   unsigned long long* n);
int tbv_ar_cap(void);          // clamps at INT_MAX
size_t tbv_ar_cap64(void);
int tbv_ar_async(void);
int tbv_ar_err(void);
void tbv_ar_rails(void);
void tbv_ar_hist(void);
int tbv_ar_sync(void);
int tbv_ar_fini(void);
tbv_comm* tbv_ar_comm(void);   // the global communicator (NULL before init)

#ifdef __cplusplus
}
#endif
