// gemm_ar.cu — row-parallel linear fused with its all-reduce, the residual add and the
// RMSNorm that follows it, in ONE kernel over peer memory:
//
//   partial = X[T, K/tp] @ W[H, K/tp]^T            tcgen05 tiles, TMA-fed, TMEM accumulators
//   Every CTA is a GEMM CTA: a finished tile slice is rounded to bf16 and stored straight into the LL
//   packet area of EVERY rank (8-byte pieces through the NVLink peer mappings, each carrying 4 bytes
//   of payload and the call's sequence number — the epilogue IS the transfer, there is no fence and
//   no flag).  The CTA then takes a ticket from a per-rank counter.  All but the last few give their
//   SM back; the LAST min(T, 16) CTAs of a rank to finish stay as finishers, one or more token rows
//   each: they poll the row's packets of all ranks as they land, add the N copies in rank order in
//   fp32, round, add the residual, and apply RMSNorm.
//
// Nothing waits for a kernel boundary between the GEMM and the reduction, nobody sits idle while the
// weights stream (an earlier form kept dedicated finisher CTAs resident from the start: they held
// GEMM-sized shared-memory slots and delayed the last tiles), and the push is spread over every SM
// that ran a tile — an SM hands only one 32-byte sector per clock to the fabric.  This is what the
// reference's hook wraps as two separate steps (RowParallelLinear, then GroupCoordinator.all_reduce:
// step3b/vllm_tp_bench.py:87-124) plus the norm it lists as future work ("fuse k_acc + next RMSNorm",
// reports/12_references.md:136).
//
// Semantics are those of the unfused pipeline, bit for bit: the all-reduce operands are the bf16
// partial sums, the sum is fp32 in rank order with one rounding, and the row normalisation forms
// its sums in the order of the plain RMSNorm kernel (rmsnorm_row_store_virtual).
//
// Messages too large for LL packets (TBV_LL_MAX) are declined (TBV_FALLBACK): the caller composes
// GEMM + fused all-reduce/norm, or the sequence-parallel GEMM -> reduce-scatter pair.
//
// Also here: the emulated-ranks form (blockIdx.y = rank, all ranks on one GPU) used to test
// the protocol on a single GPU.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include <algorithm>

#include "../comm.h"
#include "gemm.cuh"
#include "ops.h"

using namespace sm100;
using namespace tbv;

namespace {

struct Maps {
  CUtensorMap a[TBV_MAXRANK];  // weights of (emulated) rank r
  CUtensorMap b[TBV_MAXRANK];  // activations of rank r
};
struct FusedPtrs {
  const __nv_bfloat16* residual[TBV_MAXRANK];
  __nv_bfloat16* residual_out[TBV_MAXRANK];
  __nv_bfloat16* y[TBV_MAXRANK];
};
// 256 threads and at most 128 registers: two CTAs fit on an SM, like the plain GEMM kernel when its grid is
// larger than the GPU (512-thread CTAs ran the 256 tiles of a down projection in two waves and doubled its time).
constexpr int kFusedThreads = 256;   // warps 0..5 have the GEMM roles; all 8 warps work in a finisher CTA
constexpr int kMaxFinishers = 16;    // finisher CTAs per rank (rows are dealt round robin beyond that)
constexpr int kFusedVPT = 4;         // 16-byte units per finisher thread: hidden <= 8 * 4 * 256 = 8192

// grid (m_tiles, ranks, S), cluster (1, 1, S)
__global__ void __launch_bounds__(kFusedThreads, 2)
k_gemm_ar_rmsnorm(const __grid_constant__ Maps maps, const gemm::Params p, const RankCtx* ctxs, const __grid_constant__ FusedPtrs fp,
                  const __nv_bfloat16* gamma, float eps, int finishers, int norm_threads, int mute) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ gemm::Smem s;
  __shared__ unsigned long long sh_seq;
  __shared__ float sh_red[64];
  __shared__ int sh_fid;
  const int er = blockIdx.y;  // (emulated) rank index into the per-rank arrays; 0 for a real rank
  if (er == mute) return;     // emulated world, host-made fault: this rank never makes the call
  const RankCtx& c = ctxs[er];
  const int S = p.splits;
  const int split = S > 1 ? int(cluster_ctarank()) : 0;
  const int T = p.N, H = p.M;
  const unsigned n_cta = unsigned(gridDim.x) * unsigned(S);

  // ---------------- GEMM CTA: one 128-feature tile over its K range, pushed as LL packets ----------------
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tile = blockIdx.x, m0 = m_tile * gemm::kBM;
  const bool stamp = blockIdx.x == gridDim.x - 1 && cluster_ctarank() == 0;   // the last tile in launch order
  if (stamp && threadIdx.x == 0) c.dm->ts[5] = tbv::globaltimer();           // its CTA is resident
  if (m_tile == 0 && split == 0 && threadIdx.x == 0) c.dm->ts[0] = tbv::globaltimer();   // the first tile's CTA is resident
  const int kb_per = (p.kb_total + S - 1) / S;
  const int kb0 = split * kb_per;
  int nkb = p.kb_total - kb0;
  nkb = nkb < 0 ? 0 : (nkb > kb_per ? kb_per : nkb);

  uint8_t* sm = gemm::mainloop(&maps.a[er], &maps.b[er], p, s, smem_raw, m0, 0, kb0, nkb);
  volatile int* abortp = &s.abort_flag;
  float* stage_f = reinterpret_cast<float*>(sm);
  const bool epi = warp >= 2 && warp < 6;

  if (epi) {
    const int quarter = warp & 3, ml = quarter * 32 + lane;
    bool ok = nkb > 0 ? mbar_wait(smem_u32(&s.accum), 0, abortp, p.limit_ns) : true;
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    // The accumulator is complete, so the producer has passed its dependency wait: the
    // previous collective has finished and the device sequence number is stable.
    if (threadIdx.x == 64) {
      sh_seq = *(volatile unsigned long long*)&c.st->seq + 1ull;
      if (stamp) c.dm->ts[6] = tbv::globaltimer();   // its accumulator is complete
    }
    for (int col = 0; col < p.bn; col += 16) {
      uint32_t r[16];
      if (ok && nkb > 0) {
        tmem_ld16(s.tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(col), r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 16; j++) r[j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 16; j++) stage_f[(col + j) * 128 + ml] = __uint_as_float(r[j]);
    }
  }
  __syncwarp();
  if (S > 1) cluster_sync_all(); else __syncthreads();
  CallInfo ci;
  ci.seq = sh_seq;   // every CTA of the cluster read the same device word; this is the CTA's own copy
  ci.want = unsigned(ci.seq);
  ci.slot = int(ci.seq % (unsigned long long)c.nslot);

  if (epi) {
    // deterministic split-K (CTA j reduces feature slice j over the cluster's K ranges), then the
    // bf16 slice goes to EVERY rank's LL area [src = me], own rank included: the finishers read all
    // sources the same way
    const int te = threadIdx.x - 64;
    const int fs = 128 / S, q4 = fs / 4;
    const uint32_t stage_addr = smem_u32(sm);
    for (int idx = te; idx < T * q4; idx += 128) {
      const int t = idx / q4, f = split * fs + (idx % q4) * 4;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (S > 1) {
        acc = dsmem_sum_f32x4(stage_addr + uint32_t((t * 128 + f) * 4), S);
      } else {
        acc = *reinterpret_cast<const float4*>(stage_f + t * 128 + f);
      }
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      const size_t off = (size_t(t) * H + m0 + f) * 2;   // payload byte offset; packets take twice that
      for (int d = 0; d < c.world; d++) {
        const int peer = (c.rank + d) % c.world;
        st_v4(ll_region(c, peer, ci.slot, c.rank) + off * 2, pk.x, ci.want, pk.y, ci.want);
      }
    }
  }
  __syncwarp();
  if (S > 1) cluster_sync_all(); else __syncthreads();  // peers' shared memory is no longer needed; this CTA's packets are issued
  if (threadIdx.x == 0) {
    // ticket: the last `finishers` CTAs of this rank to get here reduce and normalise the rows
    const unsigned old = atomicAdd(&c.st->gemm_done, 1u);
    sh_fid = old + unsigned(finishers) >= n_cta ? int(old + unsigned(finishers) - n_cta) : -1;
    if (stamp) c.dm->ts[7] = tbv::globaltimer();     // its packets are issued
    if (m_tile == 0 && split == 0) c.dm->bc[1] = ci.seq;
  }
  gemm::teardown(p, s);      // tensor memory goes back before any waiting starts
  __syncthreads();
  const int fid = sh_fid;
  unsigned long long t_enter = 0, t_ready = 0;
  if (fid >= 0) {
    // ---------------- finisher: reduce + residual + RMSNorm of its token rows ----------------
    const bool lead = fid == 0 && threadIdx.x == 0;
    if (lead) { t_enter = c.dm->ts[0]; c.dm->bc[0] = ci.seq; c.dm->ts[1] = c.dm->ts[0]; c.dm->ts[2] = tbv::globaltimer(); }   // nearly all of this rank's tiles are pushed
    const int upr = H / 8;
    const unsigned all = (1u << c.world) - 1u;   // own rank included: its CTAs write packets here too
    for (int row = fid; row < T; row += finishers) {
      float h[kFusedVPT][8];
#pragma unroll
      for (int j = 0; j < kFusedVPT; j++) {
        const int u = threadIdx.x + j * blockDim.x;
        if (u < upr) {
          const size_t off = size_t(row) * upr + u;
          uint4 got[TBV_MAXRANK];
          ll_pull_all(c, ci.slot, off, ci.want, all, fid, ci.seq, got);
          float acc[8];
          ll_sum_unit<__nv_bfloat16>(c, got, all, got[0], acc);
          float res[8];
          Pack<__nv_bfloat16>::unpack(reinterpret_cast<const uint4*>(fp.residual[er])[off], res);
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const float sum = __bfloat162float(__float2bfloat16_rn(acc[i]));
            h[j][i] = __bfloat162float(__float2bfloat16_rn(sum + res[i]));
          }
          reinterpret_cast<uint4*>(fp.residual_out[er])[off] = Pack<__nv_bfloat16>::pack(h[j]);
        }
      }
      if (row == fid && lead) { t_ready = tbv::globaltimer(); c.dm->bc[2] = ci.seq; c.dm->ts[3] = t_ready; }   // first row's packets pulled
      rmsnorm_row_store_virtual<kFusedVPT>(h, upr, H, eps, reinterpret_cast<const uint4*>(gamma),
                                           reinterpret_cast<uint4*>(fp.y[er]) + size_t(row) * upr, sh_red, norm_threads);
    }
    if (lead) c.dm->ts[4] = tbv::globaltimer();   // rows normalised
  }
  call_end(c, ci, n_cta, t_enter, t_ready, size_t(T) * H * 2, TBV_ALGO_LL);
}

bool g_attr_done = false;

}  // namespace

// w/x/residual/residual_out/y: one pointer per (emulated) rank; a real rank passes arrays of 1.
static int launch_fused(tbv_comm* c, const void* const* ws, const void* const* xs, const void* const* residuals, const void* gamma,
                        void* const* residual_outs, void* const* ys, int tokens, int hidden, int k_local, int ldx, float eps,
                        void* stream) {
  const int nr = c->local ? c->world : 1;
  if (c->cpu || c->ranks.empty() || c->world < 2) return TBV_FALLBACK;
  if (c->sticky_err.load()) return TBV_FAIL;
  for (auto& g : c->ranks)
    if (*(volatile unsigned*)&g.hm->err != 0) { c->sticky_err.store(1); return TBV_FAIL; }
  const size_t nbytes = size_t(tokens) * hidden * 2;
  // every condition below depends on the shape and the knobs only, so all ranks decide alike
  if (tokens <= 0 || tokens > 256 || hidden % 128 || hidden > 8 * kFusedVPT * kFusedThreads || (k_local % 8) || (ldx % 8)) return TBV_FALLBACK;
  if (!(c->knobs.algo == TBV_ALGO_AUTO || c->knobs.algo == TBV_ALGO_LL) || nbytes * 2 > c->ll_cap || long(nbytes) > c->knobs.ll_max)
    return TBV_FALLBACK;
  for (int r = 0; r < nr; r++)
    if ((reinterpret_cast<uintptr_t>(residuals[r]) | reinterpret_cast<uintptr_t>(residual_outs[r]) | reinterpret_cast<uintptr_t>(ys[r]) |
         reinterpret_cast<uintptr_t>(gamma)) & 15u)
      return TBV_FAIL;   // a per-rank property: declining would leave the other ranks alone in the call
  if (c->skip.load() > 0) { c->skip.fetch_sub(1); return TBV_OK; }
  int bn, splits, stages;
  tbvops::gemm_config(hidden, tokens, k_local, 0, &bn, &splits, &stages);
  if ((tokens + bn - 1) / bn != 1) return TBV_FALLBACK;
  const int n_gemm = (hidden / 128) * splits;
  const int finishers = std::min(std::min(tokens, kMaxFinishers), n_gemm);
  if (c->local) {
    // Emulated ranks share one GPU and their finishers wait for the other ranks' tiles: every rank's finishers
    // and at least one more cluster must fit on the GPU at the same time.
    if (nr * finishers + splits > tbvops::sm_count()) return TBV_FALLBACK;
  }
  // The two-CTAs-per-SM shared-memory budget: the next kernel's CTAs must find room beside this kernel's
  // finishers, or they cannot stream their weights while the finishers wait for the peers.
  {
    const int stage_bytes = gemm::kATileBytes + bn * 128;
    const int fit = (108 * 1024) / stage_bytes;
    if (stages > fit) stages = fit < 2 ? 2 : fit;
  }
  while (stages * (gemm::kATileBytes + bn * 128) < bn * 512) stages++;  // fp32 staging reuses the ring
  Maps maps;
  FusedPtrs fp{};
  for (int r = 0; r < nr; r++) {
    if (tbvops::make_tensor_map_bf16(&maps.a[r], ws[r], hidden, k_local, k_local, 128) != 0) return TBV_FAIL;
    if (tbvops::make_tensor_map_bf16(&maps.b[r], xs[r], tokens, k_local, ldx, bn) != 0) return TBV_FAIL;
    fp.residual[r] = static_cast<const __nv_bfloat16*>(residuals[r]);
    fp.residual_out[r] = static_cast<__nv_bfloat16*>(residual_outs[r]);
    fp.y[r] = static_cast<__nv_bfloat16*>(ys[r]);
  }
  gemm::Params p{};
  p.M = hidden; p.N = tokens; p.K = k_local; p.ldy = hidden; p.bn = bn; p.splits = splits; p.stages = stages;
  p.kb_total = (k_local + 63) / 64;
  p.limit_ns = 2000000000ull;
  p.err = tbvops::gemm_err_flag();
  p.pf_bytes = tbvops::take_next_prefetch(&p.pf_ptr, (unsigned long long)hidden * (unsigned long long)k_local * 2ull);
  const size_t smem = size_t(stages) * (gemm::kATileBytes + bn * 128) + 1024;
  if (!g_attr_done) {
    if (cudaFuncSetAttribute(k_gemm_ar_rmsnorm, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) return TBV_FAIL;
    g_attr_done = true;
  }
  const RankCtx* ctxs = c->ctxs_dev;
  int mute = -1;
  if (c->local && c->mute_left.load() > 0) { c->mute_left.fetch_sub(1); mute = c->mute_rank; }
  cudaError_t e = pdl::launch(k_gemm_ar_rmsnorm, dim3(hidden / 128, nr, splits), dim3(kFusedThreads), smem,
                              static_cast<cudaStream_t>(stream), splits, maps, p, ctxs, fp, static_cast<const __nv_bfloat16*>(gamma), eps,
                              finishers, tbvops::norm_threads(hidden), mute);
  if (e != cudaSuccess) {
    fprintf(stderr, "[tbvcoll] fused gemm+all-reduce launch failed: %s\n", cudaGetErrorString(e));
    c->sticky_err.store(1);
    return TBV_FAIL;
  }
  c->host_seq++;
  return TBV_OK;
}

extern "C" {

// y = RMSNorm(h) * gamma with h = bf16(sum over ranks of bf16(x @ w^T)) + residual; residual_out = h.
// x: [tokens, k_local] (row stride ldx), w: [hidden, k_local] — this rank's shard of a row-parallel layer.
// hidden % 128 == 0, hidden <= 8192, tokens * hidden * 2 bytes within the LL packet limit (TBV_LL_MAX).
// TBV_FALLBACK (-2): compose gemm + all-reduce + add-norm instead (decided from shape and knobs only,
// so every rank gets the same answer).
int tbv_comm_gemm_allreduce_rmsnorm(tbv_comm* c, const void* w, const void* x, const void* residual, const void* gamma,
                                    void* residual_out, void* y, int tokens, int hidden, int k_local, int ldx, float eps,
                                    void* stream) {
  if (!c || c->local) return TBV_FAIL;
  tbv::NvtxRange nvtx("tbv.gemm_allreduce_rmsnorm", size_t(tokens) * hidden * 2);
  return launch_fused(c, &w, &x, &residual, gamma, &residual_out, &y, tokens, hidden, k_local, ldx, eps, stream);
}

int tbv_comm_gemm_allreduce_rmsnorm_local(tbv_comm* c, const void* const* ws, const void* const* xs, const void* const* residuals,
                                          const void* gamma, void* const* residual_outs, void* const* ys, int tokens, int hidden,
                                          int k_local, int ldx, float eps, void* stream) {
  if (!c || !c->local) return TBV_FAIL;
  return launch_fused(c, ws, xs, residuals, gamma, residual_outs, ys, tokens, hidden, k_local, ldx, eps, stream);
}

}  // extern "C"
