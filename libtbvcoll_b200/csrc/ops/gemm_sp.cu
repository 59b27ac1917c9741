// gemm_sp.cu — the two fused GEMM + collective pairs of sequence-parallel prefill.
//
//  GEMM -> reduce-scatter (row-parallel layer, tokens end up sharded):
//    k_gemm_scatter   tcgen05 GEMM; the epilogue of every 128 x BN tile stores the bf16 tile
//                     straight into the slot memory of the rank that owns those token rows and
//                     raises one flag per tile there — the transfer rides on the math, tile by tile.
//    k_rs_reduce_norm one CTA per owned row: waits for the row's tiles from every rank, adds
//                     them in rank order (fp32, one rounding) and optionally applies
//                     residual add + RMSNorm on the local T/N rows.
//  all-gather -> GEMM (column-parallel layer, input tokens sharded):
//    k_ag_push        copies this rank's rows into every rank's gather buffer, one flag per
//                     BN-row chunk.
//    k_ag_gemm        tcgen05 GEMM whose TMA producer waits for the flag of the chunk a tile
//                     needs and then loads it from THIS GPU's memory (plain tiled TMA, no cluster
//                     multicast, never a peer address); tiles over local rows start at once.
//
// The reference has no sequence-parallel path (it only cites the idea of running RMSNorm on
// 1/N of the tokens after a reduce-scatter, reports/12_references.md:45-46).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include <vector>

#include "../comm.h"
#include "gemm.cuh"
#include "ops.h"

using namespace sm100;
using namespace tbv;

namespace {

struct Maps {
  CUtensorMap a[TBV_MAXRANK];
  CUtensorMap b[TBV_MAXRANK];
};

// ---------------------------------------------------------------- GEMM -> scatter
// grid (n_tiles * nr, m_tiles, 1): token tiles are the fastest launch index, so the CTAs that share one 128-row
// weight tile run together and the weights stream from HBM once; tokens [T], rows_per_rank = T / world, rows_per_rank % bn == 0.
__global__ void __launch_bounds__(gemm::kThreads, 1)
k_gemm_scatter(const __grid_constant__ Maps maps, const gemm::Params p, const RankCtx* ctxs, int n_tiles, int rows_per_rank) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ gemm::Smem s;
  __shared__ unsigned long long sh_seq;
  const int er = blockIdx.x / n_tiles, n_tile = blockIdx.x % n_tiles;
  const RankCtx& c = ctxs[er];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tile = blockIdx.y, m0 = m_tile * gemm::kBM, n0 = n_tile * p.bn;
  const unsigned long long t_enter = (threadIdx.x == 0 && m_tile == 0 && n_tile == 0) ? tbv::globaltimer() : 0;
  uint8_t* sm = gemm::mainloop(&maps.a[er], &maps.b[er], p, s, smem_raw, m0, n0, 0, p.kb_total);
  volatile int* abortp = &s.abort_flag;
  __nv_bfloat16* stage_h = reinterpret_cast<__nv_bfloat16*>(sm);
  const int H = p.M;
  if (warp >= 2) {
    const int quarter = warp & 3, ml = quarter * 32 + lane;
    bool ok = mbar_wait(smem_u32(&s.accum), 0, abortp, p.limit_ns);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    if (threadIdx.x == 64) sh_seq = *(volatile unsigned long long*)&c.st->seq + 1ull;  // stable: the producer passed its dependency wait
    for (int col = 0; col < p.bn; col += 16) {
      uint32_t r[16];
      if (ok) {
        tmem_ld16(s.tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(col), r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 16; j++) r[j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 16; j++) stage_h[(col + j) * 128 + ml] = __float2bfloat16_rn(__uint_as_float(r[j]));
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const unsigned long long seq = sh_seq;
    const int slot = int(seq % (unsigned long long)c.nslot);
    const int dest = n0 / rows_per_rank, row0 = n0 % rows_per_rank;
    char* region = slot_region(c, dest, slot, c.rank);
    const int te = threadIdx.x - 64;
    for (int idx = te; idx < p.bn * 16; idx += 128) {  // 16 pieces of 16 bytes per 128-feature row
      const int t = idx >> 4, pc = idx & 15;
      *reinterpret_cast<uint4*>(region + (size_t(row0 + t) * H + m0 + pc * 8) * 2) =
          *reinterpret_cast<const uint4*>(stage_h + t * 128 + pc * 8);
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (threadIdx.x == 64) {
      fence_sys();
      const int chan = (row0 / p.bn) * gridDim.y + m_tile;
      st_relaxed_sys(c.flags[dest] + flag_index(c, slot, 0, c.rank, chan), unsigned(seq));
    }
  }
  __syncwarp();
  gemm::teardown(p, s);
  CallInfo ci;
  ci.seq = sh_seq;   // written before the epilogue barrier; teardown's __syncthreads publishes it to all warps
  ci.want = unsigned(ci.seq);
  ci.slot = int(ci.seq % (unsigned long long)c.nslot);
  call_end(c, ci, gridDim.y * unsigned(n_tiles), t_enter, 0, size_t(p.N) * H * 2, TBV_ALGO_TWOSHOT);
}

// grid (rows_per_rank, nr); block = norm_threads(H).  mode 0: out = sum; mode 1: h = sum + residual ->
// residual_out, y = RMSNorm(h) * gamma.
struct RsPtrs {
  __nv_bfloat16* out[TBV_MAXRANK];
  const __nv_bfloat16* residual[TBV_MAXRANK];
  __nv_bfloat16* residual_out[TBV_MAXRANK];
  __nv_bfloat16* y[TBV_MAXRANK];
};
__global__ void __launch_bounds__(1024)
k_rs_reduce_norm(const RankCtx* ctxs, const __grid_constant__ RsPtrs ptrs, const __nv_bfloat16* gamma, int H, int bn, int m_tiles,
                 float eps, int mode) {
  __shared__ float sh[32];
  pdl::launch_dependents();
  pdl::grid_dependency_wait();   // the local GEMM has finished: the device sequence number names this call
  const int er = blockIdx.y, row = blockIdx.x;
  const RankCtx& c = ctxs[er];
  const unsigned long long seq = *(volatile unsigned long long*)&c.st->seq;
  const int slot = int(seq % (unsigned long long)c.nslot);
  const int chan0 = (row / bn) * m_tiles;
  for (int i = threadIdx.x; i < c.world * m_tiles; i += blockDim.x) {
    const int src = i / m_tiles, mt = i % m_tiles;
    wait_flag(c, c.flags[c.rank] + flag_index(c, slot, 0, src, chan0 + mt), unsigned(seq), kWhereFused, src, chan0 + mt, seq);
  }
  __syncthreads();
  const int upr = H / 8;
  float h[kNormMaxUnits][8];
#pragma unroll
  for (int k = 0; k < kNormMaxUnits; k++) {
    const int u = threadIdx.x + k * blockDim.x;
    if (u < upr) {
      const size_t off = size_t(row) * upr + u;
      float acc[8];
      uint4 got[TBV_MAXRANK];
      const unsigned all = (1u << c.world) - 1u;
      gather_units(c, c.rank, slot, off, all, got);
      sum_units_rank_order<__nv_bfloat16>(c, got, all, got[0], acc);
      if (mode == 0) {
        reinterpret_cast<uint4*>(ptrs.out[er])[off] = Pack<__nv_bfloat16>::pack(acc);
      } else {
        float res[8];
        Pack<__nv_bfloat16>::unpack(reinterpret_cast<const uint4*>(ptrs.residual[er])[off], res);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float sum = __bfloat162float(__float2bfloat16_rn(acc[i]));
          h[k][i] = __bfloat162float(__float2bfloat16_rn(sum + res[i]));
        }
        reinterpret_cast<uint4*>(ptrs.residual_out[er])[off] = Pack<__nv_bfloat16>::pack(h[k]);
      }
    }
  }
  if (mode != 0)
    rmsnorm_row_store(h, upr, H, eps, reinterpret_cast<const uint4*>(gamma), reinterpret_cast<uint4*>(ptrs.y[er]) + size_t(row) * upr, sh);
}

// ---------------------------------------------------------------- all-gather -> GEMM
// grid (chunks, nr); chunk = bn rows of this rank's [rows_per_rank, K] block.
struct AgPtrs { const __nv_bfloat16* x[TBV_MAXRANK]; };
__global__ void __launch_bounds__(512)
k_ag_push(const RankCtx* ctxs, const __grid_constant__ AgPtrs ptrs, int K, int ldx, int bn, int rows_per_rank) {
  __shared__ unsigned long long sh_seq;
  pdl::launch_dependents();
  pdl::grid_dependency_wait();
  const int er = blockIdx.y, chunk = blockIdx.x;
  const RankCtx& c = ctxs[er];
  const unsigned long long t_enter = (threadIdx.x == 0 && chunk == 0) ? tbv::globaltimer() : 0;
  CallInfo ci = call_begin(c, &sh_seq);
  const int upr = K / 8;
  const int r0 = chunk * bn, r1 = min(rows_per_rank, r0 + bn);
  for (int idx = threadIdx.x; idx < (r1 - r0) * upr; idx += blockDim.x) {
    const int t = r0 + idx / upr, u = idx % upr;
    const uint4 v = *reinterpret_cast<const uint4*>(ptrs.x[er] + size_t(t) * ldx + u * 8);
    for (int d = 0; d < c.world; d++) {
      const int peer = (c.rank + d) % c.world;
      reinterpret_cast<uint4*>(slot_region(c, peer, ci.slot, c.rank))[size_t(t) * upr + u] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_sys();
    for (int peer = 0; peer < c.world; peer++) st_relaxed_sys(c.flags[peer] + flag_index(c, ci.slot, 0, c.rank, chunk), ci.want);
  }
  call_end(c, ci, gridDim.x, t_enter, 0, size_t(rows_per_rank) * K * 2, TBV_ALGO_TWOSHOT);
}

// grid (n_tiles_total, m_tiles, nr): token tiles fastest (the per-rank weights stream from HBM once, not once per
// token tile); the n tile order is rotated so that this rank's own rows come first.
struct AgOut { __nv_bfloat16* y[TBV_MAXRANK]; const CUtensorMap* gathered[TBV_MAXRANK]; };  // gathered[er]: [nslot * world] maps
__global__ void __launch_bounds__(gemm::kThreads, 1)
k_ag_gemm(const __grid_constant__ Maps maps, const gemm::Params p, const RankCtx* ctxs, const __grid_constant__ AgOut ao, int tiles_per_src) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ gemm::Smem s;
  const int er = blockIdx.z;
  const RankCtx& c = ctxs[er];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int src = (c.rank + blockIdx.x / tiles_per_src) % c.world, j = blockIdx.x % tiles_per_src;
  const int m0 = blockIdx.y * gemm::kBM;
  const int rows_per_rank = tiles_per_src * p.bn;
  const int n0_global = src * rows_per_rank + j * p.bn;
  // -- set-up identical to gemm::mainloop, but the producer resolves its activation tile first
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const uint32_t b_tile_bytes = uint32_t(p.bn) * 128u;
  const uint32_t a_base = base, b_base = base + uint32_t(p.stages) * gemm::kATileBytes;
  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; i++) { mbar_init(smem_u32(&s.full[i]), 1); mbar_init(smem_u32(&s.empty[i]), 1); }
    mbar_init(smem_u32(&s.accum), 1);
    s.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(&s.tmem_base), gemm::tmem_cols(p.bn)); tmem_relinquish(); }
  if (warp == 0 && lane == 0) tma_prefetch_desc(&maps.a[er]);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl::launch_dependents();
  const uint32_t tmem_d = s.tmem_base;
  volatile int* abortp = &s.abort_flag;
  const int nkb = p.kb_total;
  if (warp == 0 && lane == 0) {
    const uint64_t pol_w = policy_evict_last();   // prefill: weights are re-read by every token tile
    const uint64_t pol_x = policy_evict_last();
    const int pre = nkb < p.stages ? nkb : p.stages;
    for (int i = 0; i < pre; i++) {
      const uint32_t fb = smem_u32(&s.full[i]);
      mbar_expect_tx(fb, gemm::kATileBytes + b_tile_bytes);
      tma_load_2d_hint(a_base + i * gemm::kATileBytes, &maps.a[er], i * gemm::kBK, m0, fb, pol_w);
    }
    pdl::grid_dependency_wait();  // my own push kernel has finished: seq names this gather
    const unsigned long long seq = *(volatile unsigned long long*)&c.st->seq;
    const int slot = int(seq % (unsigned long long)c.nslot);
    // rows of another rank: wait until that chunk has landed in MY memory, then make the
    // (generic-proxy) peer stores visible to the TMA (async proxy) reads that follow
    wait_flag(c, c.flags[c.rank] + flag_index(c, slot, 0, src, j), unsigned(seq), kWherePhase0, src, j, seq);
    asm volatile("fence.proxy.async;" ::: "memory");
    const CUtensorMap* tmB = ao.gathered[er] + slot * c.world + src;
    for (int i = 0; i < pre; i++)
      tma_load_2d_hint(b_base + i * b_tile_bytes, tmB, i * gemm::kBK, j * p.bn, smem_u32(&s.full[i]), pol_x);
    for (int i = pre; i < nkb; i++) {
      const int st = i % p.stages;
      const uint32_t ph = uint32_t(i / p.stages) & 1u;
      if (!mbar_wait(smem_u32(&s.empty[st]), ph ^ 1u, abortp, p.limit_ns)) break;
      const uint32_t fb = smem_u32(&s.full[st]);
      mbar_expect_tx(fb, gemm::kATileBytes + b_tile_bytes);
      tma_load_2d_hint(a_base + st * gemm::kATileBytes, &maps.a[er], i * gemm::kBK, m0, fb, pol_w);
      tma_load_2d_hint(b_base + st * b_tile_bytes, tmB, i * gemm::kBK, j * p.bn, fb, pol_x);
    }
  } else if (warp == 1 && lane == 0) {
    const uint32_t idesc = umma_idesc_bf16(gemm::kBM, uint32_t(p.bn));
    for (int i = 0; i < nkb; i++) {
      const int st = i % p.stages;
      const uint32_t ph = uint32_t(i / p.stages) & 1u;
      if (!mbar_wait(smem_u32(&s.full[st]), ph, abortp, p.limit_ns)) break;
      tc_fence_after();
      const uint64_t ad = umma_desc_sw128(a_base + st * gemm::kATileBytes);
      const uint64_t bd = umma_desc_sw128(b_base + st * b_tile_bytes);
#pragma unroll
      for (int k = 0; k < gemm::kBK / 16; k++) umma_bf16(tmem_d, ad + uint64_t(2 * k), bd + uint64_t(2 * k), idesc, (i | k) != 0 ? 1u : 0u);
      umma_commit(smem_u32(&s.empty[st]));
    }
    umma_commit(smem_u32(&s.accum));
  }
  if (warp >= 2) {
    const int quarter = warp & 3, ml = quarter * 32 + lane;
    bool ok = mbar_wait(smem_u32(&s.accum), 0, abortp, p.limit_ns);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    __nv_bfloat16* stage_h = reinterpret_cast<__nv_bfloat16*>(sm);
    for (int col = 0; col < p.bn; col += 16) {
      uint32_t r[16];
      if (ok) { tmem_ld16(s.tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(col), r); tmem_ld_wait(); }
      else {
#pragma unroll
        for (int q = 0; q < 16; q++) r[q] = 0u;
      }
#pragma unroll
      for (int q = 0; q < 16; q++) stage_h[(col + q) * 128 + ml] = __float2bfloat16_rn(__uint_as_float(r[q]));
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int te = threadIdx.x - 64;
    for (int idx = te; idx < p.bn * 16; idx += 128) {
      const int t = idx >> 4, pc = idx & 15, m = m0 + pc * 8;
      if (m + 8 <= p.M)
        *reinterpret_cast<uint4*>(ao.y[er] + size_t(n0_global + t) * p.ldy + m) = *reinterpret_cast<const uint4*>(stage_h + t * 128 + pc * 8);
      else
        for (int e = 0; e < 8 && m + e < p.M; e++) ao.y[er][size_t(n0_global + t) * p.ldy + m + e] = stage_h[t * 128 + pc * 8 + e];
    }
  }
  __syncwarp();
  gemm::teardown(p, s);
}

bool g_attr = false;
int set_attrs() {
  if (g_attr) return 0;
  if (cudaFuncSetAttribute(k_gemm_scatter, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) return -1;
  if (cudaFuncSetAttribute(k_ag_gemm, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) return -1;
  g_attr = true;
  return 0;
}

// Device array of tensor maps over the gather buffers of (emulated) rank `er`, one map per (slot, source).
// The communicator owns it (built on first use per shape, freed in tbv_comm_destroy): the maps name
// addresses inside that communicator's slot memory and must not outlive it.
const CUtensorMap* gather_maps(tbv_comm* c, int er, int rows_per_rank, int K, int bn) {
  auto key = std::make_tuple(er, rows_per_rank, K, bn);
  auto it = c->gather_maps.find(key);
  if (it != c->gather_maps.end()) return static_cast<const CUtensorMap*>(it->second);
  const RankCtx& x = c->ranks[er].ctx;
  std::vector<CUtensorMap> host(size_t(x.nslot) * x.world);
  for (int slot = 0; slot < x.nslot; slot++)
    for (int src = 0; src < x.world; src++) {
      const char* base = x.data[x.rank] + size_t(slot) * x.slot_stride + size_t(src) * x.cap;
      if (tbvops::make_tensor_map_bf16(&host[size_t(slot) * x.world + src], base, rows_per_rank, K, K, bn, /*cache=*/false) != 0) return nullptr;
    }
  CUtensorMap* dev = nullptr;
  if (cudaMalloc(&dev, host.size() * sizeof(CUtensorMap)) != cudaSuccess) return nullptr;  // first use must not be under stream capture
  if (cudaMemcpy(dev, host.data(), host.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice) != cudaSuccess) { cudaFree(dev); return nullptr; }
  c->gather_maps[key] = dev;
  return dev;
}

int precheck(tbv_comm* c) {
  if (!c || c->cpu || c->ranks.empty() || c->world < 2) return TBV_FALLBACK;
  if (c->sticky_err.load()) return TBV_FAIL;
  for (auto& g : c->ranks)
    if (*(volatile unsigned*)&g.hm->err != 0) { c->sticky_err.store(1); return TBV_FAIL; }
  return TBV_OK;
}

int pick_bn(int rows_per_rank) {
  for (int bn : {256, 128, 64, 32, 16})
    if (rows_per_rank % bn == 0) return bn;
  return 0;
}

}  // namespace

// ---- GEMM -> reduce-scatter (+ residual + RMSNorm on the local rows) ---------------------------
// x: [T, k_local] (all tokens, this rank's input features), w: [H, k_local].  The rank-ordered sum
// of all ranks' x @ w^T is scattered by token rows: this rank receives rows [rank*T/N, (rank+1)*T/N).
// mode 0: out[T/N, H] = the sum.  mode 1: h = sum + residual[T/N, H] -> residual_out; y = RMSNorm(h) * gamma.
static int launch_gemm_rs(tbv_comm* c, const void* const* ws, const void* const* xs, void* const* outs, const void* const* residuals,
                          const void* gamma, void* const* residual_outs, void* const* ys, int T, int H, int k_local, int ldx,
                          float eps, int mode, void* stream) {
  int rc = precheck(c);
  if (rc != TBV_OK) return rc;
  const int nr = c->local ? c->world : 1, W = c->world;
  if (T <= 0 || T % W || H % 128 || (k_local % 8) || (ldx % 8) || H > 8 * kNormMaxUnits * 1024) return TBV_FALLBACK;
  const int rpr = T / W, bn = pick_bn(rpr);
  if (!bn || size_t(rpr) * H * 2 > c->cap || (rpr / bn) * (H / 128) > TBV_MAXCHAN) return TBV_FALLBACK;
  if (c->skip.load() > 0) { c->skip.fetch_sub(1); return TBV_OK; }
  if (set_attrs() != 0) return TBV_FAIL;
  const int n_tiles = T / bn, m_tiles = H / 128;
  const int stage_bytes = gemm::kATileBytes + bn * 128;
  int stages = (200 * 1024) / stage_bytes;
  stages = stages > gemm::kMaxStages ? gemm::kMaxStages : (stages < 2 ? 2 : stages);
  Maps maps;
  RsPtrs rp{};
  for (int r = 0; r < nr; r++) {
    if (tbvops::make_tensor_map_bf16(&maps.a[r], ws[r], H, k_local, k_local, 128) != 0) return TBV_FALLBACK;
    if (tbvops::make_tensor_map_bf16(&maps.b[r], xs[r], T, k_local, ldx, bn) != 0) return TBV_FALLBACK;
    rp.out[r] = static_cast<__nv_bfloat16*>(outs ? outs[r] : nullptr);
    rp.residual[r] = static_cast<const __nv_bfloat16*>(residuals ? residuals[r] : nullptr);
    rp.residual_out[r] = static_cast<__nv_bfloat16*>(residual_outs ? residual_outs[r] : nullptr);
    rp.y[r] = static_cast<__nv_bfloat16*>(ys ? ys[r] : nullptr);
  }
  gemm::Params p{};
  p.M = H; p.N = T; p.K = k_local; p.ldy = H; p.bn = bn; p.splits = 1; p.stages = stages; p.kb_total = (k_local + 63) / 64;
  p.limit_ns = 2000000000ull;
  p.err = tbvops::gemm_err_flag();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const RankCtx* ctxs = c->ctxs_dev;
  cudaError_t e = pdl::launch(k_gemm_scatter, dim3(n_tiles * nr, m_tiles, 1), dim3(gemm::kThreads), size_t(stages) * stage_bytes + 1024, st, 1,
                              maps, p, ctxs, n_tiles, rpr);
  if (e == cudaSuccess)
    e = pdl::launch(k_rs_reduce_norm, dim3(rpr, nr), dim3(tbvops::norm_threads(H)), 0, st, 1, ctxs, rp,
                    static_cast<const __nv_bfloat16*>(gamma), H, bn, m_tiles, eps, mode);
  if (e != cudaSuccess) {
    fprintf(stderr, "[tbvcoll] gemm->reduce-scatter launch failed: %s\n", cudaGetErrorString(e));
    c->sticky_err.store(1);
    return TBV_FAIL;
  }
  c->host_seq++;
  return TBV_OK;
}

// ---- all-gather -> GEMM ---------------------------------------------------------------------------
// x: [T/N, K] this rank's token rows (row stride ldx), w: [M, K] this rank's output features.
// y[T, M] = gather_over_ranks(x) @ w^T  (rows in rank order).
static int launch_ag_gemm(tbv_comm* c, const void* const* ws, const void* const* xs, void* const* ys, int rows_per_rank, int M, int K,
                          int ldx, int ldy, void* stream) {
  int rc = precheck(c);
  if (rc != TBV_OK) return rc;
  const int nr = c->local ? c->world : 1, W = c->world;
  const int bn = pick_bn(rows_per_rank);
  if (rows_per_rank <= 0 || !bn || (K % 8) || (ldx % 8) || (ldy % 8) || size_t(rows_per_rank) * K * 2 > c->cap ||
      rows_per_rank / bn > TBV_MAXCHAN)
    return TBV_FALLBACK;
  if (c->skip.load() > 0) { c->skip.fetch_sub(1); return TBV_OK; }
  if (set_attrs() != 0) return TBV_FAIL;
  const int tiles_per_src = rows_per_rank / bn;
  const int stage_bytes = gemm::kATileBytes + bn * 128;
  int stages = (200 * 1024) / stage_bytes;
  stages = stages > gemm::kMaxStages ? gemm::kMaxStages : (stages < 2 ? 2 : stages);
  Maps maps;
  AgPtrs ap{};
  AgOut ao{};
  for (int r = 0; r < nr; r++) {
    if (tbvops::make_tensor_map_bf16(&maps.a[r], ws[r], M, K, K, 128) != 0) return TBV_FALLBACK;
    ap.x[r] = static_cast<const __nv_bfloat16*>(xs[r]);
    ao.y[r] = static_cast<__nv_bfloat16*>(ys[r]);
    ao.gathered[r] = gather_maps(c, r, rows_per_rank, K, bn);
    if (!ao.gathered[r]) return TBV_FALLBACK;
  }
  gemm::Params p{};
  p.M = M; p.N = rows_per_rank * W; p.K = K; p.ldy = ldy; p.bn = bn; p.splits = 1; p.stages = stages; p.kb_total = (K + 63) / 64;
  p.limit_ns = 2000000000ull;
  p.err = tbvops::gemm_err_flag();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const RankCtx* ctxs = c->ctxs_dev;
  cudaError_t e = pdl::launch(k_ag_push, dim3(tiles_per_src, nr), dim3(512), 0, st, 1, ctxs, ap, K, ldx, bn, rows_per_rank);
  if (e == cudaSuccess)
    e = pdl::launch(k_ag_gemm, dim3(tiles_per_src * W, (M + 127) / 128, nr), dim3(gemm::kThreads), size_t(stages) * stage_bytes + 1024, st, 1,
                    maps, p, ctxs, ao, tiles_per_src);
  if (e != cudaSuccess) {
    fprintf(stderr, "[tbvcoll] all-gather->gemm launch failed: %s\n", cudaGetErrorString(e));
    c->sticky_err.store(1);
    return TBV_FAIL;
  }
  c->host_seq++;
  return TBV_OK;
}

extern "C" {

int tbv_comm_gemm_reduce_scatter(tbv_comm* c, const void* w, const void* x, void* out, const void* residual, const void* gamma,
                                 void* residual_out, void* y, int tokens, int hidden, int k_local, int ldx, float eps, int mode,
                                 void* stream) {
  if (!c || c->local) return TBV_FAIL;
  tbv::NvtxRange nvtx("tbv.gemm_reduce_scatter", size_t(tokens) * hidden * 2);
  return launch_gemm_rs(c, &w, &x, &out, &residual, gamma, &residual_out, &y, tokens, hidden, k_local, ldx, eps, mode, stream);
}
int tbv_comm_gemm_reduce_scatter_local(tbv_comm* c, const void* const* ws, const void* const* xs, void* const* outs,
                                       const void* const* residuals, const void* gamma, void* const* residual_outs, void* const* ys,
                                       int tokens, int hidden, int k_local, int ldx, float eps, int mode, void* stream) {
  if (!c || !c->local) return TBV_FAIL;
  return launch_gemm_rs(c, ws, xs, outs, residuals, gamma, residual_outs, ys, tokens, hidden, k_local, ldx, eps, mode, stream);
}
int tbv_comm_allgather_gemm(tbv_comm* c, const void* w, const void* x, void* y, int rows_per_rank, int M, int K, int ldx, int ldy,
                            void* stream) {
  if (!c || c->local) return TBV_FAIL;
  tbv::NvtxRange nvtx("tbv.allgather_gemm", size_t(rows_per_rank) * K * 2);
  return launch_ag_gemm(c, &w, &x, &y, rows_per_rank, M, K, ldx, ldy, stream);
}
int tbv_comm_allgather_gemm_local(tbv_comm* c, const void* const* ws, const void* const* xs, void* const* ys, int rows_per_rank, int M,
                                  int K, int ldx, int ldy, void* stream) {
  if (!c || !c->local) return TBV_FAIL;
  return launch_ag_gemm(c, ws, xs, ys, rows_per_rank, M, K, ldx, ldy, stream);
}

}  // extern "C"
