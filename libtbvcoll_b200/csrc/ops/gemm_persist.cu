// gemm_persist.cu — the many-token (prefill) form of the bf16 tcgen05 GEMM: a persistent kernel, one CTA per SM.
//
//   Y[n, m] = epilogue( sum_k X[n, k] * W[m, k] )      X: [N tokens, K], W: [M features, K], both bf16 row-major
//
// The decode form (gemm.cu) puts features on the 128-row UMMA M axis because a handful of tokens would
// waste it.  With hundreds of tokens the natural orientation is the other one: 128 tokens on UMMA M and 256
// features on UMMA N.  A thread of the epilogue then owns one token row and reads 16 consecutive features
// per TMEM load, which it stores as 32 contiguous bytes; gate/up pairs of the SiLU-mul epilogue sit in the
// same thread, so that epilogue needs no shuffles.
//
// Two tile shapes (template TH), both filling the 512 TMEM columns of the SM:
//   TH = 1  128 tokens x 256 features, two accumulators: the epilogue of tile i runs under the MMAs of tile
//           i + 1.  Every 512 tensor-core clocks consume 48 KB of operands; measured, the tensor pipe is
//           68 % busy and L2 -> shared memory is the limit.
//   TH = 2  256 tokens x 256 features as two 128-row MMAs that share one 256-row weight tile: 64 KB of operands
//           per 1024 tensor-core clocks, a third less traffic per FLOP.  Both accumulators belong to one tile,
//           so the epilogue (eight warps here, four per half) is exposed once per tile.  Measured at 4096
//           tokens: down_proj (K 14336) 1450 TFLOP/s against 1144 for TH = 1 and 1560 for cuBLAS.
//
// The CTAs walk tiles id = blockIdx.x + i * gridDim.x with the token tile fastest: the CTAs running at any
// moment share a few 256-row weight tiles (streamed from HBM once) and the activations stay in L2.  Warp 0
// lane 0 feeds a TMA ring that runs ahead across tile boundaries, warp 1 lane 0 issues tcgen05.mma, warps 2..
// drain TMEM.  Every wait is bounded; a wait that gives up raises the CTA's abort flag, all roles leave their
// loops, TMEM is freed and the host-visible error flag is set.  (The reference has no GEMM; see gemm.cu for
// what this path replaces.)
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include "gemm.cuh"
#include "ops.h"

using namespace sm100;

namespace {

constexpr int kFeatTile = 256;                    // UMMA N
constexpr int kHalfBytes = 128 * gemm::kBK * 2;      // one 128-token operand tile: 16 KB
constexpr int kWBytes = kFeatTile * gemm::kBK * 2;   // 32 KB
constexpr int kMaxStages = 4;

template <int TH> struct Shape {
  static constexpr int kTok = 128 * TH;                        // tokens per tile
  static constexpr int kXBytes = kHalfBytes * TH;
  static constexpr int kStageBytes = kXBytes + kWBytes;        // 48 KB / 64 KB
  static constexpr int kStages = TH == 1 ? 4 : 3;              // 192 KB of ring either way
  static constexpr int kBuffers = TH == 1 ? 2 : 1;             // accumulator sets that alternate between tiles
  static constexpr int kEpiWarps = 4 * TH;
  static constexpr int kThreads = 64 + 32 * kEpiWarps;
};

// Fraction of the nominal tensor rate each form sustains (measured; see gemm_tok_choose).
constexpr double kEffDecode[2] = {0.59, 0.43};   // decode-form kernel: store / SiLU-mul epilogue
constexpr double kEffTok1 = 0.62;                // 128-token tiles: gate_up 4096 x 28672 x 4096 in 25 rounds, 722 us
constexpr double kEffTok2 = 0.69;                // 256-token tiles: 0.66 (K 4096, SiLU-mul) .. 0.75 (K 14336) per round

struct PSmem {
  unsigned long long full[kMaxStages], empty[kMaxStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {  // 32 lanes x 32 consecutive fp32 columns
  tmem_ld16(taddr, r);
  tmem_ld16(taddr + 16u, r + 16);
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
// Same arithmetic as the decode kernel's SiLU-mul: every intermediate an unfused bf16 pipeline would
// have stored is rounded to bf16.
__device__ __forceinline__ float silu_mul_bf16(float g, float u) {
  g = bf16_round(g);
  u = bf16_round(u);
  const float s = bf16_round(g / (1.0f + __expf(-g)));
  return s * u;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One token row, 16 features starting at f: convert, apply the epilogue, store.
template <int EPI>
__device__ __forceinline__ void store16(const gemm::Params& p, int n, int f, const uint32_t* q) {
  float v[16];
#pragma unroll
  for (int j = 0; j < 16; j++) v[j] = __uint_as_float(q[j]);
  if (p.bias) {
#pragma unroll
    for (int j = 0; j < 16; j++) v[j] += __bfloat162float(p.bias[f + j]);
  }
  if (EPI == 1) {
    uint4 o;
    o.x = pack_bf16(silu_mul_bf16(v[0], v[1]), silu_mul_bf16(v[2], v[3]));
    o.y = pack_bf16(silu_mul_bf16(v[4], v[5]), silu_mul_bf16(v[6], v[7]));
    o.z = pack_bf16(silu_mul_bf16(v[8], v[9]), silu_mul_bf16(v[10], v[11]));
    o.w = pack_bf16(silu_mul_bf16(v[12], v[13]), silu_mul_bf16(v[14], v[15]));
    *reinterpret_cast<uint4*>(p.y + size_t(n) * p.ldy + (f >> 1)) = o;
  } else {
    uint4 o0, o1;
    o0.x = pack_bf16(v[0], v[1]);   o0.y = pack_bf16(v[2], v[3]);   o0.z = pack_bf16(v[4], v[5]);   o0.w = pack_bf16(v[6], v[7]);
    o1.x = pack_bf16(v[8], v[9]);   o1.y = pack_bf16(v[10], v[11]); o1.z = pack_bf16(v[12], v[13]); o1.w = pack_bf16(v[14], v[15]);
    uint4* dst = reinterpret_cast<uint4*>(p.y + size_t(n) * p.ldy + f);
    dst[0] = o0;
    dst[1] = o1;
  }
}

// EPI 0: store (+bias); 1: SiLU-mul over interleaved gate/up features (output has M / 2 features).
template <int EPI, int TH>
__global__ void __launch_bounds__(Shape<TH>::kThreads, 1)
k_gemm_tok(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const gemm::Params p) {
  using S = Shape<TH>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ PSmem s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const int tok_tiles = (p.N + S::kTok - 1) / S::kTok, feat_tiles = (p.M + kFeatTile - 1) / kFeatTile;
  const int tiles = tok_tiles * feat_tiles;
  const int nkb = p.kb_total;
  const int my_tiles = int(blockIdx.x) < tiles ? (tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S::kStages; i++) {
      mbar_init(smem_u32(&s.full[i]), 1);
      mbar_init(smem_u32(&s.empty[i]), 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(smem_u32(&s.acc_full[i]), 1);
      mbar_init(smem_u32(&s.acc_empty[i]), S::kEpiWarps);   // one arrival per epilogue warp
    }
    s.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&s.tmem_base), 512);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl::launch_dependents();
  const uint32_t tmem0 = s.tmem_base;
  volatile int* abortp = &s.abort_flag;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer: one flat sequence of k-blocks over all of this CTA's tiles ----
    const uint64_t pol_x = policy_evict_last();
    const long total = long(my_tiles) * nkb;
    long issued = 0;
    // Weights are never written by a kernel: the first ring fill of weight tiles goes out before the
    // preceding kernel has finished; the activations follow once it has.
    const int pre = total < S::kStages ? int(total) : S::kStages;
    for (int i = 0; i < pre; i++) {
      const int tile = int(blockIdx.x) + (i / nkb) * int(gridDim.x), kb = i % nkb;
      const uint32_t fb = smem_u32(&s.full[i]);
      mbar_expect_tx(fb, S::kStageBytes);
      tma_load_2d(base + i * S::kStageBytes + S::kXBytes, &tmW, kb * gemm::kBK, (tile / tok_tiles) * kFeatTile, fb);
    }
    pdl::grid_dependency_wait();
    for (int i = 0; i < pre; i++) {
      const int tile = int(blockIdx.x) + (i / nkb) * int(gridDim.x), kb = i % nkb;
      tma_load_2d_hint(base + i * S::kStageBytes, &tmX, kb * gemm::kBK, (tile % tok_tiles) * S::kTok, smem_u32(&s.full[i]), pol_x);
    }
    issued = pre;
    for (long i = pre; i < total; i++) {
      const int st = int(i % S::kStages);
      const uint32_t ph = uint32_t(i / S::kStages) & 1u;
      if (!mbar_wait(smem_u32(&s.empty[st]), ph ^ 1u, abortp, p.limit_ns)) break;
      const int tile = int(blockIdx.x) + int(i / nkb) * int(gridDim.x), kb = int(i % nkb);
      const uint32_t fb = smem_u32(&s.full[st]);
      mbar_expect_tx(fb, S::kStageBytes);
      tma_load_2d_hint(base + st * S::kStageBytes, &tmX, kb * gemm::kBK, (tile % tok_tiles) * S::kTok, fb, pol_x);
      tma_load_2d(base + st * S::kStageBytes + S::kXBytes, &tmW, kb * gemm::kBK, (tile / tok_tiles) * kFeatTile, fb);
      issued = i + 1;
    }
    if (*abortp) {
      // gave up: let the copies already in flight land before this CTA's shared memory goes away
      for (long i = issued > S::kStages ? issued - S::kStages : 0; i < issued; i++) {
        const uint32_t fb = smem_u32(&s.full[i % S::kStages]);
        const uint32_t ph = uint32_t(i / S::kStages) & 1u;
        for (int spin = 0; spin < 20000 && !mbar_try_wait(fb, ph); spin++) __nanosleep(50);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer ----
    const uint32_t idesc = umma_idesc_bf16(128, kFeatTile);
    long i = 0;
    bool ok = true;
    for (int t = 0; t < my_tiles && ok; t++) {
      const int buf = t % S::kBuffers, use = t / S::kBuffers;
      // the epilogue must have drained this accumulator set (kBuffers tiles ago); passes at once on first use
      if (!mbar_wait(smem_u32(&s.acc_empty[buf]), (uint32_t(use) & 1u) ^ 1u, abortp, p.limit_ns)) break;
      tc_fence_after();
      for (int kb = 0; kb < nkb; kb++, i++) {
        const int st = int(i % S::kStages);
        const uint32_t ph = uint32_t(i / S::kStages) & 1u;
        if (!mbar_wait(smem_u32(&s.full[st]), ph, abortp, p.limit_ns)) { ok = false; break; }
        tc_fence_after();
        const uint64_t bd = umma_desc_sw128(base + st * S::kStageBytes + S::kXBytes);
#pragma unroll
        for (int h = 0; h < TH; h++) {           // the 128-token halves share the weight tile
          const uint64_t ad = umma_desc_sw128(base + st * S::kStageBytes + h * kHalfBytes);
          const uint32_t tmem_d = tmem0 + uint32_t((TH == 1 ? buf : h) * kFeatTile);
#pragma unroll
          for (int k = 0; k < gemm::kBK / 16; k++)
            umma_bf16(tmem_d, ad + uint64_t(2 * k), bd + uint64_t(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&s.empty[st]));
      }
      if (ok) umma_commit(smem_u32(&s.acc_full[buf]));
    }
  } else if (warp >= 2) {
    // ---- epilogue: thread = one token row of the tile (TH = 2: warps 2..5 first half, 6..9 second half) ----
    const int quarter = warp & 3, half = TH == 1 ? 0 : (warp - 2) >> 2;
    for (int t = 0; t < my_tiles; t++) {
      const int buf = t % S::kBuffers, use = t / S::kBuffers;
      bool ok = mbar_wait(smem_u32(&s.acc_full[buf]), uint32_t(use) & 1u, abortp, p.limit_ns);
      ok = __all_sync(0xffffffffu, ok);   // reconverge before the warp-wide TMEM loads
      if (!ok) break;
      tc_fence_after();
      const int tile = int(blockIdx.x) + t * int(gridDim.x);
      const int n = (tile % tok_tiles) * S::kTok + half * 128 + quarter * 32 + lane;   // token row
      const int f0 = (tile / tok_tiles) * kFeatTile;
      const uint32_t trow = tmem0 + (uint32_t(quarter * 32) << 16) + uint32_t((TH == 1 ? buf : half) * kFeatTile);
      const bool row_ok = n < p.N;
      for (int c = 0; c < kFeatTile; c += 32) {
        uint32_t r[32];
        __syncwarp();   // rows past the end skip the stores below: reconverge before the warp-wide load
        tmem_ld32(trow + uint32_t(c), r);
        tmem_ld_wait();
        if (c + 32 == kFeatTile) {
          // accumulator fully read by this warp: hand it back to the MMA warp before the last stores go out
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&s.acc_empty[buf]));
        }
        if (!row_ok) continue;
        if (f0 + c < p.M) store16<EPI>(p, n, f0 + c, r);               // M is a multiple of 16
        if (f0 + c + 16 < p.M) store16<EPI>(p, n, f0 + c + 16, r + 16);
      }
    }
  }

  // ---- teardown: everybody is done with TMEM ----
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(s.tmem_base, 512);
  }
  if (threadIdx.x == 0 && s.abort_flag && p.err) atomicExch(p.err, 1);
}

bool g_attr = false;

template <int EPI, int TH>
cudaError_t launch(const void* w, const void* x, const gemm::Params& p, int ldx, cudaStream_t st, int* map_rc) {
  using S = Shape<TH>;
  CUtensorMap tmX, tmW;
  *map_rc = 0;
  if (tbvops::make_tensor_map_bf16(&tmX, x, p.N, p.K, ldx, S::kTok) != 0 || tbvops::make_tensor_map_bf16(&tmW, w, p.M, p.K, p.K, kFeatTile) != 0) {
    *map_rc = -3;
    return cudaSuccess;
  }
  const int tiles = ((p.N + S::kTok - 1) / S::kTok) * ((p.M + kFeatTile - 1) / kFeatTile);
  const int sms = tbvops::sm_count();
  const size_t smem = size_t(S::kStages) * S::kStageBytes + 1024;
  return pdl::launch(k_gemm_tok<EPI, TH>, dim3(tiles < sms ? tiles : sms), dim3(S::kThreads), smem, st, 1, tmX, tmW, p);
}

}  // namespace

namespace tbvops {

// Which form takes an [N tokens] x [M features] problem: 0 = the decode-form kernel (gemm.cu), 1 / 2 = this
// kernel with 128- / 256-token tiles.  `mode`: 1 = choose by estimated time, 2 / 3 = force TH 1 / 2 wherever
// the shape allows (tests, measurements).
//
// Estimated time in units of one 128 x 256 x K tile at full tensor rate.  Tiles are equal-sized and every CTA
// walks ceil(tiles / SMs) of them, so a persistent schedule costs rounds * tile size / efficiency; the
// decode-form kernel runs 2 CTAs per SM scheduled by the hardware and costs tiles / SMs / efficiency.
// Efficiencies are measured on B200 at 4096 tokens (Llama-3-8B shapes).
int gemm_tok_choose(int M, int N, int K, int ldy, int epi, int mode) {
  if (!(N >= 384 && (M % 16) == 0 && (K % 8) == 0 && (ldy % 8) == 0 && (epi == 0 || epi == 1))) return 0;
  if (mode == 2) return 1;
  if (mode == 3) return 2;
  const double sms = sm_count();
  const long ft = (M + kFeatTile - 1) / kFeatTile;
  const long t1 = long((N + 127) / 128) * ft, t2 = long((N + 255) / 256) * ft;
  const double r1 = double((t1 + long(sms) - 1) / long(sms)), r2 = double((t2 + long(sms) - 1) / long(sms));
  const double e_dec = double((M + 127) / 128) * ((N + 255) / 256) / sms / kEffDecode[epi];
  const double e1 = r1 / kEffTok1, e2 = 2.0 * r2 / kEffTok2;
  if (e_dec <= e1 && e_dec <= e2) return 0;
  return e1 <= e2 ? 1 : 2;
}

int gemm_tok_launch(const void* w, const void* x, void* y, const void* bias, int M, int N, int K, int ldx, int ldy, int epi, int th,
                    void* stream) {
  gemm::Params p{};
  p.M = M; p.N = N; p.K = K; p.ldy = ldy; p.bn = kFeatTile; p.splits = 1; p.stages = th == 1 ? 4 : 3;
  p.kb_total = (K + 63) / 64;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.y = static_cast<__nv_bfloat16*>(y);
  p.limit_ns = 2000000000ull;
  p.err = gemm_err_flag();
  if (!g_attr) {
    cudaError_t a[4] = {cudaFuncSetAttribute(k_gemm_tok<0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024),
                        cudaFuncSetAttribute(k_gemm_tok<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024),
                        cudaFuncSetAttribute(k_gemm_tok<0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024),
                        cudaFuncSetAttribute(k_gemm_tok<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024)};
    for (cudaError_t e : a)
      if (e != cudaSuccess) return -1;
    g_attr = true;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int map_rc = 0;
  cudaError_t e = th == 2 ? (epi == 1 ? launch<1, 2>(w, x, p, ldx, st, &map_rc) : launch<0, 2>(w, x, p, ldx, st, &map_rc))
                          : (epi == 1 ? launch<1, 1>(w, x, p, ldx, st, &map_rc) : launch<0, 1>(w, x, p, ldx, st, &map_rc));
  if (map_rc != 0) return map_rc;
  if (e != cudaSuccess) {
    fprintf(stderr, "[tbvops] many-token gemm launch failed: %s (M=%d N=%d K=%d tile %dx256)\n", cudaGetErrorString(e), M, N, K, 128 * th);
    return -1;
  }
  return 0;
}

}  // namespace tbvops
