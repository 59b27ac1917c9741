// gemm_streamk.cu — the decode-form bf16 tcgen05 GEMM with its work split EVENLY over the SMs.
//
//   Y[n, m] = epilogue( sum_k W[m, k] * X[n, k] )     W: [M, K] (a Linear weight), X: [N <= 64 tokens, K]
//
// The tile kernel (gemm.cu) hands out whole 128-feature tiles (or equal K slices of them): a gate_up
// projection of 224 tiles on 148 SMs leaves 76 SMs with two 1 MB weight tiles and 72 with one, and the
// two-tile SMs set the duration (measured 0.79-0.83 of the HBM copy rate).  Here the unit of work is one
// (tile, 64-wide K block) pair — 16 KB of weights — and CTA g of a persistent grid (one per SM) takes the
// contiguous unit range [g*U/G, (g+1)*U/G): every SM streams the same number of bytes.  A range crosses
// tile boundaries, so a tile's K range may be covered by several consecutive CTAs:
//   * the CTA that holds the START of a tile's K range finishes the tile (it reaches that segment LAST);
//   * every other CTA covering the tile reaches its segment FIRST, stores its fp32 partial in a per-CTA
//     scratch block in global memory and raises a flag;
//   * the finishing CTA adds the partials in ascending K order (fixed: deterministic), applies the epilogue
//     (bias, SiLU-mul) and stores; it then clears the flags it consumed, so nothing needs resetting between
//     launches and a captured graph replays correctly.
// All CTAs are resident (grid <= SM count, one CTA per SM), every wait is bounded.  Warp 0 lane 0 feeds the
// TMA ring across segment boundaries, warp 1 lane 0 issues tcgen05.mma into two alternating TMEM
// accumulators, warps 2-5 drain them.  The scratch block and the flags belong to the device (allocated on
// first use, outside stream capture): calls must be stream-ordered, like everything else in this library.
//
// The sum of one output element is formed in K order but split where the unit ranges happen to fall, so the
// low bits can differ from the tile kernel's; it is the same on every run and on every rank of a TP group.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>

#include "gemm.cuh"
#include "ops.h"

using namespace sm100;

namespace {

constexpr int kSkMaxBn = 64;
constexpr int kSkMaxGrid = 320;

struct SkSmem {
  unsigned long long full[gemm::kMaxStages], empty[gemm::kMaxStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct SkArgs {
  float* scratch;      // [grid][bn][128] fp32 partials
  unsigned* flags;     // [grid]: 1 = the CTA's partial is in its scratch block
  int m_tiles;
  long long units;     // m_tiles * kb_total
  int stage_f_off;     // byte offsets of the epilogue staging areas behind the ring
  int stage_h_off;
};

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float silu_mul_bf16(float g, float u) {   // same arithmetic as the tile kernel
  g = bf16_round(g);
  u = bf16_round(u);
  float s = bf16_round(g / (1.0f + __expf(-g)));
  return s * u;
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ long long range_begin(long long units, int g, int G) { return units * g / G; }

template <int EPI>
__global__ void __launch_bounds__(gemm::kThreads, 2)
k_gemm_streamk(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const gemm::Params p, const SkArgs a) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ SkSmem s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const int nkb = p.kb_total, G = gridDim.x, g = blockIdx.x;
  const long long u0 = range_begin(a.units, g, G), u1 = range_begin(a.units, g + 1, G);
  const long long total = u1 - u0;
  const uint32_t b_tile_bytes = uint32_t(p.bn) * 128u;
  const uint32_t a_base = base, b_base = base + uint32_t(p.stages) * gemm::kATileBytes;
  const uint32_t acc_cols = gemm::tmem_cols(p.bn);

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; i++) {
      mbar_init(smem_u32(&s.full[i]), 1);
      mbar_init(smem_u32(&s.empty[i]), 1);
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(smem_u32(&s.acc_full[i]), 1);
      mbar_init(smem_u32(&s.acc_empty[i]), 4);   // one arrival per epilogue warp
    }
    s.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&s.tmem_base), 2 * acc_cols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl::launch_dependents();
  const uint32_t tmem0 = s.tmem_base;
  volatile int* abortp = &s.abort_flag;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer: one flat sequence of units; the weight tiles of the first ring fill go out before the
    // preceding kernel has finished (weights are constant), the activations follow once it has ----
    const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
    const int pre = total < p.stages ? int(total) : p.stages;
    for (int i = 0; i < pre; i++) {
      const long long u = u0 + i;
      const uint32_t fb = smem_u32(&s.full[i]);
      mbar_expect_tx(fb, gemm::kATileBytes + b_tile_bytes);
      tma_load_2d_hint(a_base + i * gemm::kATileBytes, &tmA, int(u % nkb) * gemm::kBK, int(u / nkb) * gemm::kBM, fb, pol_w);
    }
    pdl::grid_dependency_wait();
    for (int i = 0; i < pre; i++)
      tma_load_2d_hint(b_base + i * b_tile_bytes, &tmB, int((u0 + i) % nkb) * gemm::kBK, 0, smem_u32(&s.full[i]), pol_x);
    long long issued = pre;
    for (long long i = pre; i < total; i++) {
      const int st = int(i % p.stages);
      const uint32_t ph = uint32_t(i / p.stages) & 1u;
      if (!mbar_wait(smem_u32(&s.empty[st]), ph ^ 1u, abortp, p.limit_ns)) break;
      const long long u = u0 + i;
      const uint32_t fb = smem_u32(&s.full[st]);
      mbar_expect_tx(fb, gemm::kATileBytes + b_tile_bytes);
      tma_load_2d_hint(a_base + st * gemm::kATileBytes, &tmA, int(u % nkb) * gemm::kBK, int(u / nkb) * gemm::kBM, fb, pol_w);
      tma_load_2d_hint(b_base + st * b_tile_bytes, &tmB, int(u % nkb) * gemm::kBK, 0, fb, pol_x);
      issued = i + 1;
    }
    if (*abortp) {
      // gave up: let the copies already in flight land before this CTA's shared memory goes away
      for (long long i = issued > p.stages ? issued - p.stages : 0; i < issued; i++) {
        const uint32_t fb = smem_u32(&s.full[i % p.stages]);
        const uint32_t ph = uint32_t(i / p.stages) & 1u;
        for (int spin = 0; spin < 20000 && !mbar_try_wait(fb, ph); spin++) __nanosleep(50);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer: one accumulator per segment (the part of a tile's K range inside this CTA's units) ----
    const uint32_t idesc = umma_idesc_bf16(gemm::kBM, uint32_t(p.bn));
    long long i = 0;
    bool ok = true;
    for (int seg = 0; i < total && ok; seg++) {
      const int buf = seg & 1;
      if (!mbar_wait(smem_u32(&s.acc_empty[buf]), (uint32_t(seg >> 1) & 1u) ^ 1u, abortp, p.limit_ns)) break;
      tc_fence_after();
      const long long u = u0 + i;
      const int kb_lo = int(u % nkb);
      const long long left = total - i;
      const int n_in = int(left < (nkb - kb_lo) ? left : (nkb - kb_lo));
      const uint32_t tmem_d = tmem0 + uint32_t(buf) * acc_cols;
      for (int j = 0; j < n_in; j++, i++) {
        const int st = int(i % p.stages);
        const uint32_t ph = uint32_t(i / p.stages) & 1u;
        if (!mbar_wait(smem_u32(&s.full[st]), ph, abortp, p.limit_ns)) { ok = false; break; }
        tc_fence_after();
        const uint64_t ad = umma_desc_sw128(a_base + st * gemm::kATileBytes);
        const uint64_t bd = umma_desc_sw128(b_base + st * b_tile_bytes);
#pragma unroll
        for (int k = 0; k < gemm::kBK / 16; k++)
          umma_bf16(tmem_d, ad + uint64_t(2 * k), bd + uint64_t(2 * k), idesc, (j | k) != 0 ? 1u : 0u);
        umma_commit(smem_u32(&s.empty[st]));
      }
      if (ok) umma_commit(smem_u32(&s.acc_full[buf]));
    }
  } else if (warp >= 2) {
    // ---- epilogue warps: thread = one feature row of the tile ----
    const int quarter = warp & 3, ml = quarter * 32 + lane, te = threadIdx.x - 64;
    float* stage_f = reinterpret_cast<float*>(sm + a.stage_f_off);             // [bn][128] fp32
    __nv_bfloat16* stage_h = reinterpret_cast<__nv_bfloat16*>(sm + a.stage_h_off);   // [bn][OUTW] bf16
    constexpr int OUTW = EPI == 1 ? 64 : 128;
    const int rows = p.N < p.bn ? p.N : p.bn;
    long long i = 0;
    for (int seg = 0; i < total; seg++) {
      const int buf = seg & 1;
      const long long u = u0 + i;
      const int tile = int(u / nkb), kb_lo = int(u % nkb);
      const long long left = total - i;
      const int n_in = int(left < (nkb - kb_lo) ? left : (nkb - kb_lo));
      i += n_in;
      bool ok = mbar_wait(smem_u32(&s.acc_full[buf]), uint32_t(seg >> 1) & 1u, abortp, p.limit_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool whole = kb_lo == 0 && n_in == nkb;
      const bool finisher = kb_lo == 0;
      float* dst_f = finisher ? stage_f : a.scratch + size_t(g) * size_t(p.bn) * 128;
      for (int c = 0; c < p.bn; c += 16) {
        uint32_t r[16];
        tmem_ld16(tmem0 + uint32_t(buf) * acc_cols + (uint32_t(quarter * 32) << 16) + uint32_t(c), r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; j++) dst_f[(c + j) * 128 + ml] = __uint_as_float(r[j]);
      }
      // the accumulator is in registers / memory: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s.acc_empty[buf]));
      if (!finisher) {
        // contributor: publish the partial (device scope), then go on with the next segment
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (te == 0) st_release_gpu(a.flags + g, 1u);
        continue;
      }
      if (!whole) {
        // finisher of a tile that later CTAs contribute to: add their partials in ascending K order
        const long long tile_end = (long long)(tile + 1) * nkb;
        for (int gg = g + 1; gg < G && range_begin(a.units, gg, G) < tile_end; gg++) {
          if (te == 0) {
            unsigned long long t0 = 0;
            for (unsigned it = 0; ld_acquire_gpu(a.flags + gg) == 0u; it++) {
              if ((it & 63u) == 63u) {
                if (*abortp) break;
                const unsigned long long now = globaltimer();
                if (t0 == 0) t0 = now;
                else if (now - t0 > p.limit_ns) { *abortp = 1; break; }
                __nanosleep(100);
              }
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const float* part = a.scratch + size_t(gg) * size_t(p.bn) * 128;
          for (int c = 0; c < p.bn; c++) stage_f[c * 128 + ml] += __ldcg(part + c * 128 + ml);
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (te == 0) a.flags[gg] = 0u;   // consumed: the next launch starts from cleared flags
        }
      }
      // ---- tile epilogue from the staged fp32 sums: bias, SiLU-mul, bf16, coalesced store ----
      const int m0 = tile * gemm::kBM;
      const float bias = (p.bias && m0 + ml < p.M) ? __bfloat162float(p.bias[m0 + ml]) : 0.f;
      if (EPI == 1) {
        // even lanes hold gate rows, odd lanes the matching up rows: per pair of token columns the two lanes swap
        // one value each, so that every lane does useful SiLU work
        for (int c = 0; c < p.bn; c += 2) {
          const float v0 = stage_f[c * 128 + ml] + bias, v1 = stage_f[(c + 1) * 128 + ml] + bias;
          const float recv = __shfl_xor_sync(0xffffffffu, (lane & 1) ? v0 : v1, 1);
          const float o = (lane & 1) ? silu_mul_bf16(recv, v1) : silu_mul_bf16(v0, recv);
          stage_h[(c + (lane & 1)) * 64 + (ml >> 1)] = __float2bfloat16_rn(o);
        }
      } else {
        for (int c = 0; c < p.bn; c++) stage_h[c * 128 + ml] = __float2bfloat16_rn(stage_f[c * 128 + ml] + bias);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      constexpr int PPR = OUTW / 8;   // 16-byte pieces per token row
      const int out_m0 = EPI == 1 ? (m0 >> 1) : m0;
      const int out_M = EPI == 1 ? (p.M >> 1) : p.M;
      for (int idx = te; idx < rows * PPR; idx += 128) {
        const int t = idx / PPR, pc = idx % PPR;
        const int m = out_m0 + pc * 8;
        if (m + 8 <= out_M) {
          *reinterpret_cast<uint4*>(p.y + size_t(t) * p.ldy + m) = *reinterpret_cast<const uint4*>(stage_h + t * OUTW + pc * 8);
        } else {
          for (int e = 0; e < 8 && m + e < out_M; e++) p.y[size_t(t) * p.ldy + m + e] = stage_h[t * OUTW + pc * 8 + e];
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");   // the staging areas are free for the next segment
    }
  }

  // ---- teardown ----
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(s.tmem_base, 2 * acc_cols);
  }
  if (threadIdx.x == 0 && s.abort_flag && p.err) atomicExch(p.err, 1);
}

struct DevScratch { float* scratch = nullptr; unsigned* flags = nullptr; };
DevScratch g_sk[16];
bool g_attr = false;
long g_min_bytes = -2;   // -2: read TBV_GEMM_SK_MIN on first use

}  // namespace

namespace tbvops {

// Smallest weight matrix (bytes) that takes the evenly-split kernel; below it the latency of the tile kernel's
// cluster split-K is lower.  TBV_GEMM_SK_MIN (bytes; 0 = always where the shape allows, -1 = never, the default).
long gemm_streamk_min_bytes() {
  if (g_min_bytes == -2) {
    const char* e = getenv("TBV_GEMM_SK_MIN");
    g_min_bytes = e ? atol(e) : -1;   // off unless asked for
  }
  return g_min_bytes;
}
void gemm_streamk_set_min_bytes(long v) { g_min_bytes = v; }

bool gemm_streamk_wants(int M, int N, int K, int epi, int splits_hint, bool w_not_constant) {
  const long mn = gemm_streamk_min_bytes();
  if (mn < 0 || splits_hint > 0 || w_not_constant || N > kSkMaxBn) return false;
  (void)epi;
  return long(M) * K * 2 >= mn && (long((M + 127) / 128) * ((K + 63) / 64)) >= 2 * sm_count();
}

int gemm_streamk_launch(const void* w, const void* x, void* y, const void* bias, int M, int N, int K, int ldx, int ldy, int epi,
                        void* stream) {
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 15;
  // CTAs per SM (TBV_GEMM_SK_PER_SM, 1 or 2): all of them must be resident at once because finishing CTAs wait for others
  static const int per_sm = [] { const char* e = getenv("TBV_GEMM_SK_PER_SM"); int v = e ? atoi(e) : 2; return v < 1 ? 1 : (v > 2 ? 2 : v); }();
  const int G = sm_count() * per_sm < kSkMaxGrid ? sm_count() * per_sm : kSkMaxGrid;
  if (!g_sk[dev].scratch) {
    // first use on this device (must not happen under stream capture): one partial block and one flag per CTA
    if (cudaMalloc(&g_sk[dev].scratch, size_t(kSkMaxGrid) * kSkMaxBn * 128 * sizeof(float)) != cudaSuccess) return -1;
    if (cudaMalloc(&g_sk[dev].flags, kSkMaxGrid * sizeof(unsigned)) != cudaSuccess) return -1;
    if (cudaMemset(g_sk[dev].flags, 0, kSkMaxGrid * sizeof(unsigned)) != cudaSuccess) return -1;
    cudaDeviceSynchronize();
  }
  const int bn = N <= 16 ? 16 : (N <= 32 ? 32 : 64);
  CUtensorMap tmA, tmB;
  if (make_tensor_map_bf16(&tmA, w, M, K, K, 128) != 0) return -3;
  if (make_tensor_map_bf16(&tmB, x, N, K, ldx, bn) != 0) return -3;
  gemm::Params p{};
  p.M = M; p.N = N; p.K = K; p.ldy = ldy; p.bn = bn; p.splits = 1;
  p.kb_total = (K + 63) / 64;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.y = static_cast<__nv_bfloat16*>(y);
  p.limit_ns = 2000000000ull;
  p.err = gemm_err_flag();
  const int stage_bytes = gemm::kATileBytes + bn * 128;
  const int stage_f = bn * 128 * 4, stage_h = bn * 128 * 2;
  int stages = ((per_sm == 2 ? 112 : 225) * 1024 - 1024 - stage_f - stage_h) / stage_bytes;
  stages = stages > gemm::kMaxStages ? gemm::kMaxStages : stages;
  if (stages < 2) return -2;
  p.stages = stages;
  SkArgs a{};
  a.scratch = g_sk[dev].scratch;
  a.flags = g_sk[dev].flags;
  a.m_tiles = (M + 127) / 128;
  a.units = (long long)a.m_tiles * p.kb_total;
  a.stage_f_off = stages * stage_bytes;
  a.stage_h_off = a.stage_f_off + stage_f;
  const size_t smem = size_t(stages) * stage_bytes + stage_f + stage_h + 1024;
  if (!g_attr) {
    if (cudaFuncSetAttribute(k_gemm_streamk<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(k_gemm_streamk<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess)
      return -1;
    g_attr = true;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = epi == 1 ? pdl::launch(k_gemm_streamk<1>, dim3(G), dim3(gemm::kThreads), smem, st, 1, tmA, tmB, p, a)
                           : pdl::launch(k_gemm_streamk<0>, dim3(G), dim3(gemm::kThreads), smem, st, 1, tmA, tmB, p, a);
  if (e != cudaSuccess) {
    fprintf(stderr, "[tbvops] stream-K gemm launch failed: %s (M=%d N=%d K=%d bn=%d stages=%d)\n", cudaGetErrorString(e), M, N, K, bn, stages);
    return -1;
  }
  return 0;
}

}  // namespace tbvops

extern "C" {
// Smallest weight matrix in bytes that takes the evenly-split (stream-K) decode GEMM: 0 = wherever the shape allows,
// -1 = never, -2 = read TBV_GEMM_SK_MIN again.
void tbv_op_gemm_streamk_min_bytes(long v) { tbvops::gemm_streamk_set_min_bytes(v); }
}
