// gemm.cuh — tcgen05/TMEM GEMM main loop shared by the plain and the fused kernels.
//
//   D[m, n] = sum_k W[m, k] * X[n, k]        W: [M, K] bf16 row-major (a torch Linear weight)
//                                            X: [N, K] bf16 row-major (activations, N tokens)
// "Swap-AB": output features sit on the 128-row UMMA M axis and tokens on the UMMA N axis
// (16..256), so a decode batch of 1..64 tokens wastes no tensor-core rows and the weight
// matrix streams through shared memory exactly once.
//
// Per CTA: one 128 x BN output tile over a K range.  Warp 0 issues TMA loads (128-byte
// swizzle, K blocks of 64) into a multi-stage ring, warp 1 issues tcgen05.mma into a TMEM
// accumulator, warps 2-5 read the accumulator back with tcgen05.ld.  With split-K the
// CTAs of one cluster cover disjoint K ranges and reduce through distributed shared
// memory in a fixed order (deterministic).
#pragma once
#include "../pdl.cuh"
#include "sm100.cuh"

namespace gemm {

constexpr int kBM = 128;        // UMMA M: output features per tile
constexpr int kBK = 64;         // one 128-byte swizzle span of bf16
constexpr int kMaxStages = 8;
constexpr int kThreads = 192;   // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int kATileBytes = kBM * kBK * 2;

struct Params {
  int M, N, K;
  int ldy;             // output row stride in elements
  int bn;              // tokens per tile (multiple of 16, <= 256)
  int splits;          // cluster size along K: 1, 2, 4 or 8
  int stages;
  int kb_total;        // ceil(K / 64)
  int raster;          // 0: blockIdx.x = feature tile, .y = token tile; 1: swapped (token tiles launch first)
  int a_after_wait;    // 1: operand A (w) may have been written by the preceding kernel: fetch it only after the dependency wait
  const __nv_bfloat16* bias;  // [M] or null
  __nv_bfloat16* y;
  unsigned long long limit_ns;  // bound on every barrier wait
  int* err;                     // device flag: set to 1 if a wait gave up
  const char* pf_ptr;           // weights of the GEMM that runs next (or null): see the producer's last step
  unsigned long long pf_bytes;  // how much of them to ask into L2 (a multiple of 16), shared out over the CTAs
};

struct Smem {  // static shared state of one CTA
  unsigned long long full[kMaxStages], empty[kMaxStages], accum;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t tmem_cols(int bn) {
  uint32_t c = 32;
  while (int(c) < bn) c <<= 1;
  return c;
}

// Runs the TMA/MMA pipeline.  On return (for all threads) the accumulator for this CTA's
// K range is complete in TMEM (unless s.abort_flag is set).  Returns the aligned dynamic
// shared memory base, which the epilogue may reuse as staging space.
__device__ __forceinline__ uint8_t* mainloop(const CUtensorMap* tmA, const CUtensorMap* tmB, const Params& p, Smem& s,
                                             uint8_t* smem_raw, int m0, int n0, int kb0, int nkb) {
  using namespace sm100;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const uint32_t b_tile_bytes = uint32_t(p.bn) * 128u;
  const uint32_t a_base = base, b_base = base + uint32_t(p.stages) * kATileBytes;

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; i++) {
      mbar_init(smem_u32(&s.full[i]), 1);
      mbar_init(smem_u32(&s.empty[i]), 1);
    }
    mbar_init(smem_u32(&s.accum), 1);
    s.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&s.tmem_base), tmem_cols(p.bn));
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(tmA);
    tma_prefetch_desc(tmB);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl::launch_dependents();  // the next kernel may set itself up while this one computes
  const uint32_t tmem_d = s.tmem_base;
  volatile int* abortp = &s.abort_flag;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer ----
    const uint64_t pol_w = policy_evict_first();  // weights are read once
    const uint64_t pol_x = policy_evict_last();   // activations are re-read by every M tile
    int issued = 0;
    // Weights are never written by any kernel: start streaming them into the ring before the
    // preceding kernel has finished, then wait for it and fetch the activations.
    // (Contract: operand A is constant — a weight.  A caller whose A was produced by the kernel just
    // before this one sets a_after_wait, and the early fetch is skipped.)
    const int pre = nkb < p.stages ? nkb : p.stages;
    if (p.a_after_wait) pdl::grid_dependency_wait();
    for (int i = 0; i < pre; i++) {
      const uint32_t fb = smem_u32(&s.full[i]);
      mbar_expect_tx(fb, kATileBytes + b_tile_bytes);
      tma_load_2d_hint(a_base + i * kATileBytes, tmA, (kb0 + i) * kBK, m0, fb, pol_w);
    }
    if (!p.a_after_wait) pdl::grid_dependency_wait();
    for (int i = 0; i < pre; i++)
      tma_load_2d_hint(b_base + i * b_tile_bytes, tmB, (kb0 + i) * kBK, n0, smem_u32(&s.full[i]), pol_x);
    issued = pre;
    for (int i = pre; i < nkb; i++) {
      const int st = i % p.stages;
      const uint32_t ph = uint32_t(i / p.stages) & 1u;
      if (!mbar_wait(smem_u32(&s.empty[st]), ph ^ 1u, abortp, p.limit_ns)) break;
      const uint32_t fb = smem_u32(&s.full[st]);
      mbar_expect_tx(fb, kATileBytes + b_tile_bytes);
      tma_load_2d_hint(a_base + st * kATileBytes, tmA, (kb0 + i) * kBK, m0, fb, pol_w);
      tma_load_2d_hint(b_base + st * b_tile_bytes, tmB, (kb0 + i) * kBK, n0, fb, pol_x);
      issued = i + 1;
    }
    // This CTA's own weight tiles are all requested.  Between here and the moment the NEXT GEMM may start (this
    // kernel's epilogue, the kernel boundary, an attention or all-reduce kernel in between) HBM would idle: the next
    // kernel's CTAs get an SM slot only when this kernel's leave, and then fetch no more than their ring holds before
    // their dependency wait.  So each CTA asks for its share of the next GEMM's weights to be brought into L2
    // (126 MB); the requests queue behind this kernel's own loads, and the next kernel's TMA loads find them there.
    if (p.pf_bytes && !*abortp) {
      const unsigned long long ncta = (unsigned long long)gridDim.x * gridDim.y * gridDim.z;
      const unsigned long long id = blockIdx.x + (unsigned long long)gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
      const unsigned long long per = ((p.pf_bytes + ncta - 1) / ncta + 4095ull) & ~4095ull;
      const unsigned long long off = id * per;
      if (off < p.pf_bytes) {
        const unsigned long long n = p.pf_bytes - off < per ? p.pf_bytes - off : per;
        for (unsigned long long o = 0; o < n; o += 4096ull)
          l2_prefetch_bulk(p.pf_ptr + off + o, uint32_t(n - o < 4096ull ? n - o : 4096ull));
      }
    }
    if (*abortp) {
      // gave up: let the copies already in flight land before this CTA's memory goes away
      for (int i = issued > p.stages ? issued - p.stages : 0; i < issued; i++) {
        const uint32_t fb = smem_u32(&s.full[i % p.stages]);
        const uint32_t ph = uint32_t(i / p.stages) & 1u;
        for (int spin = 0; spin < 20000 && !mbar_try_wait(fb, ph); spin++) __nanosleep(50);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer ----
    const uint32_t idesc = umma_idesc_bf16(kBM, uint32_t(p.bn));
    for (int i = 0; i < nkb; i++) {
      const int st = i % p.stages;
      const uint32_t ph = uint32_t(i / p.stages) & 1u;
      if (!mbar_wait(smem_u32(&s.full[st]), ph, abortp, p.limit_ns)) break;
      tc_fence_after();
      const uint64_t ad = umma_desc_sw128(a_base + st * kATileBytes);
      const uint64_t bd = umma_desc_sw128(b_base + st * b_tile_bytes);
#pragma unroll
      for (int k = 0; k < kBK / 16; k++)  // UMMA K = 16 bf16 = 32 bytes: +2 in the (addr >> 4) field
        umma_bf16(tmem_d, ad + uint64_t(2 * k), bd + uint64_t(2 * k), idesc, (i | k) != 0 ? 1u : 0u);
      umma_commit(smem_u32(&s.empty[st]));  // frees the stage when these MMAs are done
    }
    umma_commit(smem_u32(&s.accum));
  }
  return sm;
}

// Called by all threads at the very end (after the epilogue warps are done with TMEM).
__device__ __forceinline__ void teardown(const Params& p, Smem& s) {
  using namespace sm100;
  tc_fence_before();
  __syncthreads();
  if ((threadIdx.x >> 5) == 1) {
    tc_fence_after();
    tmem_dealloc(s.tmem_base, tmem_cols(p.bn));
  }
  if (threadIdx.x == 0 && s.abort_flag && p.err) atomicExch(p.err, 1);
}

}  // namespace gemm
