// attention.cu — paged attention over the block KV cache (GQA, head_dim 128), used for
// decode (one query token per sequence) and, with one query row per prompt token, for
// causal prefill.
//
// The reference leaves attention to vLLM; its own engine is described only ("GQA, KV cache",
// reports/11_custom_engine.md:10-20).  This is a flash-decoding kernel: one CTA per
// (kv head, query row, kv split); the G query heads that share a kv head are processed
// together so every K/V byte is read once; a half-warp owns one cached token at a time
// (16 lanes x 16 bytes = one 256-byte head row, fully coalesced); online softmax in fp32
// (base-2 exponent); partial results of kv splits are merged by the last CTA to finish,
// in split order (deterministic).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../pdl.cuh"

namespace {

constexpr int kD = 128;        // head_dim
constexpr int kU = 4;          // tokens in flight per half-warp (8 x 16-byte loads per thread)
constexpr int kMaxSplits = 8;  // portable cluster size
constexpr int kMaxBlocksPerCta = 64;  // block-table entries staged per pass
constexpr float kNegBig = -1e30f;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(r) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

struct AttnParams {
  const __nv_bfloat16* q;   // [Nq, nq, D], row stride ldq
  const __nv_bfloat16* k_cache;  // [slots, nkv, D]
  const __nv_bfloat16* v_cache;
  const int* block_tables;  // [nseq, max_blocks]
  const int* seq_of_query;  // [Nq] or null (identity)
  const int* ctx_lens;      // [Nq]: keys visible to this query row
  __nv_bfloat16* out;       // [Nq, nq, D], row stride ldo
  float scale_log2;         // softmax scale * log2(e)
  int ldq, ldo, nkv, block_size, max_blocks, splits;
};

// grid (Nq, nkv, splits), cluster (1, 1, splits): the CTAs of one cluster cover disjoint
// ranges of the cached tokens of one (query row, kv head) and merge their partial softmax
// results through distributed shared memory in split order — no global scratch, no atomics.
// kThreads: 256 (16 half-warps) while the per-half-warp partials fit in 48 KB of static shared memory, else 128.
template <int G, int kThreads>
__global__ void __launch_bounds__(kThreads) k_paged_attn(const AttnParams p) {
  constexpr int kHW = kThreads / 16;
  __shared__ float sh_o[kHW][G][kD];   // per half-warp partials, then [0] holds the CTA's result
  __shared__ float sh_ml[kHW][G][2];
  __shared__ int sh_bt[kMaxBlocksPerCta];
  pdl::launch_dependents();
  pdl::grid_dependency_wait();
  const int qi = blockIdx.x, h = blockIdx.y, sp = blockIdx.z, S = p.splits;
  const int hw = threadIdx.x >> 4, l16 = threadIdx.x & 15;
  const int ctx = min(p.ctx_lens[qi], p.max_blocks * p.block_size);  // never walk past the block table (a captured loop replayed beyond the reserved length)
  const int seq = p.seq_of_query ? p.seq_of_query[qi] : qi;
  const int* bt = p.block_tables + size_t(seq) * p.max_blocks;
  int chunk = (ctx + S - 1) / S;
  chunk = (chunk + p.block_size - 1) / p.block_size * p.block_size;
  const int t0 = sp * chunk, t1 = min(ctx, t0 + chunk);

  float qf[G][8], acc[G][8], m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; g++) {
    const uint4 qv = *reinterpret_cast<const uint4*>(p.q + size_t(qi) * p.ldq + (h * G + g) * kD + l16 * 8);
    unpack8(qv, qf[g]);
#pragma unroll
    for (int i = 0; i < 8; i++) { qf[g][i] *= p.scale_log2; acc[g][i] = 0.f; }
    m[g] = kNegBig;
    l[g] = 0.f;
  }

  // Passes of up to kMaxBlocksPerCta cache blocks: their table entries are staged in shared
  // memory first so that the K/V loads below depend on one global round trip, not two.
  const int span = kMaxBlocksPerCta * p.block_size;
  for (int pass0 = t0; pass0 < t1; pass0 += span) {
    const int pass1 = min(t1, pass0 + span);
    const int b0 = pass0 / p.block_size, nb = (pass1 - pass0 + p.block_size - 1) / p.block_size;
    __syncthreads();
    if (threadIdx.x < nb) sh_bt[threadIdx.x] = bt[b0 + threadIdx.x];
    __syncthreads();
    // The trip count is the same for every thread of the CTA (the shuffles below name the
    // whole warp); tokens past the end are masked per half-warp.
    for (int base = pass0; base < pass1; base += kHW * kU) {
      const int tok = base + hw;
      uint4 kv[kU], vv[kU];
      bool valid[kU];
#pragma unroll
      for (int j = 0; j < kU; j++) {
        const int tj = tok + j * kHW;
        valid[j] = tj < pass1;
        if (valid[j]) {
          const long long slot = (long long)sh_bt[tj / p.block_size - b0] * p.block_size + tj % p.block_size;
          const size_t off = (size_t(slot) * p.nkv + h) * kD + l16 * 8;
          kv[j] = *reinterpret_cast<const uint4*>(p.k_cache + off);
          vv[j] = *reinterpret_cast<const uint4*>(p.v_cache + off);
        } else {
          kv[j] = make_uint4(0, 0, 0, 0);
          vv[j] = make_uint4(0, 0, 0, 0);
        }
      }
      float s[kU][G];
#pragma unroll
      for (int j = 0; j < kU; j++) {
        float kf[8];
        unpack8(kv[j], kf);
#pragma unroll
        for (int g = 0; g < G; g++) {
          float d = 0.f;
#pragma unroll
          for (int i = 0; i < 8; i++) d = fmaf(qf[g][i], kf[i], d);
          s[j][g] = d;
        }
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1)
#pragma unroll
        for (int j = 0; j < kU; j++)
#pragma unroll
          for (int g = 0; g < G; g++) s[j][g] += __shfl_xor_sync(0xffffffffu, s[j][g], o);
#pragma unroll
      for (int g = 0; g < G; g++) {
        float mx = m[g];
#pragma unroll
        for (int j = 0; j < kU; j++) if (valid[j]) mx = fmaxf(mx, s[j][g]);
        const float corr = exp2f(m[g] - mx);
        float pj[kU], ps = 0.f;
#pragma unroll
        for (int j = 0; j < kU; j++) { pj[j] = valid[j] ? exp2f(s[j][g] - mx) : 0.f; ps += pj[j]; }
        l[g] = l[g] * corr + ps;
        m[g] = mx;
#pragma unroll
        for (int i = 0; i < 8; i++) acc[g][i] *= corr;
#pragma unroll
        for (int j = 0; j < kU; j++) {
          float vf[8];
          unpack8(vv[j], vf);
#pragma unroll
          for (int i = 0; i < 8; i++) acc[g][i] = fmaf(pj[j], vf[i], acc[g][i]);
        }
      }
    }
  }

  // combine the half-warps of this CTA
#pragma unroll
  for (int g = 0; g < G; g++) {
#pragma unroll
    for (int i = 0; i < 8; i++) sh_o[hw][g][l16 * 8 + i] = acc[g][i];
    if (l16 == 0) { sh_ml[hw][g][0] = m[g]; sh_ml[hw][g][1] = l[g]; }
  }
  __syncthreads();
  float res_o[(G * kD + kThreads - 1) / kThreads], res_m[(G * kD + kThreads - 1) / kThreads], res_l[(G * kD + kThreads - 1) / kThreads];
#pragma unroll
  for (int k = 0; k < (G * kD + kThreads - 1) / kThreads; k++) {
    const int idx = threadIdx.x + k * kThreads;
    if (idx < G * kD) {
      const int g = idx / kD, d = idx % kD;
      float mx = kNegBig;
      for (int w = 0; w < kHW; w++) mx = fmaxf(mx, sh_ml[w][g][0]);
      float a = 0.f, ls = 0.f;
      for (int w = 0; w < kHW; w++) {
        const float c = exp2f(sh_ml[w][g][0] - mx);
        a = fmaf(sh_o[w][g][d], c, a);
        ls = fmaf(sh_ml[w][g][1], c, ls);
      }
      res_o[k] = a; res_m[k] = mx; res_l[k] = ls;
    }
  }
  if (S == 1) {
#pragma unroll
    for (int k = 0; k < (G * kD + kThreads - 1) / kThreads; k++) {
      const int idx = threadIdx.x + k * kThreads;
      if (idx < G * kD)
        p.out[size_t(qi) * p.ldo + h * G * kD + idx] = __float2bfloat16_rn(res_l[k] > 0.f ? res_o[k] / res_l[k] : 0.f);
    }
    return;
  }
  // publish this CTA's result in its own shared memory (slot [0] of the partial arrays)
  __syncthreads();
#pragma unroll
  for (int k = 0; k < (G * kD + kThreads - 1) / kThreads; k++) {
    const int idx = threadIdx.x + k * kThreads;
    if (idx < G * kD) {
      const int g = idx / kD, d = idx % kD;
      sh_o[0][g][d] = res_o[k];
      if (d == 0) { sh_ml[0][g][0] = res_m[k]; sh_ml[0][g][1] = res_l[k]; }
    }
  }
  cluster_sync();
  // CTA `sp` merges outputs [sp * per, (sp + 1) * per) of the G * D values, in split order
  const int per = (G * kD + S - 1) / S;
  for (int i = threadIdx.x; i < per; i += kThreads) {
    const int idx = sp * per + i;
    if (idx < G * kD) {
      const int g = idx / kD, d = idx % kD;
      const uint32_t a_ml = smem_addr(&sh_ml[0][g][0]), a_o = smem_addr(&sh_o[0][g][d]);
      float ms[kMaxSplits], mx = kNegBig;
      for (int r = 0; r < S; r++) { ms[r] = ld_cluster_f32(a_ml, r); mx = fmaxf(mx, ms[r]); }
      float a = 0.f, ls = 0.f;
      for (int r = 0; r < S; r++) {
        const float c = exp2f(ms[r] - mx);
        a = fmaf(ld_cluster_f32(a_o, r), c, a);
        ls = fmaf(ld_cluster_f32(a_ml + 4, r), c, ls);
      }
      p.out[size_t(qi) * p.ldo + h * G * kD + idx] = __float2bfloat16_rn(ls > 0.f ? a / ls : 0.f);
    }
  }
  cluster_sync();  // keep this CTA's shared memory alive until every peer has read it
}

// ---------------------------------------------------------------------------------------------
// Tensor-core form: S = Q K^T and O = P V as m16n8k16 bf16 MMAs (the G query heads of one kv
// head are the rows of a 16-row tile, zero padded), K/V tiles of 16 cached tokens staged in
// shared memory by cp.async (3 stages per warp, XOR-swizzled 16-byte chunks) and fed with
// ldmatrix.  ~7 warp instructions per cached token instead of ~78 in the CUDA-core kernel, which
// is what makes the kernel memory-bound instead of issue-bound.  Same grid, cluster merge and
// numerics contract (fp32 softmax, base-2 exponent) as k_paged_attn.
constexpr int kMW = 4;            // warps per CTA
constexpr int kTile = 16;         // cached tokens per MMA tile
constexpr int kStages = 3;
constexpr int kTileBytes = kTile * kD * 2;            // 4 KB for K, 4 KB for V
constexpr int kMmaSmem = kMW * kStages * 2 * kTileBytes;  // 96 KB

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int G>
__global__ void __launch_bounds__(kMW * 32) k_paged_attn_mma(const AttnParams p) {
  extern __shared__ __align__(1024) uint8_t dsm[];
  __shared__ float sh_o[kMW][G][kD];
  __shared__ float sh_ml[kMW][G][2];
  __shared__ int sh_bt[kMaxBlocksPerCta];
  pdl::launch_dependents();
  pdl::grid_dependency_wait();
  const int qi = blockIdx.x, h = blockIdx.y, sp = blockIdx.z, S = p.splits;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = lane >> 2, quad = lane & 3;       // MMA row (query head) and column pair of this lane
  const int ctx = min(p.ctx_lens[qi], p.max_blocks * p.block_size);  // never walk past the block table (a captured loop replayed beyond the reserved length)
  const int seq = p.seq_of_query ? p.seq_of_query[qi] : qi;
  const int* bt = p.block_tables + size_t(seq) * p.max_blocks;
  int chunk = (ctx + S - 1) / S;
  chunk = (chunk + p.block_size - 1) / p.block_size * p.block_size;
  const int t0 = sp * chunk, t1 = min(ctx, t0 + chunk);

  // Q fragments (A operand): rows >= G are zero
  uint32_t qa0[kD / 16], qa2[kD / 16];
#pragma unroll
  for (int ks = 0; ks < kD / 16; ks++) {
    qa0[ks] = qa2[ks] = 0u;
    if (row < G) {
      const __nv_bfloat16* qp = p.q + size_t(qi) * p.ldq + (h * G + row) * kD + ks * 16 + quad * 2;
      qa0[ks] = *reinterpret_cast<const uint32_t*>(qp);
      qa2[ks] = *reinterpret_cast<const uint32_t*>(qp + 8);
    }
  }
  float o[kD / 8][4];
#pragma unroll
  for (int dn = 0; dn < kD / 8; dn++) o[dn][0] = o[dn][1] = o[dn][2] = o[dn][3] = 0.f;
  float m_run = kNegBig, l_run = 0.f;   // of row `row` (partial over this lane's columns for l)

  const uint32_t wbase = static_cast<uint32_t>(__cvta_generic_to_shared(dsm)) + warp * (kStages * 2 * kTileBytes);
  const int span = kMaxBlocksPerCta * p.block_size;
  for (int pass0 = t0; pass0 < t1; pass0 += span) {
    const int pass1 = min(t1, pass0 + span);
    const int b0 = pass0 / p.block_size, nb = (pass1 - pass0 + p.block_size - 1) / p.block_size;
    __syncthreads();
    if (threadIdx.x < nb) sh_bt[threadIdx.x] = bt[b0 + threadIdx.x];
    __syncthreads();
    const int ntiles = (pass1 - pass0 + kTile - 1) / kTile;
    const int my_tiles = ntiles > warp ? (ntiles - warp + kMW - 1) / kMW : 0;

    auto issue = [&](int i) {   // stage tile i of this warp (tokens tok0 .. tok0+15)
      if (i < my_tiles) {
        const int tok0 = pass0 + (warp + i * kMW) * kTile;
        const uint32_t sk = wbase + (i % kStages) * 2 * kTileBytes, sv = sk + kTileBytes;
#pragma unroll
        for (int c = 0; c < 8; c++) {
          const int id = lane + 32 * c, r = id >> 4, ch = id & 15;
          const int tok = tok0 + r;
          const uint32_t off = uint32_t(r * 256 + ((ch ^ (r & 7)) << 4));
          if (tok < pass1) {
            const long long slot = (long long)sh_bt[tok / p.block_size - b0] * p.block_size + tok % p.block_size;
            const size_t g = (size_t(slot) * p.nkv + h) * kD + ch * 8;
            cp_async16(sk + off, p.k_cache + g);
            cp_async16(sv + off, p.v_cache + g);
          } else {  // masked tokens: zero V so that 0 * garbage cannot make a NaN
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(sv + off), "r"(0u) : "memory");
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(sk + off), "r"(0u) : "memory");
          }
        }
      }
      cp_async_commit();
    };
    issue(0);
    issue(1);
    for (int i = 0; i < my_tiles; i++) {
      issue(i + 2);
      cp_async_wait<2>();
      __syncwarp();
      const int tok0 = pass0 + (warp + i * kMW) * kTile;
      const uint32_t sk = wbase + (i % kStages) * 2 * kTileBytes, sv = sk + kTileBytes;
      // ---- S = Q K^T for 16 tokens (two n tiles of 8)
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < kD / 16; ks++) {
        uint32_t b[4];
        const int mi = lane >> 3, r = ((mi >> 1) << 3) + (lane & 7), ch = ks * 2 + (mi & 1);
        ldmatrix_x4(sk + uint32_t(r * 256 + ((ch ^ (r & 7)) << 4)), b);
        mma_bf16(sc[0], qa0[ks], 0u, qa2[ks], 0u, b[0], b[1]);
        mma_bf16(sc[1], qa0[ks], 0u, qa2[ks], 0u, b[2], b[3]);
      }
      // ---- online softmax on this lane's 4 columns of row `row`
      float mx = m_run;
#pragma unroll
      for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int j = 0; j < 2; j++) {
          const int tok = tok0 + nt * 8 + quad * 2 + j;
          sc[nt][j] = tok < pass1 ? sc[nt][j] * p.scale_log2 : kNegBig;
          mx = fmaxf(mx, sc[nt][j]);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float corr = exp2f(m_run - mx);
      m_run = mx;
      float pr[2][2];
      float ps = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int j = 0; j < 2; j++) {
          const int tok = tok0 + nt * 8 + quad * 2 + j;
          pr[nt][j] = tok < pass1 ? exp2f(sc[nt][j] - mx) : 0.f;
          ps += pr[nt][j];
        }
      l_run = l_run * corr + ps;
#pragma unroll
      for (int dn = 0; dn < kD / 8; dn++) { o[dn][0] *= corr; o[dn][1] *= corr; }
      // ---- O += P V  (P: 16 heads x 16 tokens from the score registers; rows >= 8 are zero)
      const uint32_t pa0 = pack_bf16(pr[0][0], pr[0][1]), pa2 = pack_bf16(pr[1][0], pr[1][1]);
#pragma unroll
      for (int dp = 0; dp < kD / 16; dp++) {   // two 8-dim n tiles per ldmatrix
        uint32_t b[4];
        const int mi = lane >> 3, r = ((mi & 1) << 3) + (lane & 7), ch = dp * 2 + (mi >> 1);
        ldmatrix_x4_trans(sv + uint32_t(r * 256 + ((ch ^ (r & 7)) << 4)), b);
        mma_bf16(o[dp * 2], pa0, 0u, pa2, 0u, b[0], b[1]);
        mma_bf16(o[dp * 2 + 1], pa0, 0u, pa2, 0u, b[2], b[3]);
      }
      __syncwarp();
    }
    cp_async_wait<0>();
  }
  // row sums: add the 4 lanes of a row
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (row < G) {
#pragma unroll
    for (int dn = 0; dn < kD / 8; dn++) {
      sh_o[warp][row][dn * 8 + quad * 2] = o[dn][0];
      sh_o[warp][row][dn * 8 + quad * 2 + 1] = o[dn][1];
    }
    if (quad == 0) { sh_ml[warp][row][0] = m_run; sh_ml[warp][row][1] = l_run; }
  }
  __syncthreads();
  // ---- combine the warps, then the CTAs of the cluster (same as the CUDA-core kernel)
  constexpr int kThreads = kMW * 32;
  constexpr int kPer = (G * kD + kThreads - 1) / kThreads;
  float res_o[kPer], res_m[kPer], res_l[kPer];
#pragma unroll
  for (int k = 0; k < kPer; k++) {
    const int idx = threadIdx.x + k * kThreads;
    if (idx < G * kD) {
      const int g = idx / kD, d = idx % kD;
      float mx = kNegBig;
      for (int w = 0; w < kMW; w++) mx = fmaxf(mx, sh_ml[w][g][0]);
      float a = 0.f, ls = 0.f;
      for (int w = 0; w < kMW; w++) {
        const float c = exp2f(sh_ml[w][g][0] - mx);
        a = fmaf(sh_o[w][g][d], c, a);
        ls = fmaf(sh_ml[w][g][1], c, ls);
      }
      res_o[k] = a; res_m[k] = mx; res_l[k] = ls;
    }
  }
  if (S == 1) {
#pragma unroll
    for (int k = 0; k < kPer; k++) {
      const int idx = threadIdx.x + k * kThreads;
      if (idx < G * kD) p.out[size_t(qi) * p.ldo + h * G * kD + idx] = __float2bfloat16_rn(res_l[k] > 0.f ? res_o[k] / res_l[k] : 0.f);
    }
    return;
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kPer; k++) {
    const int idx = threadIdx.x + k * kThreads;
    if (idx < G * kD) {
      const int g = idx / kD, d = idx % kD;
      sh_o[0][g][d] = res_o[k];
      if (d == 0) { sh_ml[0][g][0] = res_m[k]; sh_ml[0][g][1] = res_l[k]; }
    }
  }
  cluster_sync();
  const int per = (G * kD + S - 1) / S;
  for (int i = threadIdx.x; i < per; i += kThreads) {
    const int idx = sp * per + i;
    if (idx < G * kD) {
      const int g = idx / kD, d = idx % kD;
      const uint32_t a_ml = smem_addr(&sh_ml[0][g][0]), a_o = smem_addr(&sh_o[0][g][d]);
      float ms[kMaxSplits], mx = kNegBig;
      for (int r = 0; r < S; r++) { ms[r] = ld_cluster_f32(a_ml, r); mx = fmaxf(mx, ms[r]); }
      float a = 0.f, ls = 0.f;
      for (int r = 0; r < S; r++) {
        const float c = exp2f(ms[r] - mx);
        a = fmaf(ld_cluster_f32(a_o, r), c, a);
        ls = fmaf(ld_cluster_f32(a_ml + 4, r), c, ls);
      }
      p.out[size_t(qi) * p.ldo + h * G * kD + idx] = __float2bfloat16_rn(ls > 0.f ? a / ls : 0.f);
    }
  }
  cluster_sync();
}

// ---------------------------------------------------------------------------------------------
// Prefill form: a CTA owns up to QT = 64 / G consecutive query tokens of ONE sequence for one kv
// head — 64 MMA rows (token, query head) on 4 warps — and all four warps consume the same K/V
// tiles from shared memory, so a cached token is read once per 64 rows instead of once per query
// row.  Causal: row (t, g) sees keys [0, ctx_lens[t]).  Tiles never straddle sequences: the
// host passes a list of (first row, row count) segments.
constexpr int kPfWarps = 4;
constexpr int kPfStages = 4;
constexpr int kPfSmem = kPfStages * 2 * kTileBytes;   // 32 KB

struct PrefillParams {
  AttnParams a;
  const int* tiles;   // [ntiles, 2]: first query row, number of rows (<= 64 / G)
};

template <int G>
__global__ void __launch_bounds__(kPfWarps * 32) k_prefill_attn_mma(const PrefillParams pp) {
  extern __shared__ __align__(1024) uint8_t dsm[];
  __shared__ int sh_bt[kMaxBlocksPerCta];
  pdl::launch_dependents();
  pdl::grid_dependency_wait();
  const AttnParams& p = pp.a;
  constexpr int QT = 64 / G;
  const int row0 = pp.tiles[2 * blockIdx.x], nrows = pp.tiles[2 * blockIdx.x + 1], h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rlo = warp * 16 + (lane >> 2), rhi = rlo + 8;      // CTA-level MMA rows of this lane
  const int quad = lane & 3;
  const int tlo = rlo / G, glo = rlo % G, thi = rhi / G, ghi = rhi % G;   // (token in tile, query head)
  const bool vlo = tlo < nrows, vhi = thi < nrows;
  const int seq = p.seq_of_query ? p.seq_of_query[row0] : row0;
  const int* bt = p.block_tables + size_t(seq) * p.max_blocks;
  const int ctx_cap = p.max_blocks * p.block_size;             // never walk past the block table
  const int ctx_lo = vlo ? min(p.ctx_lens[row0 + tlo], ctx_cap) : 0, ctx_hi = vhi ? min(p.ctx_lens[row0 + thi], ctx_cap) : 0;
  const int ctx_max = min(p.ctx_lens[row0 + nrows - 1], ctx_cap);   // rows are in position order
  (void)QT;

  uint32_t qa[kD / 16][4];
#pragma unroll
  for (int ks = 0; ks < kD / 16; ks++) {
    qa[ks][0] = qa[ks][1] = qa[ks][2] = qa[ks][3] = 0u;
    if (vlo) {
      const __nv_bfloat16* qp = p.q + size_t(row0 + tlo) * p.ldq + (h * G + glo) * kD + ks * 16 + quad * 2;
      qa[ks][0] = *reinterpret_cast<const uint32_t*>(qp);
      qa[ks][2] = *reinterpret_cast<const uint32_t*>(qp + 8);
    }
    if (vhi) {
      const __nv_bfloat16* qp = p.q + size_t(row0 + thi) * p.ldq + (h * G + ghi) * kD + ks * 16 + quad * 2;
      qa[ks][1] = *reinterpret_cast<const uint32_t*>(qp);
      qa[ks][3] = *reinterpret_cast<const uint32_t*>(qp + 8);
    }
  }
  float o[kD / 8][4];
#pragma unroll
  for (int dn = 0; dn < kD / 8; dn++) o[dn][0] = o[dn][1] = o[dn][2] = o[dn][3] = 0.f;
  float m_lo = kNegBig, m_hi = kNegBig, l_lo = 0.f, l_hi = 0.f;

  const uint32_t sbase = static_cast<uint32_t>(__cvta_generic_to_shared(dsm));
  const int span = kMaxBlocksPerCta * p.block_size;
  for (int pass0 = 0; pass0 < ctx_max; pass0 += span) {
    const int pass1 = min(ctx_max, pass0 + span);
    const int b0 = pass0 / p.block_size, nb = (pass1 - pass0 + p.block_size - 1) / p.block_size;
    __syncthreads();
    if (threadIdx.x < nb) sh_bt[threadIdx.x] = bt[b0 + threadIdx.x];
    __syncthreads();
    const int ntiles = (pass1 - pass0 + kTile - 1) / kTile;
    auto issue = [&](int i) {   // all 128 threads stage tile i: 256 K chunks + 256 V chunks
      if (i < ntiles) {
        const int tok0 = pass0 + i * kTile;
        const uint32_t sk = sbase + (i % kPfStages) * 2 * kTileBytes, sv = sk + kTileBytes;
#pragma unroll
        for (int c = 0; c < 2; c++) {
          const int id = threadIdx.x + 128 * c, r = id >> 4, ch = id & 15;
          const int tok = tok0 + r;
          const uint32_t off = uint32_t(r * 256 + ((ch ^ (r & 7)) << 4));
          if (tok < pass1) {
            const long long slot = (long long)sh_bt[tok / p.block_size - b0] * p.block_size + tok % p.block_size;
            const size_t g = (size_t(slot) * p.nkv + h) * kD + ch * 8;
            cp_async16(sk + off, p.k_cache + g);
            cp_async16(sv + off, p.v_cache + g);
          } else {
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(sv + off), "r"(0u) : "memory");
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(sk + off), "r"(0u) : "memory");
          }
        }
      }
      cp_async_commit();
    };
    issue(0); issue(1); issue(2);
    for (int i = 0; i < ntiles; i++) {
      issue(i + 3);
      cp_async_wait<3>();
      __syncthreads();
      const int tok0 = pass0 + i * kTile;
      const uint32_t sk = sbase + (i % kPfStages) * 2 * kTileBytes, sv = sk + kTileBytes;
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < kD / 16; ks++) {
        uint32_t b[4];
        const int mi = lane >> 3, r = ((mi >> 1) << 3) + (lane & 7), ch = ks * 2 + (mi & 1);
        ldmatrix_x4(sk + uint32_t(r * 256 + ((ch ^ (r & 7)) << 4)), b);
        mma_bf16(sc[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[0], b[1]);
        mma_bf16(sc[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[2], b[3]);
      }
      float mx_lo = m_lo, mx_hi = m_hi;
#pragma unroll
      for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int j = 0; j < 2; j++) {
          const int tok = tok0 + nt * 8 + quad * 2 + j;
          sc[nt][j] = tok < ctx_lo ? sc[nt][j] * p.scale_log2 : kNegBig;
          sc[nt][2 + j] = tok < ctx_hi ? sc[nt][2 + j] * p.scale_log2 : kNegBig;
          mx_lo = fmaxf(mx_lo, sc[nt][j]);
          mx_hi = fmaxf(mx_hi, sc[nt][2 + j]);
        }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float c_lo = exp2f(m_lo - mx_lo), c_hi = exp2f(m_hi - mx_hi);
      m_lo = mx_lo; m_hi = mx_hi;
      float pr[2][4], s_lo = 0.f, s_hi = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int j = 0; j < 2; j++) {
          const int tok = tok0 + nt * 8 + quad * 2 + j;
          pr[nt][j] = tok < ctx_lo ? exp2f(sc[nt][j] - mx_lo) : 0.f;
          pr[nt][2 + j] = tok < ctx_hi ? exp2f(sc[nt][2 + j] - mx_hi) : 0.f;
          s_lo += pr[nt][j];
          s_hi += pr[nt][2 + j];
        }
      l_lo = l_lo * c_lo + s_lo;
      l_hi = l_hi * c_hi + s_hi;
#pragma unroll
      for (int dn = 0; dn < kD / 8; dn++) { o[dn][0] *= c_lo; o[dn][1] *= c_lo; o[dn][2] *= c_hi; o[dn][3] *= c_hi; }
      const uint32_t pa0 = pack_bf16(pr[0][0], pr[0][1]), pa1 = pack_bf16(pr[0][2], pr[0][3]);
      const uint32_t pa2 = pack_bf16(pr[1][0], pr[1][1]), pa3 = pack_bf16(pr[1][2], pr[1][3]);
#pragma unroll
      for (int dp = 0; dp < kD / 16; dp++) {
        uint32_t b[4];
        const int mi = lane >> 3, r = ((mi & 1) << 3) + (lane & 7), ch = dp * 2 + (mi >> 1);
        ldmatrix_x4_trans(sv + uint32_t(r * 256 + ((ch ^ (r & 7)) << 4)), b);
        mma_bf16(o[dp * 2], pa0, pa1, pa2, pa3, b[0], b[1]);
        mma_bf16(o[dp * 2 + 1], pa0, pa1, pa2, pa3, b[2], b[3]);
      }
      __syncthreads();   // everyone is done with this stage before it is refilled
    }
    cp_async_wait<0>();
  }
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
#pragma unroll
  for (int dn = 0; dn < kD / 8; dn++) {
    if (vlo) *reinterpret_cast<__nv_bfloat162*>(p.out + size_t(row0 + tlo) * p.ldo + (h * G + glo) * kD + dn * 8 + quad * 2) =
        __floats2bfloat162_rn(o[dn][0] * inv_lo, o[dn][1] * inv_lo);
    if (vhi) *reinterpret_cast<__nv_bfloat162*>(p.out + size_t(row0 + thi) * p.ldo + (h * G + ghi) * kD + dn * 8 + quad * 2) =
        __floats2bfloat162_rn(o[dn][2] * inv_hi, o[dn][3] * inv_hi);
  }
}

}  // namespace

extern "C" {

// kv splits merge through cluster shared memory: no scratch is needed.  Kept for callers
// that size a workspace: returns a token amount.
size_t tbv_op_attn_workspace(int nq_rows, int nq_heads, int nkv, int max_splits) {
  (void)nq_rows; (void)nq_heads; (void)nkv; (void)max_splits;
  return 256;
}

// splits: 1..8 CTAs (one thread-block cluster) per (query row, kv head).
int tbv_op_paged_attention(const void* q, const void* k_cache, const void* v_cache, const void* block_tables,
                           const void* seq_of_query, const void* ctx_lens, void* out, void* workspace, int nq_rows, int nq_heads,
                           int nkv, int head_dim, int ldq, int ldo, int block_size, int max_blocks, int splits, float scale,
                           void* stream) {
  (void)workspace;
  if (nq_rows <= 0) return 0;
  if (head_dim != kD || nq_heads % nkv || (ldq % 8) || block_size <= 0) return -2;
  const int G = nq_heads / nkv;
  splits = splits < 1 ? 1 : (splits > kMaxSplits ? kMaxSplits : splits);
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.block_tables = static_cast<const int*>(block_tables);
  p.seq_of_query = static_cast<const int*>(seq_of_query);
  p.ctx_lens = static_cast<const int*>(ctx_lens);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.ldq = ldq; p.ldo = ldo; p.nkv = nkv; p.block_size = block_size; p.max_blocks = max_blocks; p.splits = splits;
  dim3 grid(nq_rows, nkv, splits);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaSuccess;
  static int impl = -1;  // TBV_ATTN=simt selects the CUDA-core kernel (kept for comparison)
  if (impl < 0) {
    const char* ev = getenv("TBV_ATTN");
    impl = (ev && !strcmp(ev, "simt")) ? 0 : 1;
    cudaFuncSetAttribute(k_paged_attn_mma<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmem);
    cudaFuncSetAttribute(k_paged_attn_mma<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmem);
    cudaFuncSetAttribute(k_paged_attn_mma<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmem);
    cudaFuncSetAttribute(k_paged_attn_mma<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmem);
  }
  if (impl == 1) {
    const dim3 blk(kMW * 32);
    switch (G) {
      case 1: e = pdl::launch(k_paged_attn_mma<1>, grid, blk, kMmaSmem, st, splits, p); break;
      case 2: e = pdl::launch(k_paged_attn_mma<2>, grid, blk, kMmaSmem, st, splits, p); break;
      case 4: e = pdl::launch(k_paged_attn_mma<4>, grid, blk, kMmaSmem, st, splits, p); break;
      case 8: e = pdl::launch(k_paged_attn_mma<8>, grid, blk, kMmaSmem, st, splits, p); break;
      default: return -2;
    }
    return e == cudaSuccess ? 0 : -1;
  }
  switch (G) {
    case 1: e = pdl::launch(k_paged_attn<1, 256>, grid, dim3(256), 0, st, splits, p); break;
    case 2: e = pdl::launch(k_paged_attn<2, 256>, grid, dim3(256), 0, st, splits, p); break;
    case 4: e = pdl::launch(k_paged_attn<4, 256>, grid, dim3(256), 0, st, splits, p); break;
    case 8: e = pdl::launch(k_paged_attn<8, 128>, grid, dim3(128), 0, st, splits, p); break;
    default: return -2;
  }
  return e == cudaSuccess ? 0 : -1;
}


// Causal prefill over the paged cache.  tiles: int32 [ntiles, 2] = (first query row, rows <= 64 / G) with all
// rows of a tile belonging to one sequence in position order; ctx_lens[row] = keys visible to that row.
int tbv_op_prefill_attention(const void* q, const void* k_cache, const void* v_cache, const void* block_tables,
                             const void* seq_of_query, const void* ctx_lens, const void* tiles, void* out, int ntiles,
                             int nq_heads, int nkv, int head_dim, int ldq, int ldo, int block_size, int max_blocks, float scale,
                             void* stream) {
  if (ntiles <= 0) return 0;
  if (head_dim != kD || nq_heads % nkv || (ldq % 8) || block_size <= 0) return -2;
  const int G = nq_heads / nkv;
  PrefillParams pp{};
  AttnParams& p = pp.a;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.block_tables = static_cast<const int*>(block_tables);
  p.seq_of_query = static_cast<const int*>(seq_of_query);
  p.ctx_lens = static_cast<const int*>(ctx_lens);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.ldq = ldq; p.ldo = ldo; p.nkv = nkv; p.block_size = block_size; p.max_blocks = max_blocks; p.splits = 1;
  pp.tiles = static_cast<const int*>(tiles);
  const dim3 grid(ntiles, nkv), blk(kPfWarps * 32);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  switch (G) {
    case 1: e = pdl::launch(k_prefill_attn_mma<1>, grid, blk, kPfSmem, st, 1, pp); break;
    case 2: e = pdl::launch(k_prefill_attn_mma<2>, grid, blk, kPfSmem, st, 1, pp); break;
    case 4: e = pdl::launch(k_prefill_attn_mma<4>, grid, blk, kPfSmem, st, 1, pp); break;
    case 8: e = pdl::launch(k_prefill_attn_mma<8>, grid, blk, kPfSmem, st, 1, pp); break;
    default: return -2;
  }
  return e == cudaSuccess ? 0 : -1;
}

}  // extern "C"
