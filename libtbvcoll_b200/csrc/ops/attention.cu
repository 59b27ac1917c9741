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
  const int ctx = p.ctx_lens[qi];
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
  switch (G) {
    case 1: e = pdl::launch(k_paged_attn<1, 256>, grid, dim3(256), 0, st, splits, p); break;
    case 2: e = pdl::launch(k_paged_attn<2, 256>, grid, dim3(256), 0, st, splits, p); break;
    case 4: e = pdl::launch(k_paged_attn<4, 256>, grid, dim3(256), 0, st, splits, p); break;
    case 8: e = pdl::launch(k_paged_attn<8, 128>, grid, dim3(128), 0, st, splits, p); break;
    default: return -2;
  }
  return e == cudaSuccess ? 0 : -1;
}

}  // extern "C"
