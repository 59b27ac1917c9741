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
constexpr int kThreads = 128;  // 8 half-warps
constexpr int kHW = kThreads / 16;
constexpr int kU = 4;          // tokens in flight per half-warp (8 x 16-byte loads per thread)
constexpr float kNegBig = -1e30f;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}

struct AttnParams {
  const __nv_bfloat16* q;   // [Nq, nq, D], row stride ldq
  const __nv_bfloat16* k_cache;  // [slots, nkv, D]
  const __nv_bfloat16* v_cache;
  const int* block_tables;  // [nseq, max_blocks]
  const int* seq_of_query;  // [Nq] or null (identity)
  const int* ctx_lens;      // [Nq]: keys visible to this query row
  __nv_bfloat16* out;       // [Nq, nq, D], row stride ldo
  float* part_o;            // [Nq, nkv, splits, G, D]   (scratch, splits > 1)
  float* part_ml;           // [Nq, nkv, splits, G, 2]
  unsigned* tickets;        // [Nq, nkv], zero between launches
  float scale_log2;         // softmax scale * log2(e)
  int ldq, ldo, nkv, block_size, max_blocks, splits;
};

template <int G>
__global__ void __launch_bounds__(kThreads) k_paged_attn(const AttnParams p) {
  pdl::launch_dependents();
  pdl::grid_dependency_wait();
  const int qi = blockIdx.x, h = blockIdx.y, sp = blockIdx.z;
  const int hw = threadIdx.x >> 4, l16 = threadIdx.x & 15;
  const int ctx = p.ctx_lens[qi];
  const int seq = p.seq_of_query ? p.seq_of_query[qi] : qi;
  const int* bt = p.block_tables + size_t(seq) * p.max_blocks;
  int chunk = (ctx + p.splits - 1) / p.splits;
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

  // The trip count is the same for every thread of the CTA (the shuffles below name the
  // whole warp); tokens past the end are masked per half-warp.
  for (int base = t0; base < t1; base += kHW * kU) {
    const int tok = base + hw;
    uint4 kv[kU], vv[kU];
    bool valid[kU];
#pragma unroll
    for (int j = 0; j < kU; j++) {
      const int tj = tok + j * kHW;
      valid[j] = tj < t1;
      if (valid[j]) {
        const long long slot = (long long)bt[tj / p.block_size] * p.block_size + tj % p.block_size;
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
    float vf[kU][8];
#pragma unroll
    for (int j = 0; j < kU; j++) unpack8(vv[j], vf[j]);
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
      for (int i = 0; i < 8; i++) {
        float a = acc[g][i] * corr;
#pragma unroll
        for (int j = 0; j < kU; j++) a = fmaf(pj[j], vf[j][i], a);
        acc[g][i] = a;
      }
    }
  }

  // combine the 8 half-warps
  __shared__ float sh_o[kHW][G][kD];
  __shared__ float sh_ml[kHW][G][2];
#pragma unroll
  for (int g = 0; g < G; g++) {
#pragma unroll
    for (int i = 0; i < 8; i++) sh_o[hw][g][l16 * 8 + i] = acc[g][i];
    if (l16 == 0) { sh_ml[hw][g][0] = m[g]; sh_ml[hw][g][1] = l[g]; }
  }
  __syncthreads();
  const int d = threadIdx.x;  // one thread per output dim
  float o[G], lm[G], ll[G];
#pragma unroll
  for (int g = 0; g < G; g++) {
    float mx = kNegBig;
    for (int w = 0; w < kHW; w++) mx = fmaxf(mx, sh_ml[w][g][0]);
    float a = 0.f, ls = 0.f;
    for (int w = 0; w < kHW; w++) {
      const float c = exp2f(sh_ml[w][g][0] - mx);
      a = fmaf(sh_o[w][g][d], c, a);
      ls = fmaf(sh_ml[w][g][1], c, ls);
    }
    o[g] = a; lm[g] = mx; ll[g] = ls;
  }
  if (p.splits == 1) {
#pragma unroll
    for (int g = 0; g < G; g++)
      p.out[size_t(qi) * p.ldo + (h * G + g) * kD + d] = __float2bfloat16_rn(ll[g] > 0.f ? o[g] / ll[g] : 0.f);
    return;
  }
  const size_t pbase = (size_t(qi) * p.nkv + h) * p.splits;
#pragma unroll
  for (int g = 0; g < G; g++) {
    p.part_o[((pbase + sp) * G + g) * kD + d] = o[g];
    if (d == 0) { p.part_ml[((pbase + sp) * G + g) * 2] = lm[g]; p.part_ml[((pbase + sp) * G + g) * 2 + 1] = ll[g]; }
  }
  __shared__ bool last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(&p.tickets[size_t(qi) * p.nkv + h], 1u) == unsigned(p.splits - 1);
  __syncthreads();
  if (!last) return;
  __threadfence();
#pragma unroll
  for (int g = 0; g < G; g++) {
    float mx = kNegBig;
    for (int s2 = 0; s2 < p.splits; s2++) mx = fmaxf(mx, *(volatile float*)&p.part_ml[((pbase + s2) * G + g) * 2]);
    float a = 0.f, ls = 0.f;
    for (int s2 = 0; s2 < p.splits; s2++) {
      const float c = exp2f(*(volatile float*)&p.part_ml[((pbase + s2) * G + g) * 2] - mx);
      a = fmaf(*(volatile float*)&p.part_o[((pbase + s2) * G + g) * kD + d], c, a);
      ls = fmaf(*(volatile float*)&p.part_ml[((pbase + s2) * G + g) * 2 + 1], c, ls);
    }
    p.out[size_t(qi) * p.ldo + (h * G + g) * kD + d] = __float2bfloat16_rn(ls > 0.f ? a / ls : 0.f);
  }
  if (threadIdx.x == 0) p.tickets[size_t(qi) * p.nkv + h] = 0;
}

}  // namespace

extern "C" {

// Scratch for kv splits: tickets (u32 per (query, kv head), must be zero before the first
// launch; the kernel leaves them zero) followed by the fp32 partials.
size_t tbv_op_attn_workspace(int nq_rows, int nq_heads, int nkv, int max_splits) {
  const size_t tick = (size_t(nq_rows) * nkv * 4 + 255) & ~size_t(255);
  return tick + size_t(nq_rows) * nq_heads * max_splits * (kD + 2) * 4;
}

int tbv_op_paged_attention(const void* q, const void* k_cache, const void* v_cache, const void* block_tables,
                           const void* seq_of_query, const void* ctx_lens, void* out, void* workspace, int nq_rows, int nq_heads,
                           int nkv, int head_dim, int ldq, int ldo, int block_size, int max_blocks, int splits, float scale,
                           void* stream) {
  if (nq_rows <= 0) return 0;
  if (head_dim != kD || nq_heads % nkv || (ldq % 8) || block_size <= 0) return -2;
  const int G = nq_heads / nkv;
  if (splits < 1) splits = 1;
  if (splits > 1 && !workspace) return -2;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.block_tables = static_cast<const int*>(block_tables);
  p.seq_of_query = static_cast<const int*>(seq_of_query);
  p.ctx_lens = static_cast<const int*>(ctx_lens);
  p.out = static_cast<__nv_bfloat16*>(out);
  char* ws = static_cast<char*>(workspace);
  const size_t tick = (size_t(nq_rows) * nkv * 4 + 255) & ~size_t(255);
  p.tickets = reinterpret_cast<unsigned*>(ws);
  p.part_o = reinterpret_cast<float*>(ws + tick);
  p.part_ml = p.part_o + size_t(nq_rows) * nq_heads * splits * kD;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.ldq = ldq; p.ldo = ldo; p.nkv = nkv; p.block_size = block_size; p.max_blocks = max_blocks; p.splits = splits;
  dim3 grid(nq_rows, nkv, splits);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaSuccess;
  switch (G) {
    case 1: e = pdl::launch(k_paged_attn<1>, grid, dim3(kThreads), 0, st, 1, p); break;
    case 2: e = pdl::launch(k_paged_attn<2>, grid, dim3(kThreads), 0, st, 1, p); break;
    case 4: e = pdl::launch(k_paged_attn<4>, grid, dim3(kThreads), 0, st, 1, p); break;
    case 8: e = pdl::launch(k_paged_attn<8>, grid, dim3(kThreads), 0, st, 1, p); break;
    default: return -2;
  }
  return e == cudaSuccess ? 0 : -1;
}

}  // extern "C"
