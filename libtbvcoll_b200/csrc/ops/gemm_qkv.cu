// gemm_qkv.cu — the qkv projection with RoPE and the KV-cache write in its epilogue.
//
// With output features on the UMMA M axis, one 128-row tile is exactly one attention head
// (head_dim 128), so the rotation partners (d, d + 64) of every token are in the same tile.
// The epilogue rounds the accumulator (+ bias) to bf16 — the value an unfused pipeline would
// have stored — applies the HF rotate_half rotation in bf16 arithmetic, writes q / k / v into the
// qkv activation buffer and scatters the k and v heads into the paged cache.  Results are bit
// for bit those of `tbv_op_gemm` followed by `tbv_op_rope_kv`; one launch per layer is saved.
// (The reference's engine lists RoPE and the q/k/v -> qkv weight fusion without code:
// reports/11_custom_engine.md:12,38.)
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include "gemm.cuh"
#include "ops.h"

using namespace sm100;

namespace {

struct RopeArgs {
  const int* positions;            // [N]
  const float* cos_sin;            // [max_pos, 128]: cos(0..63), sin(0..63)
  const long long* slot_mapping;   // [N] cache row per token (< 0: skip) or null
  __nv_bfloat16* k_cache;          // [slots, nkv, 128]
  __nv_bfloat16* v_cache;
  int nq, nkv, max_pos;
};

__device__ __forceinline__ float bfr(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ void rotate(float x1, float x2, float c, float s, float& o1, float& o2) {
  o1 = bfr(bfr(x1 * c) + bfr(-x2 * s));
  o2 = bfr(bfr(x2 * c) + bfr(x1 * s));
}

__global__ void __launch_bounds__(gemm::kThreads, 1)
k_gemm_qkv_rope(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const gemm::Params p, const RopeArgs ra) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ gemm::Smem s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = p.raster ? blockIdx.y : blockIdx.x, m0 = head * gemm::kBM, n0 = (p.raster ? blockIdx.x : blockIdx.y) * p.bn;
  const int S = p.splits;
  const int split = S > 1 ? int(cluster_ctarank()) : 0;
  const int kb_per = (p.kb_total + S - 1) / S;
  const int kb0 = split * kb_per;
  int nkb = p.kb_total - kb0;
  nkb = nkb < 0 ? 0 : (nkb > kb_per ? kb_per : nkb);
  uint8_t* sm = gemm::mainloop(&tmA, &tmB, p, s, smem_raw, m0, n0, kb0, nkb);
  volatile int* abortp = &s.abort_flag;
  const int rows = (p.N - n0 < p.bn) ? (p.N - n0) : p.bn;
  const bool rot = head < ra.nq + ra.nkv;                         // q and k heads rotate
  const int kvh = head < ra.nq ? -1 : (head < ra.nq + ra.nkv ? head - ra.nq : head - ra.nq - ra.nkv);
  __nv_bfloat16* cache = head < ra.nq ? nullptr : (head < ra.nq + ra.nkv ? ra.k_cache : ra.v_cache);

  // Split-K form: the rotation of an output piece needs its token's position, then the cos / sin entries of that
  // position, then the cache slot — a chain of dependent global loads.  The epilogue threads fetch them for their first
  // piece while the MMAs run (after their own dependency wait: positions and slots are written by the previous step),
  // instead of after the reduction.
  const int pf_half = S > 1 ? 64 / S : 0, pf_q4 = pf_half / 4 > 0 ? pf_half / 4 : 1;
  const int pf_idx = int(threadIdx.x) - 64;
  bool pf_ok = false;
  int pf_pos = 0;
  long long pf_slot = -1;
  float4 pf_cos = make_float4(1.f, 1.f, 1.f, 1.f), pf_sin = make_float4(0.f, 0.f, 0.f, 0.f);
  if (S > 1 && warp >= 2 && pf_idx < rows * pf_q4 && pf_half >= 4) {
    pdl::grid_dependency_wait();
    const int t = pf_idx / pf_q4, d = split * pf_half + (pf_idx % pf_q4) * 4;
    int pos = ra.positions[n0 + t];
    pos = pos < 0 ? 0 : (pos >= ra.max_pos ? ra.max_pos - 1 : pos);
    pf_pos = pos;
    if (rot) {
      pf_cos = *reinterpret_cast<const float4*>(ra.cos_sin + size_t(pos) * 128 + d);
      pf_sin = *reinterpret_cast<const float4*>(ra.cos_sin + size_t(pos) * 128 + 64 + d);
    }
    if (cache && ra.slot_mapping) pf_slot = ra.slot_mapping[n0 + t];
    pf_ok = true;
  }

  if (warp >= 2) {
    const int quarter = warp & 3, ml = quarter * 32 + lane;
    bool ok = nkb > 0 ? mbar_wait(smem_u32(&s.accum), 0, abortp, p.limit_ns) : true;
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const float bias = p.bias ? __bfloat162float(p.bias[m0 + ml]) : 0.f;
    float* stage_f = reinterpret_cast<float*>(sm);
    __nv_bfloat16* stage_h = reinterpret_cast<__nv_bfloat16*>(sm);
    for (int col = 0; col < p.bn; col += 16) {
      uint32_t r[16];
      if (ok && nkb > 0) {
        tmem_ld16(s.tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(col), r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 16; j++) r[j] = 0u;
      }
      if (S > 1) {
#pragma unroll
        for (int j = 0; j < 16; j++) stage_f[(col + j) * 128 + ml] = __uint_as_float(r[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 16; j++) stage_h[(col + j) * 128 + ml] = __float2bfloat16_rn(__uint_as_float(r[j]) + bias);
      }
    }
    if (S == 1) {
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int te = threadIdx.x - 64;
      if (rot) {
        for (int idx = te; idx < rows * 64; idx += 128) {
          const int t = idx >> 6, d = idx & 63;
          int pos = ra.positions[n0 + t];
          pos = pos < 0 ? 0 : (pos >= ra.max_pos ? ra.max_pos - 1 : pos);
          const float c = bfr(ra.cos_sin[size_t(pos) * 128 + d]), sn = bfr(ra.cos_sin[size_t(pos) * 128 + 64 + d]);
          float o1, o2;
          rotate(__bfloat162float(stage_h[t * 128 + d]), __bfloat162float(stage_h[t * 128 + d + 64]), c, sn, o1, o2);
          stage_h[t * 128 + d] = __float2bfloat16_rn(o1);
          stage_h[t * 128 + d + 64] = __float2bfloat16_rn(o2);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      for (int idx = te; idx < rows * 16; idx += 128) {   // 16-byte pieces: 16 per 128-feature row
        const int t = idx >> 4, pc = idx & 15;
        const uint4 v = *reinterpret_cast<const uint4*>(stage_h + t * 128 + pc * 8);
        *reinterpret_cast<uint4*>(p.y + size_t(n0 + t) * p.ldy + m0 + pc * 8) = v;
        if (cache) {
          const long long slot = ra.slot_mapping ? ra.slot_mapping[n0 + t] : -1;
          if (slot >= 0) *reinterpret_cast<uint4*>(cache + (size_t(slot) * ra.nkv + kvh) * 128 + pc * 8) = v;
        }
      }
    }
  }

  if (S > 1) {
    // deterministic split-K; CTA j of the cluster owns dims [j*half, (j+1)*half) of BOTH halves of
    // the head so that it holds both rotation partners
    __syncwarp();
    cluster_sync_all();
    if (warp >= 2) {
      const int te = threadIdx.x - 64;
      const int half = 64 / S, q4 = half / 4 > 0 ? half / 4 : 1;
      const uint32_t stage_addr = smem_u32(sm);
      for (int idx = te; idx < rows * q4; idx += 128) {
        const int t = idx / q4, d = split * half + (idx % q4) * 4;
        const float4 a = dsmem_sum_f32x4(stage_addr + uint32_t((t * 128 + d) * 4), S);
        const float4 b = dsmem_sum_f32x4(stage_addr + uint32_t((t * 128 + d + 64) * 4), S);
        float lo[4] = {a.x, a.y, a.z, a.w}, hi[4] = {b.x, b.y, b.z, b.w};
        const bool pre = pf_ok && idx == pf_idx;   // this thread's first piece: its position, cos / sin and slot are in registers
        int pos = pf_pos;
        float cs[4] = {pf_cos.x, pf_cos.y, pf_cos.z, pf_cos.w}, sn[4] = {pf_sin.x, pf_sin.y, pf_sin.z, pf_sin.w};
        if (!pre) {
          pos = ra.positions[n0 + t];
          pos = pos < 0 ? 0 : (pos >= ra.max_pos ? ra.max_pos - 1 : pos);
          if (rot) {
#pragma unroll
            for (int e = 0; e < 4; e++) { cs[e] = ra.cos_sin[size_t(pos) * 128 + d + e]; sn[e] = ra.cos_sin[size_t(pos) * 128 + 64 + d + e]; }
          }
        }
        __nv_bfloat16 ol[4], oh[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float x1 = bfr(lo[e] + (p.bias ? __bfloat162float(p.bias[m0 + d + e]) : 0.f));
          const float x2 = bfr(hi[e] + (p.bias ? __bfloat162float(p.bias[m0 + d + 64 + e]) : 0.f));
          float o1 = x1, o2 = x2;
          if (rot) rotate(x1, x2, bfr(cs[e]), bfr(sn[e]), o1, o2);
          ol[e] = __float2bfloat16_rn(o1);
          oh[e] = __float2bfloat16_rn(o2);
        }
        const uint2 vl = *reinterpret_cast<const uint2*>(ol), vh = *reinterpret_cast<const uint2*>(oh);
        __nv_bfloat16* dst = p.y + size_t(n0 + t) * p.ldy + m0 + d;
        *reinterpret_cast<uint2*>(dst) = vl;
        *reinterpret_cast<uint2*>(dst + 64) = vh;
        if (cache) {
          const long long slot = pre ? pf_slot : (ra.slot_mapping ? ra.slot_mapping[n0 + t] : -1);
          if (slot >= 0) {
            __nv_bfloat16* cd = cache + (size_t(slot) * ra.nkv + kvh) * 128 + d;
            *reinterpret_cast<uint2*>(cd) = vl;
            *reinterpret_cast<uint2*>(cd + 64) = vh;
          }
        }
      }
    }
    __syncwarp();
    cluster_sync_all();
  }
  __syncwarp();
  gemm::teardown(p, s);
}

bool g_attr = false;

}  // namespace

extern "C" int tbv_op_gemm_qkv_rope(const void* w, const void* x, void* qkv, const void* bias, int M, int N, int K, int ldx, int ldy,
                                    const void* positions, const void* cos_sin, const void* slot_mapping, void* k_cache, void* v_cache,
                                    int nq, int nkv, int max_pos, int splits_hint, void* stream) {
  const char* pf_ptr = nullptr;   // an announcement holds for exactly one launch
  const unsigned long long pf_bytes = tbvops::take_next_prefetch(&pf_ptr, (unsigned long long)(M > 0 ? M : 0) * (unsigned long long)(K > 0 ? K : 0) * 2ull);
  if (M != (nq + 2 * nkv) * 128 || N <= 0 || (K % 8) || (ldx % 8) || (ldy % 8)) return -2;
  int bn, splits, stages;
  tbvops::gemm_config(M, N, K, splits_hint, &bn, &splits, &stages);
  CUtensorMap tmA, tmB;
  if (tbvops::make_tensor_map_bf16(&tmA, w, M, K, K, 128) != 0) return -3;
  if (tbvops::make_tensor_map_bf16(&tmB, x, N, K, ldx, bn) != 0) return -3;
  gemm::Params p{};
  p.M = M; p.N = N; p.K = K; p.ldy = ldy; p.bn = bn; p.splits = splits; p.stages = stages;
  p.kb_total = (K + 63) / 64;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.y = static_cast<__nv_bfloat16*>(qkv);
  p.limit_ns = 2000000000ull;
  p.err = tbvops::gemm_err_flag();
  p.pf_ptr = pf_ptr;
  p.pf_bytes = pf_bytes;
  RopeArgs ra{static_cast<const int*>(positions), static_cast<const float*>(cos_sin), static_cast<const long long*>(slot_mapping),
              static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), nq, nkv, max_pos};
  if (!g_attr) {
    if (cudaFuncSetAttribute(k_gemm_qkv_rope, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) return -1;
    g_attr = true;
  }
  const size_t smem = size_t(stages) * (gemm::kATileBytes + bn * 128) + 1024;
  const int mt = M / 128, nt = (N + bn - 1) / bn;
  p.raster = nt > 1 ? 1 : 0;   // token tiles of one head launch together: its weights stream from HBM once
  cudaError_t e = pdl::launch(k_gemm_qkv_rope, dim3(p.raster ? nt : mt, p.raster ? mt : nt, splits), dim3(gemm::kThreads), smem,
                              static_cast<cudaStream_t>(stream), splits, tmA, tmB, p, ra);
  if (e != cudaSuccess) {
    fprintf(stderr, "[tbvops] qkv+rope gemm launch failed: %s\n", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}
