// gemm.cu — bf16 GEMM on tcgen05 tensor cores (TMA-fed, TMEM accumulators) with fused
// epilogues, and its host-side launcher (tensor-map cache, tile/split heuristics).
//
// The reference has no GEMM of its own: linear layers run inside vLLM / PyTorch on
// rocBLAS (reports/11_custom_engine.md:38 describes q/k/v -> qkv and gate/up -> gate_up
// weight fusion in the absent engine).  These kernels are the sm_100a replacement for
// that path: qkv, gate_up (+ SiLU-mul in the epilogue), o_proj, down_proj, lm_head.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "gemm.cuh"
#include "ops.h"

using namespace sm100;
using gemm::Params;

namespace {

enum Epi : int { kEpiStore = 0, kEpiSiluMul = 1 };

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
// silu(g) * u with every intermediate rounded to bf16, which is what an unfused bf16
// pipeline (gate, act(gate), act * up as separate bf16 tensors) produces.
__device__ __forceinline__ float silu_mul_bf16(float g, float u) {
  g = bf16_round(g);
  u = bf16_round(u);
  float s = bf16_round(g / (1.0f + __expf(-g)));
  return s * u;
}

template <int EPI>
__global__ void __launch_bounds__(gemm::kThreads, 1)
k_gemm(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ gemm::Smem s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Launch order follows blockIdx.x.  With many token tiles the CTAs that share one 128-row weight tile
  // must run together, so that the weights stream from HBM once and the activations stay in L2.
  const int m0 = (p.raster ? blockIdx.y : blockIdx.x) * gemm::kBM, n0 = (p.raster ? blockIdx.x : blockIdx.y) * p.bn;
  const int S = p.splits;
  const int split = S > 1 ? int(cluster_ctarank()) : 0;
  const int kb_per = (p.kb_total + S - 1) / S;
  const int kb0 = split * kb_per;
  int nkb = p.kb_total - kb0;
  nkb = nkb < 0 ? 0 : (nkb > kb_per ? kb_per : nkb);

  uint8_t* sm = gemm::mainloop(&tmA, &tmB, p, s, smem_raw, m0, n0, kb0, nkb);
  volatile int* abortp = &s.abort_flag;
  const int rows = (p.N - n0 < p.bn) ? (p.N - n0) : p.bn;  // valid tokens in this tile
  constexpr int OUTW = EPI == kEpiSiluMul ? 64 : 128;       // output features per tile

  if (warp >= 2) {
    const int quarter = warp & 3;             // TMEM lane quarter this warp may read
    const int ml = quarter * 32 + lane;       // feature row inside the tile
    bool ok = nkb > 0 ? mbar_wait(smem_u32(&s.accum), 0, abortp, p.limit_ns) : true;
    // lanes leave the polling loop at different times: reconverge before the warp-wide
    // (.sync.aligned) TMEM loads, and make the decision to load warp-uniform
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const float bias = (p.bias && m0 + ml < p.M) ? __bfloat162float(p.bias[m0 + ml]) : 0.f;
    float* stage_f = reinterpret_cast<float*>(sm);
    __nv_bfloat16* stage_h = reinterpret_cast<__nv_bfloat16*>(sm);
    for (int c = 0; c < p.bn; c += 16) {
      uint32_t r[16];
      if (ok && nkb > 0) {
        tmem_ld16(s.tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(c), r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 16; j++) r[j] = 0u;
      }
      if (S > 1) {
#pragma unroll
        for (int j = 0; j < 16; j++) stage_f[(c + j) * 128 + ml] = __uint_as_float(r[j]);
      } else if (EPI == kEpiSiluMul) {
        // Even lanes hold gate rows, odd lanes the matching up rows.  Per pair of token columns the two lanes
        // swap one value each, so that the even lane finishes column j and the odd lane column j + 1: every
        // lane does useful SiLU work and one shuffle serves two outputs.
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const float v0 = __uint_as_float(r[j]) + bias, v1 = __uint_as_float(r[j + 1]) + bias;
          const float recv = __shfl_xor_sync(0xffffffffu, (lane & 1) ? v0 : v1, 1);
          const float o = (lane & 1) ? silu_mul_bf16(recv, v1) : silu_mul_bf16(v0, recv);
          stage_h[(c + j + (lane & 1)) * 64 + (ml >> 1)] = __float2bfloat16_rn(o);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; j++) stage_h[(c + j) * 128 + ml] = __float2bfloat16_rn(__uint_as_float(r[j]) + bias);
      }
    }
    if (S == 1) {
      // coalesced copy-out of the staged tile: 16-byte pieces, OUTW features per token row
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int te = threadIdx.x - 64;
      constexpr int PPR = OUTW / 8;  // 16-byte pieces per row
      const int out_m0 = EPI == kEpiSiluMul ? (m0 >> 1) : m0;
      const int out_M = EPI == kEpiSiluMul ? (p.M >> 1) : p.M;
      for (int idx = te; idx < rows * PPR; idx += 128) {
        const int t = idx / PPR, pc = idx % PPR;
        const int m = out_m0 + pc * 8;
        if (m + 8 <= out_M) {
          *reinterpret_cast<uint4*>(p.y + size_t(n0 + t) * p.ldy + m) =
              *reinterpret_cast<const uint4*>(stage_h + t * OUTW + pc * 8);
        } else {
          for (int e = 0; e < 8 && m + e < out_M; e++) p.y[size_t(n0 + t) * p.ldy + m + e] = stage_h[t * OUTW + pc * 8 + e];
        }
      }
    }
  }

  if (S > 1) {
    // ---- deterministic split-K: CTA j of the cluster reduces feature slice j over all K ranges ----
    __syncwarp();
    cluster_sync_all();
    if (warp >= 2) {
      const int te = threadIdx.x - 64;
      const int fs = 128 / S;            // features per CTA
      const int q4 = fs / 4;             // float4 pieces per row
      const uint32_t stage_addr = smem_u32(sm);
      for (int idx = te; idx < rows * q4; idx += 128) {
        const int t = idx / q4, f = split * fs + (idx % q4) * 4;
        float4 acc = dsmem_sum_f32x4(stage_addr + uint32_t((t * 128 + f) * 4), S);
        const int m = m0 + f;
        if (p.bias) {
          if (m + 0 < p.M) acc.x += __bfloat162float(p.bias[m + 0]);
          if (m + 1 < p.M) acc.y += __bfloat162float(p.bias[m + 1]);
          if (m + 2 < p.M) acc.z += __bfloat162float(p.bias[m + 2]);
          if (m + 3 < p.M) acc.w += __bfloat162float(p.bias[m + 3]);
        }
        if (EPI == kEpiSiluMul) {
          __nv_bfloat162 o = __floats2bfloat162_rn(silu_mul_bf16(acc.x, acc.y), silu_mul_bf16(acc.z, acc.w));
          if (m + 4 <= p.M) *reinterpret_cast<__nv_bfloat162*>(p.y + size_t(n0 + t) * p.ldy + (m >> 1)) = o;
        } else {
          __nv_bfloat16* dst = p.y + size_t(n0 + t) * p.ldy + m;
          if (m + 4 <= p.M) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst) = pk;
          } else {
            float a4[4] = {acc.x, acc.y, acc.z, acc.w};
            for (int e = 0; e < 4 && m + e < p.M; e++) dst[e] = __float2bfloat16_rn(a4[e]);
          }
        }
      }
    }
    __syncwarp();
    cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
  }
  __syncwarp();
  gemm::teardown(p, s);
}

// ---- host side -------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

struct MapKey {
  const void* ptr;
  unsigned long long rows, cols, ld;
  unsigned box_rows;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ k.rows; h = h * 1000003u ^ k.cols; h = h * 1000003u ^ k.ld; h = h * 1000003u ^ k.box_rows;
    return h;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
std::mutex g_maps_mu;
int g_persist_mode = -1;   // TBV_GEMM_PERSIST, read on first use; tbv_op_gemm_persist_mode overrides it
int* g_err_flag[16] = {nullptr};
int g_sm_count[16] = {0};
bool g_attr_done = false;

}  // namespace

namespace tbvops {

// [rows, cols] bf16 row-major with row stride ld (elements); box = box_rows x 64, 128-byte swizzle.
// The encoded map is a pure function of the arguments (it names addresses, it holds no
// reference), so the memo below can never go stale; `cache = false` skips it for maps that a
// caller keeps itself.
int make_tensor_map_bf16(CUtensorMap* out, const void* ptr, unsigned long long rows, unsigned long long cols,
                         unsigned long long ld, unsigned box_rows, bool cache) {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  });
  if (!g_encode) return -1;
  MapKey key{ptr, rows, cols, ld, box_rows};
  if (cache) {
    std::lock_guard<std::mutex> g(g_maps_mu);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return 0; }
  }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) || (ld * 2) % 16 || box_rows > 256 || box_rows == 0) return -2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -3;
  if (cache) {
    std::lock_guard<std::mutex> g(g_maps_mu);
    if (g_maps.size() > 65536) g_maps.clear();
    g_maps[key] = m;
  }
  *out = m;
  return 0;
}

// ---- weights of the GEMM that follows, to be asked into L2 by the kernel launched next ------------------------------
namespace {
thread_local const char* t_pf_ptr = nullptr;
thread_local unsigned long long t_pf_bytes = 0;
}
unsigned long long take_next_prefetch(const char** ptr, unsigned long long own_bytes) {
  // Measured on the Llama-3-8B decode step (batch 8), one edge of the layer at a time: only "o_proj announces gate_up" pays
  // (-3.0 % of the step at TP=1 shapes, -2.0 % at TP=2 shapes: a 117-235 MB weight stream that starts after a small kernel
  // in between); at TP=4 shapes the same edge costs 6.7 % (gate_up is 58 MB, o_proj 8 MB: the bulk requests delay the small
  // loads of the kernels in between more than they save), and with every GEMM announcing 32 MB the TP=8 shapes lose 20 %.
  // So a launch takes an announcement only when its own weight matrix is large enough to give the requests cover
  // (TBV_L2_PREFETCH_MIN_OWN_MB) and the announced matrix is a long stream (TBV_L2_PREFETCH_MIN_NEXT_MB), and it never asks for
  // more than TBV_L2_PREFETCH_MB.
  static const long cap_mb = [] { const char* e = getenv("TBV_L2_PREFETCH_MB"); long v = e ? atol(e) : 32; return v < 0 ? 0 : v; }();
  static const long min_own_mb = [] { const char* e = getenv("TBV_L2_PREFETCH_MIN_OWN_MB"); long v = e ? atol(e) : 12; return v < 0 ? 0 : v; }();
  static const long min_next_mb = [] { const char* e = getenv("TBV_L2_PREFETCH_MIN_NEXT_MB"); long v = e ? atol(e) : 96; return v < 0 ? 0 : v; }();
  unsigned long long n = t_pf_bytes;
  *ptr = t_pf_ptr;
  t_pf_ptr = nullptr;
  t_pf_bytes = 0;
  if (!*ptr || (reinterpret_cast<uintptr_t>(*ptr) & 15u) || own_bytes < ((unsigned long long)min_own_mb << 20) ||
      n < ((unsigned long long)min_next_mb << 20))
    return 0;
  const unsigned long long cap = (unsigned long long)cap_mb << 20;
  if (n > cap) n = cap;
  return n & ~15ull;
}
void set_next_prefetch(const void* ptr, unsigned long long bytes) {
  t_pf_ptr = static_cast<const char*>(ptr);
  t_pf_bytes = bytes;
}

int* gemm_err_flag() {
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 15;
  if (!g_err_flag[dev]) {
    cudaMalloc(&g_err_flag[dev], sizeof(int));
    cudaMemset(g_err_flag[dev], 0, sizeof(int));
    cudaDeviceProp prop;
    cudaGetDeviceProperties(&prop, dev);
    g_sm_count[dev] = prop.multiProcessorCount;
  }
  return g_err_flag[dev];
}
int sm_count() {
  int dev = 0;
  cudaGetDevice(&dev);
  gemm_err_flag();
  return g_sm_count[dev & 15];
}

void gemm_config(int M, int N, int K, int splits_hint, int* bn_out, int* splits_out, int* stages_out) {
  int bn = N <= 16 ? 16 : (N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : 256)));
  const int kb = (K + 63) / 64;
  const int tiles = ((M + 127) / 128) * ((N + bn - 1) / bn);
  const int sms = sm_count();
  int splits = 1;
  if (splits_hint > 0) {
    splits = splits_hint;
  } else {
    // a K range per CTA of at least `min_kb` 64-wide blocks (TBV_GEMM_MIN_KB, read once)
    static const int min_kb = [] { const char* e = getenv("TBV_GEMM_MIN_KB"); int v = e ? atoi(e) : 8; return v < 1 ? 1 : v; }();
    while (splits < 8 && tiles * splits * 2 <= 2 * sms && kb / (splits * 2) >= min_kb) splits *= 2;
  }
  while (splits > 1 && (kb + splits - 1) / splits * (splits - 1) >= kb) splits /= 2;  // every split gets work
  const int stage_bytes = gemm::kATileBytes + bn * 128;
  const int budget = (tiles * splits > sms) ? 108 * 1024 : 200 * 1024;  // two CTAs per SM when the grid is larger than the GPU
  int stages = budget / stage_bytes;
  stages = stages < 2 ? 2 : (stages > gemm::kMaxStages ? gemm::kMaxStages : stages);
  const int need = splits > 1 ? bn * 512 : bn * 256;  // epilogue staging reuses the ring
  while (stages * stage_bytes < need) stages++;
  *bn_out = bn; *splits_out = splits; *stages_out = stages;
}

}  // namespace tbvops

extern "C" {

// y[N, M(/2)] = epilogue(x[N, K] @ w[M, K]^T).  ldx / ldy: row strides in elements.
// epi (low byte): 0 = store (+bias), 1 = SiLU-mul over row-interleaved gate/up weights (M = 2 * out features).
// CONTRACT: w is treated as a constant — its tiles are fetched before this kernel has waited for its
// predecessor in the stream (that is what hides the weight stream behind the previous kernel).  If w was
// written by a kernel launched just before (a dequantised or copied weight, an activation used as w), add
// TBV_GEMM_W_NOT_CONSTANT (0x100) to epi: the fetch then follows the dependency wait.
int tbv_op_gemm(const void* w, const void* x, void* y, const void* bias, int M, int N, int K, int ldx, int ldy, int epi,
                int splits_hint, void* stream) {
  const int w_not_constant = (epi & 0x100) ? 1 : 0;
  epi &= 0xff;
  const char* pf_ptr = nullptr;   // an announcement holds for exactly one launch, whichever kernel that launch picks
  const unsigned long long pf_bytes = tbvops::take_next_prefetch(&pf_ptr, (unsigned long long)(M > 0 ? M : 0) * (unsigned long long)(K > 0 ? K : 0) * 2ull);
  if (M <= 0 || N <= 0 || K <= 0 || (K % 8) || (ldx % 8) || (ldy % 8) || (reinterpret_cast<uintptr_t>(y) & 15u)) return -2;
  if (epi == kEpiSiluMul && (M % 2)) return -2;
  // Hundreds of tokens: the persistent kernel with tokens on the UMMA M axis.  TBV_GEMM_PERSIST: 0 = never,
  // 1 (default) = where it is estimated to be faster, 2 / 3 = its 128- / 256-token tile wherever the shape allows.
  if (g_persist_mode == -1) { const char* pe = getenv("TBV_GEMM_PERSIST"); g_persist_mode = pe ? atoi(pe) : 1; }  // read once, not per launch
  const int persist = g_persist_mode;
  if (persist > 0 && splits_hint <= 0) {
    const int th = w_not_constant ? 0 : tbvops::gemm_tok_choose(M, N, K, ldy, epi, persist);   // the many-token kernel always prefetches w
    if (th > 0) return tbvops::gemm_tok_launch(w, x, y, bias, M, N, K, ldx, ldy, epi, th, stream);
  }
  // Large weight matrices at decode batch sizes: the persistent kernel that splits the work evenly over the SMs.
  if (tbvops::gemm_streamk_wants(M, N, K, epi, splits_hint, w_not_constant != 0))
    return tbvops::gemm_streamk_launch(w, x, y, bias, M, N, K, ldx, ldy, epi, stream);
  int bn, splits, stages;
  tbvops::gemm_config(M, N, K, splits_hint, &bn, &splits, &stages);
  CUtensorMap tmA, tmB;
  if (tbvops::make_tensor_map_bf16(&tmA, w, M, K, K, 128) != 0) return -3;
  if (tbvops::make_tensor_map_bf16(&tmB, x, N, K, ldx, bn) != 0) return -3;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.ldy = ldy; p.bn = bn; p.splits = splits; p.stages = stages;
  p.kb_total = (K + 63) / 64;
  p.a_after_wait = w_not_constant;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.y = static_cast<__nv_bfloat16*>(y);
  p.limit_ns = 2000000000ull;
  p.err = tbvops::gemm_err_flag();
  p.pf_ptr = pf_ptr;
  p.pf_bytes = pf_bytes;
  const size_t smem = size_t(stages) * (gemm::kATileBytes + bn * 128) + 1024;
  if (!g_attr_done) {
    // 227 KB per CTA in total; the kernel's static shared state comes out of the same budget
    cudaError_t a1 = cudaFuncSetAttribute(k_gemm<kEpiStore>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
    cudaError_t a2 = cudaFuncSetAttribute(k_gemm<kEpiSiluMul>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
    if (a1 != cudaSuccess || a2 != cudaSuccess) {
      fprintf(stderr, "[tbvops] cudaFuncSetAttribute(max dynamic smem) failed: %s\n", cudaGetErrorString(a1 != cudaSuccess ? a1 : a2));
      return -1;
    }
    g_attr_done = true;
  }
  const int mt = (M + 127) / 128, nt = (N + bn - 1) / bn;
  p.raster = nt > 1 ? 1 : 0;
  const dim3 grid(p.raster ? nt : mt, p.raster ? mt : nt, splits);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = epi == kEpiSiluMul ? pdl::launch(k_gemm<kEpiSiluMul>, grid, dim3(gemm::kThreads), smem, st, splits, tmA, tmB, p)
                                     : pdl::launch(k_gemm<kEpiStore>, grid, dim3(gemm::kThreads), smem, st, splits, tmA, tmB, p);
  if (e != cudaSuccess) {
    fprintf(stderr, "[tbvops] gemm launch failed: %s (M=%d N=%d K=%d bn=%d splits=%d stages=%d)\n", cudaGetErrorString(e), M, N, K,
            bn, splits, stages);
    return -1;
  }
  return 0;
}

// Announce the weights of the GEMM that will run after the next one launched from this host thread: that launch's CTAs ask
// for them to be brought into L2 once their own weight tiles are requested (decode-size kernels only; others ignore it).
void tbv_op_gemm_prefetch_next(const void* ptr, size_t bytes) { tbvops::set_next_prefetch(ptr, bytes); }

// Many-token kernel selection: 0 never, 1 where estimated faster, 2 / 3 force its 128- / 256-token tile;
// -1 = take TBV_GEMM_PERSIST from the environment again at the next call.
void tbv_op_gemm_persist_mode(int mode) { g_persist_mode = mode < -1 ? -1 : mode; }

// 1 if any GEMM wait ever gave up on the current device (synchronises the device).
int tbv_op_gemm_error(void) {
  int v = 0;
  cudaMemcpy(&v, tbvops::gemm_err_flag(), sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}

void tbv_op_gemm_config(int M, int N, int K, int splits_hint, int* bn, int* splits, int* stages) {
  tbvops::gemm_config(M, N, K, splits_hint, bn, splits, stages);
}

}  // extern "C"
