// misc.cu — the small memory-bound decode operators: RoPE + KV-cache write, SiLU-mul,
// embedding gather (vocab-parallel), greedy argmax.
//
// The reference's engine layer is described only (TP weight sharding, RoPE, GQA, KV cache,
// greedy: reports/11_custom_engine.md:10-20); these are the sm_100a kernels for it.  All
// arithmetic follows HF Llama's bf16 semantics op by op (each elementwise op rounds to
// bf16), so logits can be compared with a plain PyTorch reference.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "../pdl.cuh"

namespace {

__device__ __forceinline__ float bfr(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// qkv: [T, (nq + 2*nkv) * D] (q heads, then k heads, then v heads).  Rotates q and k in
// place (HF "rotate_half" pairing: i <-> i + D/2, cos/sin rounded to bf16, products and
// the sum each rounded to bf16) and scatters k, v into the paged cache:
// k_cache/v_cache: [num_blocks * block_size, nkv, D], row = slot_mapping[t] (< 0: skip).
__global__ void k_rope_kv(__nv_bfloat16* qkv, const int* __restrict__ positions, const float* __restrict__ cos_sin,
                          const long long* __restrict__ slot_mapping, __nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
                          int nq, int nkv, int D, int max_pos) {
  pdl::launch_dependents();
  pdl::grid_dependency_wait();
  // one CTA per (token, head): q heads and k heads rotate, v heads are copied to the cache
  const int t = blockIdx.x, h = blockIdx.y;
  const int half = D / 2;
  __nv_bfloat16* row = qkv + size_t(t) * (nq + 2 * nkv) * D;
  const long long slot = slot_mapping ? slot_mapping[t] : -1;
  if (h >= nq + nkv) {
    if (slot >= 0) {
      const uint4* vs = reinterpret_cast<const uint4*>(row + h * D);
      uint4* vd = reinterpret_cast<uint4*>(v_cache + (size_t(slot) * nkv + (h - nq - nkv)) * D);
      for (int i = threadIdx.x; i < D / 8; i += blockDim.x) vd[i] = vs[i];
    }
    return;
  }
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
  const float* cs = cos_sin + size_t(pos) * D;  // [cos(0..half-1), sin(0..half-1)]
  __nv_bfloat16* v = row + h * D;
  for (int d = threadIdx.x; d < half; d += blockDim.x) {
    const float c = bfr(cs[d]), s = bfr(cs[half + d]);
    const float x1 = __bfloat162float(v[d]), x2 = __bfloat162float(v[d + half]);
    const float o1 = bfr(bfr(x1 * c) + bfr(-x2 * s));
    const float o2 = bfr(bfr(x2 * c) + bfr(x1 * s));
    const __nv_bfloat16 b1 = __float2bfloat16_rn(o1), b2 = __float2bfloat16_rn(o2);
    v[d] = b1;
    v[d + half] = b2;
    if (h >= nq && slot >= 0) {
      __nv_bfloat16* kc = k_cache + (size_t(slot) * nkv + (h - nq)) * D;
      kc[d] = b1;
      kc[d + half] = b2;
    }
  }
}

// out[t, i] = bf16( bf16(silu(gate)) * up ),  x: [T, 2*I] = [gate | up]
__global__ void k_silu_mul(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int I) {
  pdl::launch_dependents();
  pdl::grid_dependency_wait();
  const size_t t = blockIdx.y;
  const int i8 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i8 >= I) return;
  const uint4 g4 = *reinterpret_cast<const uint4*>(x + t * 2 * I + i8);
  const uint4 u4 = *reinterpret_cast<const uint4*>(x + t * 2 * I + I + i8);
  const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(&g4);
  const __nv_bfloat16* u = reinterpret_cast<const __nv_bfloat16*>(&u4);
  uint4 o4;
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&o4);
#pragma unroll
  for (int k = 0; k < 8; k++) {
    const float gf = __bfloat162float(g[k]);
    o[k] = __float2bfloat16_rn(bfr(gf / (1.0f + __expf(-gf))) * __bfloat162float(u[k]));
  }
  *reinterpret_cast<uint4*>(out + t * I + i8) = o4;
}

// same, for row-interleaved gate/up columns: x[t, 2i] = gate_i, x[t, 2i+1] = up_i
__global__ void k_silu_mul_interleaved(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int I) {
  pdl::launch_dependents();
  pdl::grid_dependency_wait();
  const size_t t = blockIdx.y;
  const int i8 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i8 >= I) return;
  const uint4 a4 = *reinterpret_cast<const uint4*>(x + t * 2 * I + 2 * i8);
  const uint4 b4 = *reinterpret_cast<const uint4*>(x + t * 2 * I + 2 * i8 + 8);
  const __nv_bfloat16* a = reinterpret_cast<const __nv_bfloat16*>(&a4);
  const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&b4);
  uint4 o4;
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&o4);
#pragma unroll
  for (int k = 0; k < 8; k++) {
    const __nv_bfloat16* src = k < 4 ? a : b;
    const float gf = __bfloat162float(src[(2 * k) & 7]), uf = __bfloat162float(src[(2 * k + 1) & 7]);
    o[k] = __float2bfloat16_rn(bfr(gf / (1.0f + __expf(-gf))) * uf);
  }
  *reinterpret_cast<uint4*>(out + t * I + i8) = o4;
}

// out[t] = table[ids[t] - vocab_start] if in [vocab_start, vocab_end) else 0  (vocab-parallel shard)
__global__ void k_embedding(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                            __nv_bfloat16* __restrict__ out, int hidden, long long vocab_start, long long vocab_end) {
  pdl::launch_dependents();
  pdl::grid_dependency_wait();
  const size_t t = blockIdx.x;
  const long long id = ids[t];
  const bool mine = id >= vocab_start && id < vocab_end;
  const uint4* src = reinterpret_cast<const uint4*>(table + size_t(mine ? id - vocab_start : 0) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + t * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = mine ? src[i] : make_uint4(0, 0, 0, 0);
}

// Greedy sampling over a vocab shard: per row the maximum logit and the smallest index
// holding it.  Stage 1: `nblk` CTAs per row write partials; stage 2: the last CTA of a row
// (atomic ticket) folds them in block order — deterministic, first index wins ties like
// torch.argmax.
__global__ void k_argmax(const __nv_bfloat16* __restrict__ logits, int vocab, int ld, long long index_offset,
                         float* part_val, long long* part_idx, unsigned* tickets, float* out_val, long long* out_idx) {
  pdl::launch_dependents();
  pdl::grid_dependency_wait();
  const int row = blockIdx.y, nblk = gridDim.x;
  const int per = (vocab + nblk - 1) / nblk;
  const int v0 = blockIdx.x * per, v1 = min(vocab, v0 + per);
  const __nv_bfloat16* x = logits + size_t(row) * ld;
  float best = -FLT_MAX;
  int bi = 0x7fffffff;
  for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
    const float f = __bfloat162float(x[i]);
    if (f > best) { best = f; bi = i; }  // ascending i per thread: first index kept on ties
  }
  __shared__ float sv[32];
  __shared__ int si[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  __shared__ bool last;
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x + 31) / 32; w++)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    part_val[row * nblk + blockIdx.x] = best;
    part_idx[row * nblk + blockIdx.x] = bi;
    __threadfence();
    last = atomicAdd(&tickets[row], 1u) == unsigned(nblk - 1);
  }
  __syncthreads();
  if (last && threadIdx.x == 0) {
    __threadfence();
    float b = -FLT_MAX;
    long long i = 0x7fffffff;
    for (int k = 0; k < nblk; k++) {
      const float v = *(volatile float*)&part_val[row * nblk + k];
      const long long vi = *(volatile long long*)&part_idx[row * nblk + k];
      if (v > b || (v == b && vi < i)) { b = v; i = vi; }
    }
    out_val[row] = b;
    out_idx[row] = i + index_offset;
    tickets[row] = 0;  // ready for the next launch
  }
}

// Fold per-rank (value, index) candidates gathered from all ranks: out[t] = index of the
// largest value, lowest index on ties.  vals/idx: [world, T].
__global__ void k_argmax_merge(const float* __restrict__ vals, const long long* __restrict__ idx, int world, int T,
                               long long rank_stride_bytes, long long* __restrict__ out) {
  pdl::launch_dependents();
  pdl::grid_dependency_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float b = vals[t];
  long long bi = idx[t];
  for (int r = 1; r < world; r++) {
    const float v = *reinterpret_cast<const float*>(reinterpret_cast<const char*>(vals) + r * rank_stride_bytes + size_t(t) * 4);
    const long long vi = *reinterpret_cast<const long long*>(reinterpret_cast<const char*>(idx) + r * rank_stride_bytes + size_t(t) * 8);
    if (v > b || (v == b && vi < bi)) { b = v; bi = vi; }
  }
  out[t] = bi;
}

// Device-side bookkeeping between two decode steps, so that a captured step can be
// replayed back to back without the host: feed the sampled token back, advance position
// and context length, look up the cache slot of the new position, log the token.
__global__ void k_decode_advance(const long long* __restrict__ next_ids, long long* ids, int* positions, int* ctx_lens,
                                 long long* slot_mapping, const int* __restrict__ block_tables, int max_blocks, int block_size,
                                 int batch, long long* history, int* step_counter, int max_steps) {
  pdl::launch_dependents();
  pdl::grid_dependency_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  const int step = *step_counter;
  if (b < batch) {
    const long long tok = next_ids[b];
    ids[b] = tok;
    if (history && step < max_steps) history[size_t(step) * batch + b] = tok;
    const int pos = positions[b] + 1;
    positions[b] = pos;
    ctx_lens[b] = min(pos + 1, max_blocks * block_size);   // past the reserved length the step still runs, over the last full context
    const int blk = pos / block_size;
    slot_mapping[b] = blk < max_blocks ? (long long)block_tables[size_t(b) * max_blocks + blk] * block_size + pos % block_size : -1;
  }
  __syncthreads();
  if (b == 0) *step_counter = step + 1;
}

}  // namespace

extern "C" {

int tbv_op_decode_advance(const void* next_ids, void* ids, void* positions, void* ctx_lens, void* slot_mapping,
                          const void* block_tables, int max_blocks, int block_size, int batch, void* history, void* step_counter,
                          int max_steps, void* stream) {
  if (batch <= 0 || batch > 1024) return -2;  // one CTA: the step counter is read before it is bumped
  cudaError_t e = pdl::launch(k_decode_advance, dim3(1), dim3((batch + 31) / 32 * 32), 0, static_cast<cudaStream_t>(stream), 1,
                              static_cast<const long long*>(next_ids), static_cast<long long*>(ids), static_cast<int*>(positions),
                              static_cast<int*>(ctx_lens), static_cast<long long*>(slot_mapping),
                              static_cast<const int*>(block_tables), max_blocks, block_size, batch,
                              static_cast<long long*>(history), static_cast<int*>(step_counter), max_steps);
  return e == cudaSuccess ? 0 : -1;
}

// One plain asynchronous copy on `stream` (pinned host <-> device, or device <-> device): what a serving loop uses to
// bring a step's packed inputs in and the sampled tokens out.  It can be captured into a CUDA graph together with the
// step's kernels, so that a step costs the host one graph launch.
int tbv_op_copy_async(void* dst, const void* src, size_t bytes, void* stream) {
  if (!dst || !src) return -2;
  if (bytes == 0) return 0;
  return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : -1;
}

int tbv_op_rope_kv(void* qkv, const void* positions, const void* cos_sin, const void* slot_mapping, void* k_cache, void* v_cache,
                   int tokens, int nq, int nkv, int D, int max_pos, void* stream) {
  if (tokens <= 0) return 0;
  if (D % 16) return -2;
  cudaError_t e = pdl::launch(k_rope_kv, dim3(tokens, nq + 2 * nkv), dim3(D / 2), 0, static_cast<cudaStream_t>(stream), 1,
                              static_cast<__nv_bfloat16*>(qkv), static_cast<const int*>(positions), static_cast<const float*>(cos_sin),
                              static_cast<const long long*>(slot_mapping), static_cast<__nv_bfloat16*>(k_cache),
                              static_cast<__nv_bfloat16*>(v_cache), nq, nkv, D, max_pos);
  return e == cudaSuccess ? 0 : -1;
}

int tbv_op_silu_mul(const void* x, void* out, int tokens, int inter, void* stream) {
  if (tokens <= 0) return 0;
  if (inter % 8) return -2;
  dim3 grid((inter / 8 + 255) / 256, tokens);
  cudaError_t e = pdl::launch(k_silu_mul, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), 1,
                              static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), inter);
  return e == cudaSuccess ? 0 : -1;
}

int tbv_op_silu_mul_interleaved(const void* x, void* out, int tokens, int inter, void* stream) {
  if (tokens <= 0) return 0;
  if (inter % 8) return -2;
  dim3 grid((inter / 8 + 255) / 256, tokens);
  cudaError_t e = pdl::launch(k_silu_mul_interleaved, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), 1,
                              static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), inter);
  return e == cudaSuccess ? 0 : -1;
}

int tbv_op_embedding(const void* ids, const void* table, void* out, int tokens, int hidden, long long vocab_start,
                     long long vocab_end, void* stream) {
  if (tokens <= 0) return 0;
  if (hidden % 8) return -2;
  cudaError_t e = pdl::launch(k_embedding, dim3(tokens), dim3(256), 0, static_cast<cudaStream_t>(stream), 1,
                              static_cast<const long long*>(ids), static_cast<const __nv_bfloat16*>(table),
                              static_cast<__nv_bfloat16*>(out), hidden, vocab_start, vocab_end);
  return e == cudaSuccess ? 0 : -1;
}

// workspace layout (caller-provided scratch, >= tbv_op_argmax_workspace(tokens) bytes, zeroed once):
//   [tickets: tokens u32 (padded to 256 B)] [part_val: tokens*64 f32] [part_idx: tokens*64 i64]
size_t tbv_op_argmax_workspace(int tokens) {
  return ((size_t(tokens) * 4 + 255) & ~size_t(255)) + size_t(tokens) * 64 * 4 + size_t(tokens) * 64 * 8;
}
int tbv_op_argmax(const void* logits, int tokens, int vocab, int ld, long long index_offset, void* workspace, void* out_val,
                  void* out_idx, void* stream) {
  if (tokens <= 0) return 0;
  int nblk = (vocab + 4095) / 4096;
  nblk = nblk < 1 ? 1 : (nblk > 64 ? 64 : nblk);
  char* ws = static_cast<char*>(workspace);
  unsigned* tickets = reinterpret_cast<unsigned*>(ws);
  float* pv = reinterpret_cast<float*>(ws + ((size_t(tokens) * 4 + 255) & ~size_t(255)));
  long long* pi = reinterpret_cast<long long*>(reinterpret_cast<char*>(pv) + size_t(tokens) * 64 * 4);
  cudaError_t e = pdl::launch(k_argmax, dim3(nblk, tokens), dim3(256), 0, static_cast<cudaStream_t>(stream), 1,
                              static_cast<const __nv_bfloat16*>(logits), vocab, ld, index_offset, pv, pi, tickets,
                              static_cast<float*>(out_val), static_cast<long long*>(out_idx));
  return e == cudaSuccess ? 0 : -1;
}
// vals / idx point at rank 0's candidates; rank r's are rank_stride_bytes further on.
int tbv_op_argmax_merge(const void* vals, const void* idx, int world, int tokens, long long rank_stride_bytes, void* out,
                        void* stream) {
  if (tokens <= 0) return 0;
  cudaError_t e = pdl::launch(k_argmax_merge, dim3((tokens + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream), 1,
                              static_cast<const float*>(vals), static_cast<const long long*>(idx), world, tokens, rank_stride_bytes,
                              static_cast<long long*>(out));
  return e == cudaSuccess ? 0 : -1;
}

}  // extern "C"
