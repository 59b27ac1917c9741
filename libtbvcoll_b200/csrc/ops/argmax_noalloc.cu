// argmax_noalloc.cu — greedy arg-max whose scratch is a fixed array in the library image,
// for callers that cannot allocate device memory (see noalloc.h for who they are and why).
// A separate variant of the arg-max kernel in misc.cu; nothing here touches that path.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdio.h>

#include "noalloc.h"

namespace {

constexpr int kMaxTokens = TBV_ARGMAX_NOALLOC_MAX_TOKENS;
constexpr int kMaxBlk = 64;  // CTAs per row, as in tbv_op_argmax
constexpr size_t kTicketBytes = size_t(kMaxTokens) * sizeof(unsigned);
constexpr size_t kValBytes = size_t(kMaxTokens) * kMaxBlk * sizeof(float);
constexpr size_t kIdxBytes = size_t(kMaxTokens) * kMaxBlk * sizeof(long long);
constexpr size_t kIdxOff = kTicketBytes + kValBytes;  // 8-byte aligned: both terms are multiples of 1024

// The scratch itself: tickets | partial values | partial indices.  Every GPU that loads the
// library holds one copy until the process exits.  In HOST code this name is only a handle
// for the symbol, not a device address — the address is fetched with cudaGetSymbolAddress
// below and that pointer is what the kernel receives.
static __device__ __align__(256) unsigned char g_scratch[kTicketBytes + kValBytes + kIdxBytes];

__global__ void k_argmax_noalloc(const __nv_bfloat16* __restrict__ logits, int vocab, int ld, long long index_offset,
                                 unsigned char* scratch, float* out_val, long long* out_idx) {
  unsigned* tickets = reinterpret_cast<unsigned*>(scratch);
  float* part_val = reinterpret_cast<float*>(scratch + kTicketBytes);
  long long* part_idx = reinterpret_cast<long long*>(scratch + kIdxOff);
  const int row = blockIdx.y, nblk = gridDim.x;
  const int per = (vocab + nblk - 1) / nblk;
  const int v0 = blockIdx.x * per, v1 = min(vocab, v0 + per);
  const __nv_bfloat16* x = logits + size_t(row) * ld;
  float best = -FLT_MAX;
  int bi = 0x7fffffff;
  for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
    const float f = __bfloat162float(x[i]);
    if (f > best) { best = f; bi = i; }  // ascending i per thread: the first index is kept on ties
  }
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ bool last;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x + 31) / 32; w++)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    part_val[row * kMaxBlk + blockIdx.x] = best;
    part_idx[row * kMaxBlk + blockIdx.x] = bi;
    __threadfence();
    last = atomicAdd(&tickets[row], 1u) == unsigned(nblk - 1);
  }
  __syncthreads();
  if (last && threadIdx.x == 0) {
    __threadfence();
    float b = -FLT_MAX;
    long long i = 0x7fffffff;
    for (int k = 0; k < nblk; k++) {  // block order: deterministic
      const float v = *(volatile float*)&part_val[row * kMaxBlk + k];
      const long long vi = *(volatile long long*)&part_idx[row * kMaxBlk + k];
      if (v > b || (v == b && vi < i)) { b = v; i = vi; }
    }
    out_val[row] = b;
    out_idx[row] = i + index_offset;
  }
}

constexpr int kMaxDev = 64;
unsigned char* g_scratch_dev[kMaxDev] = {nullptr};  // device address of g_scratch, per device

}  // namespace

extern "C" int tbv_op_argmax_noalloc(const void* logits, int tokens, int vocab, int ld, long long index_offset, void* out_val,
                                     void* out_idx, void* stream) {
  if (tokens < 0 || vocab <= 0 || tokens > kMaxTokens) {
    fprintf(stderr, "[tbvops] tbv_op_argmax_noalloc: tokens=%d vocab=%d is outside what the built-in scratch holds "
                    "(at most %d rows per call); split the batch or use tbv_op_argmax with your own workspace\n",
            tokens, vocab, kMaxTokens);
    return -2;
  }
  if (tokens == 0) return 0;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return -1;
  if (!g_scratch_dev[dev]) {
    // Set-up, once per device, with that device current: the device address of the array.
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_scratch);
    if (e != cudaSuccess || !ptr) {
      fprintf(stderr, "[tbvops] tbv_op_argmax_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
      return -1;
    }
    g_scratch_dev[dev] = static_cast<unsigned char*>(ptr);
  }
  unsigned char* scratch = g_scratch_dev[dev];
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array still holds the previous call's contents; only the tickets must start at zero.
  if (cudaMemsetAsync(scratch, 0, size_t(tokens) * sizeof(unsigned), st) != cudaSuccess) return -1;
  int nblk = (vocab + 4095) / 4096;
  nblk = nblk < 1 ? 1 : (nblk > kMaxBlk ? kMaxBlk : nblk);
  k_argmax_noalloc<<<dim3(nblk, tokens), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), vocab, ld, index_offset, scratch,
                                                       static_cast<float*>(out_val), static_cast<long long*>(out_idx));
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
