// ops.h — internal declarations shared by the operator translation units.
#pragma once
#include <cuda.h>

namespace tbvops {
int make_tensor_map_bf16(CUtensorMap* out, const void* ptr, unsigned long long rows, unsigned long long cols,
                         unsigned long long ld, unsigned box_rows, bool cache = true);
int* gemm_err_flag();
// The weights announced by tbv_op_gemm_prefetch_next for the next GEMM launch of this host thread: returns the byte count
// (0 = none or `own_bytes`, the launch's own weight matrix, too small to give cover; capped by TBV_L2_PREFETCH_MB) and forgets
// the announcement.
unsigned long long take_next_prefetch(const char** ptr, unsigned long long own_bytes);
void set_next_prefetch(const void* ptr, unsigned long long bytes);
int sm_count();
void gemm_config(int M, int N, int K, int splits_hint, int* bn_out, int* splits_out, int* stages_out);
// many-token (prefill) persistent kernel, gemm_persist.cu
int gemm_tok_choose(int M, int N, int K, int ldy, int epi, int mode);
int gemm_tok_launch(const void* w, const void* x, void* y, const void* bias, int M, int N, int K, int ldx, int ldy, int epi, int th,
                    void* stream);
// evenly-split (stream-K) decode GEMM, gemm_streamk.cu
bool gemm_streamk_wants(int M, int N, int K, int epi, int splits_hint, bool w_not_constant);
int gemm_streamk_launch(const void* w, const void* x, void* y, const void* bias, int M, int N, int K, int ldx, int ldy, int epi,
                        void* stream);
// threads per CTA for the row-normalisation kernels; the fused collective uses the same
// mapping so that both produce identical bits
inline int norm_threads(int hidden) {
  const int upr = hidden / 8;                 // 16-byte units per row
  const int k = (upr + 1023) / 1024;          // units per thread
  return ((upr + k - 1) / k + 31) / 32 * 32;
}
}  // namespace tbvops
