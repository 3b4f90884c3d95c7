// Epilogue semantics shared by both GEMM kernels (tcgen05 product path and the mma.sync cross-check).
#pragma once
#include "common.cuh"

namespace hb200 {

enum GemmEpilogue : int { EPI_STORE = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_SCATTER_ADD = 3 };

struct GemmParams {
  const __nv_bfloat16* A;
  const __nv_bfloat16* W;
  __nv_bfloat16* C;
  int M, N, K;
  int64_t lda, ldw, ldc;
  int epilogue;
  const __nv_bfloat16* resid;
  float alpha;
  const int32_t* rows;    // SCATTER_ADD target rows
  const int32_t* m_dev;   // optional live row count on the device
  int32_t* err_flag;
  // tcgen05 kernel only: rows of A gathered through `a_rows` (A row of tile row m = a_rows[m]; A then needs no compact
  // copy), and the SwiGLU epilogue applied to  row_scale[a_rows[m]] * (acc + col_bias[col])  instead of acc - the
  // pre-MLP norm folded into the contraction: norm(x + rec) W^T = inv_rms * (x W'^T + rec W'^T) with W' = W diag(gain).
  const int32_t* a_rows = nullptr;
  const float* row_scale = nullptr;
  const float* col_bias = nullptr;
  int32_t* m_hint = nullptr;   // skinny kernel only: the live row count this launch site saw the last time (written by
                               // the kernel, read before the wait on the predecessor): 0 -> no speculative weight prefetch
};

// Consume `n` consecutive fp32 accumulator columns [col, col+n) of logical output row `m`
// (n is a multiple of 16; `col` a multiple of 16). Handles the N tail column by column.
template <int NV>
__device__ __forceinline__ void epilogue_row_chunk(const GemmParams& p, int m, int col, const float (&acc)[NV]) {
  if (p.epilogue == EPI_SWIGLU) {
    // groups of 16 columns = 8 gate + 8 up of the same hidden units -> 8 outputs at column col/2
    __nv_bfloat16* dst = p.C + (size_t)m * p.ldc + (col >> 1);
#pragma unroll
    for (int g16 = 0; g16 < NV / 16; ++g16) {
      if (col + g16 * 16 + 16 <= p.N) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = silu_mul(acc[g16 * 16 + j], acc[g16 * 16 + 8 + j]);
        store_bf16x8(dst + g16 * 8, o);
      }
    }
    return;
  }
  const size_t row = (p.epilogue == EPI_SCATTER_ADD) ? (size_t)__ldcg(p.rows + m) : (size_t)m;
  __nv_bfloat16* dst = p.C + row * p.ldc + col;
  const __nv_bfloat16* src = (p.epilogue == EPI_RESID) ? p.resid + row * p.ldc + col
                                                       : (p.epilogue == EPI_SCATTER_ADD ? dst : nullptr);
#pragma unroll
  for (int v8 = 0; v8 < NV / 8; ++v8) {
    const int c = col + v8 * 8;
    if (c + 8 <= p.N) {
      float o[8];
      if (src != nullptr) {
        float r[8];
        load_bf16x8_cg(src + v8 * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r[j] + p.alpha * acc[v8 * 8 + j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = p.alpha * acc[v8 * 8 + j];
      }
      store_bf16x8(dst + v8 * 8, o);
    } else {
      for (int j = 0; j < 8 && c + j < p.N; ++j) {
        float val = p.alpha * acc[v8 * 8 + j];
        if (src != nullptr) val += ldcg_bf16(src + v8 * 8 + j);
        dst[v8 * 8 + j] = __float2bfloat16_rn(val);
      }
    }
  }
}

int launch_gemm_tcgen05(const GemmParams& p, cudaStream_t st);
int launch_gemm_mma(const GemmParams& p, cudaStream_t st);
// M <= 128 rows: one CTA per (128 weight rows, K slice), split-K reduced across a thread-block cluster
// chained: launched as a link of a programmatic-dependent-launch chain (see common.cuh)
int launch_gemm_skinny(const GemmParams& p, cudaStream_t st, bool chained = false);

}  // namespace hb200
