// Row kernels and helpers shared by the prefill executor (model.cu) and the decode executor (decode.cu):
// per-launch event recorder, register-resident row loads, router-score / gather-norm / exit-norm / embedding kernels.
#pragma once
#include <vector>

#include "common.cuh"

namespace hb200 {

int launch_mod_select(const float* scores, int B, int L, int k, int32_t* idx_out, const int32_t* depth, int min_active,
                      int32_t* rows_out, int32_t* count, const int32_t* forced_idx, cudaStream_t st);
int launch_compact_active(const int32_t* depth, int64_t n, int min_active, int32_t* rows_out, int32_t* count,
                          cudaStream_t st);

// ---- per-launch event recorder ---------------------------------------------------------------------------
struct Profile {
  std::vector<cudaEvent_t> ev;          // 2 per launch
  std::vector<hb200_launch_record> rec;
  int count = 0;
  int capacity = 0;
  int dropped = 0;                      // launches that found the recorder full (reported by hb200_profile_read)
};

struct ProfScope {
  Profile* p;
  cudaStream_t st;
  int slot;
  ProfScope(void* prof, cudaStream_t s, int kind, int block, int rec, int m, int n, int k)
      : p(static_cast<Profile*>(prof)), st(s), slot(-1) {
    if (p != nullptr && p->count < p->capacity) {
      slot = p->count++;
      p->rec[slot] = hb200_launch_record{kind, block, rec, m, n, k};
      cudaEventRecord(p->ev[2 * slot], st);
    } else if (p != nullptr) {
      ++p->dropped;
    }
  }
  ~ProfScope() {
    if (slot >= 0) cudaEventRecord(p->ev[2 * slot + 1], st);
  }
};

constexpr int ROW_NCH = 8;   // row kernels keep up to 8 x 256 elements of a row in registers (dim <= 2048)

// Launch a row kernel template with the smallest register-resident row that covers `dim`.
#define HB_DISPATCH_NCH(dim, ...)                 \
  do {                                            \
    if ((dim) <= 256) { constexpr int NCH = 1; __VA_ARGS__; }        \
    else if ((dim) <= 512) { constexpr int NCH = 2; __VA_ARGS__; }   \
    else if ((dim) <= 1024) { constexpr int NCH = 4; __VA_ARGS__; }  \
    else { constexpr int NCH = 8; __VA_ARGS__; }                     \
  } while (0)

// Loads row `src` (+ optional fp32 per-column offset), returns sum of squares; values stay in v.
template <int NCH>
__device__ __forceinline__ float load_row_add(const __nv_bfloat16* __restrict__ src, const float* __restrict__ add,
                                              int D, int lane, float (&v)[NCH][8]) {
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * 8;
    if (i < D) load_bf16x8(src + i, v[c]);   // all loads of the row are issued before any is consumed
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * 8;
    if (i < D) {
      if (add != nullptr) {
        const float4 a0 = *reinterpret_cast<const float4*>(add + i);
        const float4 a1 = *reinterpret_cast<const float4*>(add + i + 4);
        v[c][0] += a0.x; v[c][1] += a0.y; v[c][2] += a0.z; v[c][3] += a0.w;
        v[c][4] += a1.x; v[c][5] += a1.y; v[c][6] += a1.z; v[c][7] += a1.w;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[c][j] * v[c][j];
    }
  }
  return warp_sum(ss);
}

// v <- bf16-rounded (v * r * w)
template <int NCH>
__device__ __forceinline__ void scale_row(const float* __restrict__ w, float r, int D, int lane, float (&v)[NCH][8]) {
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * 8;
    if (i < D) {
      const float4 w0 = *reinterpret_cast<const float4*>(w + i);
      const float4 w1 = *reinterpret_cast<const float4*>(w + i + 4);
      const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) v[c][j] = __bfloat162float(__float2bfloat16_rn(v[c][j] * r * ww[j]));
    }
  }
}

// Router pass over ALL tokens, streaming (no activation is written): four rows per warp so that the per-column
// vectors are fetched once per four rows.
//   MoD score   s = rsqrt(mean((x+rec)^2) + eps) * sum_d (x_d + rec_d) * wn_d + b,  wn = norm2 gain * MoD weight
//               (the fp32 value of Linear(AdaRMSNorm(x + rec)) without rounding the normalised row to bf16)
//   MoR depth   from l = sum_d x_d * mor_w_d + b on the raw row (recursion 0 only)
//   norm scale  inv_rms = rsqrt(mean((x+rec)^2) + eps) of every row (HAS_SS): what the MLP's first contraction applies
//               in its epilogue when the pre-MLP norm is folded into it
constexpr int SCORE_ROWS = 4;
template <int NCH, bool HAS_MOD, bool HAS_ROUTER, bool HAS_SS = false>
__global__ void __launch_bounds__(256) mor_score_kernel(const __nv_bfloat16* __restrict__ cur,
                                                        const float* __restrict__ rec, const float* __restrict__ mod_wn,
                                                        const float* __restrict__ mod_b,
                                                        const float* __restrict__ mor_w, const float* __restrict__ mor_b,
                                                        float* __restrict__ scores, float* __restrict__ logits,
                                                        int32_t* __restrict__ depth, int64_t T, int D, float eps,
                                                        int n_rec, int min_d, float* __restrict__ inv_rms = nullptr) {
  const int lane = threadIdx.x & 31;
  const int64_t row0 = ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * SCORE_ROWS;
  if (row0 >= T) return;
  // issue every load of the four rows first (up to 16 x 16 bytes in flight per lane)
  uint4 raw[SCORE_ROWS][NCH];
#pragma unroll
  for (int r = 0; r < SCORE_ROWS; ++r)
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int i = (c * 32 + lane) * 8;
      raw[r][c] = (i < D && row0 + r < T) ? *reinterpret_cast<const uint4*>(cur + (row0 + r) * D + i)
                                         : make_uint4(0, 0, 0, 0);
    }
  float ss[SCORE_ROWS], dm[SCORE_ROWS], lm[SCORE_ROWS];
#pragma unroll
  for (int r = 0; r < SCORE_ROWS; ++r) ss[r] = dm[r] = lm[r] = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * 8;
    float wn[8], rc[8], wr[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) wn[j] = rc[j] = wr[j] = 0.f;
    if (i < D) {
      if (HAS_MOD) {
        const float4 a0 = *reinterpret_cast<const float4*>(mod_wn + i), a1 = *reinterpret_cast<const float4*>(mod_wn + i + 4);
        wn[0] = a0.x; wn[1] = a0.y; wn[2] = a0.z; wn[3] = a0.w; wn[4] = a1.x; wn[5] = a1.y; wn[6] = a1.z; wn[7] = a1.w;
      }
      if (HAS_MOD || HAS_SS) {
        const float4 b0 = *reinterpret_cast<const float4*>(rec + i), b1 = *reinterpret_cast<const float4*>(rec + i + 4);
        rc[0] = b0.x; rc[1] = b0.y; rc[2] = b0.z; rc[3] = b0.w; rc[4] = b1.x; rc[5] = b1.y; rc[6] = b1.z; rc[7] = b1.w;
      }
      if (HAS_ROUTER) {
        const float4 a0 = *reinterpret_cast<const float4*>(mor_w + i), a1 = *reinterpret_cast<const float4*>(mor_w + i + 4);
        wr[0] = a0.x; wr[1] = a0.y; wr[2] = a0.z; wr[3] = a0.w; wr[4] = a1.x; wr[5] = a1.y; wr[6] = a1.z; wr[7] = a1.w;
      }
    }
#pragma unroll
    for (int r = 0; r < SCORE_ROWS; ++r) {
      const uint32_t w4[4] = {raw[r][c].x, raw[r][c].y, raw[r][c].z, raw[r][c].w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float x = (j & 1) ? __uint_as_float(w4[j >> 1] & 0xffff0000u) : __uint_as_float(w4[j >> 1] << 16);
        if (HAS_MOD || HAS_SS) {
          const float xr = x + rc[j];
          ss[r] += xr * xr;
          if (HAS_MOD) dm[r] += xr * wn[j];
        }
        if (HAS_ROUTER) lm[r] += x * wr[j];
      }
    }
  }
#pragma unroll
  for (int r = 0; r < SCORE_ROWS; ++r) {
    float s2 = 0.f, d2 = 0.f, l2 = 0.f;
    if (HAS_MOD || HAS_SS) s2 = warp_sum(ss[r]);
    if (HAS_MOD) d2 = warp_sum(dm[r]);
    if (HAS_ROUTER) l2 = warp_sum(lm[r]);
    if (lane == 0 && row0 + r < T) {
      if (HAS_MOD) scores[row0 + r] = rsqrtf(s2 / (float)D + eps) * d2 + mod_b[0];
      if (HAS_SS) inv_rms[row0 + r] = rsqrtf(s2 / (float)D + eps);
      if (HAS_ROUTER) {
        const float l = l2 + mor_b[0];
        if (logits != nullptr) logits[row0 + r] = l;
        if (depth != nullptr) depth[row0 + r] = mor_depth_from_logit(l, n_rec, min_d);
      }
    }
  }
}

// ug[j] = AdaRMSNorm(cur[rows[j]] + rec) for j < *count.  One warp per compact row.
template <int NCH>
__global__ void __launch_bounds__(256) norm_gather_kernel(const __nv_bfloat16* __restrict__ cur,
                                                          const float* __restrict__ rec, const float* __restrict__ w2,
                                                          const int32_t* __restrict__ rows,
                                                          const int32_t* __restrict__ count,
                                                          __nv_bfloat16* __restrict__ ug, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t j = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (j >= *count) return;
  const int64_t src = rows[j];
  float v[NCH][8];
  const float ss = load_row_add<NCH>(cur + src * D, rec, D, lane, v);
  scale_row<NCH>(w2, rsqrtf(ss / (float)D + eps), D, lane, v);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * 8;
    if (i < D) store_bf16x8(ug + j * D + i, v[c]);
  }
}

// inv_rms[rows[j]] = rsqrt(mean((cur[rows[j]] + rec)^2) + eps) for j < *count: the norm scale of the rows routed to
// the MLP in a block without a score pass (one warp per listed row, nothing but 4 bytes written).
template <int NCH>
__global__ void __launch_bounds__(256) rows_inv_rms_kernel(const __nv_bfloat16* __restrict__ cur,
                                                           const float* __restrict__ rec,
                                                           const int32_t* __restrict__ rows,
                                                           const int32_t* __restrict__ count,
                                                           float* __restrict__ inv_rms, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t j = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (j >= *count) return;
  const int64_t src = rows[j];
  float v[NCH][8];
  const float ss = load_row_add<NCH>(cur + src * D, rec, D, lane, v);
  if (lane == 0) inv_rms[src] = rsqrtf(ss / (float)D + eps);
}

// y = RMSNorm(src; w1) rounded to bf16 (the block output), z = RMSNorm(y; w2) (the next block's pre-attention norm,
// or the model's final norm): one read of src instead of three passes.  Either output may be omitted.  w1 == nullptr
// (a block without an exit norm): y = src.  y may be src itself (a row is read completely before any of it is
// written), which is why neither pointer is declared restrict.
template <int NCH>
__global__ void __launch_bounds__(256) dual_norm_kernel(const __nv_bfloat16* src,
                                                        const float* __restrict__ w1, __nv_bfloat16* y,
                                                        const float* __restrict__ w2, __nv_bfloat16* __restrict__ z,
                                                        int64_t T, int D, float eps) {
  chain_release();
  chain_wait();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= T) return;
  float v[NCH][8];
  const float ss = load_row_add<NCH>(src + row * D, nullptr, D, lane, v);
  if (w1 != nullptr) scale_row<NCH>(w1, rsqrtf(ss / (float)D + eps), D, lane, v);
  float ss2 = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * 8;
    if (i < D) {
      if (y != nullptr) store_bf16x8(y + row * D + i, v[c]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss2 += v[c][j] * v[c][j];
    }
  }
  if (z == nullptr) return;
  ss2 = warp_sum(ss2);
  scale_row<NCH>(w2, rsqrtf(ss2 / (float)D + eps), D, lane, v);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * 8;
    if (i < D) store_bf16x8(z + row * D + i, v[c]);
  }
}

// x = bf16(table[clamp(id)] * scale), a = AdaRMSNorm(x; w): embedding and the first block's pre-attention norm.
template <int NCH>
__global__ void __launch_bounds__(256) embed_norm_kernel(const int64_t* __restrict__ ids,
                                                         const __nv_bfloat16* __restrict__ table,
                                                         __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                         __nv_bfloat16* __restrict__ a, int64_t T, int D, int V,
                                                         float scale, float eps) {
  chain_release();
  chain_wait();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= T) return;
  int64_t id = __ldcg(ids + row);   // written by the previous decode step's argmax (see load_bf16x8_cg)
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  float v[NCH][8];
  load_row_add<NCH>(table + id * D, nullptr, D, lane, v);
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * 8;
    if (i < D) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[c][j] = __bfloat162float(__float2bfloat16_rn(v[c][j] * scale));
        ss += v[c][j] * v[c][j];
      }
      store_bf16x8(x + row * D + i, v[c]);
    }
  }
  ss = warp_sum(ss);
  scale_row<NCH>(w, rsqrtf(ss / (float)D + eps), D, lane, v);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * 8;
    if (i < D) store_bf16x8(a + row * D + i, v[c]);
  }
}


}  // namespace hb200
