// Coalesced elementwise / row kernels behind the exported fused-op signatures:
// RMSNorm, RoPE, QK L2-norm, SwiGLU activation, token embedding, MoR depth mapping.
// All are HBM-bound: 128-bit accesses where alignment allows, fp32 arithmetic,
// warp-shuffle row reductions.
#include "common.cuh"

namespace hb200 {

template <typename T> struct VecOf { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float* f) {
  constexpr int N = VecOf<T>::N;
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) f[i] = Cvt<T>::to_f(e[i]);
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float* f) {
  constexpr int N = VecOf<T>::N;
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < N; ++i) e[i] = Cvt<T>::from_f(f[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// V consecutive weights (fp32 or the activation dtype) through 16-byte loads
template <typename WT, int V>
__device__ __forceinline__ void load_weights(const WT* p, float* f) {
  if constexpr (sizeof(WT) == 4) {
#pragma unroll
    for (int j = 0; j < V; j += 4) {
      const float4 t = *reinterpret_cast<const float4*>(p + j);
      f[j] = t.x; f[j + 1] = t.y; f[j + 2] = t.z; f[j + 3] = t.w;
    }
  } else {
    static_assert(V == 8, "16-bit weights come with 16-bit activations");
    load_vec<WT>(p, f);
  }
}

// ---------------------------------------------------------------------------------
// RMSNorm: one warp per row; the row stays in registers between the two passes when it fits.
// ---------------------------------------------------------------------------------
template <typename T, typename WT, int NCH>
__global__ void __launch_bounds__(256) rms_norm_vec_kernel(const T* __restrict__ x, const WT* __restrict__ w,
                                                           T* __restrict__ y, int64_t rows, int dim, float eps) {
  constexpr int V = VecOf<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * dim;
  T* yr = y + row * dim;
  float v[NCH][V];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * V;
    if (i < dim) {
      load_vec<T>(xr + i, v[c]);
#pragma unroll
      for (int j = 0; j < V; ++j) ss += v[c][j] * v[c][j];
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)dim + eps);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * V;
    if (i < dim) {
      float o[V], wv[V];
      load_weights<WT, V>(w + i, wv);
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = v[c][j] * r * wv[j];
      store_vec<T>(yr + i, o);
    }
  }
}

template <typename T, typename WT>
__global__ void __launch_bounds__(256) rms_norm_generic_kernel(const T* __restrict__ x, const WT* __restrict__ w,
                                                               T* __restrict__ y, int64_t rows, int dim, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * dim;
  T* yr = y + row * dim;
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) {
    const float a = Cvt<T>::to_f(xr[i]);
    ss += a * a;
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)dim + eps);
  for (int i = lane; i < dim; i += 32) yr[i] = Cvt<T>::from_f(Cvt<T>::to_f(xr[i]) * r * Cvt<WT>::to_f(w[i]));
}

template <typename T, typename WT>
static int launch_rms_norm(const void* x, const void* w, void* y, int64_t rows, int dim, float eps, cudaStream_t st) {
  constexpr int V = VecOf<T>::N;
  const int warps = 8;
  const unsigned grid = (unsigned)ceil_div64(rows, warps);
  const bool vec_ok = (dim % V == 0) && aligned16(x) && aligned16(y) && aligned16(w);
  if (vec_ok && dim <= 32 * V * 4) {
    rms_norm_vec_kernel<T, WT, 4><<<grid, warps * 32, 0, st>>>((const T*)x, (const WT*)w, (T*)y, rows, dim, eps);
  } else if (vec_ok && dim <= 32 * V * 8) {
    rms_norm_vec_kernel<T, WT, 8><<<grid, warps * 32, 0, st>>>((const T*)x, (const WT*)w, (T*)y, rows, dim, eps);
  } else {
    rms_norm_generic_kernel<T, WT><<<grid, warps * 32, 0, st>>>((const T*)x, (const WT*)w, (T*)y, rows, dim, eps);
  }
  HB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------
// RoPE (interleaved pairs). Strided input view, contiguous output.
// ---------------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) rope_kernel(const T* __restrict__ x, const float* __restrict__ cs,
                                                   const float* __restrict__ sn, T* __restrict__ y, int H, int S,
                                                   int hd, int64_t sb, int64_t sh, int64_t ss, int table_ld,
                                                   int64_t total_units) {
  constexpr int V = VEC ? VecOf<T>::N : 2;   // elements handled by one thread
  const int upr = hd / V;                    // units per head row
  const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= total_units) return;
  const int iu = (int)(u % upr);
  const int64_t row = u / upr;               // (b*H + h)*S + s
  const int s = (int)(row % S);
  const int64_t bh = row / S;
  const int h = (int)(bh % H);
  const int64_t b = bh / H;
  const T* xp = x + b * sb + h * sh + s * ss + iu * V;
  T* yp = y + row * hd + iu * V;
  const float* c = cs + (int64_t)s * table_ld + iu * (V / 2);
  const float* sp = sn + (int64_t)s * table_ld + iu * (V / 2);
  float f[V], o[V];
  if (VEC) {
    load_vec<T>(xp, f);
  } else {
    f[0] = Cvt<T>::to_f(xp[0]);
    f[1] = Cvt<T>::to_f(xp[1]);
  }
  float ct[V / 2], stt[V / 2];
  if (VEC && (V / 2) % 4 == 0) {
#pragma unroll
    for (int p = 0; p < V / 2; p += 4) {
      const float4 a = *reinterpret_cast<const float4*>(c + p), b = *reinterpret_cast<const float4*>(sp + p);
      ct[p] = a.x; ct[p + 1] = a.y; ct[p + 2] = a.z; ct[p + 3] = a.w;
      stt[p] = b.x; stt[p + 1] = b.y; stt[p + 2] = b.z; stt[p + 3] = b.w;
    }
  } else {
#pragma unroll
    for (int p = 0; p < V / 2; ++p) { ct[p] = c[p]; stt[p] = sp[p]; }
  }
#pragma unroll
  for (int p = 0; p < V / 2; ++p) {
    const float cv = ct[p], sv = stt[p];
    o[2 * p] = f[2 * p] * cv - f[2 * p + 1] * sv;
    o[2 * p + 1] = f[2 * p] * sv + f[2 * p + 1] * cv;
  }
  if (VEC) {
    store_vec<T>(yp, o);
  } else {
    yp[0] = Cvt<T>::from_f(o[0]);
    yp[1] = Cvt<T>::from_f(o[1]);
  }
}

template <typename T>
static int launch_rope(const void* x, const float* cs, const float* sn, void* y, int B, int H, int S, int hd,
                       int64_t sb, int64_t sh, int64_t ss, int table_ld, cudaStream_t st) {
  constexpr int V = VecOf<T>::N;
  const bool vec = (hd % V == 0) && (sb % V == 0) && (sh % V == 0) && (ss % V == 0) && aligned16(x) && aligned16(y) &&
                   (V != 8 || (aligned16(cs) && aligned16(sn) && table_ld % 4 == 0));
  const int64_t rows = (int64_t)B * H * S;
  if (vec) {
    const int64_t units = rows * (hd / V);
    rope_kernel<T, true><<<(unsigned)ceil_div64(units, 256), 256, 0, st>>>((const T*)x, cs, sn, (T*)y, H, S, hd, sb,
                                                                            sh, ss, table_ld, units);
  } else {
    const int64_t units = rows * (hd / 2);
    rope_kernel<T, false><<<(unsigned)ceil_div64(units, 256), 256, 0, st>>>((const T*)x, cs, sn, (T*)y, H, S, hd, sb,
                                                                             sh, ss, table_ld, units);
  }
  HB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------
// QK L2 norm: LPR lanes cooperate on one head vector (hd elements).
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) qk_norm_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                      T* __restrict__ qo, T* __restrict__ ko, int64_t rows_q,
                                                      int64_t rows_k, int hd, float scale_q, float scale_k, int mode,
                                                      int lanes_per_row) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = t / lanes_per_row;
  const int sub = (int)(t % lanes_per_row);
  const bool valid = row < rows_q + rows_k;
  const bool is_k = row >= rows_q;
  const T* src = nullptr;
  T* dst = nullptr;
  if (valid) {
    src = is_k ? k + (row - rows_q) * hd : q + row * hd;
    dst = is_k ? ko + (row - rows_q) * hd : qo + row * hd;
  }
  float ss = 0.f;
  if (valid)
    for (int i = sub; i < hd; i += lanes_per_row) {
      const float a = Cvt<T>::to_f(src[i]);
      ss += a * a;
    }
  // lanes_per_row is a power of two <= 32 and rows never straddle a warp
  for (int o = lanes_per_row >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (!valid) return;
  const float inv = (mode == 0) ? 1.0f / fmaxf(sqrtf(ss), 1e-12f) : rsqrtf(ss + 1e-8f);
  const float m = inv * (is_k ? scale_k : scale_q);
  for (int i = sub; i < hd; i += lanes_per_row) dst[i] = Cvt<T>::from_f(Cvt<T>::to_f(src[i]) * m);
}

// ---------------------------------------------------------------------------------
// SwiGLU activation
// ---------------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ g, const T* __restrict__ u,
                                                     T* __restrict__ o, int64_t rows, int cols, int64_t ldg,
                                                     int64_t ldu) {
  constexpr int V = VEC ? VecOf<T>::N : 1;
  const int upr = cols / V;
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * upr) return;
  const int64_t r = t / upr;
  const int c = (int)(t % upr) * V;
  if (VEC) {
    float a[V], b[V], y[V];
    load_vec<T>(g + r * ldg + c, a);
    load_vec<T>(u + r * ldu + c, b);
#pragma unroll
    for (int i = 0; i < V; ++i) y[i] = a[i] / (1.0f + expf(-a[i])) * b[i];
    store_vec<T>(o + r * cols + c, y);
  } else {
    const float a = Cvt<T>::to_f(g[r * ldg + c]);
    const float b = Cvt<T>::to_f(u[r * ldu + c]);
    o[r * cols + c] = Cvt<T>::from_f(a / (1.0f + expf(-a)) * b);
  }
}

template <typename T>
static int launch_swiglu(const void* g, const void* u, void* o, int64_t rows, int cols, int64_t ldg, int64_t ldu,
                         cudaStream_t st) {
  constexpr int V = VecOf<T>::N;
  const bool vec = (cols % V == 0) && (ldg % V == 0) && (ldu % V == 0) && aligned16(g) && aligned16(u) && aligned16(o);
  if (vec) {
    const int64_t n = rows * (cols / V);
    swiglu_kernel<T, true><<<(unsigned)ceil_div64(n, 256), 256, 0, st>>>((const T*)g, (const T*)u, (T*)o, rows, cols,
                                                                          ldg, ldu);
  } else {
    const int64_t n = rows * cols;
    swiglu_kernel<T, false><<<(unsigned)ceil_div64(n, 256), 256, 0, st>>>((const T*)g, (const T*)u, (T*)o, rows, cols,
                                                                           ldg, ldu);
  }
  HB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------
// Embedding gather with id clamp and sqrt(dim) scale: one warp per token.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embed_kernel(const int64_t* __restrict__ ids,
                                                    const __nv_bfloat16* __restrict__ table,
                                                    __nv_bfloat16* __restrict__ out, int64_t T, int D, int V,
                                                    float scale) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  int64_t id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const __nv_bfloat16* src = table + id * D;
  __nv_bfloat16* dst = out + t * D;
  for (int i = lane * 8; i < D; i += 256) {
    float f[8];
    load_bf16x8(src + i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= scale;
    store_bf16x8(dst + i, f);
  }
}

// ---------------------------------------------------------------------------------
// MoR depth mapping
// ---------------------------------------------------------------------------------
__global__ void mor_depths_kernel(const float* __restrict__ logits, int32_t* __restrict__ depth, int64_t n, int n_rec,
                                  int min_d) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) depth[i] = mor_depth_from_logit(logits[i], n_rec, min_d);
}

// Greedy token choice: index of the largest value of each bf16 row (lowest index among equal maxima; NaN never wins).
__global__ void __launch_bounds__(256) argmax_rows_kernel(const __nv_bfloat16* __restrict__ x, int cols, int64_t ld,
                                                          int64_t* __restrict__ out) {
  __shared__ float s_val[8];
  __shared__ int s_idx[8];
  chain_release();
  chain_wait();
  const __nv_bfloat16* row = x + (int64_t)blockIdx.x * ld;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  auto take = [&](float v, int i) {
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  };
  int done = 0;
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    // 16-byte pieces, four in flight per thread
    const int vec = cols / 8;
    constexpr int UN = 4;
    for (int v0 = threadIdx.x; v0 < vec; v0 += blockDim.x * UN) {
      uint4 raw[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int vi = v0 + u * blockDim.x;
        raw[u] = vi < vec ? __ldcg(reinterpret_cast<const uint4*>(row + (size_t)vi * 8)) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int vi = v0 + u * blockDim.x;
        if (vi < vec) {
          const uint32_t w4[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            take(__uint_as_float(w4[j] << 16), vi * 8 + 2 * j);
            take(__uint_as_float(w4[j] & 0xffff0000u), vi * 8 + 2 * j + 1);
          }
        }
      }
    }
    done = vec * 8;
  }
  for (int i = done + threadIdx.x; i < cols; i += blockDim.x) take(ldcg_bf16(row + i), i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = best_i; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (s_val[w] > best || (s_val[w] == best && s_idx[w] < best_i)) { best = s_val[w]; best_i = s_idx[w]; }
    out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

// Per-row negative log-likelihood of bf16 logits: nll[r] = logsumexp(row r) - row[target[r]] in fp32 (0 where the
// target is `ignore_index`).  One pass: each thread keeps a running maximum and a sum of exponentials relative to it.
__global__ void __launch_bounds__(256) cross_entropy_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                                 const int64_t* __restrict__ targets, int cols, int64_t ld,
                                                                 int64_t ignore_index, float* __restrict__ nll) {
  __shared__ float s_max[8], s_sum[8];
  const int64_t tgt = targets[blockIdx.x];
  if (tgt == ignore_index) {
    if (threadIdx.x == 0) nll[blockIdx.x] = 0.f;
    return;
  }
  const __nv_bfloat16* row = x + (int64_t)blockIdx.x * ld;
  float mx = -INFINITY, sum = 0.f;
  auto take = [&](float v) {
    if (v > mx) { sum = sum * __expf(mx - v) + 1.f; mx = v; }      // exp(-inf) = 0 covers the first element
    else if (v > -INFINITY) sum += __expf(v - mx);                  // -inf adds nothing (and -inf - -inf is NaN)
  };
  int done = 0;
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const int vec = cols / 8;
    constexpr int UN = 4;
    for (int v0 = threadIdx.x; v0 < vec; v0 += blockDim.x * UN) {
      uint4 raw[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int vi = v0 + u * blockDim.x;
        raw[u] = vi < vec ? __ldcg(reinterpret_cast<const uint4*>(row + (size_t)vi * 8)) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        if (v0 + u * (int)blockDim.x < vec) {
          const uint32_t w4[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            take(__uint_as_float(w4[j] << 16));
            take(__uint_as_float(w4[j] & 0xffff0000u));
          }
        }
      }
    }
    done = vec * 8;
  }
  for (int i = done + threadIdx.x; i < cols; i += blockDim.x) take(ldcg_bf16(row + i));
  // merge (max, sum) pairs: lanes, then warps
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, mx, o), os = __shfl_xor_sync(0xffffffffu, sum, o);
    const float nm = fmaxf(mx, om);
    sum = (mx == -INFINITY ? 0.f : sum * __expf(mx - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    mx = nm;
  }
  if ((threadIdx.x & 31) == 0) { s_max[threadIdx.x >> 5] = mx; s_sum[threadIdx.x >> 5] = sum; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = s_max[0], t = s_sum[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
      const float nm = fmaxf(m, s_max[w]);
      t = (m == -INFINITY ? 0.f : t * __expf(m - nm)) + (s_max[w] == -INFINITY ? 0.f : s_sum[w] * __expf(s_max[w] - nm));
      m = nm;
    }
    const int64_t ti = tgt < 0 ? 0 : (tgt >= cols ? cols - 1 : tgt);       // the host has checked the range
    nll[blockIdx.x] = m + logf(t) - ldcg_bf16(row + ti);
  }
}

}  // namespace hb200

namespace hb200 {
int launch_argmax_rows(const void* x, int64_t rows, int cols, int64_t ld, int64_t* out, cudaStream_t st, bool chained) {
  return launch_chained(argmax_rows_kernel, dim3((unsigned)rows), dim3(256), 0, st, chained, 1,
                        (const __nv_bfloat16*)x, cols, ld, out);
}
}  // namespace hb200

using namespace hb200;

extern "C" int hb200_argmax_rows(const void* x, int64_t rows, int cols, int64_t ld, int64_t* out, void* stream) {
  HB_REQUIRE(x && out, HB200_ERR_INVALID, "argmax_rows: null pointer");
  HB_REQUIRE(rows >= 0 && cols >= 1 && ld >= cols, HB200_ERR_INVALID, "argmax_rows: bad shape");
  if (rows == 0) return 0;
  argmax_rows_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, cols, ld, out);
  HB_LAUNCH_CHECK();
  return 0;
}

extern "C" int hb200_cross_entropy_rows(const void* logits, const int64_t* targets, int64_t rows, int cols, int64_t ld,
                                        int64_t ignore_index, float* nll, void* stream) {
  HB_REQUIRE(logits && targets && nll, HB200_ERR_INVALID, "cross_entropy_rows: null pointer");
  HB_REQUIRE(rows >= 0 && cols >= 1 && ld >= cols, HB200_ERR_INVALID, "cross_entropy_rows: bad shape");
  if (rows == 0) return 0;
  cross_entropy_rows_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, targets, cols,
                                                                             ld, ignore_index, nll);
  HB_LAUNCH_CHECK();
  return 0;
}

extern "C" int hb200_rms_norm(const void* x, const void* w, void* y, int64_t rows, int dim, float eps, int dtype,
                              int w_dtype, void* stream) {
  HB_REQUIRE(x && w && y, HB200_ERR_INVALID, "rms_norm: null pointer");
  HB_REQUIRE(rows >= 0 && dim > 0, HB200_ERR_INVALID, "rms_norm: bad shape rows=%lld dim=%d", (long long)rows, dim);
  if (rows == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
#define HB_RMS_CASE(DT, T)                                                                              \
  if (dtype == DT) {                                                                                    \
    if (w_dtype == HB200_F32) return launch_rms_norm<T, float>(x, w, y, rows, dim, eps, st);            \
    if (w_dtype == DT) return launch_rms_norm<T, T>(x, w, y, rows, dim, eps, st);                       \
  }
  HB_RMS_CASE(HB200_F32, float)
  HB_RMS_CASE(HB200_BF16, __nv_bfloat16)
  HB_RMS_CASE(HB200_F16, __half)
#undef HB_RMS_CASE
  set_error("rms_norm: unsupported dtype combination x=%d w=%d (weight must be fp32 or match x)", dtype, w_dtype);
  return HB200_ERR_UNSUPPORTED;
}

extern "C" int hb200_rope(const void* x, const float* cos_t, const float* sin_t, void* y, int B, int H, int S, int hd,
                          int64_t sb, int64_t sh, int64_t ss, int table_ld, int dtype, void* stream) {
  HB_REQUIRE(x && cos_t && sin_t && y, HB200_ERR_INVALID, "rope: null pointer");
  HB_REQUIRE(B >= 0 && H > 0 && S >= 0 && hd > 0 && (hd % 2) == 0, HB200_ERR_INVALID,
             "rope: bad shape B=%d H=%d S=%d hd=%d (head_dim must be even)", B, H, S, hd);
  HB_REQUIRE(table_ld >= hd / 2, HB200_ERR_INVALID, "rope: table row stride %d < hd/2", table_ld);
  if ((int64_t)B * S == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == HB200_F32) return launch_rope<float>(x, cos_t, sin_t, y, B, H, S, hd, sb, sh, ss, table_ld, st);
  if (dtype == HB200_BF16) return launch_rope<__nv_bfloat16>(x, cos_t, sin_t, y, B, H, S, hd, sb, sh, ss, table_ld, st);
  if (dtype == HB200_F16) return launch_rope<__half>(x, cos_t, sin_t, y, B, H, S, hd, sb, sh, ss, table_ld, st);
  set_error("rope: unsupported dtype %d", dtype);
  return HB200_ERR_UNSUPPORTED;
}

extern "C" int hb200_qk_norm(const void* q, const void* k, void* q_out, void* k_out, int64_t rows_q, int64_t rows_k,
                             int hd, float scale, float temperature, int mode, int dtype, void* stream) {
  HB_REQUIRE(q && k && q_out && k_out, HB200_ERR_INVALID, "qk_norm: null pointer");
  HB_REQUIRE(rows_q >= 0 && rows_k >= 0 && hd > 0, HB200_ERR_INVALID, "qk_norm: bad shape");
  HB_REQUIRE(mode == 0 || mode == 1, HB200_ERR_INVALID, "qk_norm: mode must be 0 or 1");
  const int64_t rows = rows_q + rows_k;
  if (rows == 0) return 0;
  int lpr = 1;
  while (lpr < 8 && lpr * 4 < hd) lpr <<= 1;   // ~4 elements per lane, at most 8 lanes per row
  const int64_t threads = rows * lpr;
  const unsigned grid = (unsigned)ceil_div64(threads, 256);
  cudaStream_t st = (cudaStream_t)stream;
  const float sk = scale * temperature;
  if (dtype == HB200_F32)
    qk_norm_kernel<float><<<grid, 256, 0, st>>>((const float*)q, (const float*)k, (float*)q_out, (float*)k_out, rows_q,
                                                rows_k, hd, scale, sk, mode, lpr);
  else if (dtype == HB200_BF16)
    qk_norm_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
                                                        (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out, rows_q, rows_k,
                                                        hd, scale, sk, mode, lpr);
  else if (dtype == HB200_F16)
    qk_norm_kernel<__half><<<grid, 256, 0, st>>>((const __half*)q, (const __half*)k, (__half*)q_out, (__half*)k_out,
                                                 rows_q, rows_k, hd, scale, sk, mode, lpr);
  else {
    set_error("qk_norm: unsupported dtype %d", dtype);
    return HB200_ERR_UNSUPPORTED;
  }
  HB_LAUNCH_CHECK();
  return 0;
}

extern "C" int hb200_swiglu(const void* gate, const void* up, void* out, int64_t rows, int cols, int64_t ld_gate,
                            int64_t ld_up, int dtype, void* stream) {
  HB_REQUIRE(gate && up && out, HB200_ERR_INVALID, "swiglu: null pointer");
  HB_REQUIRE(rows >= 0 && cols > 0 && ld_gate >= cols && ld_up >= cols, HB200_ERR_INVALID, "swiglu: bad shape");
  if (rows == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == HB200_F32) return launch_swiglu<float>(gate, up, out, rows, cols, ld_gate, ld_up, st);
  if (dtype == HB200_BF16) return launch_swiglu<__nv_bfloat16>(gate, up, out, rows, cols, ld_gate, ld_up, st);
  if (dtype == HB200_F16) return launch_swiglu<__half>(gate, up, out, rows, cols, ld_gate, ld_up, st);
  set_error("swiglu: unsupported dtype %d", dtype);
  return HB200_ERR_UNSUPPORTED;
}

extern "C" int hb200_embed(const int64_t* ids, const void* table, void* out, int64_t T, int D, int V, float scale,
                           void* stream) {
  HB_REQUIRE(ids && table && out, HB200_ERR_INVALID, "embed: null pointer");
  HB_REQUIRE(T >= 0 && D > 0 && V > 0 && (D % 8) == 0, HB200_ERR_INVALID, "embed: dim must be a multiple of 8");
  HB_REQUIRE(aligned16(table) && aligned16(out), HB200_ERR_INVALID, "embed: pointers must be 16-byte aligned");
  if (T == 0) return 0;
  embed_kernel<<<(unsigned)ceil_div64(T, 8), 256, 0, (cudaStream_t)stream>>>(
      ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, T, D, V, scale);
  HB_LAUNCH_CHECK();
  return 0;
}

extern "C" int hb200_mor_depths(const float* logits, int32_t* depth, int64_t n, int n_rec, int min_depth,
                                void* stream) {
  HB_REQUIRE(logits && depth, HB200_ERR_INVALID, "mor_depths: null pointer");
  HB_REQUIRE(n >= 0 && n_rec >= 1 && min_depth >= 0 && min_depth <= n_rec - 1, HB200_ERR_INVALID,
             "mor_depths: bad arguments");
  if (n == 0) return 0;
  mor_depths_kernel<<<(unsigned)ceil_div64(n, 256), 256, 0, (cudaStream_t)stream>>>(logits, depth, n, n_rec,
                                                                                    min_depth);
  HB_LAUNCH_CHECK();
  return 0;
}
