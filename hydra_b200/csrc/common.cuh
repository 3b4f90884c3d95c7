// Shared helpers for the sm_100a kernels: status/error plumbing, dtype traits,
// vector loads, warp reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/hydra_b200.h"

namespace hb200 {

// ---- host-side status plumbing ------------------------------------------------
void set_error(const char* fmt, ...);   // defined in api.cu (thread-local buffer)

#define HB_REQUIRE(cond, code, ...)          \
  do {                                       \
    if (!(cond)) {                           \
      ::hb200::set_error(__VA_ARGS__);       \
      return (code);                         \
    }                                        \
  } while (0)

#define HB_CUDA(expr)                                                                    \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess) {                                                             \
      ::hb200::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, \
                         __LINE__);                                                      \
      return HB200_ERR_CUDA;                                                             \
    }                                                                                    \
  } while (0)

#define HB_LAUNCH_CHECK()                                                             \
  do {                                                                                \
    cudaError_t _e = cudaGetLastError();                                              \
    if (_e != cudaSuccess) {                                                          \
      ::hb200::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e),  \
                         __FILE__, __LINE__);                                         \
      return HB200_ERR_CUDA;                                                          \
    }                                                                                 \
  } while (0)

#define HB_PROPAGATE(expr)      \
  do {                          \
    int _s = (expr);            \
    if (_s != 0) return _s;     \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- device helpers -------------------------------------------------------------
template <typename T> struct Cvt;
template <> struct Cvt<float> {
  __device__ static float to_f(float v) { return v; }
  __device__ static float from_f(float v) { return v; }
};
template <> struct Cvt<__nv_bfloat16> {
  __device__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Cvt<__half> {
  __device__ static float to_f(__half v) { return __half2float(v); }
  __device__ static __half from_f(float v) { return __float2half_rn(v); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// 8 bf16 <-> 8 floats through one 16-byte access
struct alignas(16) bf16x8 { __nv_bfloat162 h[4]; };

__device__ __forceinline__ void load_bf16x8(const __nv_bfloat16* p, float (&f)[8]) {
  bf16x8 v = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(v.h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store_bf16x8(__nv_bfloat16* p, const float (&f)[8]) {
  bf16x8 v;
#pragma unroll
  for (int i = 0; i < 4; ++i) v.h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = v;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float silu_mul(float g, float u) {
  return g / (1.0f + __expf(-g)) * u;
}

// MoR depth from a raw router logit: clamp(round_half_even(min_d + sigmoid(3 tanh(l/2)) * (R-1-min_d))).
__device__ __forceinline__ int mor_depth_from_logit(float l, int n_rec, int min_d) {
  const float sq = tanhf(l * 0.5f) * 3.0f;
  const float p = 1.0f / (1.0f + expf(-sq));
  const float cont = (min_d > 0) ? (float)min_d + p * (float)(n_rec - 1 - min_d) : p * (float)(n_rec - 1);
  int d = (int)rintf(cont);   // round half to even, as torch.round
  d = d < min_d ? min_d : d;
  d = d > n_rec - 1 ? n_rec - 1 : d;
  return d;
}

// Exclusive prefix sum of one int per thread over the whole CTA (thread order). `total` is the CTA sum.
// `warp_buf` is shared scratch of at least 33 ints; contains a trailing __syncthreads().
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_buf, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_buf[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = lane < nwarps ? warp_buf[lane] : 0;
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    warp_buf[lane] = wi - w;          // exclusive warp offsets
    if (lane == 31) warp_buf[32] = wi;  // CTA total
  }
  __syncthreads();
  const int off = warp_buf[warp];
  total = warp_buf[32];
  __syncthreads();
  return off + incl - v;
}

}  // namespace hb200
