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

// Weight of the output projection: the untied matrix when the model carries one, else the embedding table.
inline const void* output_weight(const hb200_model* m) { return m->lm_head ? m->lm_head : m->tok_emb; }

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

// ---- programmatic dependent launch ------------------------------------------------------------------------------
// A chain of kernels in one stream in which each kernel lets its successor be scheduled early (chain_release, at the
// top) and touches global memory only after its predecessor has completed and flushed (chain_wait).  The successor's
// launch latency and prologue (barrier set-up, TMEM allocation) then overlap the predecessor's tail.  Both
// instructions are no-ops in a kernel that was launched without the attribute.
#ifdef __CUDACC__
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launch `kern` as a link of such a chain (chained = false: an ordinary launch).  cluster_x > 1 adds a cluster shape.
template <typename... KArgs, typename... Args>
inline int launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool chained,
                          int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (chained) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) {
    set_error("kernel launch failed: %s", cudaGetErrorString(e));
    return HB200_ERR_CUDA;
  }
  return 0;
}
#endif

// Raises a kernel's dynamic shared memory limit to at least `bytes` on the current device (the attribute is a
// per-device property of the kernel; the sizes already set are remembered per (kernel, device)).  Defined in api.cu.
int ensure_dynamic_smem(const void* kernel, size_t bytes);

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

// 8 bf16 <-> 8 floats through ONE 16-byte access (explicit uint4: a struct-of-bfloat162 copy is not guaranteed to
// become a single vector instruction)
__device__ __forceinline__ void load_bf16x8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // bf16 -> fp32 is a 16-bit shift
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
// Loads that bypass L1 (ld.global.cg).  Kernels of a programmatic-dependent-launch chain start before their
// predecessor has finished, so the L1 invalidation of a kernel boundary no longer separates a predecessor's reads of a
// buffer from a later kernel's reads of the same buffer after another SM rewrote it: everything such kernels read
// that other kernels of the chain write goes through L2.
__device__ __forceinline__ void load_bf16x8_cg(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ float ldcg_bf16(const __nv_bfloat16* p) {
  return __uint_as_float((uint32_t)__ldcg(reinterpret_cast<const unsigned short*>(p)) << 16);
}
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void store_bf16x8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 raw;
  raw.x = pack_bf16x2_rn(f[0], f[1]);
  raw.y = pack_bf16x2_rn(f[2], f[3]);
  raw.z = pack_bf16x2_rn(f[4], f[5]);
  raw.w = pack_bf16x2_rn(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = raw;
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
