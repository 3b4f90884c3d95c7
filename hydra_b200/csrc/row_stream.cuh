// Streaming row kernels of the prefill executor: router scores, gather + pre-MLP norm, exit norm + next input norm.
//
// Rows travel HBM -> shared memory as bulk copies (cp.async.bulk, 2 KB or more each) through a ring of stages fed by
// one producer warp; sixteen consumer warps work out of shared memory and write their results from registers.  A
// register-resident row kernel has to hold every byte it wants in flight in registers, which caps it at two CTAs per
// SM and leaves a CTA's loads un-overlapped with its own arithmetic; here up to 192 KB per SM are in flight whatever
// the consumers are doing, one persistent CTA per SM.  The per-column vectors (gains, offsets, router weights) sit in
// shared memory once per CTA.  The arithmetic, and its order, is that of the register-resident kernels in
// row_kernels.cuh, so both forms give the same bits.
//
// Every mbarrier wait is bounded; on expiry the CTA raises its abort flag, all roles leave their loops, the error is
// reported through err_flag and the kernel returns after the copies in flight have had time to land.
#pragma once
#include "row_kernels.cuh"
#include "tcgen05.cuh"

namespace hb200 {

constexpr int STREAM_CONSUMERS = 16;
constexpr int STREAM_THREADS = (STREAM_CONSUMERS + 1) * 32;

template <int NCH_, int NVEC_> struct StreamCfg {
  static constexpr int NCH = NCH_;
  static constexpr int NVEC = NVEC_;                                 // fp32 per-column vectors kept in shared memory
  static constexpr int RPW = NCH <= 4 ? 2 : 1;                       // rows per consumer warp and tile
  static constexpr int TILE_ROWS = STREAM_CONSUMERS * RPW;
  static constexpr int DPAD = NCH * 256;                             // elements of a per-column vector
  static constexpr int STAGE_BYTES = TILE_ROWS * DPAD * 2;           // rows are packed at D*2 bytes: an upper bound
  static constexpr int VEC_BYTES = NVEC * DPAD * 4;
  static constexpr int BUDGET = 226 * 1024 - VEC_BYTES;
  static constexpr int STAGES = BUDGET / STAGE_BYTES >= 4 ? 4 : BUDGET / STAGE_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + VEC_BYTES + 256 + 128;
  static_assert(STAGES >= 2, "the ring needs two stages");
};

struct StreamCtx {
  uint32_t ring;                   // shared-memory address of stage 0
  uint32_t bars;                   // full barriers, then empty barriers
  float* vec;                      // NVEC vectors of DPAD floats, in the lane-interleaved layout of stream_vec_slot
  volatile uint32_t* abort_flag;
};

// Element (c*32 + lane)*8 + j of a per-column vector sits at ((c*2 + j/4)*32 + lane)*4 + j%4, so that the two float4
// reads a lane makes per 8-column chunk are contiguous across the warp (no bank conflicts).
__device__ __forceinline__ int stream_vec_slot(int i) {
  return (((i >> 8) * 2 + ((i >> 2) & 1)) * 32 + ((i & 255) >> 3)) * 4 + (i & 3);
}
__device__ __forceinline__ void stream_vec_load(const float* vec, int c, int lane, float (&o)[8]) {
  const int v0 = (c * 64 + lane) * 4;
  const float4 a0 = *reinterpret_cast<const float4*>(vec + v0), a1 = *reinterpret_cast<const float4*>(vec + v0 + 128);
  o[0] = a0.x; o[1] = a0.y; o[2] = a0.z; o[3] = a0.w; o[4] = a1.x; o[5] = a1.y; o[6] = a1.z; o[7] = a1.w;
}

// Carves the dynamic shared memory and initialises the barriers.  The caller fills the vectors and then synchronises
// the CTA before any role starts.
template <class Cfg>
__device__ __forceinline__ StreamCtx stream_setup(unsigned char* smem) {
  StreamCtx cx;
  cx.ring = (s_addr(smem) + 127u) & ~127u;
  unsigned char* base_ptr = smem + (cx.ring - s_addr(smem));
  cx.vec = reinterpret_cast<float*>(base_ptr + Cfg::STAGES * Cfg::STAGE_BYTES);
  cx.bars = cx.ring + Cfg::STAGES * Cfg::STAGE_BYTES + Cfg::VEC_BYTES;
  cx.abort_flag = reinterpret_cast<volatile uint32_t*>(base_ptr + Cfg::STAGES * Cfg::STAGE_BYTES + Cfg::VEC_BYTES + 128);
  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(cx.bars + 8u * s, 1);
      mbar_init(cx.bars + 8u * (Cfg::STAGES + s), STREAM_CONSUMERS);
    }
    *cx.abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  return cx;
}

// Producer warp: tiles of TILE_ROWS rows, this CTA's tiles blockIdx.x, blockIdx.x + gridDim.x, ...  Contiguous rows
// (rows == nullptr) are copied one consumer warp's share at a time; listed rows (row j of the tile = src row rows[j])
// one row per lane.
template <class Cfg>
__device__ __forceinline__ void stream_produce(const StreamCtx& cx, const __nv_bfloat16* src, const int32_t* rows,
                                               int64_t n_rows, int D) {
  const int lane = threadIdx.x & 31;
  const int64_t n_tiles = (n_rows + Cfg::TILE_ROWS - 1) / Cfg::TILE_ROWS;
  const uint32_t row_bytes = (uint32_t)D * 2u;
  int it = 0;
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
    const int s = it % Cfg::STAGES;
    const uint32_t ph = (uint32_t)(it / Cfg::STAGES) & 1u;
    const int64_t row0 = tile * Cfg::TILE_ROWS;
    const int rows_here = (int)((n_rows - row0) < (int64_t)Cfg::TILE_ROWS ? (n_rows - row0) : (int64_t)Cfg::TILE_ROWS);
    // the index of a listed row is fetched before the wait for the stage, so its latency hides behind that wait
    int64_t listed = 0;
    if (rows != nullptr && lane < rows_here) listed = (int64_t)rows[row0 + lane];
    bool ok = true;
    if (lane == 0) ok = mbar_wait(cx.bars + 8u * (Cfg::STAGES + s), ph ^ 1u, cx.abort_flag, 64u);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const uint32_t full = cx.bars + 8u * s;
    const uint32_t dst = cx.ring + (uint32_t)s * Cfg::STAGE_BYTES;
    if (lane == 0) mbar_arrive_expect_tx(full, (uint32_t)rows_here * row_bytes);
    __syncwarp();
    if (rows != nullptr) {
      if (lane < rows_here) bulk_load_1d(dst + (uint32_t)lane * row_bytes, src + listed * D, row_bytes, full);
    } else if (lane < STREAM_CONSUMERS) {
      const int r0 = lane * Cfg::RPW;
      const int n = rows_here - r0 < Cfg::RPW ? rows_here - r0 : Cfg::RPW;
      if (n > 0) bulk_load_1d(dst + (uint32_t)r0 * row_bytes, src + (row0 + r0) * D, (uint32_t)n * row_bytes, full);
    }
  }
}

// Consumer warps: f(j0, raw) once per tile and warp with the raw 16-byte pieces of rows j0 .. j0+RPW-1 (zeros for rows
// at or past n_rows); the stage is handed back to the producer as soon as the rows are in registers.
template <class Cfg, class F>
__device__ __forceinline__ void stream_consume(const StreamCtx& cx, int64_t n_rows, int D, F&& f) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n_tiles = (n_rows + Cfg::TILE_ROWS - 1) / Cfg::TILE_ROWS;
  const uint32_t row_bytes = (uint32_t)D * 2u;
  int it = 0;
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
    const int s = it % Cfg::STAGES;
    const uint32_t ph = (uint32_t)(it / Cfg::STAGES) & 1u;
    bool ok = mbar_wait(cx.bars + 8u * s, ph, cx.abort_flag, 32u);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const int64_t j0 = tile * Cfg::TILE_ROWS + warp * Cfg::RPW;
    const uint32_t src = cx.ring + (uint32_t)s * Cfg::STAGE_BYTES + (uint32_t)(warp * Cfg::RPW) * row_bytes;
    uint4 raw[Cfg::RPW][Cfg::NCH];
#pragma unroll
    for (int r = 0; r < Cfg::RPW; ++r)
#pragma unroll
      for (int c = 0; c < Cfg::NCH; ++c) {
        const int i = (c * 32 + lane) * 8;
        raw[r][c] = (i < D && j0 + r < n_rows) ? ld_shared_v4(src + (uint32_t)r * row_bytes + (uint32_t)i * 2u)
                                              : make_uint4(0, 0, 0, 0);
      }
    __syncwarp();
    if (lane == 0) mbar_arrive(cx.bars + 8u * (Cfg::STAGES + s));
    f(j0, raw);
  }
}

// After the roles have left their loops: report an abandoned wait and give copies in flight time to land.
__device__ __forceinline__ void stream_teardown(const StreamCtx& cx, int32_t* err_flag, int code) {
  __syncthreads();
  if (*cx.abort_flag != 0u) {
    if (threadIdx.x == 0 && err_flag != nullptr) atomicExch(err_flag, code);
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& u, float (&x)[8]) {
  const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] = (j & 1) ? __uint_as_float(w4[j >> 1] & 0xffff0000u) : __uint_as_float(w4[j >> 1] << 16);
}

// ---- router scores over all tokens (mor_score_kernel's arithmetic) ---------------------------------------------
template <int NCH, bool HAS_MOD, bool HAS_ROUTER, bool HAS_SS>
__global__ void __launch_bounds__(STREAM_THREADS, 1)
    mor_score_stream_kernel(const __nv_bfloat16* __restrict__ cur, const float* __restrict__ rec,
                            const float* __restrict__ mod_wn, const float* __restrict__ mod_b,
                            const float* __restrict__ mor_w, const float* __restrict__ mor_b, float* __restrict__ scores,
                            float* __restrict__ logits, int32_t* __restrict__ depth, int64_t T, int D, float eps, int n_rec,
                            int min_d, float* __restrict__ inv_rms, int32_t* err_flag) {
  using Cfg = StreamCfg<NCH, 3>;
  extern __shared__ unsigned char stream_smem[];
  const StreamCtx cx = stream_setup<Cfg>(stream_smem);
  for (int i = threadIdx.x; i < Cfg::DPAD; i += STREAM_THREADS) {
    const bool in = i < D;
    const int slot = stream_vec_slot(i);
    cx.vec[slot] = (HAS_MOD && in) ? mod_wn[i] : 0.f;
    cx.vec[Cfg::DPAD + slot] = ((HAS_MOD || HAS_SS) && in) ? rec[i] : 0.f;
    cx.vec[2 * Cfg::DPAD + slot] = (HAS_ROUTER && in) ? mor_w[i] : 0.f;
  }
  __syncthreads();
  if ((threadIdx.x >> 5) == STREAM_CONSUMERS) {
    stream_produce<Cfg>(cx, cur, nullptr, T, D);
  } else {
    const int lane = threadIdx.x & 31;
    const float b_mod = HAS_MOD ? mod_b[0] : 0.f;
    const float b_mor = HAS_ROUTER ? mor_b[0] : 0.f;
    stream_consume<Cfg>(cx, T, D, [&](int64_t j0, uint4 (&raw)[Cfg::RPW][NCH]) {
      float ss[Cfg::RPW], dm[Cfg::RPW], lm[Cfg::RPW];
#pragma unroll
      for (int r = 0; r < Cfg::RPW; ++r) ss[r] = dm[r] = lm[r] = 0.f;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        if ((c * 32 + lane) * 8 >= D) continue;
        float wn[8], rc[8], wr[8];
        if (HAS_MOD) stream_vec_load(cx.vec, c, lane, wn);
        if (HAS_MOD || HAS_SS) stream_vec_load(cx.vec + Cfg::DPAD, c, lane, rc);
        if (HAS_ROUTER) stream_vec_load(cx.vec + 2 * Cfg::DPAD, c, lane, wr);
#pragma unroll
        for (int r = 0; r < Cfg::RPW; ++r) {
          float x[8];
          unpack_bf16x8(raw[r][c], x);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (HAS_MOD || HAS_SS) {
              const float xr = x[j] + rc[j];
              ss[r] += xr * xr;
              if (HAS_MOD) dm[r] += xr * wn[j];
            }
            if (HAS_ROUTER) lm[r] += x[j] * wr[j];
          }
        }
      }
#pragma unroll
      for (int r = 0; r < Cfg::RPW; ++r) {
        float s2 = 0.f, d2 = 0.f, l2 = 0.f;
        if (HAS_MOD || HAS_SS) s2 = warp_sum(ss[r]);
        if (HAS_MOD) d2 = warp_sum(dm[r]);
        if (HAS_ROUTER) l2 = warp_sum(lm[r]);
        if (lane == 0 && j0 + r < T) {
          if (HAS_MOD) scores[j0 + r] = rsqrtf(s2 / (float)D + eps) * d2 + b_mod;
          if (HAS_SS) inv_rms[j0 + r] = rsqrtf(s2 / (float)D + eps);
          if (HAS_ROUTER) {
            const float l = l2 + b_mor;
            if (logits != nullptr) logits[j0 + r] = l;
            if (depth != nullptr) depth[j0 + r] = mor_depth_from_logit(l, n_rec, min_d);
          }
        }
      }
    });
  }
  stream_teardown(cx, err_flag, 4);
}

// ---- ug[j] = AdaRMSNorm(cur[rows[j]] + rec) for j < *count (norm_gather_kernel's arithmetic) -------------------
template <int NCH>
__global__ void __launch_bounds__(STREAM_THREADS, 1)
    norm_gather_stream_kernel(const __nv_bfloat16* __restrict__ cur, const float* __restrict__ rec,
                              const float* __restrict__ w2, const int32_t* __restrict__ rows,
                              const int32_t* __restrict__ count, __nv_bfloat16* __restrict__ ug, int D, float eps,
                              int32_t* err_flag) {
  using Cfg = StreamCfg<NCH, 2>;
  extern __shared__ unsigned char stream_smem[];
  const int64_t n = *count;
  // a CTA without a tile (few routed rows: the late recursions) leaves before it sets anything up
  if ((int64_t)blockIdx.x * Cfg::TILE_ROWS >= n) return;
  const StreamCtx cx = stream_setup<Cfg>(stream_smem);
  {
    for (int i = threadIdx.x; i < Cfg::DPAD; i += STREAM_THREADS) {
      const bool in = i < D;
      const int slot = stream_vec_slot(i);
      cx.vec[slot] = in ? rec[i] : 0.f;
      cx.vec[Cfg::DPAD + slot] = in ? w2[i] : 0.f;
    }
  }
  __syncthreads();
  if ((threadIdx.x >> 5) == STREAM_CONSUMERS) {
    stream_produce<Cfg>(cx, cur, rows, n, D);
  } else {
    const int lane = threadIdx.x & 31;
    stream_consume<Cfg>(cx, n, D, [&](int64_t j0, uint4 (&raw)[Cfg::RPW][NCH]) {
#pragma unroll
      for (int r = 0; r < Cfg::RPW; ++r) {
        if (j0 + r >= n) break;                                   // warp-uniform
        float v[NCH][8];
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          if ((c * 32 + lane) * 8 >= D) continue;
          float rc[8];
          stream_vec_load(cx.vec, c, lane, rc);
          unpack_bf16x8(raw[r][c], v[c]);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[c][j] += rc[j];
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += v[c][j] * v[c][j];
        }
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const int i = (c * 32 + lane) * 8;
          if (i >= D) continue;
          float ww[8];
          stream_vec_load(cx.vec + Cfg::DPAD, c, lane, ww);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[c][j] = v[c][j] * inv * ww[j];     // store_bf16x8 rounds to nearest even
          store_bf16x8(ug + (j0 + r) * D + i, v[c]);
        }
      }
    });
  }
  stream_teardown(cx, err_flag, 4);
}

// ---- y = RMSNorm(src; w1) (bf16), z = RMSNorm(y; w2) (dual_norm_kernel's arithmetic) ---------------------------
// Either output may be omitted; w1 == nullptr: y = src.  y may be src itself: a tile is in shared memory before any of
// its rows is written, and no other tile covers those rows.
template <int NCH>
__global__ void __launch_bounds__(STREAM_THREADS, 1)
    dual_norm_stream_kernel(const __nv_bfloat16* src, const float* __restrict__ w1, __nv_bfloat16* y,
                            const float* __restrict__ w2, __nv_bfloat16* __restrict__ z, int64_t T, int D, float eps,
                            int32_t* err_flag) {
  using Cfg = StreamCfg<NCH, 2>;
  extern __shared__ unsigned char stream_smem[];
  const StreamCtx cx = stream_setup<Cfg>(stream_smem);
  for (int i = threadIdx.x; i < Cfg::DPAD; i += STREAM_THREADS) {
    const bool in = i < D;
    const int slot = stream_vec_slot(i);
    cx.vec[slot] = (in && w1 != nullptr) ? w1[i] : 0.f;
    cx.vec[Cfg::DPAD + slot] = (in && z != nullptr) ? w2[i] : 0.f;
  }
  __syncthreads();
  if ((threadIdx.x >> 5) == STREAM_CONSUMERS) {
    stream_produce<Cfg>(cx, src, nullptr, T, D);
  } else {
    const int lane = threadIdx.x & 31;
    stream_consume<Cfg>(cx, T, D, [&](int64_t j0, uint4 (&raw)[Cfg::RPW][NCH]) {
#pragma unroll
      for (int r = 0; r < Cfg::RPW; ++r) {
        if (j0 + r >= T) break;                                   // warp-uniform
        float v[NCH][8];
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          if ((c * 32 + lane) * 8 >= D) continue;
          unpack_bf16x8(raw[r][c], v[c]);
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += v[c][j] * v[c][j];
        }
        ss = warp_sum(ss);
        const float inv1 = rsqrtf(ss / (float)D + eps);
        float ss2 = 0.f;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const int i = (c * 32 + lane) * 8;
          if (i >= D) continue;
          if (w1 != nullptr) {
            float ww[8];
            stream_vec_load(cx.vec, c, lane, ww);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[c][j] = __bfloat162float(__float2bfloat16_rn(v[c][j] * inv1 * ww[j]));
          }
          if (y != nullptr) store_bf16x8(y + (j0 + r) * D + i, v[c]);
#pragma unroll
          for (int j = 0; j < 8; ++j) ss2 += v[c][j] * v[c][j];
        }
        if (z == nullptr) continue;
        ss2 = warp_sum(ss2);
        const float inv2 = rsqrtf(ss2 / (float)D + eps);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const int i = (c * 32 + lane) * 8;
          if (i >= D) continue;
          float ww[8];
          stream_vec_load(cx.vec + Cfg::DPAD, c, lane, ww);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[c][j] = v[c][j] * inv2 * ww[j];
          store_bf16x8(z + (j0 + r) * D + i, v[c]);
        }
      }
    });
  }
  stream_teardown(cx, err_flag, 4);
}

}  // namespace hb200
