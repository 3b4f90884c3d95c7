// Causal grouped-query attention on the 5th-generation tensor cores (tcgen05 + TMEM, operands fed by TMA).
//
// One CTA = 128 query rows of one (batch, q-head).  Per tile of 128 keys:
//   warp 0     TMA producer: Q once, then K and V tiles ([128 keys, hd], swizzle = row width) through a 2-stage ring;
//   warp 1     one thread issues  S = Q K^T   (tcgen05.mma M128 x N128 x K=hd, fp32 S in TMEM columns 0..127)
//              and, once the probabilities are in shared memory,  O += P V  (M128 x N=hd x K128, V as the MN-major
//              B operand exactly as TMA delivered it, O accumulating in TMEM columns 128..128+hd across ALL tiles);
//   warps 2-9  softmax: two warps per TMEM lane quadrant, each owning 64 of the tile's 128 keys; thread = query row;
//              tcgen05.ld 32 columns of S at a time, p = 2^(s*scale*log2e - bound), causal mask on the diagonal tile,
//              P as bf16 into a 128B-swizzled K-major A-operand tile in shared memory (double buffered).
//   The softmax denominator is produced by the tensor core as well: a third, 16-column accumulator receives
//   P x ones (the same bf16 P that multiplies V), so the softmax threads issue one FFMA, one ex2 and half a
//   byte-permute per score, and numerator and denominator see identical probabilities (which is also why P may
//   be truncated to bf16 instead of rounded: the bias divides out).
//
// No running maximum and no rescaling of O: the caller supplies an upper bound of |q.k|*scale (in CCGQA q is a
// unit vector and |k| is the key temperature, both after RoPE, so the bound is temperature/sqrt(hd)); softmax is
// shift-invariant, so subtracting the bound instead of the row maximum gives the same result while every exponent
// stays <= 0.  That makes the kernel a single pass over S limited by the exp (MUFU) rate - the attention core at
// head_dim <= 32 costs one exp per 128 tensor FLOPs - and lets O stay in TMEM untouched until the end.
//
// Two CTAs fit per SM (104 KB of shared memory and 256 TMEM columns each at hd 32), so one CTA's softmax overlaps
// the other's MMAs.  Every mbarrier wait is bounded; on expiry the CTA flags the error, frees TMEM and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "common.cuh"
#include "tcgen05.cuh"

namespace hb200 {

constexpr int AQ = 128;   // query rows per CTA
constexpr int AK = 128;   // keys per tile
constexpr int SOFTMAX_WARPS = 8;
constexpr int ATT_THREADS = (2 + SOFTMAX_WARPS) * 32;

template <int HD> struct AttCfg {
  static constexpr int ROW_BYTES = HD * 2;                               // 32 / 64 / 128: also the swizzle width
  static constexpr uint32_t LAYOUT = HD == 64 ? 2u : (HD == 32 ? 4u : 6u);
  static constexpr int SBO = 8 * ROW_BYTES;                              // stride between 8-row groups
  static constexpr int Q_BYTES = AQ * ROW_BYTES;
  static constexpr int KV_BYTES = AK * ROW_BYTES;
  static constexpr int P_BYTES = AQ * AK * 2;                            // two 64-key halves of 16 KB
  static constexpr int STAGES = 2;
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + STAGES * KV_BYTES;
  static constexpr int OFF_P = OFF_V + STAGES * KV_BYTES;
  static constexpr int OFF_ONES = OFF_P + 2 * P_BYTES;                   // [128 keys][16] bf16, all 1.0
  static constexpr int ONES_BYTES = AK * 32;
  static constexpr int OFF_BAR = OFF_ONES + ONES_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr uint32_t TMEM_COLS = 256;                             // S: 0..127, O: 128..128+HD, row sums: 192..207
};

struct AttParams {
  __nv_bfloat16* o;
  int S, H, KV;
  float scale_log2;    // scale * log2(e)
  float bound_log2;    // upper bound of s * scale_log2
  int32_t* err_flag;
};

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_q,
                                                                const __grid_constant__ CUtensorMap tma_k,
                                                                const __grid_constant__ CUtensorMap tma_v,
                                                                const AttParams p) {
  using Cfg = AttCfg<HD>;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t base = (s_addr(smem_dyn) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - s_addr(smem_dyn));
  const uint32_t bars = base + Cfg::OFF_BAR;
  // barrier slots (8 bytes each)
  const uint32_t q_full = bars, s_full = bars + 8, s_free = bars + 16, o_full = bars + 24;
  auto kv_full = [&](int s) { return bars + 32u + 8u * s; };
  auto kv_empty = [&](int s) { return bars + 48u + 8u * s; };
  auto p_full = [&](int b) { return bars + 64u + 8u * b; };
  auto p_free = [&](int b) { return bars + 80u + 8u * b; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + Cfg::OFF_BAR + 96);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.S, H = p.H, KV = p.KV;
  const int n_qt = (S + AQ - 1) / AQ;
  const int qt = n_qt - 1 - (int)blockIdx.x;   // late query tiles (most keys) first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (H / KV);
  const int q0 = qt * AQ;
  const int n_kt = qt + 1;                     // causal: key tiles 0..qt
  const int q_row0 = (b * H + h) * S + q0;     // row of the [B*H*S, hd] view
  const int kv_row0 = (b * KV + kvh) * S;      // row of the [B*KV*S, hd] view

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(s_full, 1);
    mbar_init(s_free, SOFTMAX_WARPS);
    mbar_init(o_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(kv_full(i), 1);
      mbar_init(kv_empty(i), 1);
      mbar_init(p_full(i), SOFTMAX_WARPS);
      mbar_init(p_free(i), 1);
    }
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // constant all-ones B operand for the row-sum MMA (any layout of ones is the same matrix)
  for (int i = threadIdx.x; i < Cfg::ONES_BYTES / 16; i += blockDim.x)
    st_shared_v4(base + Cfg::OFF_ONES + (uint32_t)i * 16u, make_uint4(0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u));
  fence_proxy_async_smem();
  if (warp == 1) tmem_alloc(s_addr(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128u, tmem_l = tmem_base + 192u;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, Cfg::Q_BYTES);
      tma_load_2d(base, &tma_q, 0, q_row0, q_full);
      for (int j = 0; j < n_kt; ++j) {
        const int s = j & 1;
        if (!mbar_wait(kv_empty(s), (uint32_t)(((j >> 1) & 1) ^ 1), abort_flag)) break;
        mbar_arrive_expect_tx(kv_full(s), 2 * Cfg::KV_BYTES);
        tma_load_2d(base + Cfg::OFF_K + s * Cfg::KV_BYTES, &tma_k, 0, kv_row0 + j * AK, kv_full(s));
        tma_load_2d(base + Cfg::OFF_V + s * Cfg::KV_BYTES, &tma_v, 0, kv_row0 + j * AK, kv_full(s));
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(AQ, AK);          // Q, K both K-major
      constexpr uint32_t idesc_pv = make_idesc_b_mn(AQ, HD);    // P K-major, V MN-major
      constexpr uint32_t idesc_l = make_idesc_b_mn(AQ, 16);     // P x ones -> row sums
      bool ok = mbar_wait(q_full, 0u, abort_flag);
      const uint64_t dq = make_smem_desc_ex(base, Cfg::SBO, Cfg::LAYOUT, 16);
      auto issue_s = [&](int j) {   // S = Q K_j^T into the (single) S accumulator
        const uint64_t dk = make_smem_desc_ex(base + Cfg::OFF_K + (j & 1) * Cfg::KV_BYTES, Cfg::SBO, Cfg::LAYOUT, 16);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma_bf16(tmem_s, dq + 2u * k, dk + 2u * k, idesc_s, k ? 1u : 0u);
        umma_commit(s_full);
      };
      if (ok && (ok = mbar_wait(kv_full(0), 0u, abort_flag))) {
        tcgen05_fence_after();
        issue_s(0);
      }
      for (int j = 0; ok && j < n_kt; ++j) {
        const int s = j & 1, pb = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        if (j + 1 < n_kt) {
          // QK^T of the NEXT tile goes out as soon as the softmax warps have pulled S of this tile into registers,
          // so it runs in the shadow of their exponentials
          if (!mbar_wait(kv_full((j + 1) & 1), (uint32_t)(((j + 1) >> 1) & 1), abort_flag)) break;
          if (!mbar_wait(s_free, (uint32_t)(j & 1), abort_flag)) break;
          tcgen05_fence_after();
          issue_s(j + 1);
        }
        if (!mbar_wait(p_full(pb), ph, abort_flag)) break;
        tcgen05_fence_after();
        const uint32_t pbase = base + Cfg::OFF_P + pb * Cfg::P_BYTES;
        const uint32_t vbase = base + Cfg::OFF_V + s * Cfg::KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < AK / 16; ++kk) {
          // A: P, K-major, 128B swizzle, two 64-key halves 16 KB apart, 32 bytes per 16 keys inside a half
          const uint64_t dp = make_smem_desc(pbase + (kk >> 2) * (AQ * 128) + (kk & 3) * 32);
          // B: V as stored [key][dim] = MN-major; 16 keys = two 8-key groups SBO apart
          const uint64_t dv = make_smem_desc_ex(vbase + kk * 16 * Cfg::ROW_BYTES, Cfg::SBO, Cfg::LAYOUT, Cfg::KV_BYTES);
          umma_bf16(tmem_o, dp, dv, idesc_pv, (j | kk) ? 1u : 0u);
          const uint64_t d1 = make_smem_desc_ex(base + Cfg::OFF_ONES + kk * 16 * 32, 256, 6u, Cfg::ONES_BYTES);
          umma_bf16(tmem_l, dp, d1, idesc_l, (j | kk) ? 1u : 0u);
        }
        umma_commit(kv_empty(s));    // K/V stage reusable once these MMAs have read it
        umma_commit(p_free(pb));     // P buffer reusable
      }
      umma_commit(o_full);
    }
    __syncwarp();
  } else {
    // ------------------------------ softmax warps (2..9): thread = query row, half of the keys ------------------
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;          // keys [64*half, 64*half + 64) of every tile
    const int r = quad * 32 + lane;            // row inside the tile
    const int qrow = q0 + r;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    bool ok = true;
    for (int j = 0; j < n_kt; ++j) {
      const int pb = j & 1;
      if (!mbar_wait(s_full, (uint32_t)(j & 1), abort_flag)) ok = false;
      if (ok && !mbar_wait(p_free(pb), (uint32_t)(((j >> 1) & 1) ^ 1), abort_flag)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const bool diag = (j == n_kt - 1);
      const uint32_t prow = base + Cfg::OFF_P + pb * Cfg::P_BYTES + (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u;
      // both 32-column loads of this thread's 64 keys go out before one wait; S is then free for the next QK^T
      uint32_t sraw[2][32];
      tmem_ld_32x32_nowait(tmem_s + lane_off + (uint32_t)(half * 64), sraw[0]);
      tmem_ld_32x32_nowait(tmem_s + lane_off + (uint32_t)(half * 64 + 32), sraw[1]);
      tmem_wait_ld();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        const int key0 = j * AK + c * 32;
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(sraw[cc][i]), p.scale_log2, -p.bound_log2));
          float p1 = ex2_approx(fmaf(__uint_as_float(sraw[cc][i + 1]), p.scale_log2, -p.bound_log2));
          if (diag) {
            if (key0 + i > qrow) p0 = 0.f;
            if (key0 + i + 1 > qrow) p1 = 0.f;
          }
          // bf16 by truncation: one byte-permute on the integer pipe instead of a conversion on the (saturated)
          // special-function pipe.  The truncation bias cancels: the denominator is summed from the same bf16 values.
          packed[i >> 1] = __byte_perm(__float_as_uint(p0), __float_as_uint(p1), 0x7632);
        }
        // 32 keys = 64 bytes = four 16-byte pieces of this row inside half (c >> 1)
        const uint32_t half_base = prow + (uint32_t)(c >> 1) * (AQ * 128);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int piece = (c & 1) * 4 + q4;
          st_shared_v4(half_base + (uint32_t)((piece ^ (r & 7)) << 4),
                       make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]));
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(pb));
    }
    // ---- finish: O / l -> bf16, token-major ----
    if (ok && !mbar_wait(o_full, 0u, abort_flag)) ok = false;
    ok = __all_sync(0xffffffffu, ok);
    if (ok && half == 0) {
      tcgen05_fence_after();
      float lsum[16];
      tmem_ld_32x16(tmem_l + lane_off, lsum);     // every column of the ones-MMA holds the row sum
      const float inv = 1.0f / lsum[0];
      __nv_bfloat16* dst = p.o + ((size_t)b * S + qrow) * ((size_t)H * HD) + (size_t)h * HD;
      if constexpr (HD == 16) {
        float v[16];
        tmem_ld_32x16(tmem_o + lane_off, v);
        if (qrow < S) {
          float a[8], c8[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) { a[i] = v[i] * inv; c8[i] = v[8 + i] * inv; }
          store_bf16x8(dst, a);
          store_bf16x8(dst + 8, c8);
        }
      } else {
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          float v[32];
          tmem_ld_32x32(tmem_o + lane_off + (uint32_t)(c * 32), v);
          if (qrow < S) {
#pragma unroll
            for (int q8 = 0; q8 < 4; ++q8) {
              float a[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) a[i] = v[q8 * 8 + i] * inv;
              store_bf16x8(dst + c * 32 + q8 * 8, a);
            }
          }
        }
      }
    }
  }

  // ------------------------------ teardown ------------------------------
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (threadIdx.x == 0 && p.err_flag != nullptr) atomicExch(p.err_flag, 2);
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  tcgen05_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ---- host side -------------------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  });
  return fn;
}

// [rows, hd] bf16 matrix, boxes of 128 rows x hd columns, swizzle width = row width
static int make_rows_map(CUtensorMap* map, const void* ptr, uint64_t rows, int hd) {
  auto fn = encode_fn();
  HB_REQUIRE(fn != nullptr, HB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[2] = {(cuuint64_t)hd, rows};
  cuuint64_t gstride[1] = {(cuuint64_t)hd * 2};
  cuuint32_t box[2] = {(cuuint32_t)hd, 128};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = hd == 64 ? CU_TENSOR_MAP_SWIZZLE_128B
                                         : (hd == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  HB_REQUIRE(r == CUDA_SUCCESS, HB200_ERR_CUDA, "cuTensorMapEncodeTiled (attention) failed with CUresult %d", (int)r);
  return 0;
}

template <int HD>
static int launch_att(const void* q, const void* k, const void* v, const AttParams& p, int B, cudaStream_t st) {
  using Cfg = AttCfg<HD>;
  CUtensorMap tq, tk, tv;
  HB_PROPAGATE(make_rows_map(&tq, q, (uint64_t)B * p.H * p.S, HD));
  HB_PROPAGATE(make_rows_map(&tk, k, (uint64_t)B * p.KV * p.S, HD));
  HB_PROPAGATE(make_rows_map(&tv, v, (uint64_t)B * p.KV * p.S, HD));
  auto kern = attention_tcgen05_kernel<HD>;
  HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, (size_t)(Cfg::SMEM_BYTES)));
  dim3 grid((p.S + AQ - 1) / AQ, p.H, B);
  kern<<<grid, ATT_THREADS, Cfg::SMEM_BYTES, st>>>(tq, tk, tv, p);
  HB_LAUNCH_CHECK();
  return 0;
}

// Returns HB200_ERR_UNSUPPORTED (without touching the error text) when the shape is not built for this path.
int launch_attention_tcgen05(const void* q, const void* k, const void* v, void* o, int B, int S, int H, int KV, int hd,
                             float scale, float logit_bound, int32_t* err_flag, cudaStream_t st) {
  AttParams p{(__nv_bfloat16*)o, S, H, KV, scale * 1.4426950408889634f, logit_bound * 1.4426950408889634f, err_flag};
  if (hd == 16) return launch_att<16>(q, k, v, p, B, st);
  if (hd == 32) return launch_att<32>(q, k, v, p, B, st);
  if (hd == 64) return launch_att<64>(q, k, v, p, B, st);
  return HB200_ERR_UNSUPPORTED;
}

}  // namespace hb200
