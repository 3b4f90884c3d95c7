// Causal grouped-query attention on the 5th-generation tensor cores (tcgen05 + TMEM, operands fed by TMA).
//
// One CTA = 128 query rows of one (batch, q-head).  Per tile of 128 keys:
//   warp 0     TMA producer: Q once, then K and V tiles ([128 keys, hd], swizzle = row width) through a 5- or 6-stage ring
//              (a tile takes ~2500 clocks to arrive from L2; with fewer stages that latency sets the pace);
//   warp 1     one thread issues  S = Q K^T   (tcgen05.mma M128 x N128 x K=hd, fp32 S in TMEM columns 0..127)
//              and, once the probabilities are back in TMEM,  O += P V  (M128 x N=hd x K128: P is the A operand READ
//              FROM TENSOR MEMORY, V the MN-major B operand exactly as TMA delivered it; O accumulates in TMEM across
//              ALL tiles);
//   warps 2-9  softmax: two warps per TMEM lane quadrant, each owning 64 of the tile's 128 keys; thread = query row;
//              tcgen05.ld 32 columns of S at a time, p = 2^(s*scale*log2e - bound), causal mask on the diagonal tile,
//              P as packed bf16 pairs straight back into 64 TMEM columns (tcgen05.st).
//   Why P lives in tensor memory: a K = 16 slice of a 128-row operand tile in shared memory is 128 separate 32-byte
//   pieces, one shared-memory wavefront each, so every M128 x N=hd MMA with P in shared memory occupied the tensor
//   pipe for ~128 clocks however small N was - the kernel was bound by that operand fetch, not by the exponentials.
//   Read from tensor memory the same MMA costs a few tens of clocks, and P never touches shared memory at all.
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
// CTAs are ordered heaviest first over the whole grid (the last query tile of every (batch, head) before any
// second-to-last one), so the hardware scheduler fills the tail with the short ones.  K / V / Q are addressed through
// [heads][S][hd] tensor maps: rows past the end of a sequence read as zero instead of the next head's rows.
// Two CTAs fit per SM (256 TMEM columns each at hd <= 32), so one CTA's softmax overlaps the other's MMAs.
// Every mbarrier wait is bounded; on expiry the CTA flags the error, frees TMEM and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "common.cuh"
#include "tcgen05.cuh"

namespace hb200 {

constexpr int AQ = 128;   // query rows per CTA
constexpr int AK = 128;   // keys per tile
constexpr int CPW = 2;             // 32-key chunks of a tile per softmax warp
constexpr int SOFTMAX_WARPS = 4 * (4 / CPW);
constexpr int ATT_THREADS = (2 + SOFTMAX_WARPS) * 32;

template <int HD> struct AttCfg {
  static constexpr int ROW_BYTES = HD * 2;                               // 32 / 64 / 128: also the swizzle width
  static constexpr uint32_t LAYOUT = HD == 64 ? 2u : (HD == 32 ? 4u : 6u);
  static constexpr int SBO = 8 * ROW_BYTES;                              // stride between 8-row groups
  static constexpr int Q_BYTES = AQ * ROW_BYTES;
  static constexpr int KV_BYTES = AK * ROW_BYTES;
  static constexpr int STAGES = HD == 64 ? 5 : 6;                        // K/V tiles in flight: a load takes ~2500 clocks to land
  static_assert(STAGES <= 8, "barrier slots are laid out for at most eight stages");
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + STAGES * KV_BYTES;
  static constexpr int OFF_ONES = OFF_V + STAGES * KV_BYTES;             // [128 keys][16] bf16, all 1.0
  static constexpr int ONES_BYTES = AK * 32;
  static constexpr int OFF_BAR = OFF_ONES + ONES_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  // S: 0..127, O: 128..128+HD, row sums: 128+HD..+16, P (bf16 pairs, 64 cells): the last 64 columns
  static constexpr uint32_t TMEM_COLS = HD <= 32 ? 256 : 512;
  static constexpr uint32_t COL_O = 128, COL_L = 128 + HD, COL_P = TMEM_COLS - 64;
};

struct AttParams {
  __nv_bfloat16* o;
  int S, H, KV;
  float scale_log2;    // scale * log2(e)
  float bound_log2;    // upper bound of s * scale_log2
  int32_t* err_flag;
};

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS, (HD <= 32 ? 2 : 1)) attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_q,
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
  const uint32_t p_full = bars + 32u, p_free = bars + 40u;
  auto kv_full = [&](int s) { return bars + 48u + 8u * s; };
  auto kv_empty = [&](int s) { return bars + 112u + 8u * s; };      // up to eight stages each
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + Cfg::OFF_BAR + 176);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.S, H = p.H, KV = p.KV;
  const int n_qt = (S + AQ - 1) / AQ;
  const int qt = n_qt - 1 - (int)blockIdx.y;   // late query tiles (most keys) first, over the whole grid
  const int h = (int)blockIdx.x % H, b = (int)blockIdx.x / H;
  const int kvh = h / (H / KV);
  const int q0 = qt * AQ;
  const int n_kt = qt + 1;                     // causal: key tiles 0..qt

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(s_full, 1);
    mbar_init(s_free, SOFTMAX_WARPS);
    mbar_init(o_full, 1);
    mbar_init(p_full, SOFTMAX_WARPS);
    mbar_init(p_free, 1);
    for (int i = 0; i < Cfg::STAGES; ++i) {
      mbar_init(kv_full(i), 1);
      mbar_init(kv_empty(i), 1);
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
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + Cfg::COL_O, tmem_l = tmem_base + Cfg::COL_L,
                 tmem_p = tmem_base + Cfg::COL_P;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, Cfg::Q_BYTES);
      tma_load_3d(base, &tma_q, 0, q0, b * H + h, q_full);
      int s = 0;
      uint32_t ph = 0;
      for (int j = 0; j < n_kt; ++j) {
        if (!mbar_wait(kv_empty(s), ph ^ 1u, abort_flag, 256u)) break;   // five tiles ahead: no hurry
        mbar_arrive_expect_tx(kv_full(s), 2 * Cfg::KV_BYTES);
        tma_load_3d(base + Cfg::OFF_K + s * Cfg::KV_BYTES, &tma_k, 0, j * AK, b * KV + kvh, kv_full(s));
        tma_load_3d(base + Cfg::OFF_V + s * Cfg::KV_BYTES, &tma_v, 0, j * AK, b * KV + kvh, kv_full(s));
        if (++s == Cfg::STAGES) { s = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // The whole warp runs this loop with warp-uniform values; one elected lane issues each MMA / commit (see the
    // *_elect wrappers: a fraction of the issue cost of a single-lane loop, and these MMAs are small).
    {
      constexpr uint32_t idesc_s = make_idesc(AQ, AK);          // Q, K both K-major
      constexpr uint32_t idesc_pv = make_idesc_b_mn(AQ, HD);    // P from tensor memory, V MN-major
      constexpr uint32_t idesc_l = make_idesc_b_mn(AQ, 16);     // P x ones -> row sums
      bool ok = mbar_wait(q_full, 0u, abort_flag, 64u);
      const uint64_t dq = make_smem_desc_ex(base, Cfg::SBO, Cfg::LAYOUT, 16);
      const uint64_t dk0 = make_smem_desc_ex(base + Cfg::OFF_K, Cfg::SBO, Cfg::LAYOUT, 16);
      const uint64_t dv0 = make_smem_desc_ex(base + Cfg::OFF_V, Cfg::SBO, Cfg::LAYOUT, Cfg::KV_BYTES);
      const uint64_t d10 = make_smem_desc_ex(base + Cfg::OFF_ONES, 256, 6u, Cfg::ONES_BYTES);
      auto issue_s = [&](int stage) {   // S = Q K^T into the (single) S accumulator
        const uint64_t dk = dk0 + (uint64_t)((stage * Cfg::KV_BYTES) >> 4);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma_bf16_elect(tmem_s, dq + 2u * k, dk + 2u * k, idesc_s, k ? 1u : 0u);
        umma_commit_elect(s_full);
      };
      if (ok && (ok = mbar_wait(kv_full(0), 0u, abort_flag, 64u))) {
        tcgen05_fence_after();
        issue_s(0);
      }
      int s = 0, sn = 1 % Cfg::STAGES;        // stage of tile j, stage of tile j + 1
      uint32_t phn = (Cfg::STAGES == 1) ? 1u : 0u;   // parity of kv_full(sn) for tile j + 1
      for (int j = 0; ok && j < n_kt; ++j) {
        if (j + 1 < n_kt) {
          // QK^T of the NEXT tile goes out as soon as the softmax warps have pulled S of this tile into registers,
          // so it runs in the shadow of their exponentials
          if (!mbar_wait(kv_full(sn), phn, abort_flag, 64u)) break;
          if (!mbar_wait(s_free, (uint32_t)(j & 1), abort_flag, 32u)) break;
          tcgen05_fence_after();
          issue_s(sn);
        }
        if (!mbar_wait(p_full, (uint32_t)(j & 1), abort_flag, 32u)) break;
        tcgen05_fence_after();
        const uint64_t dvs = dv0 + (uint64_t)((s * Cfg::KV_BYTES) >> 4);
        const uint32_t first = j ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < AK / 16; ++kk) {
          // A: P in tensor memory, 16 keys = 8 cells; B: V as stored [key][dim] = MN-major, 16 keys = two 8-key groups
          umma_bf16_ts_elect(tmem_o, tmem_p + (uint32_t)(kk * 8), dvs + (uint64_t)((kk * 16 * Cfg::ROW_BYTES) >> 4), idesc_pv,
                             kk ? 1u : first);
          umma_bf16_ts_elect(tmem_l, tmem_p + (uint32_t)(kk * 8), d10 + (uint64_t)((kk * 16 * 32) >> 4), idesc_l, kk ? 1u : first);
        }
        umma_commit_elect(kv_empty(s));    // K/V stage reusable once these MMAs have read it
        umma_commit_elect(p_free);         // P cells reusable
        s = sn;
        if (++sn == Cfg::STAGES) { sn = 0; phn ^= 1u; }
      }
      umma_commit_elect(o_full);
    }
    __syncwarp();
  } else {
    // ------------------------------ softmax warps (2..9): thread = query row, half of the keys ------------------
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;          // keys [32*CPW*part, +32*CPW) of every tile
    const int r = quad * 32 + lane;            // row inside the tile
    const int qrow = q0 + r;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    bool ok = true;
    for (int j = 0; j < n_kt; ++j) {
      if (!mbar_wait(s_full, (uint32_t)(j & 1), abort_flag)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const bool diag = (j == n_kt - 1);
      // both 32-column loads of this thread's 64 keys go out before one wait; S is then free for the next QK^T
      uint32_t sraw[CPW][32];
#pragma unroll
      for (int cc = 0; cc < CPW; ++cc) tmem_ld_32x32_nowait(tmem_s + lane_off + (uint32_t)((part * CPW + cc) * 32), sraw[cc]);
      tmem_wait_ld();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      uint32_t packed[CPW * 16];     // probabilities as bf16 pairs: cell i = keys 2i (low half), 2i+1 (high half)
#pragma unroll
      for (int cc = 0; cc < CPW; ++cc) {
        const int c = part * CPW + cc;
        const int key0 = j * AK + c * 32;
        // Three separately compiled bodies, chosen by a warp-uniform branch: the common tile carries no mask code at all
        // (as one loop with the mask predicated in, every tile paid two compares and two selects per pair of scores,
        // more than the exponentials themselves cost to issue).
        if (!diag) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(sraw[cc][i]), p.scale_log2, -p.bound_log2));
            const float p1 = ex2_approx(fmaf(__uint_as_float(sraw[cc][i + 1]), p.scale_log2, -p.bound_log2));
            // bf16 by truncation: one byte-permute on the integer pipe instead of a conversion on the special-function
            // pipe.  The truncation bias cancels: the denominator is summed from the same bf16 values.
            packed[cc * 16 + (i >> 1)] = __byte_perm(__float_as_uint(p0), __float_as_uint(p1), 0x7632);
          }
        } else if (c > quad) {       // every key of these 32 lies after every row of this warp: no exponentials needed
#pragma unroll
          for (int i = 0; i < 16; ++i) packed[cc * 16 + i] = 0u;
        } else {                     // the diagonal tile: causal mask
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = ex2_approx(fmaf(__uint_as_float(sraw[cc][i]), p.scale_log2, -p.bound_log2));
            float p1 = ex2_approx(fmaf(__uint_as_float(sraw[cc][i + 1]), p.scale_log2, -p.bound_log2));
            if (key0 + i > qrow) p0 = 0.f;
            if (key0 + i + 1 > qrow) p1 = 0.f;
            packed[cc * 16 + (i >> 1)] = __byte_perm(__float_as_uint(p0), __float_as_uint(p1), 0x7632);
          }
        }
      }
      // the P cells may be overwritten once the PV MMAs of the previous tile have read them
      if (!mbar_wait(p_free, (uint32_t)((j & 1) ^ 1), abort_flag)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      if constexpr (CPW == 2) tmem_st_32x32(tmem_p + lane_off + (uint32_t)(part * 32), reinterpret_cast<const uint32_t(&)[32]>(packed));
      else tmem_st_32x16(tmem_p + lane_off + (uint32_t)(part * 16), packed);
      tmem_wait_st();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- finish: O / l -> bf16, token-major ----
    if (ok && !mbar_wait(o_full, 0u, abort_flag)) ok = false;
    ok = __all_sync(0xffffffffu, ok);
    if (ok && part == 0) {
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

// [heads, S, hd] bf16 tensor, boxes of 128 rows x hd columns of one head, swizzle width = row width; rows past S read
// as zero
static int make_rows_map(CUtensorMap* map, const void* ptr, uint64_t heads, uint64_t S, int hd) {
  auto fn = encode_fn();
  HB_REQUIRE(fn != nullptr, HB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[3] = {(cuuint64_t)hd, S, heads};
  cuuint64_t gstride[2] = {(cuuint64_t)hd * 2, (cuuint64_t)S * hd * 2};
  cuuint32_t box[3] = {(cuuint32_t)hd, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapSwizzle sw = hd == 64 ? CU_TENSOR_MAP_SWIZZLE_128B
                                         : (hd == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  HB_REQUIRE(r == CUDA_SUCCESS, HB200_ERR_CUDA, "cuTensorMapEncodeTiled (attention) failed with CUresult %d", (int)r);
  return 0;
}

template <int HD>
static int launch_att(const void* q, const void* k, const void* v, const AttParams& p, int B, cudaStream_t st) {
  using Cfg = AttCfg<HD>;
  CUtensorMap tq, tk, tv;
  HB_PROPAGATE(make_rows_map(&tq, q, (uint64_t)B * p.H, (uint64_t)p.S, HD));
  HB_PROPAGATE(make_rows_map(&tk, k, (uint64_t)B * p.KV, (uint64_t)p.S, HD));
  HB_PROPAGATE(make_rows_map(&tv, v, (uint64_t)B * p.KV, (uint64_t)p.S, HD));
  auto kern = attention_tcgen05_kernel<HD>;
  HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, (size_t)(Cfg::SMEM_BYTES)));
  dim3 grid(B * p.H, (p.S + AQ - 1) / AQ, 1);
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
