// Fused CCGQA pre-attention kernel, tcgen05 version (latent 256, kv_dim 64: the 250M-class shapes).
//
//   qkv [B,S,lat+2kvd] (read once)  ->  q [B,H,S,hd], k [B,KV,S,hd], v [B,KV,S,hd]  (written once)
//
// Persistent: one CTA per SM walks over tiles of 124 tokens (one sequence each) and keeps four things in flight at
// once - the input of the NEXT tile on its way from HBM, the two convolutions of the CURRENT tile on the tensor
// cores, the conv weights streaming from L2, and the epilogue of the PREVIOUS accumulators.
//
// Both convolutions are tcgen05.mma contractions over the same operand layout.  A tile's q|k columns sit in shared
// memory as 40 "planes" of 8 channels: plane[c8][row][8 channels], rows 16 bytes apart.  That is the tensor core's
// un-swizzled K-major core-matrix layout with the 8-row groups packed back to back, in which a shift by j rows is a
// shift of the operand's start address by 16*j bytes - so the three taps of a causal k=3 convolution are three
// A-operand descriptors over one tile, no im2col copy:
//   conv1 (grouped, per head):  y1[128 rows, hd]   = sum_j  x [rows j..j+127, head's channels] W1_j^T      K = 3*hd
//   conv2 (dense):              out[128 rows, C]   = sum_j  y1[rows j..j+127, all channels]    W2_j^T      K = 3*C
// y1 row r is token t0-2+r, x row r is token t0-4+r, output row m is token t0+m.  x and y1 hold 128 rows each, and
// the taps of rows near the end read up to two rows past the plane (the first rows of the next plane: finite data),
// so y1 rows 0..125 and output rows 0..123 are exact: 124 tokens per tile, the rest is thrown away.  (At 2048 tokens
// per sequence that is 17 tiles, the same count as 126 would give.)
// Rows before the sequence start are zero in x, hence zero in y1 (no bias): the reference's causal padding of both
// convolutions.  The x planes are written by TMA: one [8 channels x 128 rows] box per plane from a [B][S][C] tensor
// map, whose out-of-range rows (before the sequence, after it) arrive as zeros.
//
// Roles (15 warps):
//   warp 0      weight producer: TMA streams, in consumption order, the conv1 weight of 64 channels at a time (two swizzled
//               boxes), the query conv2 weight in [128 out-channels x 64 K] blocks and the key conv2 weight in [64 x 64]
//               blocks (128B-swizzled, 128-byte rows) through a ring of four 16 KB stages.  The TMA unit works through
//               a box one row at a time, about 1.6 clocks per row whatever its width, so every weight box has the
//               widest rows its layout allows: with 16- or 64-byte rows the unit itself set the pace of the kernel;
//   warp 1      MMA issuer: the whole warp runs the loop with warp-uniform operands and one elected lane issues (a
//               single-lane loop costs ~46 clocks per MMA to issue, this form 24-34, and the conv1 / key MMAs hold less
//               math than that): conv1 in five rounds of 64 channels into a double-buffered 64-column accumulator, then
//               conv2 of the queries (two M128 x N128 halves per K block, one weight stage each) and of the keys (N64);
//   warps 2-5   drain each conv1 round (TMEM -> bf16 -> y1 planes), nothing else on their critical path; between tiles
//               they copy the value columns with the one-token shift;
//   warps 6-13  epilogue, thread = token, two warps per TMEM lane quadrant: + 0.5 * mean key / mean query (summed from
//               the x planes while they are in shared memory), L2 norm, key temperature, RoPE, 64-byte stores - five
//               32-column chunks per warp (queries 0-2 and the keys, or queries 3-7) while the next tile's conv1 runs;
//   warp 14     x loader: as soon as conv1 and the mean readers are done with the x planes, one lane issues the 40 TMA
//               loads of the next tile's planes (a 16-byte-row box is slow to issue, ~230 clocks each, which is why
//               this is nobody else's job); they land while conv2 of the current tile runs.
// The conv2 K blocks of a tile are visited in an order rotated by the tile's position in its sequence: CTAs that run
// side by side then stream different weight blocks instead of all hitting the same L2 lines at once, and the order
// (hence the fp32 summation order) stays a function of the token position alone, so a sequence gives the same bits
// whatever batch it is part of.
//
// TMEM (512 columns): queries at 0, keys at 256, conv1 rounds at 320 / 384.
// Every mbarrier wait is bounded; on expiry the CTA raises its abort flag, every role leaves its loop, the error is
// reported through err_flag, TMEM is released and the kernel returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "common.cuh"
#include "tcgen05.cuh"
#include "tma_host.cuh"

namespace hb200 {

namespace pretc {
constexpr int TT = 124;                  // output tokens per tile
constexpr int MR = 128;                  // rows of every MMA
constexpr int LAT = 256, KVD = 64, C = LAT + KVD;
constexpr int PLANES = C / 8;            // 40 planes of 8 channels
constexpr int XROWS = MR;                // x rows held: tokens t0-4 .. t0+123 (one TMA box of 128 rows per plane)
constexpr int XP_PLANE = XROWS * 16;
constexpr int XP_BYTES = PLANES * XP_PLANE;
constexpr int Y1_PLANE = MR * 16;
constexpr int Y1_BYTES = PLANES * Y1_PLANE;
constexpr int STAGE_BYTES = 16384;
constexpr int STAGES = 4;
constexpr int OFF_RING = 0;
constexpr int OFF_XP = STAGES * STAGE_BYTES;
constexpr int OFF_Y1 = OFF_XP + XP_BYTES;
constexpr int OFF_TAIL = OFF_Y1 + Y1_BYTES;   // 64 zero bytes: the last plane's two overhanging rows
constexpr int OFF_BAR = OFF_TAIL + 64;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
constexpr int ROUND_CH = 64;             // channels per conv1 round
constexpr int ROUNDS = C / ROUND_CH;     // 5
constexpr int QBLOCKS = 2 * (3 * LAT / 64);   // q conv2: 12 K blocks of 64, each as two [128 out-channels x 64 K] stages
constexpr int KBLOCKS = 3 * KVD / 64;    // 3 K blocks of 64 of the k conv2
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_Q = 0, COL_K = 256, COL_C1 = 320;
constexpr int WARPS = 15, THREADS = WARPS * 32;
constexpr int DL_WARP0 = 2, DL_WARPS = 4, DL_THREADS = DL_WARPS * 32;
constexpr int E_WARP0 = 6, X_WARP = 14;
}  // namespace pretc

struct PreTcParams {
  const __nv_bfloat16* qkv;
  const float* cos_t;
  const float* sin_t;
  const float* temp;
  __nv_bfloat16* q;
  __nv_bfloat16* k;
  __nv_bfloat16* v;
  int B, S, H, KV;
  int n_tiles, tiles_per_seq;
  int32_t* err_flag;
};

// In-thread epilogue of one head vector: + coupling, L2 norm, scale, RoPE, 16-byte stores.
template <int HD>
__device__ __forceinline__ void finish_head(const float* acc, const float* couple, float mult, const float* cs,
                                            const float* sn, __nv_bfloat16* dst, bool valid) {
  float v[HD];
  float ss = 0.f;
#pragma unroll
  for (int d = 0; d < HD; ++d) {
    v[d] = acc[d] + couple[d];
    ss += v[d] * v[d];
  }
  // mult / max(|v|, 1e-12): rsqrt of the clamped sum of squares (2 ulp, far inside the bf16 rounding of the result)
  const float inv = mult * rsqrtf(fmaxf(ss, 1e-24f));
  if (!valid) return;
#pragma unroll
  for (int d8 = 0; d8 < HD / 8; ++d8) {
    float o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int pr = d8 * 4 + i;
      const float x0 = v[2 * pr] * inv, x1 = v[2 * pr + 1] * inv;
      o[2 * i] = x0 * cs[pr] - x1 * sn[pr];
      o[2 * i + 1] = x0 * sn[pr] + x1 * cs[pr];
    }
    store_bf16x8(dst + d8 * 8, o);
  }
}

// 0.5 * mean over `heads` head vectors of HD channels, read from the x planes in shared memory: `plane0_row` is the
// address of this token's 16 bytes in the first plane of the channel range, planes are `plane_stride` bytes apart
template <int HD>
__device__ __forceinline__ void head_mean_planes(uint32_t plane0_row, uint32_t plane_stride, int heads, float (&m)[HD]) {
#pragma unroll
  for (int d = 0; d < HD; ++d) m[d] = 0.f;
  const int pieces = heads * HD / 8;
#pragma unroll 1
  for (int i0 = 0; i0 < pieces; i0 += 8) {
    uint4 raw[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) raw[u] = ld_shared_v4(plane0_row + (uint32_t)(i0 + u) * plane_stride);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t w4[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
      const int d0 = (u * 8) % HD;       // i0 is a multiple of 8 pieces = 64 channels, a multiple of HD
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        m[d0 + 2 * jj] += __uint_as_float(w4[jj] << 16);
        m[d0 + 2 * jj + 1] += __uint_as_float(w4[jj] & 0xffff0000u);
      }
    }
  }
  const float s = 0.5f / (float)heads;
#pragma unroll
  for (int d = 0; d < HD; ++d) m[d] *= s;
}

template <int HD>
__global__ void __launch_bounds__(pretc::THREADS, 1) ccgqa_pre_tc_kernel(const __grid_constant__ CUtensorMap tma_x,
                                                                         const __grid_constant__ CUtensorMap tma_w1a,
                                                                         const __grid_constant__ CUtensorMap tma_w1b,
                                                                         const __grid_constant__ CUtensorMap tma_w2q,
                                                                         const __grid_constant__ CUtensorMap tma_w2k,
                                                                         const PreTcParams p) {
  using namespace pretc;
  static_assert(HD == 16 || HD == 32, "head_dim 16 or 32");
  constexpr int QKV_LD = LAT + 2 * KVD;
  // conv1 weight of one round: 64 rows x 3*hd, as two K-major swizzled boxes - taps 0 and 1 (2*hd columns) and tap 2
  // (hd columns); the swizzle width of each is its row width
  constexpr int W1A_ROW = 4 * HD, W1B_ROW = 2 * HD;                 // bytes per row: 128 / 64 (hd 32), 64 / 32 (hd 16)
  constexpr int W1A_BYTES = ROUND_CH * W1A_ROW, W1_BYTES = ROUND_CH * (W1A_ROW + W1B_ROW);
  constexpr uint32_t W1A_LAYOUT = W1A_ROW == 128 ? 2u : 4u, W1B_LAYOUT = W1B_ROW == 64 ? 4u : 6u;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t base = (s_addr(smem_dyn) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - s_addr(smem_dyn));
  const uint32_t xp_addr = base + OFF_XP, y1_addr = base + OFF_Y1;
  const uint32_t bars = base + OFF_BAR;
  auto w_full = [&](int s) { return bars + 8u * s; };
  auto w_empty = [&](int s) { return bars + 32u + 8u * s; };
  const uint32_t xp_full = bars + 64u, y1_full = bars + 72u;
  auto c1_full = [&](int b) { return bars + 80u + 8u * b; };
  auto c1_free = [&](int b) { return bars + 96u + 8u * b; };
  const uint32_t q_full = bars + 112u, q_free = bars + 128u;
  const uint32_t k_full = bars + 144u, k_free = bars + 152u, xp_free = bars + 160u;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + OFF_BAR + 176);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int H = p.H, KV = p.KV, S = p.S;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int my_tiles = (p.n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;   // tiles blockIdx.x + it*gridDim.x

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(w_empty(s), 1);
    }
    mbar_init(xp_full, 1);
    mbar_init(xp_free, 1 + 8);                     // conv1 complete (MMA commit) + the 8 warps that read their means from x
    mbar_init(y1_full, DL_WARPS);
    for (int b = 0; b < 2; ++b) {
      mbar_init(c1_full(b), 1);
      mbar_init(c1_free(b), DL_WARPS);
    }
    mbar_init(q_full, 1);
    mbar_init(q_free, 8);
    mbar_init(k_full, 1);
    mbar_init(k_free, 4);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < 4) reinterpret_cast<uint4*>(base_ptr + OFF_TAIL)[tid] = make_uint4(0u, 0u, 0u, 0u);
  if (warp == 1) tmem_alloc(s_addr(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
  fence_proxy_async_smem();
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ weight producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      auto next_stage = [&]() -> uint32_t {      // waits for the next ring slot, returns its address (0 on abort)
        if (!mbar_wait(w_empty(stage), phase ^ 1u, abort_flag, 64u)) { ok = false; return 0u; }
        return base + OFF_RING + stage * STAGE_BYTES;
      };
      auto advance = [&]() { if (++stage == STAGES) { stage = 0; phase ^= 1u; } };
      for (int it = 0; ok && it < my_tiles; ++it) {
        for (int rd = 0; ok && rd < ROUNDS; ++rd) {                 // conv1 weight of 64 output channels
          const uint32_t dst = next_stage();
          if (!ok) break;
          mbar_arrive_expect_tx(w_full(stage), W1_BYTES);
          tma_load_2d(dst, &tma_w1a, 0, rd * ROUND_CH, w_full(stage));
          tma_load_2d(dst + W1A_BYTES, &tma_w1b, 2 * HD, rd * ROUND_CH, w_full(stage));
          advance();
        }
        const int pos = ((int)blockIdx.x + it * (int)gridDim.x) % p.tiles_per_seq;
        for (int i = 0; ok && i < QBLOCKS; ++i) {                   // conv2 weight of the queries: 128 output channels x 64 K per stage
          const uint32_t dst = next_stage();
          if (!ok) break;
          const int kb = ((i >> 1) + pos * 5) % (QBLOCKS / 2);
          mbar_arrive_expect_tx(w_full(stage), 128 * 64 * 2);
          tma_load_2d(dst, &tma_w2q, kb * 64, (i & 1) * 128, w_full(stage));
          advance();
        }
        for (int kb = 0; ok && kb < KBLOCKS; ++kb) {                // conv2 weight of the keys
          const uint32_t dst = next_stage();
          if (!ok) break;
          mbar_arrive_expect_tx(w_full(stage), KVD * 64 * 2);
          tma_load_2d(dst, &tma_w2k, kb * 64, 0, w_full(stage));
          advance();
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (whole warp, one elected lane issues) ------------------------------
    {
      constexpr uint32_t idesc_c1 = make_idesc(MR, HD);
      constexpr uint32_t idesc_q = make_idesc(MR, 128);
      constexpr uint32_t idesc_k = make_idesc(MR, KVD);
      // descriptor templates; per MMA only the start-address field (16-byte units, low bits) moves
      const uint64_t dx0 = make_smem_desc_ex(xp_addr, 128, 0u, XP_PLANE);           // x planes: 8-row groups 128 B apart
      const uint64_t dy0 = make_smem_desc_ex(y1_addr, 128, 0u, Y1_PLANE);           // y1 planes
      const uint64_t dw1a = make_smem_desc_ex(base + OFF_RING, 8 * W1A_ROW, W1A_LAYOUT, 16);             // conv1 weight, taps 0-1
      const uint64_t dw1b = make_smem_desc_ex(base + OFF_RING + W1A_BYTES, 8 * W1B_ROW, W1B_LAYOUT, 16); // conv1 weight, tap 2
      const uint64_t dwk = make_smem_desc(base + OFF_RING);                         // [64 rows][128 B], 128B swizzle
      int stage = 0;
      uint32_t phase = 0, c1_use[2] = {0u, 0u};
      bool ok = true;
      auto wait_stage = [&]() -> uint32_t {      // returns the stage's offset in 16-byte units
        if (!mbar_wait(w_full(stage), phase, abort_flag)) { ok = false; return 0u; }
        tcgen05_fence_after();
        return (uint32_t)(stage * STAGE_BYTES) >> 4;
      };
      auto release_stage = [&]() {
        umma_commit_elect(w_empty(stage));
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      };
      for (int it = 0; ok && it < my_tiles; ++it) {
        const uint32_t tpar = (uint32_t)(it & 1);
        if (!mbar_wait(xp_full, tpar, abort_flag, 32u)) { ok = false; break; }
        tcgen05_fence_after();
        // ---- conv1: five rounds of 64 channels, each head its own M128 x N=hd x K=3*hd contraction ----
        for (int rd = 0; ok && rd < ROUNDS; ++rd) {
          const int cb = rd & 1;
          const uint32_t so = wait_stage();
          if (!ok) break;
          if (!mbar_wait(c1_free(cb), (c1_use[cb] & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          tcgen05_fence_after();
          const uint64_t dx_rd = dx0 + (uint64_t)((uint32_t)(rd * (ROUND_CH / 8) * XP_PLANE) >> 4);
          const uint64_t dwa_rd = dw1a + (uint64_t)so, dwb_rd = dw1b + (uint64_t)so;
          const uint32_t d_rd = tmem_base + COL_C1 + (uint32_t)(cb * ROUND_CH);
#pragma unroll
          for (int hh = 0; hh < ROUND_CH / HD; ++hh) {
#pragma unroll
            for (int ks = 0; ks < 3 * HD / 16; ++ks) {
              const int j = (ks * 16) / HD, ci0 = (ks * 16) % HD;
              // A: x rows j..j+127 of the 16 input channels hh*HD+ci0.. of this round (two planes)
              const uint32_t a_off = (uint32_t)(((hh * HD + ci0) / 8) * XP_PLANE + j * 16) >> 4;
              // B: this head's rows of the round's weight block; K = 16 ks .. sits in the first box (taps 0, 1) or the second
              const uint64_t db = (ks * 16 < 2 * HD)
                                      ? dwa_rd + (uint64_t)((uint32_t)(hh * HD * W1A_ROW + ks * 32) >> 4)
                                      : dwb_rd + (uint64_t)((uint32_t)(hh * HD * W1B_ROW + (ks * 16 - 2 * HD) * 2) >> 4);
              umma_bf16_elect(d_rd + (uint32_t)(hh * HD), dx_rd + a_off, db, idesc_c1, ks ? 1u : 0u);
            }
          }
          release_stage();
          umma_commit_elect(c1_full(cb));
          ++c1_use[cb];
        }
        if (!ok) break;
        umma_commit_elect(xp_free);              // every conv1 MMA of this tile has read its x planes
        // ---- conv2 ----
        const int pos = ((int)blockIdx.x + it * (int)gridDim.x) % p.tiles_per_seq;   // tile position in its sequence
        if (!mbar_wait(y1_full, tpar, abort_flag, 32u)) { ok = false; break; }
        if (!mbar_wait(q_free, tpar ^ 1u, abort_flag, 32u)) { ok = false; break; }
        tcgen05_fence_after();
        for (int i = 0; ok && i < QBLOCKS; ++i) {
          const uint32_t so = wait_stage();
          if (!ok) break;
          const int kb = ((i >> 1) + pos * 5) % (QBLOCKS / 2);   // rotated start, same order as the producer's
          const int j = (kb * 64) / LAT, ch0 = (kb * 64) % LAT;
          const uint64_t da = dy0 + (uint64_t)((uint32_t)((ch0 / 8) * Y1_PLANE + j * 16) >> 4);
          const uint64_t db = dwk + (uint64_t)so;              // same [rows][128 B] 128B-swizzled form as the key weight
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_bf16_elect(tmem_base + COL_Q + (uint32_t)((i & 1) * 128), da + (uint64_t)((uint32_t)(ks * 2 * Y1_PLANE) >> 4),
                            db + (uint64_t)(ks * 2), idesc_q, ((i >> 1) | ks) ? 1u : 0u);
          release_stage();
        }
        if (!ok) break;
        umma_commit_elect(q_full);
        if (!mbar_wait(k_free, tpar ^ 1u, abort_flag, 32u)) { ok = false; break; }
        tcgen05_fence_after();
        for (int kb = 0; ok && kb < KBLOCKS; ++kb) {
          const uint32_t so = wait_stage();
          if (!ok) break;
          const int j = (kb * 64) / KVD, ch0 = LAT + (kb * 64) % KVD;
          const uint64_t da = dy0 + (uint64_t)((uint32_t)((ch0 / 8) * Y1_PLANE + j * 16) >> 4);
          const uint64_t db = dwk + (uint64_t)so;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_bf16_elect(tmem_base + COL_K, da + (uint64_t)((uint32_t)(ks * 2 * Y1_PLANE) >> 4), db + (uint64_t)(ks * 2), idesc_k,
                            (kb | ks) ? 1u : 0u);
          release_stage();
        }
        if (ok) umma_commit_elect(k_full);
      }
    }
    __syncwarp();
  } else if (warp < E_WARP0) {
    // ------------------ conv1 drain + value shift (warps 2..5) ------------------
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                        // y1 row this thread drains
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const int dt = tid - DL_WARP0 * 32;                    // 0..127
    uint32_t c1_use[2] = {0u, 0u};
    bool ok = true;
    constexpr int VP = KVD / 8;                            // 16-byte pieces of a token's value columns
    constexpr int VPT = (TT * VP + DL_THREADS - 1) / DL_THREADS;   // pieces per thread (8)
    for (int it = 0; ok && it < my_tiles; ++it) {
      const int tile = (int)blockIdx.x + it * (int)gridDim.x;
      const int b = tile / p.tiles_per_seq, t0 = (tile % p.tiles_per_seq) * TT;
      const __nv_bfloat16* qkv_b = p.qkv + (size_t)b * S * QKV_LD;
      for (int rd = 0; rd < ROUNDS; ++rd) {
        const int cb = rd & 1;
        if (!mbar_wait(c1_full(cb), c1_use[cb] & 1u, abort_flag)) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ++c1_use[cb];
        tcgen05_fence_after();
        uint32_t raw[2][32];
        tmem_ld_32x32_nowait(tmem_base + lane_off + COL_C1 + (uint32_t)(cb * ROUND_CH), raw[0]);
        tmem_ld_32x32_nowait(tmem_base + lane_off + COL_C1 + (uint32_t)(cb * ROUND_CH + 32), raw[1]);
        tmem_wait_ld();
        tcgen05_fence_before();
        // 64 channels of this row -> eight 16-byte pieces, one per plane
#pragma unroll
        for (int pc = 0; pc < 8; ++pc) {
          const uint32_t* s8 = &raw[pc >> 2][(pc & 3) * 8];
          uint4 o;
          o.x = pack_bf16x2_rn(__uint_as_float(s8[0]), __uint_as_float(s8[1]));
          o.y = pack_bf16x2_rn(__uint_as_float(s8[2]), __uint_as_float(s8[3]));
          o.z = pack_bf16x2_rn(__uint_as_float(s8[4]), __uint_as_float(s8[5]));
          o.w = pack_bf16x2_rn(__uint_as_float(s8[6]), __uint_as_float(s8[7]));
          st_shared_v4(y1_addr + (uint32_t)(rd * 8 + pc) * Y1_PLANE + (uint32_t)r * 16u, o);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(c1_free(cb));
          if (rd == ROUNDS - 1) mbar_arrive(y1_full);
        }
      }
      if (!ok) break;
      // value shift of this tile (first half of the v channels from this token, second half from the previous one):
      // a plain copy that runs while conv2 keeps the tensor cores busy
      {
        uint4 val[VPT];
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
          const int idx = u * DL_THREADS + dt;
          const int vt = t0 + idx / VP, c = (idx % VP) * 8;
          const int src_tok = (c < KVD / 2) ? vt : vt - 1;
          val[u] = make_uint4(0, 0, 0, 0);
          if (idx < TT * VP && vt < S && src_tok >= 0)
            val[u] = *reinterpret_cast<const uint4*>(qkv_b + (size_t)src_tok * QKV_LD + LAT + KVD + c);
        }
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
          const int idx = u * DL_THREADS + dt;
          const int vt = t0 + idx / VP, c = (idx % VP) * 8;
          if (idx < TT * VP && vt < S)
            *reinterpret_cast<uint4*>(p.v + (((size_t)b * KV + c / HD) * S + vt) * HD + (c % HD)) = val[u];
        }
      }
    }
  } else if (warp < X_WARP) {
    // ------------------------------ epilogue warps (6..13): thread = token ------------------------------
    // Ten 32-column chunks per tile and lane quadrant - eight of the query accumulator, two of the key accumulator,
    // which is complete last.  Warps 6-9 take query chunks 0-2 and then the keys, warps 10-13 query chunks 3-7.
    const int quad = warp & 3;
    const int half = (warp - E_WARP0) >> 2;
    const int r = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const float temp = *p.temp;
    bool ok = true;
    for (int it = 0; it < my_tiles; ++it) {
      const uint32_t tpar = (uint32_t)(it & 1);
      const int tile = (int)blockIdx.x + it * (int)gridDim.x;
      const int b = tile / p.tiles_per_seq, t0 = (tile % p.tiles_per_seq) * TT;
      const int tok = t0 + r;
      const bool valid = r < TT && tok < S;
      float km[HD], qm[HD], cs[HD / 2], sn[HD / 2];
#pragma unroll
      for (int i = 0; i < HD / 2; i += 4) {
        const float4 c4 = valid ? *reinterpret_cast<const float4*>(p.cos_t + (size_t)tok * (HD / 2) + i) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 s4 = valid ? *reinterpret_cast<const float4*>(p.sin_t + (size_t)tok * (HD / 2) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        cs[i] = c4.x; cs[i + 1] = c4.y; cs[i + 2] = c4.z; cs[i + 3] = c4.w;
        sn[i] = s4.x; sn[i + 1] = s4.y; sn[i + 2] = s4.z; sn[i + 3] = s4.w;
      }
      if (!mbar_wait(xp_full, tpar, abort_flag, 64u)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      // the means come from the x planes while they are in shared memory (x row of output row r is r + 4; rows past
      // 127 belong to no token): queries are coupled with the mean key (planes 32..39), keys with the mean query
      const uint32_t xrow = xp_addr + (uint32_t)((r + 4) & (XROWS - 1)) * 16u;
      head_mean_planes<HD>(xrow + (uint32_t)(LAT / 8) * XP_PLANE, XP_PLANE, KV, km);
      if (half == 0) head_mean_planes<HD>(xrow, XP_PLANE, H, qm);
      __syncwarp();
      if (lane == 0) mbar_arrive(xp_free);
      if (!mbar_wait(q_full, tpar, abort_flag, 64u)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int c_begin = half == 0 ? 0 : 3, c_end = half == 0 ? 3 : 8;
#pragma unroll 1
      for (int c = c_begin; c < c_end; ++c) {
        float v[32];
        tmem_ld_32x32(tmem_base + lane_off + COL_Q + (uint32_t)(c * 32), v);   // warp-collective
#pragma unroll
        for (int hh = 0; hh < 32 / HD; ++hh) {
          const int h = (c * 32) / HD + hh;
          finish_head<HD>(v + hh * HD, km, 1.0f, cs, sn, p.q + (((size_t)b * H + h) * S + tok) * HD, valid);
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_free);
      if (half != 0) continue;
      if (!mbar_wait(k_full, tpar, abort_flag, 64u)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
#pragma unroll 1
      for (int c = 0; c < KVD / 32; ++c) {
        float v[32];
        tmem_ld_32x32(tmem_base + lane_off + COL_K + (uint32_t)(c * 32), v);   // warp-collective
#pragma unroll
        for (int hh = 0; hh < 32 / HD; ++hh) {
          const int h = (c * 32) / HD + hh;
          finish_head<HD>(v + hh * HD, qm, temp, cs, sn, p.k + (((size_t)b * KV + h) * S + tok) * HD, valid);
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(k_free);
    }
  } else {
    // ------------------------------ x loader (warp 14) ------------------------------
    if (lane == 0) {
      for (int it = 0; it < my_tiles; ++it) {
        // the planes may be overwritten once conv1 of the previous tile and its mean readers are done with them
        if (it > 0 && !mbar_wait(xp_free, (uint32_t)((it - 1) & 1), abort_flag, 256u)) break;
        const int tile = (int)blockIdx.x + it * (int)gridDim.x;
        const int b = tile / p.tiles_per_seq, t0 = (tile % p.tiles_per_seq) * TT;
        mbar_arrive_expect_tx(xp_full, XP_BYTES);
#pragma unroll 1
        for (int pl = 0; pl < PLANES; ++pl) tma_load_3d(xp_addr + (uint32_t)pl * XP_PLANE, &tma_x, pl * 8, t0 - 4, b, xp_full);
      }
    }
    __syncwarp();
  }

  // ------------------------------ teardown ------------------------------
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag != 0u) {
    if (tid == 0 && p.err_flag != nullptr) atomicExch(p.err_flag, 3);
    const uint64_t ts = global_timer_ns();
    while (global_timer_ns() - ts < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  tcgen05_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, pretc::TMEM_COLS);
}

// ---- host side ---------------------------------------------------------------------------------------------------
// 2-D bf16 map over a row-major [rows, cols] weight, box [box_rows, box_cols]
static int make_weight_map(CUtensorMap* map, const void* ptr, int rows, int cols, int box_rows, int box_cols,
                           CUtensorMapSwizzle swizzle) {
  auto fn = get_encode_fn();
  HB_REQUIRE(fn != nullptr, HB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  HB_REQUIRE(r == CUDA_SUCCESS, HB200_ERR_CUDA, "cuTensorMapEncodeTiled (conv weight) failed with CUresult %d", (int)r);
  return 0;
}

// Returns HB200_ERR_UNSUPPORTED (error text untouched) for shapes this kernel is not built for.
int launch_ccgqa_pre_tc(const void* qkv, const void* w1_qk, const void* w2_q, const void* w2_k, const float* cos_t,
                        const float* sin_t, const float* key_temperature, void* q, void* k, void* v, int B, int S, int H,
                        int KV, int hd, int32_t* err_flag, cudaStream_t st) {
  using namespace pretc;
  if (H * hd != LAT || KV * hd != KVD || H == KV || (hd != 16 && hd != 32)) return HB200_ERR_UNSUPPORTED;
  CUtensorMap tx, t1a, t1b, tq, tk;
  {
    // qkv as [B][S][lat+2kvd]: boxes of 8 channels x 128 rows of one sequence, un-swizzled -> one x plane each
    auto fn = get_encode_fn();
    HB_REQUIRE(fn != nullptr, HB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t gdim[3] = {(cuuint64_t)(LAT + 2 * KVD), (cuuint64_t)S, (cuuint64_t)B};
    cuuint64_t gstride[2] = {(cuuint64_t)(LAT + 2 * KVD) * 2, (cuuint64_t)S * (LAT + 2 * KVD) * 2};
    cuuint32_t box[3] = {8, (cuuint32_t)XROWS, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(qkv), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    HB_REQUIRE(r == CUDA_SUCCESS, HB200_ERR_CUDA, "cuTensorMapEncodeTiled (qkv planes) failed with CUresult %d", (int)r);
  }
  // conv1 weight [C, 3*hd]: per round of 64 rows one box of the first two taps and one of the third, swizzle = row width
  HB_PROPAGATE(make_weight_map(&t1a, w1_qk, C, 3 * hd, ROUND_CH, 2 * hd, hd == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B));
  HB_PROPAGATE(make_weight_map(&t1b, w1_qk, C, 3 * hd, ROUND_CH, hd, hd == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B));
  // conv2 weights [C_out, 3*C_in]: blocks of 128 (queries) / 64 (keys) rows x 64 K, 128-byte swizzle
  HB_PROPAGATE(make_weight_map(&tq, w2_q, LAT, 3 * LAT, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B));
  HB_PROPAGATE(make_weight_map(&tk, w2_k, KVD, 3 * KVD, KVD, 64, CU_TENSOR_MAP_SWIZZLE_128B));
  const int tiles_per_seq = (S + TT - 1) / TT;
  const int n_tiles = B * tiles_per_seq;
  PreTcParams p{(const __nv_bfloat16*)qkv, cos_t, sin_t, key_temperature, (__nv_bfloat16*)q, (__nv_bfloat16*)k,
                (__nv_bfloat16*)v, B, S, H, KV, n_tiles, tiles_per_seq, err_flag};
  const int grid = n_tiles < sm_count() ? n_tiles : sm_count();
  if (hd == 32) {
    auto kern = ccgqa_pre_tc_kernel<32>;
    HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, (size_t)(SMEM_BYTES)));
    kern<<<grid, THREADS, SMEM_BYTES, st>>>(tx, t1a, t1b, tq, tk, p);
  } else {
    auto kern = ccgqa_pre_tc_kernel<16>;
    HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, (size_t)(SMEM_BYTES)));
    kern<<<grid, THREADS, SMEM_BYTES, st>>>(tx, t1a, t1b, tq, tk, p);
  }
  HB_LAUNCH_CHECK();
  return 0;
}

}  // namespace hb200
