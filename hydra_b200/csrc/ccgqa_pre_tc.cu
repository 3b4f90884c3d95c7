// Fused CCGQA pre-attention kernel, tcgen05 version (latent 256, kv_dim 64: the 250M-class shapes).
//
//   qkv [B,S,lat+2kvd] (read once)  ->  q [B,H,S,hd], k [B,KV,S,hd], v [B,KV,S,hd]  (written once)
//
// One CTA = 128 tokens of one sequence (+ a 4-token causal halo).
//   phase 1 (all 8 warps)
//     - the q|k columns of tokens t0-4 .. t0+141 go to shared memory (zero outside the sequence);
//     - conv1 (grouped k=3 causal conv, 1/9 of the FLOPs) per head on mma.sync; its bf16 result y1 is written to
//       shared memory in the tensor core's un-swizzled K-major "core matrix" layout with the 8-row groups packed
//       back to back: [16-byte channel chunk][row][8 channels].  In that layout a shift by j rows is a shift of
//       the operand's start address by 16*j bytes, so the three taps of the dense conv are three A-operand
//       descriptors over the same tile - no im2col copy.
//   phase 2 (warp-specialised)
//     - warp 0: TMA producer streaming the repacked conv2 weight [C_out, 3*C_in] (128B-swizzled 64-wide K blocks)
//       through a 4-stage ring that re-uses the shared memory of the phase-1 input tile;
//     - warp 1: one thread issues tcgen05.mma M128 x N256 x K16 (q) and M128 x N64 x K16 (k): conv2 is a
//       [128, 768] x [768, 256] contraction per tile with fp32 accumulators in TMEM;
//     - warps 2-3: value shift (first half of the v channels from this token, second half from the previous one),
//       a pure copy global -> global that overlaps the contraction;
//     - warps 4-7: epilogue, thread = token.  While the MMAs run each thread computes the QK-mean vectors of its
//       token from its qkv row (L2-resident) and fetches its RoPE row; then per head: tcgen05.ld of the head's
//       32 accumulator columns, + 0.5*mean, L2 norm (in-thread, no shuffles), key temperature, RoPE, 64-byte store.
//
// Every mbarrier wait is bounded; on expiry the CTA flags the error, frees its TMEM and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "common.cuh"
#include "mma.cuh"
#include "tcgen05.cuh"

namespace hb200 {

namespace pretc {
constexpr int TT = 128;                  // output tokens per tile
constexpr int LAT = 256, KVD = 64, C = LAT + KVD;
constexpr int YROWS = 144;               // y1 rows computed (t0-2 .. t0+141): nine m16 tiles, 130 are needed
constexpr int XROWS = YROWS + 2;         // x rows held (t0-4 .. t0+141)
constexpr int LDX = C + 8;               // padded x row (bf16 elements): conflict-free fragment loads
constexpr int CHUNKS = C / 8;            // 16-byte channel chunks of y1
constexpr int CHUNK_BYTES = YROWS * 16;  // one chunk: all rows, 16 bytes each
constexpr int STAGE_BYTES = 256 * 64 * 2;   // one conv2 weight block: 256 rows x 64 K (k-conv blocks use 8 KB of it)
constexpr int STAGES = 4;
constexpr int RING_BYTES = STAGES * STAGE_BYTES;          // 128 KB; its first 96 KB hold x during phase 1
constexpr int Y1_BYTES = CHUNKS * CHUNK_BYTES;            // 90 KB
constexpr int OFF_Y1 = RING_BYTES;
constexpr int OFF_BAR = OFF_Y1 + Y1_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
static_assert(XROWS * LDX * 2 <= 3 * STAGE_BYTES, "x tile must fit in the first three ring stages");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
constexpr int QBLOCKS = 3 * LAT / 64;    // 12 K blocks of the q conv2
constexpr int KBLOCKS = 3 * KVD / 64;    // 3 K blocks of the k conv2
constexpr uint32_t TMEM_COLS = 512;      // q accumulator 0..255, k accumulator 256..319
}  // namespace pretc

struct PreTcParams {
  const __nv_bfloat16* qkv;
  const __nv_bfloat16* w1;   // [lat+kvd][3*hd]
  const float* cos_t;
  const float* sin_t;
  const float* temp;
  __nv_bfloat16* q;
  __nv_bfloat16* k;
  __nv_bfloat16* v;
  int B, S, H, KV;
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
  const float inv = mult / fmaxf(sqrtf(ss), 1e-12f);
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

template <int HD>
__global__ void __launch_bounds__(256, 1) ccgqa_pre_tc_kernel(const __grid_constant__ CUtensorMap tma_w2q,
                                                              const __grid_constant__ CUtensorMap tma_w2k,
                                                              const PreTcParams p) {
  using namespace pretc;
  static_assert(HD == 16 || HD == 32, "head_dim 16 or 32");
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t base = (s_addr(smem_dyn) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - s_addr(smem_dyn));
  __nv_bfloat16* X = reinterpret_cast<__nv_bfloat16*>(base_ptr);                 // [XROWS][LDX], phase 1 only
  __nv_bfloat16* Y1 = reinterpret_cast<__nv_bfloat16*>(base_ptr + OFF_Y1);        // [CHUNKS][YROWS][8]
  const uint32_t y1_addr = base + OFF_Y1;
  const uint32_t bars = base + OFF_BAR;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 32u + 8u * s; };
  const uint32_t acc_full = bars + 64u;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + OFF_BAR + 72);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int H = p.H, KV = p.KV, S = p.S;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int tiles_per_seq = (S + TT - 1) / TT;
  const int b = blockIdx.x / tiles_per_seq;
  const int t0 = (blockIdx.x % tiles_per_seq) * TT;
  constexpr int QKV_LD = LAT + 2 * KVD;
  const __nv_bfloat16* qkv_b = p.qkv + (size_t)b * S * QKV_LD;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // the first weight block starts its trip now: ring slot i lives in physical stage (i + 3) % 4, and the last
    // physical stage is the one the input tile does not occupy during phase 1
    mbar_arrive_expect_tx(full_bar(0), LAT * 64 * 2);
    tma_load_2d(base + (STAGES - 1) * STAGE_BYTES, &tma_w2q, 0, 0, full_bar(0));
  }
  if (warp == 1) tmem_alloc(s_addr(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);

  // ---------------- phase 1a: q|k columns of the tile -> shared memory ----------------
  // every 16-byte piece is its own asynchronous copy (23 per thread, all in flight at once: one memory latency for the
  // whole tile instead of one per batch of register-staged loads); rows outside the sequence are zero
  {
    constexpr int PIECES = XROWS * (C / 8);
    const uint32_t x_s = s_addr(X);
    for (int idx = tid; idx < PIECES; idx += 256) {
      const int r = idx / (C / 8), piece = idx % (C / 8);
      const int tok = t0 - 4 + r;
      const uint32_t dst = x_s + (uint32_t)(r * LDX + piece * 8) * 2u;
      if (tok >= 0 && tok < S) cp_async16(dst, qkv_b + (size_t)tok * QKV_LD + piece * 8);
      else st_shared_v4(dst, make_uint4(0u, 0u, 0u, 0u));
    }
    cp_async16_commit();
    cp_async16_wait_all();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // ---------------- phase 1b: conv1 (grouped) on mma.sync: y1 row r <-> token t0-2+r ----------------
  // Work units are (head, m16 tile), head-major; each warp takes a contiguous range, so it changes head at most
  // twice and keeps the head's whole weight block (3*hd x hd) in registers as B fragments: the inner loop touches
  // shared memory only (the 61 KB weight would not survive in the little L1 left beside 224 KB of shared memory).
  {
    constexpr int NT1 = HD / 8, KS1 = 3 * HD / 16, MT = YROWS / 16;
    const int units = MT * (H + KV);
    const int u_begin = (units * warp) / 8, u_end = (units * (warp + 1)) / 8;
    uint32_t bfrag[KS1][NT1][2];
    int cur_head = -1;
    for (int u = u_begin; u < u_end; ++u) {
      const int hg = u / MT, mt = u % MT;
      const int cb = hg * HD;
      if (hg != cur_head) {
        cur_head = hg;
#pragma unroll
        for (int ks = 0; ks < KS1; ++ks)
#pragma unroll
          for (int nt = 0; nt < NT1; ++nt) {
            const __nv_bfloat16* wr = p.w1 + (size_t)(cb + nt * 8 + g) * (3 * HD) + ks * 16 + 2 * t4;
            bfrag[ks][nt][0] = __ldg(reinterpret_cast<const unsigned int*>(wr));
            bfrag[ks][nt][1] = __ldg(reinterpret_cast<const unsigned int*>(wr + 8));
          }
      }
      float acc[NT1][4];
#pragma unroll
      for (int i = 0; i < NT1; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS1; ++ks) {
        const int kk0 = ks * 16;
        const int j = kk0 / HD, c0 = kk0 % HD;
        const __nv_bfloat16* r0 = X + (mt * 16 + g + j) * LDX + cb + c0 + 2 * t4;
        const __nv_bfloat16* r1 = r0 + 8 * LDX;
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(r0);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(r1);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(r0 + 8);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(r1 + 8);
#pragma unroll
        for (int nt = 0; nt < NT1; ++nt) mma_bf16_16816(acc[nt], a0, a1, a2, a3, bfrag[ks][nt][0], bfrag[ks][nt][1]);
      }
      // C fragment (row, cols 2t..2t+1 of n-tile nt) -> chunk (cb/8 + nt), row, element 2t
#pragma unroll
      for (int nt = 0; nt < NT1; ++nt) {
        __nv_bfloat16* y = Y1 + (size_t)(cb / 8 + nt) * (YROWS * 8) + (mt * 16 + g) * 8 + 2 * t4;
        *reinterpret_cast<uint32_t*>(y) = pack_bf16x2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<uint32_t*>(y + 8 * 8) = pack_bf16x2(acc[nt][2], acc[nt][3]);
      }
    }
  }
  // y1 was written through the generic proxy and is read by the tensor core; x is about to be overwritten by TMA
  fence_proxy_async_smem();
  __syncthreads();

  // ---------------- phase 2: warp-specialised ----------------
  // epilogue geometry: thread = token r of the tile, for warp w and warp w + 4 alike (TMEM lane quarter w % 4)
  const int quad = warp & 3;
  const int r = quad * 32 + lane;
  const int tok = t0 + r;
  const bool valid = tok < S;
  const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
  float qm[HD], km[HD], cs[HD / 2], sn[HD / 2];
  if (warp == 0) {
    if (lane == 0) {
      int stage = 1;                                   // block 0 was issued at kernel start
      uint32_t phase = 0;
      for (int kb = 1; kb < QBLOCKS + KBLOCKS; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) break;
        const uint32_t dst = base + ((stage + STAGES - 1) % STAGES) * STAGE_BYTES;
        if (kb < QBLOCKS) {
          mbar_arrive_expect_tx(full_bar(stage), LAT * 64 * 2);
          tma_load_2d(dst, &tma_w2q, kb * 64, 0, full_bar(stage));
        } else {
          mbar_arrive_expect_tx(full_bar(stage), KVD * 64 * 2);
          tma_load_2d(dst, &tma_w2k, (kb - QBLOCKS) * 64, 0, full_bar(stage));
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_q = make_idesc(128, LAT);
      constexpr uint32_t idesc_k = make_idesc(128, KVD);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; ok && kb < QBLOCKS + KBLOCKS; ++kb) {
        if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const bool is_q = kb < QBLOCKS;
        const int kq = is_q ? kb : kb - QBLOCKS;
        const int cin = is_q ? LAT : KVD;
        const int j = (kq * 64) / cin;                         // conv tap of this K block
        const int ch0 = (kq * 64) % cin + (is_q ? 0 : LAT);    // first y1 channel of this K block
        const uint32_t sb = base + ((stage + STAGES - 1) % STAGES) * STAGE_BYTES;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          // A: y1 rows j..j+127, 16 channels = two 16-byte chunks CHUNK_BYTES apart; 8-row groups are 128 B apart
          const uint32_t a_addr = y1_addr + (uint32_t)((ch0 + ks * 16) / 8) * CHUNK_BYTES + (uint32_t)j * 16u;
          const uint64_t da = make_smem_desc_ex(a_addr, 128, 0u, CHUNK_BYTES);
          const uint64_t db = make_smem_desc(sb + ks * 32);
          if (is_q)
            umma_bf16(tmem_base, da, db, idesc_q, (kq | ks) ? 1u : 0u);
          else
            umma_bf16(tmem_base + 256u, da, db, idesc_k, (kq | ks) ? 1u : 0u);
        }
        umma_commit(empty_bar(stage));
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (ok) umma_commit(acc_full);
    }
    __syncwarp();
  } else if (warp < 4) {
    // ---- value shift: warps 2,3 copy 128 tokens x 128 bytes as 16-byte pieces, 16 loads in flight per thread ----
    const int vt = tid - 64;                       // 0..63
    constexpr int VP = KVD / 8;                    // pieces per token
#pragma unroll 1
    for (int i0 = 0; i0 < TT * VP; i0 += 64 * 16) {
      uint4 val[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int idx = i0 + u * 64 + vt;
        const int tok = t0 + idx / VP, c = (idx % VP) * 8;
        const int src_tok = (c < KVD / 2) ? tok : tok - 1;
        val[u] = make_uint4(0, 0, 0, 0);
        if (tok < S && src_tok >= 0)
          val[u] = *reinterpret_cast<const uint4*>(qkv_b + (size_t)src_tok * QKV_LD + LAT + KVD + c);
      }
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int idx = i0 + u * 64 + vt;
        const int tok = t0 + idx / VP, c = (idx % VP) * 8;
        if (tok < S)
          *reinterpret_cast<uint4*>(p.v + (((size_t)b * KV + c / HD) * S + tok) * HD + (c % HD)) = val[u];
      }
    }
  } else {
    // ---- warps 4..7 prepare the per-token vectors of the epilogue while the contraction runs ----
    // QK-mean vectors of this token (0.5 * mean over heads), straight from its qkv row
#pragma unroll
    for (int d = 0; d < HD; ++d) qm[d] = km[d] = 0.f;
    if (valid) {
      const __nv_bfloat16* row = qkv_b + (size_t)tok * QKV_LD;
      // 32 + 8 sixteen-byte pieces; piece i covers channels 8i..8i+7 = dims (8i mod HD).. of head 8i / HD
#pragma unroll
      for (int i0 = 0; i0 < LAT / 8; i0 += 8) {
        uint4 raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) raw[u] = *reinterpret_cast<const uint4*>(row + (i0 + u) * 8);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const uint32_t w4[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
          const int d0 = ((i0 + u) * 8) % HD;
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            qm[d0 + 2 * jj] += __uint_as_float(w4[jj] << 16);
            qm[d0 + 2 * jj + 1] += __uint_as_float(w4[jj] & 0xffff0000u);
          }
        }
      }
      {
        uint4 raw[KVD / 8];
#pragma unroll
        for (int u = 0; u < KVD / 8; ++u) raw[u] = *reinterpret_cast<const uint4*>(row + LAT + u * 8);
#pragma unroll
        for (int u = 0; u < KVD / 8; ++u) {
          const uint32_t w4[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
          const int d0 = (u * 8) % HD;
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            km[d0 + 2 * jj] += __uint_as_float(w4[jj] << 16);
            km[d0 + 2 * jj + 1] += __uint_as_float(w4[jj] & 0xffff0000u);
          }
        }
      }
    }
    const float sq = 0.5f / (float)H, sk = 0.5f / (float)KV;
#pragma unroll
    for (int d = 0; d < HD; ++d) { qm[d] *= sq; km[d] *= sk; }
#pragma unroll
    for (int i = 0; i < HD / 2; ++i) {
      cs[i] = valid ? p.cos_t[(size_t)tok * (HD / 2) + i] : 1.f;
      sn[i] = valid ? p.sin_t[(size_t)tok * (HD / 2) + i] : 0.f;
    }
  }

  // ---------------- epilogue: all 8 warps, thread = token, the ten 32-column chunks split 5 + 5 ----------------
  // Warps 0-3 are done with their roles by now (the producer long before).  Warps 4-7 hand their token's vectors to
  // warps 0-3 through the weight ring, which is idle once the accumulators are complete.
  {
    const float temp = *p.temp;
    bool ok = mbar_wait(acc_full, 0u, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    tcgen05_fence_after();
    float* hand = reinterpret_cast<float*>(base_ptr);        // [2*HD + HD][128] floats: field-major, token-minor
    if (warp >= 4) {
#pragma unroll
      for (int d = 0; d < HD; ++d) { hand[d * TT + r] = qm[d]; hand[(HD + d) * TT + r] = km[d]; }
#pragma unroll
      for (int i = 0; i < HD / 2; ++i) { hand[(2 * HD + i) * TT + r] = cs[i]; hand[(2 * HD + HD / 2 + i) * TT + r] = sn[i]; }
    }
    __syncthreads();
    if (warp < 4) {
#pragma unroll
      for (int d = 0; d < HD; ++d) { qm[d] = hand[d * TT + r]; km[d] = hand[(HD + d) * TT + r]; }
#pragma unroll
      for (int i = 0; i < HD / 2; ++i) { cs[i] = hand[(2 * HD + i) * TT + r]; sn[i] = hand[(2 * HD + HD / 2 + i) * TT + r]; }
    }
    if (ok) {
      constexpr int QCH = LAT / 32, KCH = KVD / 32, HALF = (QCH + KCH) / 2;
      const int c_begin = warp >= 4 ? 0 : HALF, c_end = warp >= 4 ? HALF : QCH + KCH;
#pragma unroll 1
      for (int c = c_begin; c < c_end; ++c) {
        float v[32];
        if (c < QCH) {
          // queries: LAT accumulator columns = H heads of HD
          tmem_ld_32x32(tmem_base + lane_off + (uint32_t)(c * 32), v);   // warp-collective
#pragma unroll
          for (int hh = 0; hh < 32 / HD; ++hh) {
            const int h = c * (32 / HD) + hh;
            finish_head<HD>(v + hh * HD, km, 1.0f, cs, sn, p.q + (((size_t)b * H + h) * S + tok) * HD, valid);
          }
        } else {
          // keys: KVD columns at 256..
          const int ck = c - QCH;
          tmem_ld_32x32(tmem_base + lane_off + (uint32_t)(256 + ck * 32), v);
#pragma unroll
          for (int hh = 0; hh < 32 / HD; ++hh) {
            const int h = ck * (32 / HD) + hh;
            finish_head<HD>(v + hh * HD, qm, temp, cs, sn, p.k + (((size_t)b * KV + h) * S + tok) * HD, valid);
          }
        }
      }
    }
  }

  // ---------------- teardown ----------------
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
static PFN_cuTensorMapEncodeTiled_v12000 pre_encode_fn() {
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

// repacked conv2 weight [rows, 3*cin] bf16, blocks of `rows` x 64 K, 128-byte swizzle
static int make_w2_map(CUtensorMap* map, const void* ptr, int rows, int cin) {
  auto fn = pre_encode_fn();
  HB_REQUIRE(fn != nullptr, HB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[2] = {(cuuint64_t)3 * cin, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)3 * cin * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  HB_REQUIRE(r == CUDA_SUCCESS, HB200_ERR_CUDA, "cuTensorMapEncodeTiled (conv2 weight) failed with CUresult %d", (int)r);
  return 0;
}

// Returns HB200_ERR_UNSUPPORTED (error text untouched) for shapes this kernel is not built for.
int launch_ccgqa_pre_tc(const void* qkv, const void* w1_qk, const void* w2_q, const void* w2_k, const float* cos_t,
                        const float* sin_t, const float* key_temperature, void* q, void* k, void* v, int B, int S, int H,
                        int KV, int hd, int32_t* err_flag, cudaStream_t st) {
  using namespace pretc;
  if (H * hd != LAT || KV * hd != KVD || H == KV || (hd != 16 && hd != 32)) return HB200_ERR_UNSUPPORTED;
  CUtensorMap tq, tk;
  HB_PROPAGATE(make_w2_map(&tq, w2_q, LAT, LAT));
  HB_PROPAGATE(make_w2_map(&tk, w2_k, KVD, KVD));
  PreTcParams p{(const __nv_bfloat16*)qkv, (const __nv_bfloat16*)w1_qk, cos_t, sin_t, key_temperature,
                (__nv_bfloat16*)q, (__nv_bfloat16*)k, (__nv_bfloat16*)v, B, S, H, KV, err_flag};
  const int tiles = B * ((S + TT - 1) / TT);
  if (hd == 32) {
    auto kern = ccgqa_pre_tc_kernel<32>;
    HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, (size_t)(SMEM_BYTES)));
    kern<<<tiles, 256, SMEM_BYTES, st>>>(tq, tk, p);
  } else {
    auto kern = ccgqa_pre_tc_kernel<16>;
    HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, (size_t)(SMEM_BYTES)));
    kern<<<tiles, 256, SMEM_BYTES, st>>>(tq, tk, p);
  }
  HB_LAUNCH_CHECK();
  return 0;
}

}  // namespace hb200
