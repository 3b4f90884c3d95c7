// Skinny-M bf16 GEMM for decode (M <= 512 rows, one 128-row tile per grid.y):  C = epilogue(A W^T),  A [M,K], W [N,K],
// both K-major.
//
// With a handful of rows the contraction is bound by streaming W from HBM once, so the work is cut for bandwidth,
// not for tensor throughput: one CTA per (64..128 weight rows, one slice of K), two CTAs per SM, so even a 2048 x 5632
// weight (16 row tiles) keeps 128 CTAs streaming and the CTAs of the next contraction of a chain can move in (and start
// their weight stream) while the current one drains.  Inside a CTA the pipeline is the one of the large GEMM: warp 0 issues TMA loads of
// the A slice (a 64-row box when M <= 64, else 128 rows; rows beyond M are zero-filled by the tensor map and cost no
// traffic) and the W tile [64|96|128 x 64] into a 128B-swizzled 96 KB ring (4-6 stages), warp 1 issues tcgen05.mma
// (M=128, N = tile width, K=16) into a TMEM accumulator, warps 2-5 (one per TMEM lane quadrant) drain it.  With the
// 64-row box the MMA's rows 64..127 read the bytes that follow in the stage (the W tile): finite garbage that lands
// in accumulator rows nobody reads.
//
// Split-K reduction through distributed shared memory: the CTAs that share a row tile form one thread-block cluster
// (2, 4 or 8 CTAs, cluster rank = K slice).  Each parks its fp32 partial in its own shared memory; after a cluster
// barrier every CTA sums one 1/ksplit share of the tile's columns over all peers (ld.shared::cluster, slice order
// fixed, so the result is deterministic) and applies the epilogue to that share.  No global scratch, no atomics.
// Unsplit tiles go straight from TMEM to the epilogue.
//
// Every mbarrier wait is bounded as in the large GEMM (abort flag, err_flag, TMEM freed on the way out); the two
// cluster barriers are on the common path of every thread, so a CTA that gave up still arrives at them.
#include "gemm_epilogue.cuh"
#include "tcgen05.cuh"
#include "tma_host.cuh"

namespace hb200 {

constexpr int SK_BM = 128, SK_BN = 128, SK_BK = 64;
constexpr int SK_MAX_M = 512;              // up to four 128-row tiles (grid.y); beyond that the general kernel is the better fit
constexpr int SK_RING_BYTES = 96 * 1024;   // operand ring: as many stages of (A rows + tile width) x 64 as fit, at most 12
constexpr int SK_MAX_STAGES = 12;
constexpr int SK_CTAS_PER_SM = 2;          // two CTAs share an SM, so the weight prefetch of the next contraction of a chain
                                            // overlaps the tail of the current one
constexpr int SK_THREADS = 6 * 32;          // producer, MMA issuer, 4 epilogue warps
constexpr int SK_SMEM_BYTES = SK_RING_BYTES + 512 + 1024;
constexpr int SK_MIN_KB_PER_SPLIT = 2;
static_assert(SK_BM * SK_BN * 4 <= SK_RING_BYTES, "the fp32 partial reuses the operand ring");
static_assert(8 * (2 * SK_MAX_STAGES + 1) + 16 <= 512, "barrier block");

struct SkinnyPlan {
  int bn, n_tiles, k_blocks, ksplit, kb_per;
};

// Tile width (64 / 96 / 128 weight rows) and K split (1 / 2 / 4 / 8 slices = cluster size) that put the most CTAs on
// the SMs without exceeding one wave; every slice keeps at least two K blocks and every cluster member a column share
// that is a multiple of 16 (the SwiGLU epilogue pairs columns in groups of 16).
static SkinnyPlan skinny_plan(int N, int K) {
  static const int cand[9][2] = {{128, 1}, {128, 2}, {128, 4}, {128, 8}, {96, 1}, {96, 2}, {64, 1}, {64, 2}, {64, 4}};
  const int k_blocks = ceil_div(K, SK_BK), sms = sm_count();
  int best = 0, best_ctas = -1;
  for (int i = 0; i < 9; ++i) {
    const int bn = cand[i][0], ks = cand[i][1];
    if (ks > 1 && k_blocks / ks < SK_MIN_KB_PER_SPLIT) continue;
    const int ctas = ceil_div(N, bn) * ks;
    if (ctas > SK_CTAS_PER_SM * sms) continue;
    if (ctas > best_ctas) { best = i; best_ctas = ctas; }   // earlier candidates (wider tile, fewer slices) win ties
  }
  SkinnyPlan s;
  s.bn = best_ctas < 0 ? 128 : cand[best][0];
  s.ksplit = best_ctas < 0 ? 1 : cand[best][1];
  s.n_tiles = ceil_div(N, s.bn);
  s.k_blocks = k_blocks;
  s.kb_per = ceil_div(k_blocks, s.ksplit);
  return s;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

// Row m of this CTA's column share [c_first, c_first + cw) of the tile: sum the KS partials (all loads of a 16-column
// group in flight at once, then added in slice order) and apply the epilogue.
// For the read-modify-write epilogues the old values of the row segment were requested before the mainloop finished
// (`old`, `grow` = global row); groups that were not prefetched (column tail) take the generic epilogue.
constexpr int SK_MAX_GROUPS = 4;    // column share of a cluster member: at most 64 columns = 4 groups of 16
template <int KS>
__device__ __forceinline__ void reduce_share(const GemmParams& p, uint32_t part_addr, int m, int m_glob, int tile_col0,
                                             int c_first, int cw, long long grow,
                                             const uint4 (&old)[SK_MAX_GROUPS][2]) {
  uint32_t peer[KS];
#pragma unroll
  for (int s = 0; s < KS; ++s) peer[s] = map_to_cta(part_addr + (uint32_t)((c_first * SK_BM + m) * 4), (uint32_t)s);
#pragma unroll
  for (int g = 0; g < SK_MAX_GROUPS; ++g) {
    if (g >= cw / 16) break;
    const int col = tile_col0 + c_first + g * 16;
    if (col >= p.N) break;
    float t[KS][16];
#pragma unroll
    for (int s = 0; s < KS; ++s)
#pragma unroll
      for (int j = 0; j < 16; ++j) t[s][j] = ld_dsmem_f32(peer[s] + (uint32_t)((g * 16 + j) * SK_BM * 4));
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      v[j] = t[0][j];
#pragma unroll
      for (int s = 1; s < KS; ++s) v[j] += t[s][j];
    }
    if (grow >= 0 && col + 16 <= p.N) {
      __nv_bfloat16* dst = p.C + (size_t)grow * p.ldc + col;
#pragma unroll
      for (int h8 = 0; h8 < 2; ++h8) {
        const uint32_t w4[4] = {old[g][h8].x, old[g][h8].y, old[g][h8].z, old[g][h8].w};
        uint4 o;
        uint32_t* ow = &o.x;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float r0 = __uint_as_float(w4[j] << 16), r1 = __uint_as_float(w4[j] & 0xffff0000u);
          ow[j] = pack_bf16x2_rn(r0 + p.alpha * v[h8 * 8 + 2 * j], r1 + p.alpha * v[h8 * 8 + 2 * j + 1]);
        }
        *reinterpret_cast<uint4*>(dst + h8 * 8) = o;
      }
    } else {
      epilogue_row_chunk<16>(p, m_glob, col, v);
    }
  }
}

__global__ void __launch_bounds__(SK_THREADS, SK_CTAS_PER_SM) gemm_skinny_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                                    const __grid_constant__ CUtensorMap tma_b,
                                                                    const GemmParams p, int bn, int a_rows, int ksplit,
                                                                    int kb_per, int k_blocks) {
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t base = (s_addr(smem_dyn) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - s_addr(smem_dyn));
  const uint32_t a_bytes = (uint32_t)a_rows * SK_BK * 2, stage_bytes = a_bytes + (uint32_t)bn * SK_BK * 2;
  const int n_stages = min(SK_MAX_STAGES, SK_RING_BYTES / (int)stage_bytes);
  const uint32_t bars = base + SK_RING_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (SK_MAX_STAGES + s); };
  const uint32_t tfull_bar = bars + 8u * (2 * SK_MAX_STAGES);
  volatile uint32_t* tmem_slot =
      reinterpret_cast<volatile uint32_t*>(base_ptr + SK_RING_BYTES + 8 * (2 * SK_MAX_STAGES + 1));
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* part = reinterpret_cast<float*>(base_ptr);       // [bn columns][SK_BM rows] fp32, over the operand ring
  const uint32_t stage_tx = stage_bytes;                  // bytes one stage receives (out-of-range rows count too)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  chain_release();

  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(s_addr(const_cast<uint32_t*>(tmem_slot)), SK_BN);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Everything so far is independent of earlier kernels, and so are the weights: the producer starts streaming the
  // W tiles of the first ring-full of K blocks before it waits for the predecessor (expect_tx without an arrival
  // keeps each stage's barrier open until the matching A load has been issued).  W must not be written by the
  // preceding kernels of the chain.
  const int nt = blockIdx.x / ksplit, ks = blockIdx.x - nt * ksplit;   // ks == rank in the cluster
  const int m_base = (int)blockIdx.y * SK_BM;                          // 128-row tile of A / C (batches beyond 128 rows)
  const int kb0 = ks * kb_per, kb1_full = min(k_blocks, kb0 + kb_per);
  // a launch site whose rows ran out the last time (a late MoR recursion) most likely has none now either: do not
  // stream weights for it ahead of the wait.  A wrong guess costs the prefetch, nothing else.
  const bool expect_rows = (p.m_hint == nullptr) || (__ldcg(p.m_hint) > (int)blockIdx.y * SK_BM);
  const int pre = expect_rows ? max(0, min(n_stages, kb1_full - kb0)) : 0;
  const uint32_t b_bytes = stage_bytes - a_bytes;
  if (warp == 0 && lane == 0) {
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(full_bar(i), b_bytes);
      tma_load_2d(base + i * stage_bytes + a_bytes, &tma_b, (kb0 + i) * SK_BK, nt * bn, full_bar(i));
    }
  }
  chain_wait();
  // the A slices of the prefetched stages go out before the live row count is even read: if it turns out to be zero
  // the tiles are simply not consumed
  if (warp == 0 && lane == 0) {
    for (int i = 0; i < pre; ++i) {
      mbar_arrive_expect_tx(full_bar(i), a_bytes);
      tma_load_2d(base + i * stage_bytes, &tma_a, (kb0 + i) * SK_BK, m_base, full_bar(i));
    }
  }
  const int M_all = p.m_dev ? min(__ldcg(p.m_dev), p.M) : p.M;
  const int M = min(max(M_all - m_base, 0), SK_BM);                     // live rows of this tile
  if (p.m_hint != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *p.m_hint = M_all;
  const int kb1 = (M > 0) ? kb1_full : kb0;
  const bool has_work = kb1 > kb0;                                      // a trailing slice may be empty

  long long rmw_row = -1;                       // epilogue warps only (see below)
  uint4 rmw_old[SK_MAX_GROUPS][2];
  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      if (!has_work) {
        // no live rows: let the requested tiles land, then leave
        for (int i = 0; i < pre; ++i)
          if (!mbar_wait(full_bar(i), 0u, abort_flag)) break;
      } else {
        int stage = pre % n_stages;
        uint32_t phase = (pre == n_stages) ? 1u : 0u;
        for (int kb = kb0 + pre; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) break;
          const uint32_t sa = base + stage * stage_bytes;
          mbar_arrive_expect_tx(full_bar(stage), stage_tx);
          tma_load_2d(sa, &tma_a, kb * SK_BK, m_base, full_bar(stage));
          tma_load_2d(sa + a_bytes, &tma_b, kb * SK_BK, nt * bn, full_bar(stage));
          if (++stage == n_stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && has_work) {
      const uint32_t idesc = make_idesc(SK_BM, bn);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t sa = base + stage * stage_bytes;
        const uint64_t da = make_smem_desc(sa);
        const uint64_t db = make_smem_desc(sa + a_bytes);
#pragma unroll
        for (int k = 0; k < SK_BK / 16; ++k) umma_bf16(tmem_base, da + 2u * k, db + 2u * k, idesc, (kb > kb0 || k) ? 1u : 0u);
        umma_commit(empty_bar(stage));
        if (++stage == n_stages) { stage = 0; phase ^= 1u; }
      }
      if (ok) umma_commit(tfull_bar);
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue warps (2..5): TMEM -> epilogue, or TMEM -> own partial ----------
    const int quad = warp & 3;
    const int m = quad * 32 + lane;
    bool ok = true;
    // read-modify-write epilogues of split tiles: this thread's row index and the old values of its column share are
    // requested now, so both round trips hide behind the mainloop
    if (ksplit > 1 && (p.epilogue == EPI_RESID || p.epilogue == EPI_SCATTER_ADD) && (p.N % 8 == 0) && m < M) {
      rmw_row = (p.epilogue == EPI_SCATTER_ADD) ? (long long)__ldcg(p.rows + m_base + m) : (long long)(m_base + m);
      const __nv_bfloat16* src = (p.epilogue == EPI_RESID) ? p.resid : p.C;
      const int cw = bn / ksplit;
#pragma unroll
      for (int g = 0; g < SK_MAX_GROUPS; ++g) {
        const int col = nt * bn + ks * cw + g * 16;
        if (g < cw / 16 && col + 16 <= p.N) {
          rmw_old[g][0] = __ldcg(reinterpret_cast<const uint4*>(src + (size_t)rmw_row * p.ldc + col));
          rmw_old[g][1] = __ldcg(reinterpret_cast<const uint4*>(src + (size_t)rmw_row * p.ldc + col + 8));
        }
      }
    }
    if (has_work) {
      if (!mbar_wait(tfull_bar, 0u, abort_flag)) ok = false;      // all MMAs done: the ring is free, TMEM is final
      ok = __all_sync(0xffffffffu, ok);
      tcgen05_fence_after();
    }
    const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16);
    if (ok && quad * 32 < M) {                                     // warp-uniform
      if (ksplit == 1) {
        if (has_work) {
#pragma unroll 1
          for (int c = 0; c < bn / 32; ++c) {
            float v[32];
            tmem_ld_32x32(t_row + (uint32_t)(c * 32), v);
            const int col = nt * bn + c * 32;
            if (m < M && col < p.N) epilogue_row_chunk<32>(p, m_base + m, col, v);
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < bn / 32; ++c) {
          float v[32];
          if (has_work) {
            tmem_ld_32x32(t_row + (uint32_t)(c * 32), v);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) part[(c * 32 + j) * SK_BM + m] = v[j];   // lanes = consecutive rows: no conflicts
        }
      }
    }
    tcgen05_fence_before();
  }

  if (ksplit > 1) {
    // every thread of every CTA of the cluster passes both barriers, whatever happened above
    cluster_sync_all();                                            // all partials are in place
    if (warp >= 2 && *abort_flag == 0u) {
      const int m = (warp & 3) * 32 + lane;
      if (m < M) {
        const int cw = bn / ksplit;                                // this CTA's share of the tile's columns
        if (ksplit == 2) reduce_share<2>(p, s_addr(part), m, m_base + m, nt * bn, ks * cw, cw, rmw_row, rmw_old);
        else if (ksplit == 4) reduce_share<4>(p, s_addr(part), m, m_base + m, nt * bn, ks * cw, cw, rmw_row, rmw_old);
        else reduce_share<8>(p, s_addr(part), m, m_base + m, nt * bn, ks * cw, cw, rmw_row, rmw_old);
      }
    }
    cluster_sync_all();                                            // nobody leaves while a peer may still read it
  }

  // ------------------------------ teardown ------------------------------
  __syncthreads();
  const bool aborted = (*abort_flag != 0u);
  if (aborted) {
    if (threadIdx.x == 0 && p.err_flag != nullptr) atomicExch(p.err_flag, 1);
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  tcgen05_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, SK_BN);
}

int launch_gemm_skinny(const GemmParams& p, cudaStream_t st, bool chained) {
  HB_REQUIRE(p.M >= 1 && p.M <= SK_MAX_M, HB200_ERR_UNSUPPORTED, "skinny gemm: M = %d (1..%d rows)", p.M, SK_MAX_M);
  const SkinnyPlan s = skinny_plan(p.N, p.K);
  CUtensorMap ta, tb;
  const int a_rows = p.M <= 64 ? 64 : SK_BM;
  HB_PROPAGATE(make_tmap(&ta, p.A, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)p.lda, (uint32_t)a_rows));
  HB_PROPAGATE(make_tmap(&tb, p.W, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.ldw, (uint32_t)s.bn));
  HB_PROPAGATE(ensure_dynamic_smem((const void*)gemm_skinny_kernel, (size_t)(SK_SMEM_BYTES)));
  const unsigned m_tiles = (unsigned)((p.M + SK_BM - 1) / SK_BM);     // each streams W again: from L2 after the first
  return launch_chained(gemm_skinny_kernel, dim3((unsigned)(s.n_tiles * s.ksplit), m_tiles), dim3(SK_THREADS), SK_SMEM_BYTES, st,
                        chained, s.ksplit, ta, tb, p, s.bn, a_rows, s.ksplit, s.kb_per, s.k_blocks);
}

}  // namespace hb200
