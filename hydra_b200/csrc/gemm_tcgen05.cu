// Persistent, warp-specialised bf16 GEMM for sm_100a:  C = epilogue(A W^T),  A [M,K], W [N,K] (both K-major).
//
//   warp 0      TMA producer: cp.async.bulk.tensor 2D loads of 128x64 (A) and BNx64 (W) tiles into a ring of
//               128B-swizzled shared-memory stages, completion on "full" mbarriers;
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16, kind::f16, fp32 accumulate in TMEM),
//               tcgen05.commit releases smem stages ("empty") and publishes finished accumulators ("tmem_full");
//   warps 2-9   epilogue: two warps per TMEM lane quadrant, each owning half of the tile's columns; tcgen05.ld of
//               32 lanes x 32 columns, fused epilogue, then "tmem_empty".  Plain-store and SwiGLU results are staged
//               per warp in 128B-swizzled shared memory and written with TMA bulk tensor stores (fully coalesced,
//               asynchronous, clipped at the matrix edge by the tensor map); the residual and scatter-add epilogues
//               read-modify-write their rows directly with 16-byte accesses.
//
// CTA pairs (PAIR; the 256-column tiles of the MLP and vocabulary projections): two CTAs of one cluster share a
// 256 x 256 tile.  Each stages its own 128 rows of A and HALF of the tile's W rows per K block; CTA 0 issues one
// tcgen05.mma.cta_group::2 (M = 256) per K step, which reads both CTAs' shared memory and writes each CTA's 128 rows into
// that CTA's own tensor memory; both CTAs' loads are counted on CTA 0's stage barrier, tcgen05.commit signals the stage
// and accumulator barriers of both, and the epilogue warps of both report to CTA 0.  A stage is 32 KB instead of 48 KB
// per SM - a third less shared-memory and L2 traffic per FLOP and six stages instead of four - which measured 5-11 %
// faster on the down and vocabulary projections (and lets the SMs hold a higher clock under the power cap); the
// epilogues are per CTA and unchanged.
//
// TMEM holds two BN-column accumulators so the epilogue of tile i overlaps the mainloop of tile i+1.  The live
// row count may come from device memory (MoD/MoR compaction), in which case the tile loop bounds are computed
// in-kernel and no host synchronisation is needed.
//
// GATHER variant (the MLP's first contraction behind MoD / MoR routing): A is not a compact matrix but the rows
// a_rows[0..M) of a larger one.  Four extra warps then fill the A half of every stage themselves - tile row = 8 lanes,
// 16 bytes each per 64-column block, cp.async into the same 128B-swizzled layout TMA would have written - and the
// SwiGLU epilogue applies the per-row norm scale and per-column bias, so the normalised rows never exist in memory.
// A gather thread never waits for its copies: cp.async.mbarrier.arrive.noinc makes the stage's barrier count them in
// when they land, next to the TMA transaction count of the W half, so all stages stay in flight as with TMA.  The
// copies are generic-proxy writes; the MMA thread orders them before its tensor-core (async-proxy) reads with a
// fence.proxy.async after it has acquired the barrier.
//
// Every mbarrier wait is bounded (wall-clock limit via %globaltimer): on expiry the CTA raises an abort flag that
// all roles poll, reports through err_flag, lets copies in flight land, frees its TMEM and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "gemm_epilogue.cuh"
#include "tcgen05.cuh"
#include "tma_host.cuh"

namespace hb200 {

constexpr int GBM = 128;            // tile rows  (UMMA M)
constexpr int GBK = 64;             // K per stage = one 128-byte swizzle span of bf16
constexpr int GROUP_M_DEFAULT = 16; // m-tiles per rasterisation group (keeps an A panel L2-resident)
constexpr int EPI_WARPS = 8;        // two per TMEM lane quadrant
constexpr int GEMM_THREADS = (2 + EPI_WARPS) * 32;
constexpr int GATHER_WARPS = 4;     // GATHER variant: 128 threads, 8 lanes per tile row and 64-column block
constexpr int GEMM_THREADS_GATHER = GEMM_THREADS + GATHER_WARPS * 32;


// NSTAGES = 0 selects the default ring depth for the tile width; a shallow ring (2 stages, 128-wide tiles) leaves
// room for two CTAs per SM, which is what the short-K, epilogue-bound contractions want (o_proj: K = 256).
template <int BN, int NSTAGES = 0> struct GemmCfg {
  static constexpr int A_BYTES = GBM * GBK * 2;
  static constexpr int B_BYTES = BN * GBK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = NSTAGES > 0 ? NSTAGES : ((BN == 384) ? 3 : ((BN == 256) ? 4 : 6));
  static constexpr int CTAS_PER_SM = (NSTAGES > 0 && NSTAGES <= 2 && BN == 128) ? 2 : 1;
  // 384-wide tiles (a whole qkv projection row block: A is fetched once instead of three times) fill most of TMEM,
  // so they run with a single accumulator; narrower tiles double-buffer it
  static constexpr int ACCS = (BN == 384) ? 1 : 2;
  static constexpr int TMEM_COLS = (BN == 384) ? 512 : 2 * BN;
  static constexpr int B_BOX_ROWS = (BN > 256) ? 128 : BN;             // a TMA box holds at most 256 rows
  static constexpr int BAR_BYTES = 256;
  static constexpr int STORE_BOX_BYTES = 32 * 128;                 // one TMA store box: 32 rows x 64 bf16
  static constexpr int STORE_BYTES = EPI_WARPS * STORE_BOX_BYTES;  // one staging box per epilogue warp
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STORE_BYTES + BAR_BYTES + 1024;   // + alignment slack
};

// CTA pair (cta_group::2): a 256-row x BN tile per pair of CTAs of one cluster.  Each CTA stages its own 128 rows of A
// and HALF of the tile's W rows per K block (32 KB per stage instead of 48 KB: the tensor cores of both SMs read the W
// halves from each other's shared memory), which leaves room for six stages.
// 384-column tiles (the qkv projection) as a pair: one MMA of N = 256 and one of N = 128 per K step, as in the single-CTA
// form; a CTA's half of the W rows is then rows [128 rank, +128) of the tile for the first and [256 + 64 rank, +64) for
// the second, fetched as three boxes of 64 rows.
template <int BN> struct GemmCfgPair {
  static constexpr int A_BYTES = GBM * GBK * 2;
  static constexpr int B_BYTES = (BN / 2) * GBK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = BN == 384 ? 4 : 6;
  static constexpr int CTAS_PER_SM = 1;
  static constexpr int ACCS = BN == 384 ? 1 : 2;
  static constexpr int TMEM_COLS = 512;
  static constexpr int B_BOX_ROWS = BN == 384 ? 64 : BN / 2;
  static constexpr int BAR_BYTES = 256;
  static constexpr int STORE_BOX_BYTES = 32 * 128;
  static constexpr int STORE_BYTES = EPI_WARPS * STORE_BOX_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STORE_BYTES + BAR_BYTES + 1024;
  static_assert(BN == 256 || BN == 384, "the pair kernel is built for 256- and 384-column tiles");
};

// tile index -> (m_tile, n_tile): groups of group_m m-tiles, n outer / m inner inside a group
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int group_m, int& mt, int& nt) {
  const int per_group = group_m * n_tiles;
  const int grp = tile / per_group;
  const int first_m = grp * group_m;
  const int gm = min(group_m, m_tiles - first_m);
  const int in = tile - grp * per_group;
  nt = in / gm;
  mt = first_m + in % gm;
}

template <int BN, int NSTAGES, bool GATHER = false, bool PAIR = false>
__global__ void __launch_bounds__(GATHER ? GEMM_THREADS_GATHER : GEMM_THREADS, (PAIR ? 1 : GemmCfg<BN, NSTAGES>::CTAS_PER_SM)) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                              const __grid_constant__ CUtensorMap tma_b,
                                                              const __grid_constant__ CUtensorMap tma_c,
                                                              const GemmParams p, const int group_m) {
  using Cfg = std::conditional_t<PAIR, GemmCfgPair<(PAIR && BN == 384) ? 384 : 256>, GemmCfg<BN, NSTAGES>>;
  static_assert(!(PAIR && GATHER), "the gathered form is single-CTA");
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t base = (s_addr(smem_dyn) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - s_addr(smem_dyn));
  const uint32_t store_base = base + Cfg::STAGES * Cfg::STAGE_BYTES;   // 1024-byte aligned
  const uint32_t bars = store_base + Cfg::STORE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (Cfg::STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * Cfg::STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * Cfg::STAGES + 2 + a); };
  volatile uint32_t* tmem_slot =
      reinterpret_cast<volatile uint32_t*>(base_ptr + Cfg::STAGES * Cfg::STAGE_BYTES + Cfg::STORE_BYTES +
                                           8 * (2 * Cfg::STAGES + 4));
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int M = p.m_dev ? min(*p.m_dev, p.M) : p.M;
  // PAIR: the work item is a 256-row tile of the pair; CTA `rank` of the pair owns its rows rank*128 .. rank*128+127
  const uint32_t rank = PAIR ? cluster_cta_rank() : 0u;
  const int cta_first = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;      // first work item of this CTA (pair)
  const int cta_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int m_tiles = PAIR ? (M + 2 * GBM - 1) / (2 * GBM) : (M + GBM - 1) / GBM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = (p.K + GBK - 1) / GBK;
  // Work items = tiles, except in the last, partial wave: when the tiles left over after the full waves would occupy at
  // most half of the CTAs, each of them is split into its two 128-column halves, so that the tail of the launch costs
  // half a tile time instead of a whole one (the scatter-add contraction of the MLP has 5.4 waves of tiles at the
  // benchmark's row counts).  Not for the SwiGLU epilogue, whose output boxes pair columns across the whole tile.
  const int full_items = (total_tiles / (int)gridDim.x) * (int)gridDim.x;
  const int rem_tiles = total_tiles - full_items;
  const bool split_tail = BN == 256 && !GATHER && !PAIR && p.epilogue != EPI_SWIGLU && rem_tiles > 0 && 2 * rem_tiles <= (int)gridDim.x;
  const int total_items = split_tail ? full_items + 2 * rem_tiles : total_tiles;
  auto item_tile = [&](int w, int& tile, int& col_off, int& ncols) {
    if (split_tail && w >= full_items) {
      tile = full_items + ((w - full_items) >> 1);
      col_off = ((w - full_items) & 1) * 128;
      ncols = 128;
    } else {
      tile = w;
      col_off = 0;
      ncols = BN;
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      // TMA transaction (+ every gather thread); PAIR: both CTAs' producers arrive on CTA 0's barrier
      mbar_init(full_bar(s), GATHER ? 1 + GATHER_WARPS * 32 : (PAIR ? 2 : 1));
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < Cfg::ACCS; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), PAIR ? 2 * EPI_WARPS : EPI_WARPS);      // PAIR: the epilogue warps of both CTAs, on CTA 0's
    }
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (PAIR) tmem_alloc_pair(s_addr(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
    else tmem_alloc(s_addr(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
  }
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_barrier_all();     // the peer's barriers are initialised before anything signals them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = cta_first; ok && w < total_items; w += cta_step) {
        int tile, col_off, ncols, mt, nt;
        item_tile(w, tile, col_off, ncols);
        tile_coords(tile, m_tiles, n_tiles, group_m, mt, nt);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t sa = base + stage * Cfg::STAGE_BYTES;
          if constexpr (PAIR) {
            // this CTA's 128 rows of A and its half of the W rows, counted on the barrier of the pair's CTA 0
            const uint32_t full0 = cluster_map_shared(full_bar(stage), 0u);
            mbar_arrive_expect_tx_cluster(full0, Cfg::STAGE_BYTES);
            tma_load_2d_pair(sa, &tma_a, kb * GBK, (2 * mt + (int)rank) * GBM, full0);
            if constexpr (BN == 384) {
              const uint32_t sb = sa + Cfg::A_BYTES;
              tma_load_2d_pair(sb, &tma_b, kb * GBK, nt * BN + (int)rank * 128, full0);
              tma_load_2d_pair(sb + 64 * GBK * 2, &tma_b, kb * GBK, nt * BN + (int)rank * 128 + 64, full0);
              tma_load_2d_pair(sb + 128 * GBK * 2, &tma_b, kb * GBK, nt * BN + 256 + (int)rank * 64, full0);
            } else {
              tma_load_2d_pair(sa + Cfg::A_BYTES, &tma_b, kb * GBK, nt * BN + (int)rank * Cfg::B_BOX_ROWS, full0);
            }
          } else {
            mbar_arrive_expect_tx(full_bar(stage), GATHER ? Cfg::B_BYTES : Cfg::STAGE_BYTES);
            if constexpr (!GATHER) tma_load_2d(sa, &tma_a, kb * GBK, mt * GBM, full_bar(stage));
#pragma unroll
            for (int bb = 0; bb < BN / Cfg::B_BOX_ROWS; ++bb)
              tma_load_2d(sa + Cfg::A_BYTES + bb * Cfg::B_BOX_ROWS * GBK * 2, &tma_b, kb * GBK,
                          nt * BN + bb * Cfg::B_BOX_ROWS, full_bar(stage));
          }
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && rank == 0u) {                     // PAIR: CTA 0 issues for both
      constexpr uint32_t idesc = make_idesc(PAIR ? 2 * GBM : GBM, BN > 256 ? 256 : BN);
      constexpr uint32_t idesc_tail = make_idesc(PAIR ? 2 * GBM : GBM, BN > 256 ? BN - 256 : 16);   // columns beyond one MMA's 256
      int stage = 0, as = 0;
      uint32_t phase = 0, aphase = 0;
      bool ok = true;
      for (int w = cta_first; ok && w < total_items; w += cta_step) {
        int tile, col_off, ncols;
        item_tile(w, tile, col_off, ncols);
        const uint32_t idesc_w = (ncols == BN) ? idesc : make_idesc(GBM, 128);   // a half tile: N = 128
        if (!mbar_wait(tempty_bar(as), aphase ^ 1u, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          if constexpr (GATHER) fence_proxy_async_smem();   // the A half was written by cp.async (generic proxy)
          tcgen05_fence_after();
          const uint32_t sa = base + stage * Cfg::STAGE_BYTES;
          const uint64_t da = make_smem_desc(sa);
          const uint64_t db = make_smem_desc(sa + Cfg::A_BYTES + (uint32_t)col_off * (GBK * 2));   // W rows col_off..
#pragma unroll
          for (int k = 0; k < GBK / 16; ++k) {
            // advance 16 elements (32 bytes) along K inside the swizzle span: +2 in 16-byte units
            if constexpr (PAIR) umma_bf16_pair(d_tmem, da + 2u * k, db + 2u * k, idesc_w, (kb | k) ? 1u : 0u);
            else umma_bf16(d_tmem, da + 2u * k, db + 2u * k, idesc_w, (kb | k) ? 1u : 0u);
            if constexpr (BN > 256) {
              // B rows 256.. start 256 rows x 128 bytes further on; their accumulator columns follow the first 256
              // (PAIR: this CTA's share of those rows follows its 128 rows of the first MMA)
              const uint64_t db_tail = make_smem_desc(sa + Cfg::A_BYTES + (PAIR ? 128 : 256) * GBK * 2);
              if constexpr (PAIR) umma_bf16_pair(d_tmem + 256u, da + 2u * k, db_tail + 2u * k, idesc_tail, (kb | k) ? 1u : 0u);
              else umma_bf16(d_tmem + 256u, da + 2u * k, db_tail + 2u * k, idesc_tail, (kb | k) ? 1u : 0u);
            }
          }
          // stage reusable once these MMAs have read it (PAIR: in both CTAs)
          if constexpr (PAIR) {
            umma_commit_pair(empty_bar(stage));
            umma_commit_pair(cluster_map_shared(empty_bar(stage), 1u));
          } else {
            umma_commit(empty_bar(stage));
          }
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if constexpr (PAIR) {              // accumulator complete, in both CTAs' tensor memory
          umma_commit_pair(tfull_bar(as));
          umma_commit_pair(cluster_map_shared(tfull_bar(as), 1u));
        } else {
          umma_commit(tfull_bar(as));
        }
        if (++as == Cfg::ACCS) { as = 0; aphase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (GATHER && warp >= 2 + EPI_WARPS) {
    // ------------------------------ A gather warps (10..13) ------------------------------
    // warp w covers tile rows 32w..32w+31; per 64-column block an instruction copies 4 rows x 128 bytes (8 lanes per
    // row), eight instructions per block.  Rows past the live count are zero-filled (source size 0).
    const int gw = warp - (2 + EPI_WARPS);
    const int sub = lane >> 3, piece = lane & 7;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_items; tile += gridDim.x) {   // (no split tail in this variant)
      int mt, nt;
      tile_coords(tile, m_tiles, n_tiles, group_m, mt, nt);
      const int m_lane = mt * GBM + gw * 32 + lane;
      const int my_row = m_lane < M ? __ldg(p.a_rows + m_lane) : -1;       // A row of tile row 32*gw + lane
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, 96u)) { ok = false; break; }   // sleeps, does not spin
        const uint32_t sa = base + stage * Cfg::STAGE_BYTES;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = i * 4 + sub;                                      // row inside this warp's 32
          const int src_row = __shfl_sync(0xffffffffu, my_row, rr);
          const int tr = gw * 32 + rr;                                     // tile row
          const uint32_t dst = sa + (uint32_t)((tr >> 3) * 1024 + (tr & 7) * 128 + ((piece ^ (tr & 7)) << 4));
          const int col = kb * GBK + piece * 8;
          const bool in = src_row >= 0 && col < p.K;
          const void* src = in ? (const void*)(p.A + (size_t)src_row * p.lda + col) : (const void*)p.A;
          const int nbytes = in ? 16 : 0;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(nbytes) : "memory");
        }
        // arrives on the stage's barrier once this thread's copies above have landed (no increment of the pending
        // count: the barrier was initialised expecting one such arrival per gather thread)
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(full_bar(stage)) : "memory");
        if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
    cp_async16_wait_all();      // nothing of this thread's is still in flight when the CTA tears down
  } else {
    // ------------------------------ epilogue warps (2..9) ------------------------------
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;          // which half of the tile's columns this warp drains
    constexpr int CHUNKS_FULL = BN / 32 / (EPI_WARPS / 4);
    const bool swiglu = (p.epilogue == EPI_SWIGLU);
    const bool tma_store = (p.epilogue == EPI_STORE) || swiglu;
    const bool rmw = !tma_store && (p.N % 8 == 0);   // residual / scatter-add with whole 16-byte pieces
    const int n_out = swiglu ? p.N / 2 : p.N;
    const uint32_t my_box = store_base + (uint32_t)(warp - 2) * Cfg::STORE_BOX_BYTES;
    int as = 0;
    uint32_t aphase = 0;
    bool ok = true;
    for (int w = cta_first; ok && w < total_items; w += cta_step) {
      int tile, col_off, ncols, mt, nt;
      item_tile(w, tile, col_off, ncols);
      tile_coords(tile, m_tiles, n_tiles, group_m, mt, nt);
      if constexpr (PAIR) mt = 2 * mt + (int)rank;     // this CTA's 128 rows of the pair's tile
      const int CHUNKS = (ncols == BN) ? CHUNKS_FULL : 128 / 32 / (EPI_WARPS / 4);   // 32-column chunks this warp drains
      const int col_base = nt * BN + col_off;                                        // first output column of the item
      const int m = mt * GBM + quad * 32 + lane;
      float row_scale = 1.0f;                    // norm scale of this thread's row (GATHER SwiGLU form)
      if (p.row_scale != nullptr && m < M) row_scale = __ldg(p.row_scale + __ldg(p.a_rows + m));
      // Read-modify-write epilogues (residual, scatter-add).  The accumulator comes out of TMEM with thread = row, but
      // rows are 2 KB or more apart in memory, so row-per-thread 16-byte accesses would touch 32 partial sectors per
      // request.  Instead the warp's staging box (32 rows x 64 columns, 128B-swizzled) is the meeting point: the old
      // values are fetched with eight lanes per row (whole 128-byte lines, cp.async, issued BEFORE the accumulator
      // wait so the latency hides behind the mainloop), each thread then updates its own row inside the box, and the
      // box leaves again with eight lanes per row.
      const int RMW_BOXES = CHUNKS * 32 / 64;
      const int rmw_col0 = col_base + half * CHUNKS * 32;
      long long grow = -1;                       // global row this lane's tile row reads / writes, -1 = none
      const __nv_bfloat16* rmw_src = (p.epilogue == EPI_RESID) ? p.resid : p.C;
      auto rmw_fetch = [&](int bx) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int rr = it * 4 + (lane >> 3), piece = lane & 7;
          const long long gr = __shfl_sync(0xffffffffu, grow, rr);
          const int col = rmw_col0 + bx * 64 + piece * 8;
          if (gr >= 0 && col < p.N)
            cp_async16(my_box + (uint32_t)(rr * 128 + ((piece ^ (rr & 7)) << 4)), rmw_src + (size_t)gr * p.ldc + col);
        }
        cp_async16_commit();
      };
      if (rmw) {
        if (m < M) grow = (p.epilogue == EPI_SCATTER_ADD) ? (long long)p.rows[m] : (long long)m;
        rmw_fetch(0);
      }
      if (!mbar_wait(tfull_bar(as), aphase, abort_flag)) { ok = false; }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(as * BN);
      if (tma_store) {
        // ---- staged path: 64 output columns per box, one box in flight per warp ----
        constexpr int ACC_PER_BOX = 64;                       // accumulator columns feeding one box (plain store)
        const int acc_per_box = swiglu ? 2 * ACC_PER_BOX : ACC_PER_BOX;
        const int boxes = CHUNKS * 32 / acc_per_box;
        for (int bx = 0; bx < boxes; ++bx) {
          const int acc0 = half * CHUNKS * 32 + bx * acc_per_box;      // first accumulator column of the box
          if (lane == 0) bulk_wait_read0();                            // previous box has left shared memory
          __syncwarp();
          const uint32_t row_smem = my_box + (uint32_t)lane * 128u;
          for (int c = 0; c < acc_per_box / 32; ++c) {
            float v[32];
            tmem_ld_32x32(t_row + (uint32_t)(acc0 + c * 32), v);       // warp-collective
            if (swiglu && p.row_scale != nullptr) {
              // pre-MLP norm folded in: inv_rms[row] * (acc + bias[col]) is what the activation sees
              const int col0 = col_base + acc0 + c * 32;
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4) {
                const float4 b4 = (col0 + q4 * 4 < p.N) ? __ldg(reinterpret_cast<const float4*>(p.col_bias + col0 + q4 * 4))
                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
                v[q4 * 4 + 0] = row_scale * (v[q4 * 4 + 0] + b4.x);
                v[q4 * 4 + 1] = row_scale * (v[q4 * 4 + 1] + b4.y);
                v[q4 * 4 + 2] = row_scale * (v[q4 * 4 + 2] + b4.z);
                v[q4 * 4 + 3] = row_scale * (v[q4 * 4 + 3] + b4.w);
              }
            }
            if (swiglu) {
#pragma unroll
              for (int h16 = 0; h16 < 2; ++h16) {
                uint4 o;
                o.x = pack_bf16x2_rn(silu_mul(v[h16 * 16 + 0], v[h16 * 16 + 8]), silu_mul(v[h16 * 16 + 1], v[h16 * 16 + 9]));
                o.y = pack_bf16x2_rn(silu_mul(v[h16 * 16 + 2], v[h16 * 16 + 10]), silu_mul(v[h16 * 16 + 3], v[h16 * 16 + 11]));
                o.z = pack_bf16x2_rn(silu_mul(v[h16 * 16 + 4], v[h16 * 16 + 12]), silu_mul(v[h16 * 16 + 5], v[h16 * 16 + 13]));
                o.w = pack_bf16x2_rn(silu_mul(v[h16 * 16 + 6], v[h16 * 16 + 14]), silu_mul(v[h16 * 16 + 7], v[h16 * 16 + 15]));
                const int piece = c * 2 + h16;                         // 16-byte piece inside the 128-byte row
                st_shared_v4(row_smem + (uint32_t)((piece ^ (lane & 7)) << 4), o);
              }
            } else {
#pragma unroll
              for (int q8 = 0; q8 < 4; ++q8) {
                uint4 o;
                o.x = pack_bf16x2_rn(p.alpha * v[q8 * 8 + 0], p.alpha * v[q8 * 8 + 1]);
                o.y = pack_bf16x2_rn(p.alpha * v[q8 * 8 + 2], p.alpha * v[q8 * 8 + 3]);
                o.z = pack_bf16x2_rn(p.alpha * v[q8 * 8 + 4], p.alpha * v[q8 * 8 + 5]);
                o.w = pack_bf16x2_rn(p.alpha * v[q8 * 8 + 6], p.alpha * v[q8 * 8 + 7]);
                const int piece = c * 4 + q8;
                st_shared_v4(row_smem + (uint32_t)((piece ^ (lane & 7)) << 4), o);
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int out_col = swiglu ? (col_base + acc0) / 2 : col_base + acc0;
            if (out_col < n_out) {
              tma_store_2d(&tma_c, out_col, mt * GBM + quad * 32, my_box);
              bulk_commit();
            }
          }
        }
      } else if (rmw) {
#pragma unroll 1
        for (int bx = 0; bx < RMW_BOXES; ++bx) {
          cp_async16_wait_all();
          __syncwarp();                                            // every lane's pieces of the box have landed
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            float v[32];
            tmem_ld_32x32(t_row + (uint32_t)(half * CHUNKS * 32 + bx * 64 + c2 * 32), v);   // warp-collective
            if (grow >= 0) {
#pragma unroll
              for (int q8 = 0; q8 < 4; ++q8) {
                const int piece = c2 * 4 + q8;
                if (rmw_col0 + bx * 64 + piece * 8 < p.N) {
                  const uint32_t addr = my_box + (uint32_t)(lane * 128 + ((piece ^ (lane & 7)) << 4));
                  const uint4 old4 = ld_shared_v4(addr);
                  const uint32_t w4[4] = {old4.x, old4.y, old4.z, old4.w};
                  uint4 o;
                  uint32_t* ow = &o.x;
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float r0 = __uint_as_float(w4[j] << 16), r1 = __uint_as_float(w4[j] & 0xffff0000u);
                    ow[j] = pack_bf16x2_rn(r0 + p.alpha * v[q8 * 8 + 2 * j], r1 + p.alpha * v[q8 * 8 + 2 * j + 1]);
                  }
                  st_shared_v4(addr, o);
                }
              }
            }
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + (lane >> 3), piece = lane & 7;
            const long long gr = __shfl_sync(0xffffffffu, grow, rr);
            const int col = rmw_col0 + bx * 64 + piece * 8;
            if (gr >= 0 && col < p.N)
              *reinterpret_cast<uint4*>(p.C + (size_t)gr * p.ldc + col) =
                  ld_shared_v4(my_box + (uint32_t)(rr * 128 + ((piece ^ (rr & 7)) << 4)));
          }
          __syncwarp();                                            // the box is free again
          if (bx + 1 < RMW_BOXES) rmw_fetch(bx + 1);
        }
      } else {
        // generic fallback (column counts that are not a multiple of 8)
#pragma unroll 1
        for (int c = half * CHUNKS; c < (half + 1) * CHUNKS; ++c) {
          float v[32];
          tmem_ld_32x32(t_row + (uint32_t)(c * 32), v);   // warp-collective
          const int col = col_base + c * 32;
          if (m < M && col < p.N) epilogue_row_chunk<32>(p, m, col, v);
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(cluster_map_shared(tempty_bar(as), 0u));
        else mbar_arrive(tempty_bar(as));
      }
      if (++as == Cfg::ACCS) { as = 0; aphase ^= 1u; }
    }
    if (lane == 0) bulk_wait0();   // this thread's bulk stores have completed before the CTA may exit
    __syncwarp();
  }

  // ------------------------------ teardown ------------------------------
  __syncthreads();
  const bool aborted = (*abort_flag != 0u);
  if (aborted) {
    if (threadIdx.x == 0 && p.err_flag != nullptr) atomicExch(p.err_flag, 1);
    // give copies / MMAs in flight time to land before the shared memory and TMEM are released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  tcgen05_fence_after();
  if constexpr (PAIR) {
    // nobody leaves while the peer's tensor core may still read this CTA's shared memory or signal its barriers; every
    // thread of both CTAs reaches this barrier whatever happened above
    cluster_barrier_all();
    if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  } else {
    if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---- host side -----------------------------------------------------------------------------------------------
template <int BN, int NSTAGES = 0, bool GATHER = false>
static int launch_bn(const GemmParams& p, cudaStream_t st) {
  using Cfg = GemmCfg<BN, NSTAGES>;
  CUtensorMap ta, tb, tc;
  // (the gathered form never issues a TMA load of A; the map only has to be a valid one)
  HB_PROPAGATE(make_tmap(&ta, p.A, (uint64_t)(GATHER ? GBM : p.M), (uint64_t)p.K, (uint64_t)p.lda, GBM));
  HB_PROPAGATE(make_tmap(&tb, p.W, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.ldw, Cfg::B_BOX_ROWS));
  if (p.epilogue == EPI_STORE || p.epilogue == EPI_SWIGLU) {
    // output map for the staged TMA-store epilogue: boxes of 32 rows x 64 columns, clipped at [M, n_out]
    const uint64_t n_out = p.epilogue == EPI_SWIGLU ? (uint64_t)p.N / 2 : (uint64_t)p.N;
    HB_PROPAGATE(make_tmap(&tc, p.C, (uint64_t)p.M, n_out, (uint64_t)p.ldc, 32, CU_TENSOR_MAP_L2_PROMOTION_NONE));
  } else {
    tc = ta;   // unused by the direct epilogues
  }
  auto kern = gemm_tcgen05_kernel<BN, NSTAGES, GATHER>;
  HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, (size_t)(Cfg::SMEM_BYTES)));
  const int64_t tiles = (int64_t)ceil_div(p.M, GBM) * ceil_div(p.N, BN);
  const int grid = (int)std::min<int64_t>(tiles, (int64_t)sm_count() * Cfg::CTAS_PER_SM);
  // Rasterisation group: the weight matrix is re-streamed once per group of m-tiles, so when it is too large to
  // stay in L2 next to the output stream (the vocabulary projection: 103 MB) a taller group cuts its HBM re-reads;
  // the group's A panel (group_m x 128 rows x K) must itself stay L2-resident (<= 16 MB).
  int group_m = GROUP_M_DEFAULT;
  if ((size_t)p.N * p.K * 2 > (size_t)48 << 20) group_m = (int)std::max<size_t>(16, std::min<size_t>(64, ((size_t)16 << 20) / ((size_t)GBM * p.K * 2)));
  kern<<<grid, GATHER ? GEMM_THREADS_GATHER : GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(ta, tb, tc, p, group_m);
  HB_LAUNCH_CHECK();
  return 0;
}

// CTA-pair form of the 256-column kernel: clusters of two CTAs, one 256 x 256 tile per pair.
template <int BN>
static int launch_pair(const GemmParams& p, cudaStream_t st) {
  using Cfg = GemmCfgPair<BN>;
  CUtensorMap ta, tb, tc;
  HB_PROPAGATE(make_tmap(&ta, p.A, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)p.lda, GBM));
  HB_PROPAGATE(make_tmap(&tb, p.W, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.ldw, Cfg::B_BOX_ROWS));
  if (p.epilogue == EPI_STORE || p.epilogue == EPI_SWIGLU) {
    const uint64_t n_out = p.epilogue == EPI_SWIGLU ? (uint64_t)p.N / 2 : (uint64_t)p.N;
    HB_PROPAGATE(make_tmap(&tc, p.C, (uint64_t)p.M, n_out, (uint64_t)p.ldc, 32, CU_TENSOR_MAP_L2_PROMOTION_NONE));
  } else {
    tc = ta;
  }
  auto kern = gemm_tcgen05_kernel<BN, 0, false, true>;
  HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, (size_t)(Cfg::SMEM_BYTES)));
  const int64_t tiles = (int64_t)ceil_div(p.M, 2 * GBM) * ceil_div(p.N, BN);
  const int pairs = (int)std::min<int64_t>(tiles, (int64_t)(sm_count() / 2));
  int group_m = GROUP_M_DEFAULT / 2;       // in 256-row tiles
  if ((size_t)p.N * p.K * 2 > (size_t)48 << 20)
    group_m = (int)std::max<size_t>(8, std::min<size_t>(32, ((size_t)16 << 20) / ((size_t)2 * GBM * p.K * 2)));
  return launch_chained(kern, dim3(2 * pairs), dim3(GEMM_THREADS), (size_t)Cfg::SMEM_BYTES, st, false, 2, ta, tb, tc, p, group_m);
}

int launch_gemm_tcgen05(const GemmParams& p, cudaStream_t st) {
  // 256-column tiles run as CTA pairs (below) unless HB200_GEMM_PAIR=0 asks for the single-CTA kernel
  static const bool pair_on = [] {
    const char* e = getenv("HB200_GEMM_PAIR");
    return e == nullptr || e[0] != '0';
  }();
  if (p.a_rows != nullptr) {
    // gathered A: the MLP's gate_up contraction with the norm folded in
    HB_REQUIRE(p.epilogue == EPI_SWIGLU && p.row_scale != nullptr && p.col_bias != nullptr && p.K % 8 == 0, HB200_ERR_INVALID,
               "gemm: gathered A is built for the SwiGLU epilogue with row scale and column bias");
    return launch_bn<256, 0, true>(p, st);
  }
  // wide tiles unless N is a small multiple of 128 (qkv projection: 384); the SwiGLU epilogue pairs columns inside
  // 128-column halves of a 256-wide tile and always takes the wide kernel
  // a 384-column projection (qkv of the 8q/2kv and 16q/4kv shapes at latent 256) as one tile per row block: the A
  // panel is fetched once instead of once per 128-column tile
  if (p.epilogue == EPI_STORE && p.N == 384) return (pair_on && p.M >= 2 * GBM) ? launch_pair<384>(p, st) : launch_bn<384>(p, st);
  if (p.epilogue != EPI_SWIGLU && p.N % 256 != 0 && p.N % 128 == 0 && p.N <= 1024) return launch_bn<128>(p, st);
  // short K with a read-modify-write epilogue (o_proj + residual): the epilogue dominates, so run two narrower CTAs
  // per SM (2 x 256 TMEM columns, 2 x 97 KB of shared memory) and let their epilogues overlap
  if ((p.epilogue == EPI_RESID || p.epilogue == EPI_SCATTER_ADD) && p.K <= 512 && p.N % 128 == 0)
    return launch_bn<128, 2>(p, st);
  if (pair_on && p.M >= 2 * GBM) return launch_pair<256>(p, st);
  return launch_bn<256>(p, st);
}

}  // namespace hb200
