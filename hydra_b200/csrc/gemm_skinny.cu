// Skinny-M bf16 GEMM for decode (M <= 128 rows):  C = epilogue(A W^T),  A [M,K], W [N,K], both K-major.
//
// With a handful of rows the contraction is bound by streaming W from HBM once, so the work is cut for bandwidth,
// not for tensor throughput: one CTA per (128 weight rows, one slice of K), so even a 2048 x 5632 weight (16 row
// tiles) keeps 128 SMs streaming.  Inside a CTA the pipeline is the one of the large GEMM: warp 0 issues TMA loads of
// the A slice [128 x 64] (rows beyond M are zero-filled by the tensor map and cost no traffic) and the W tile
// [128 x 64] into a 6-deep 128B-swizzled ring, warp 1 issues tcgen05.mma (M=128, N=128, K=16) into a TMEM
// accumulator, warps 2-5 (one per TMEM lane quadrant) drain it.
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
constexpr int SK_STAGES = 6;
constexpr int SK_A_BYTES = SK_BM * SK_BK * 2, SK_B_BYTES = SK_BN * SK_BK * 2, SK_STAGE_BYTES = SK_A_BYTES + SK_B_BYTES;
constexpr int SK_THREADS = 6 * 32;          // producer, MMA issuer, 4 epilogue warps
constexpr int SK_SMEM_BYTES = SK_STAGES * SK_STAGE_BYTES + 256 + 1024;
constexpr int SK_MAX_SPLIT = 8;             // portable cluster size
constexpr int SK_MIN_KB_PER_SPLIT = 2;
static_assert(SK_BM * SK_BN * 4 <= SK_STAGES * SK_STAGE_BYTES, "the fp32 partial reuses the operand ring");

struct SkinnyPlan {
  int n_tiles, k_blocks, ksplit, kb_per;
};

static SkinnyPlan skinny_plan(int N, int K) {
  SkinnyPlan s;
  s.n_tiles = ceil_div(N, SK_BN);
  s.k_blocks = ceil_div(K, SK_BK);
  const int want = std::min(sm_count() / s.n_tiles, s.k_blocks / SK_MIN_KB_PER_SPLIT);
  s.ksplit = 1;
  while (s.ksplit * 2 <= std::min(want, SK_MAX_SPLIT)) s.ksplit *= 2;   // power of two: column shares of 128 / ksplit
  s.kb_per = ceil_div(s.k_blocks, s.ksplit);
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

__global__ void __launch_bounds__(SK_THREADS, 1) gemm_skinny_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                                    const __grid_constant__ CUtensorMap tma_b,
                                                                    const GemmParams p, int ksplit, int kb_per,
                                                                    int k_blocks) {
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t base = (s_addr(smem_dyn) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - s_addr(smem_dyn));
  const uint32_t bars = base + SK_STAGES * SK_STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (SK_STAGES + s); };
  const uint32_t tfull_bar = bars + 8u * (2 * SK_STAGES);
  volatile uint32_t* tmem_slot =
      reinterpret_cast<volatile uint32_t*>(base_ptr + SK_STAGES * SK_STAGE_BYTES + 8 * (2 * SK_STAGES + 2));
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* part = reinterpret_cast<float*>(base_ptr);       // [SK_BN columns][SK_BM rows] fp32, over the operand ring

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int M = p.m_dev ? min(*p.m_dev, p.M) : p.M;
  const int nt = blockIdx.x / ksplit, ks = blockIdx.x - nt * ksplit;   // ks == rank in the cluster
  const int kb0 = ks * kb_per, kb1 = (M > 0) ? min(k_blocks, kb0 + kb_per) : kb0;
  const bool has_work = kb1 > kb0;                                      // a trailing slice may be empty

  if (threadIdx.x == 0) {
    for (int s = 0; s < SK_STAGES; ++s) {
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

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) break;
        const uint32_t sa = base + stage * SK_STAGE_BYTES;
        mbar_arrive_expect_tx(full_bar(stage), SK_STAGE_BYTES);
        tma_load_2d(sa, &tma_a, kb * SK_BK, 0, full_bar(stage));
        tma_load_2d(sa + SK_A_BYTES, &tma_b, kb * SK_BK, nt * SK_BN, full_bar(stage));
        if (++stage == SK_STAGES) { stage = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && has_work) {
      constexpr uint32_t idesc = make_idesc(SK_BM, SK_BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t sa = base + stage * SK_STAGE_BYTES;
        const uint64_t da = make_smem_desc(sa);
        const uint64_t db = make_smem_desc(sa + SK_A_BYTES);
#pragma unroll
        for (int k = 0; k < SK_BK / 16; ++k) umma_bf16(tmem_base, da + 2u * k, db + 2u * k, idesc, (kb > kb0 || k) ? 1u : 0u);
        umma_commit(empty_bar(stage));
        if (++stage == SK_STAGES) { stage = 0; phase ^= 1u; }
      }
      if (ok) umma_commit(tfull_bar);
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue warps (2..5): TMEM -> epilogue, or TMEM -> own partial ----------
    const int quad = warp & 3;
    const int m = quad * 32 + lane;
    bool ok = true;
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
          for (int c = 0; c < SK_BN / 32; ++c) {
            float v[32];
            tmem_ld_32x32(t_row + (uint32_t)(c * 32), v);
            const int col = nt * SK_BN + c * 32;
            if (m < M && col < p.N) epilogue_row_chunk<32>(p, m, col, v);
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < SK_BN / 32; ++c) {
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
      const int cw = SK_BN / ksplit;                               // this CTA's share of the tile's columns (>= 16)
      if (m < M) {
        const uint32_t part_addr = s_addr(part);
#pragma unroll 1
        for (int g = 0; g < cw / 16; ++g) {
          const int c0 = ks * cw + g * 16;                         // column inside the tile
          const int col = nt * SK_BN + c0;
          if (col >= p.N) break;
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
          for (int s = 0; s < ksplit; ++s) {                       // fixed order: deterministic sum
            const uint32_t peer = map_to_cta(part_addr + (uint32_t)((c0 * SK_BM + m) * 4), (uint32_t)s);
            float t[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) t[j] = ld_dsmem_f32(peer + (uint32_t)(j * SK_BM * 4));
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += t[j];
          }
          epilogue_row_chunk<16>(p, m, col, v);
        }
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

int launch_gemm_skinny(const GemmParams& p, cudaStream_t st) {
  HB_REQUIRE(p.M >= 1 && p.M <= SK_BM, HB200_ERR_UNSUPPORTED, "skinny gemm: M = %d (1..%d rows)", p.M, SK_BM);
  const SkinnyPlan s = skinny_plan(p.N, p.K);
  CUtensorMap ta, tb;
  HB_PROPAGATE(make_tmap(&ta, p.A, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)p.lda, SK_BM));
  HB_PROPAGATE(make_tmap(&tb, p.W, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.ldw, SK_BN));
  static bool attr_set = false;
  if (!attr_set) {
    HB_CUDA(cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_SMEM_BYTES));
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(s.n_tiles * s.ksplit), 1, 1);
  cfg.blockDim = dim3(SK_THREADS, 1, 1);
  cfg.dynamicSmemBytes = SK_SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)s.ksplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  HB_CUDA(cudaLaunchKernelEx(&cfg, gemm_skinny_kernel, ta, tb, p, s.ksplit, s.kb_per, s.k_blocks));
  HB_LAUNCH_CHECK();
  return 0;
}

}  // namespace hb200
