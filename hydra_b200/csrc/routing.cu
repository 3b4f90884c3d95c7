// Mixture-of-Depths selection: per sequence, the ascending index list of the k largest router
// scores (radix select + ordered compaction), optionally intersected with the tokens that are
// still active in the Mixture-of-Recursions loop and appended to a compact row list.
#include "common.cuh"

namespace hb200 {

// Monotone map fp32 -> uint32 (larger value <=> larger key); NaN ranks highest, -0 == +0.
__device__ __forceinline__ uint32_t score_key(float s) {
  if (s != s) return 0xFFFFFFFFu;
  s += 0.0f;
  const uint32_t b = __float_as_uint(s);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// One CTA per sequence. Dynamic shared memory: L keys (uint32).
__global__ void __launch_bounds__(1024) mod_select_kernel(const float* __restrict__ scores, int L, int k,
                                                          int32_t* __restrict__ idx_out,
                                                          const int32_t* __restrict__ depth, int min_active,
                                                          int32_t* __restrict__ rows_out, int32_t* __restrict__ count,
                                                          const int32_t* __restrict__ forced_idx) {
  extern __shared__ uint32_t keys[];
  __shared__ int hist[256];
  __shared__ int scan_buf[33];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  __shared__ int s_base;

  const int b = blockIdx.x;
  const int tid = threadIdx.x, nt = blockDim.x;
  const float* sc = scores + (int64_t)b * L;

  uint32_t kth = 0;
  int need_eq = 0;
  if (forced_idx == nullptr) {
    for (int i = tid; i < L; i += nt) keys[i] = score_key(sc[i]);
    if (tid == 0) {
      s_prefix = 0;
      s_remaining = k;
    }
    __syncthreads();
    uint32_t mask = 0;
    for (int pass = 3; pass >= 0; --pass) {
      for (int i = tid; i < 256; i += nt) hist[i] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const int remaining = s_remaining;
      const int shift = pass * 8;
      for (int i = tid; i < L; i += nt) {
        const uint32_t key = keys[i];
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xFF], 1);
      }
      __syncthreads();
      if (tid < 32) {
        int c[8], s = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          c[j] = hist[255 - (tid * 8 + j)];
          s += c[j];
        }
        int incl = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int t = __shfl_up_sync(0xffffffffu, incl, o);
          if (tid >= o) incl += t;
        }
        const int excl = incl - s;
        if (excl < remaining && remaining <= incl) {
          int acc = excl;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (acc + c[j] >= remaining) {
              s_prefix = prefix | ((uint32_t)(255 - (tid * 8 + j)) << shift);
              s_remaining = remaining - acc;
              break;
            }
            acc += c[j];
          }
        }
      }
      mask |= 0xFFu << shift;
      __syncthreads();
    }
    kth = s_prefix;
    need_eq = s_remaining;   // how many of the scores equal to the k-th largest are taken (lowest index first)
  } else {
    // forced routing: mark the given positions, then run the same ordered compaction
    for (int i = tid; i < L; i += nt) keys[i] = 0;
    __syncthreads();
    const int32_t* f = forced_idx + (int64_t)b * k;
    for (int i = tid; i < k; i += nt) {
      const int p = f[i];
      if (p >= 0 && p < L) keys[p] = 2;
    }
    __syncthreads();
    kth = 1;          // keys: 2 = selected (> kth), 0 = not selected
    need_eq = 0;
  }

  // ordered compaction: each thread owns a contiguous segment of positions
  const int seg = (L + nt - 1) / nt;
  const int p0 = min(tid * seg, L), p1 = min(p0 + seg, L);
  int n_gt = 0, n_eq = 0;
  for (int p = p0; p < p1; ++p) {
    const uint32_t key = keys[p];
    n_gt += key > kth;
    n_eq += key == kth;
  }
  int tot_gt, tot_eq;
  const int gt_before = block_exclusive_scan(n_gt, scan_buf, tot_gt);
  const int eq_before = block_exclusive_scan(n_eq, scan_buf, tot_eq);
  int rank = gt_before + min(eq_before, need_eq);
  int eq_rank = eq_before;
  // second ordered count: selected AND still active
  int n_act = 0;
  {
    int er = eq_before;
    for (int p = p0; p < p1; ++p) {
      const uint32_t key = keys[p];
      bool sel = key > kth;
      if (key == kth) sel = (er++ < need_eq);
      if (sel && depth != nullptr && depth[(int64_t)b * L + p] >= min_active) ++n_act;
    }
  }
  int tot_act = 0, act_before = 0;
  if (rows_out != nullptr) {
    act_before = block_exclusive_scan(n_act, scan_buf, tot_act);
    if (tid == 0) s_base = atomicAdd(count, tot_act);
    __syncthreads();
  }
  const int base = rows_out != nullptr ? s_base : 0;
  int arank = act_before;
  for (int p = p0; p < p1; ++p) {
    const uint32_t key = keys[p];
    bool sel = key > kth;
    if (key == kth) sel = (eq_rank++ < need_eq);
    if (sel) {
      if (idx_out != nullptr && rank < k) idx_out[(int64_t)b * k + rank] = p;
      ++rank;
      if (rows_out != nullptr && depth[(int64_t)b * L + p] >= min_active) rows_out[base + arank++] = b * L + p;
    }
  }
}

// The same selection for sequences of at most 256 * KPT positions: 256 threads, each holding KPT consecutive scores (and
// depths) in registers from one coalesced load, so the four radix passes and the compaction run out of registers with
// eight warps per barrier instead of thirty-two, and the two ordered counts share one scan.  Same rules, same results.
template <int KPT>
__global__ void __launch_bounds__(256) mod_select_reg_kernel(const float* __restrict__ scores, int L, int k,
                                                             int32_t* __restrict__ idx_out,
                                                             const int32_t* __restrict__ depth, int min_active,
                                                             int32_t* __restrict__ rows_out, int32_t* __restrict__ count,
                                                             const int32_t* __restrict__ forced_idx) {
  __shared__ int hist[256];
  __shared__ int scan_buf[33];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  __shared__ int s_base;
  __shared__ unsigned char marks[256 * KPT];

  const int b = blockIdx.x, tid = threadIdx.x;
  const int p0 = tid * KPT;
  const float* sc = scores + (int64_t)b * L;
  uint32_t key[KPT];
  bool act[KPT];
#pragma unroll
  for (int j = 0; j < KPT; ++j) act[j] = false;
  // whole 16-byte pieces when the sequence allows it (its length a multiple of 4, pointers aligned)
  const bool vec = ((L & 3) == 0) && ((reinterpret_cast<uintptr_t>(scores) & 15u) == 0) &&
                   (depth == nullptr || (reinterpret_cast<uintptr_t>(depth) & 15u) == 0);
  if (rows_out != nullptr) {
    const int32_t* dp = depth + (int64_t)b * L;
    if (vec) {
#pragma unroll
      for (int j = 0; j < KPT; j += 4)
        if (p0 + j < L) {
          const int4 d4 = *reinterpret_cast<const int4*>(dp + p0 + j);
          act[j] = d4.x >= min_active; act[j + 1] = d4.y >= min_active; act[j + 2] = d4.z >= min_active; act[j + 3] = d4.w >= min_active;
        }
    } else {
#pragma unroll
      for (int j = 0; j < KPT; ++j)
        if (p0 + j < L) act[j] = dp[p0 + j] >= min_active;
    }
  }

  uint32_t kth = 0;
  int need_eq = 0;
  if (forced_idx == nullptr) {
    // positions past L get key 0, which no score maps to (the smallest key, -inf, is 0x007FFFFF): never selected
    if (vec) {
#pragma unroll
      for (int j = 0; j < KPT; j += 4) {
        float4 f4 = make_float4(0.f, 0.f, 0.f, 0.f);
        const bool in = p0 + j < L;
        if (in) f4 = *reinterpret_cast<const float4*>(sc + p0 + j);
        key[j] = in ? score_key(f4.x) : 0u; key[j + 1] = in ? score_key(f4.y) : 0u;
        key[j + 2] = in ? score_key(f4.z) : 0u; key[j + 3] = in ? score_key(f4.w) : 0u;
      }
    } else {
#pragma unroll
      for (int j = 0; j < KPT; ++j) key[j] = (p0 + j < L) ? score_key(sc[p0 + j]) : 0u;
    }
    if (tid == 0) {
      s_prefix = 0;
      s_remaining = k;
    }
    uint32_t mask = 0;
    for (int pass = 3; pass >= 0; --pass) {
      hist[tid] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const int remaining = s_remaining;
      const int shift = pass * 8;
#pragma unroll
      for (int j = 0; j < KPT; ++j)
        if (p0 + j < L && (key[j] & mask) == prefix) atomicAdd(&hist[(key[j] >> shift) & 0xFF], 1);
      __syncthreads();
      if (tid < 32) {
        int c[8], sum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          c[j] = hist[255 - (tid * 8 + j)];
          sum += c[j];
        }
        int incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int t = __shfl_up_sync(0xffffffffu, incl, o);
          if (tid >= o) incl += t;
        }
        const int excl = incl - sum;
        if (excl < remaining && remaining <= incl) {
          int acc = excl;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (acc + c[j] >= remaining) {
              s_prefix = prefix | ((uint32_t)(255 - (tid * 8 + j)) << shift);
              s_remaining = remaining - acc;
              break;
            }
            acc += c[j];
          }
        }
      }
      mask |= 0xFFu << shift;
      __syncthreads();
    }
    kth = s_prefix;
    need_eq = s_remaining;   // how many of the scores equal to the k-th largest are taken (lowest index first)
  } else {
    // forced routing: mark the given positions, then run the same ordered compaction
#pragma unroll
    for (int j = 0; j < KPT; ++j) marks[p0 + j] = 0;
    __syncthreads();
    const int32_t* f = forced_idx + (int64_t)b * k;
    for (int i = tid; i < k; i += 256) {
      const int p = f[i];
      if (p >= 0 && p < L) marks[p] = 1;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < KPT; ++j) key[j] = marks[p0 + j] ? 2u : 0u;
    kth = 1;          // keys: 2 = selected (> kth), 0 = not selected
    need_eq = 0;
  }

  // ordered compaction over each thread's KPT consecutive positions; both counts (above / equal to the k-th key) in one scan
  int n_gt = 0, n_eq = 0;
#pragma unroll
  for (int j = 0; j < KPT; ++j) {
    n_gt += key[j] > kth;
    n_eq += key[j] == kth;
  }
  int tot_pack;
  const int before = block_exclusive_scan(n_gt | (n_eq << 16), scan_buf, tot_pack);
  const int gt_before = before & 0xFFFF, eq_before = before >> 16;
  int rank = gt_before + min(eq_before, need_eq);
  // second ordered count: selected AND still active
  bool sel[KPT];
  int n_act = 0;
  {
    int er = eq_before;
#pragma unroll
    for (int j = 0; j < KPT; ++j) {
      sel[j] = key[j] > kth;
      if (key[j] == kth) sel[j] = (er++ < need_eq);
      n_act += (sel[j] && act[j]) ? 1 : 0;
    }
  }
  int tot_act = 0, act_before = 0;
  if (rows_out != nullptr) {
    act_before = block_exclusive_scan(n_act, scan_buf, tot_act);
    if (tid == 0) s_base = atomicAdd(count, tot_act);
    __syncthreads();
  }
  const int base = rows_out != nullptr ? s_base : 0;
  int arank = act_before;
#pragma unroll
  for (int j = 0; j < KPT; ++j) {
    if (sel[j]) {
      if (idx_out != nullptr && rank < k) idx_out[(int64_t)b * k + rank] = p0 + j;
      ++rank;
      if (rows_out != nullptr && act[j]) rows_out[base + arank++] = b * L + p0 + j;
    }
  }
}

// Row list of all tokens with depth >= min_active (blocks without MoD). One CTA per 4096-token chunk;
// ascending inside a chunk, chunk order decided by the atomic reservation.
__global__ void __launch_bounds__(1024) compact_active_kernel(const int32_t* __restrict__ depth, int64_t n,
                                                              int min_active, int32_t* __restrict__ rows_out,
                                                              int32_t* __restrict__ count) {
  __shared__ int scan_buf[33];
  __shared__ int s_base;
  const int64_t c0 = (int64_t)blockIdx.x * 4096;
  const int tid = threadIdx.x;
  const int64_t p0 = c0 + tid * 4;
  int flags[4], cnt = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    flags[j] = (p0 + j < n) && (depth[p0 + j] >= min_active);
    cnt += flags[j];
  }
  int total;
  int off = block_exclusive_scan(cnt, scan_buf, total);
  if (tid == 0) s_base = atomicAdd(count, total);
  __syncthreads();
  off += s_base;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (flags[j]) rows_out[off++] = (int32_t)(p0 + j);
}

int launch_mod_select(const float* scores, int B, int L, int k, int32_t* idx_out, const int32_t* depth, int min_active,
                      int32_t* rows_out, int32_t* count, const int32_t* forced_idx, cudaStream_t st) {
  if (L <= 256 * 8) {
    mod_select_reg_kernel<8><<<B, 256, 0, st>>>(scores, L, k, idx_out, depth, min_active, rows_out, count, forced_idx);
    HB_LAUNCH_CHECK();
    return 0;
  }
  if (L <= 256 * 16) {
    mod_select_reg_kernel<16><<<B, 256, 0, st>>>(scores, L, k, idx_out, depth, min_active, rows_out, count, forced_idx);
    HB_LAUNCH_CHECK();
    return 0;
  }
  const size_t smem = (size_t)L * sizeof(uint32_t);
  HB_REQUIRE(smem <= 200 * 1024, HB200_ERR_UNSUPPORTED, "mod_topk_select: sequence length %d too long (max 51200)", L);
  if (smem > 48 * 1024) {
    HB_PROPAGATE(ensure_dynamic_smem((const void*)mod_select_kernel, (size_t)(200 * 1024)));
  }
  mod_select_kernel<<<B, 1024, smem, st>>>(scores, L, k, idx_out, depth, min_active, rows_out, count, forced_idx);
  HB_LAUNCH_CHECK();
  return 0;
}

int launch_compact_active(const int32_t* depth, int64_t n, int min_active, int32_t* rows_out, int32_t* count,
                          cudaStream_t st) {
  compact_active_kernel<<<(unsigned)ceil_div64(n, 4096), 1024, 0, st>>>(depth, n, min_active, rows_out, count);
  HB_LAUNCH_CHECK();
  return 0;
}

}  // namespace hb200

using namespace hb200;

extern "C" int hb200_mod_topk_select(const float* scores, int B, int L, int k, int32_t* idx_out, const int32_t* depth,
                                     int min_active_depth, int32_t* rows_out, int32_t* count, void* stream) {
  HB_REQUIRE(scores && idx_out, HB200_ERR_INVALID, "mod_topk_select: null pointer");
  HB_REQUIRE(B >= 0 && L >= 1 && k >= 1 && k <= L, HB200_ERR_INVALID, "mod_topk_select: need 1 <= k <= L (k=%d L=%d)", k,
             L);
  HB_REQUIRE((rows_out == nullptr) || (depth != nullptr && count != nullptr), HB200_ERR_INVALID,
             "mod_topk_select: rows_out needs depth and count");
  if (B == 0) return 0;
  return launch_mod_select(scores, B, L, k, idx_out, depth, min_active_depth, rows_out, count, nullptr,
                           (cudaStream_t)stream);
}
