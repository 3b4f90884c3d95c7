// Next-token sampling on the device: temperature, top-k and top-p (nucleus) filtering, one draw per row.
//
// Follows the sampler inside the reference's generation helper (diagnostics/eval_checkpoint.py:133-155):
//   logits / temperature;  top-k: everything below the k-th largest value is removed (ties with it stay);
//   top-p: in descending order a token is removed iff the probability mass before it exceeds top_p (the first token
//   always stays), probabilities being the softmax of what top-k left;  one draw from the renormalised rest.
// The reference draws with torch.multinomial; here the draw is the inverse CDF in descending-logit order (equal logits
// by ascending token id) at a caller-supplied uniform number per row, so a result is a function of (logits, uniform).
//
// One CTA per row, no sort: logits are bf16, so a row has at most 65536 distinct values.  The CTA builds the exact count
// of every 16-bit pattern in shared memory (128 KB, two 16-bit counters per word) and a three-level bitmap of the
// values that occur (NaNs take no part).
// The distinct values are then dealt out evenly, in descending order, to the threads (a row of 50257 logits holds a
// few thousand distinct values, packed into a few narrow ranges of the key space: dealing by rank instead of by key
// range gives every thread 3-4 of them instead of giving 50 threads 64 each), and every later decision - the top-k
// threshold, the softmax mass, the nucleus cut, the drawn value - is a short walk per thread plus a block scan.
// Masses are 64-bit fixed point (32 fractional bits relative to the largest token), so sums are exact, associative and
// the same in every run.  One last pass over the row finds the drawn token among the tokens that share the drawn
// value.  HBM/L2 traffic: the row is read twice (2 x 2 x vocab bytes).
#include "common.cuh"

namespace hb200 {

constexpr int SMP_THREADS = 1024;
constexpr int SMP_KEYS = 65536;
constexpr int SMP_KEYS_PER_THREAD = SMP_KEYS / SMP_THREADS;   // 64 consecutive values per thread
constexpr int SMP_WORDS = SMP_KEYS / 2;                       // two 16-bit counters per word
constexpr int SMP_BM_WORDS = SMP_KEYS / 32;                   // one presence bit per value
constexpr size_t SMP_SMEM = (size_t)(SMP_WORDS + SMP_BM_WORDS + 64 + 2 + SMP_THREADS) * 4;

// Values are ordered through a 16-bit key whose unsigned order is the order of the bf16 values; -0 is read as +0
// (canon_zero), so the two compare equal as they do in floating point and tie by token id.
// Keys above 0xff80 and below 0x007f are NaNs.
__device__ __forceinline__ uint32_t raw_to_key(uint32_t r) { return (r & 0x8000u) ? (~r & 0xffffu) : (r | 0x8000u); }
__device__ __forceinline__ uint32_t key_to_raw(uint32_t k) { return (k & 0x8000u) ? (k & 0x7fffu) : (~k & 0xffffu); }
__device__ __forceinline__ float order_key_value(uint32_t k) { return __uint_as_float(key_to_raw(k) << 16); }
constexpr uint32_t SMP_KEY_POS_INF = 0xff80u, SMP_KEY_NEG_INF = 0x007fu;
// The counters are indexed by the raw bf16 bits (the row pass does no conversion); groups of four words are
// XOR-swizzled so that threads reading consecutive 32-word ranges with 16-byte loads hit distinct banks.
__device__ __forceinline__ uint32_t count_word(uint32_t raw) {
  const uint32_t w = raw >> 1;
  return w ^ (((w >> 5) & 7u) << 2);
}
// presence bits of the two 16-bit counters of a word: bit 0 <=> low counter non-zero, bit 1 <=> high counter non-zero
__device__ __forceinline__ uint32_t present2(uint32_t w) {
  const uint32_t r = __vsetne2(w, 0u);
  return (r | (r >> 15)) & 3u;
}
__device__ __forceinline__ uint32_t count_of(const uint32_t* cnt, uint32_t key) {
  const uint32_t raw = key_to_raw(key);
  return (cnt[count_word(raw)] >> ((raw & 1u) << 4)) & 0xffffu;
}

// -0 (0x8000) -> +0 in both halves of a word
__device__ __forceinline__ uint32_t canon_zero(uint32_t w) { return w & ~(__vcmpeq2(w, 0x80008000u) & 0x80008000u); }
__device__ __forceinline__ uint4 canon_zero(uint4 q) {
  return make_uint4(canon_zero(q.x), canon_zero(q.y), canon_zero(q.z), canon_zero(q.w));
}
// the 8 elements [i, i + 8) of a row as four words of two bf16 each (i a multiple of 8); elements past the end read 0
__device__ __forceinline__ uint4 load_raw8(const unsigned short* bits, int i, int cols, bool vec) {
  if (vec && i + 8 <= cols) return canon_zero(__ldcg(reinterpret_cast<const uint4*>(bits + i)));
  uint32_t h[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) h[j] = (i + j < cols) ? (uint32_t)__ldcg(bits + i + j) : 0u;
  return canon_zero(make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16)));
}
// how many of the elements [i, i + 8) hold exactly the bits `raw` (pat2 = raw in both halves of a word)
__device__ __forceinline__ uint32_t count_equal8(const uint4& q, int i, int cols, uint32_t raw, uint32_t pat2) {
  if (i + 8 <= cols)
    return (__popc(__vcmpeq2(q.x, pat2)) + __popc(__vcmpeq2(q.y, pat2)) + __popc(__vcmpeq2(q.z, pat2)) +
            __popc(__vcmpeq2(q.w, pat2))) >> 4;
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  uint32_t c = 0u;
#pragma unroll
  for (int j = 0; j < 8; ++j) c += (i + j < cols && ((w[j >> 1] >> ((j & 1) << 4)) & 0xffffu) == raw) ? 1u : 0u;
  return c;
}

// exclusive scan over the block in thread order; `scratch` holds 33 values; every thread gets the block total
template <class T>
__device__ __forceinline__ T block_exclusive_scan(T v, T* scratch, T& total) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  T inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const T n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  if (lane == 31) scratch[wid] = inc;
  __syncthreads();
  if (wid == 0) {
    const T s = scratch[lane];
    T si = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const T n = __shfl_up_sync(0xffffffffu, si, o);
      if (lane >= o) si += n;
    }
    scratch[lane] = si - s;
    if (lane == 31) scratch[32] = si;
  }
  __syncthreads();
  const T res = scratch[wid] + inc - v;
  total = scratch[32];
  __syncthreads();
  return res;
}

// fixed-point softmax weight of a value relative to the row maximum: exp((v - vmax) / T) * 2^32
__device__ __forceinline__ unsigned long long mass_of(uint32_t key, uint32_t kmax, float vmax, float inv_t) {
  if (key == kmax) return 1ull << 32;
  const float e = expf((order_key_value(key) - vmax) * inv_t);
  return (unsigned long long)(e * 4294967296.0f);
}

// Walks the values present in the row in descending order.  `bm` has one bit per key, `sm` one bit per word of bm,
// `top` one bit per word of sm, so a run of absent values of any length is stepped over in constant time.
struct KeyCursor {
  int w;           // bitmap word the cursor is in
  uint32_t m;      // bits of that word not yet visited
  __device__ __forceinline__ void lower_word(const uint32_t* bm, const uint32_t* sm, unsigned long long top) {
    int sw = w >> 5;                                       // the caller knows a lower non-empty word exists
    uint32_t s = sm[sw] & ((1u << (w & 31)) - 1u);
    if (s == 0u) {
      sw = 63 - __clzll(top & ((1ull << sw) - 1ull));
      s = sm[sw];
    }
    w = sw * 32 + 31 - __clz(s);
    m = bm[w];
  }
  __device__ __forceinline__ uint32_t next(const uint32_t* bm, const uint32_t* sm, unsigned long long top) {
    if (m == 0u) lower_word(bm, sm, top);                  // the caller knows another key exists
    const int b = 31 - __clz(m);
    m &= ~(1u << b);
    return (uint32_t)w * 32u + (uint32_t)b;
  }
};

__global__ void __launch_bounds__(SMP_THREADS, 1)
sample_rows_kernel(const __nv_bfloat16* __restrict__ x, int cols, int64_t ld, float temperature, int top_k, float top_p,
                   const float* __restrict__ uniforms, int64_t* __restrict__ out) {
  extern __shared__ __align__(16) uint32_t cnt[];          // SMP_WORDS counter words, then the bitmaps and the ranks
  uint32_t* bm = cnt + SMP_WORDS;                          // SMP_BM_WORDS words: bit k%32 of word k/32 <=> key k occurs
  uint32_t* sm = bm + SMP_BM_WORDS;                        // 64 words: which words of bm are non-zero
  uint32_t* top2 = sm + 64;                                // 2 words: which words of sm are non-zero
  uint32_t* pair_rank = top2 + 2;                          // SMP_THREADS entries, see below
  __shared__ unsigned long long scratch64[33];
  __shared__ uint32_t scratch32[33];
  __shared__ uint32_t sh_key;
  __shared__ uint32_t sh_n;
  __shared__ unsigned long long sh_mass;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const __nv_bfloat16* row = x + (int64_t)blockIdx.x * ld;
  const unsigned short* bits = reinterpret_cast<const unsigned short*>(row);
  const bool vec = ((reinterpret_cast<uintptr_t>(row) & 15u) == 0);

  for (int i = tid; i < SMP_WORDS / 4; i += SMP_THREADS) reinterpret_cast<uint4*>(cnt)[i] = make_uint4(0u, 0u, 0u, 0u);
  if (tid < 2) top2[tid] = 0u;
  if (tid == 0) { sh_key = 0u; sh_n = 0u; sh_mass = 0ull; }
  __syncthreads();

  // ---- pass 1 over the row: count every bit pattern (loads issued four at a time, then consumed) -------------------
  for (int i0 = tid * 8; i0 < cols; i0 += 4 * SMP_THREADS * 8) {
    uint4 q[4];
    if (vec && i0 + 3 * SMP_THREADS * 8 + 8 <= cols) {       // all four inside the row: nothing between the loads
#pragma unroll
      for (int b = 0; b < 4; ++b)
        q[b] = canon_zero(__ldcg(reinterpret_cast<const uint4*>(bits + i0 + b * SMP_THREADS * 8)));
    } else {
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int i = i0 + b * SMP_THREADS * 8;
        q[b] = (i < cols) ? load_raw8(bits, i, cols, vec) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int i = i0 + b * SMP_THREADS * 8;
      const uint32_t w[4] = {q[b].x, q[b].y, q[b].z, q[b].w};
      if (i + 8 <= cols) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t r0 = w[j] & 0xffffu, r1 = w[j] >> 16;
          atomicAdd(&cnt[count_word(r0)], 1u << ((r0 & 1u) << 4));
          atomicAdd(&cnt[count_word(r1)], 1u << ((r1 & 1u) << 4));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t r = (w[j >> 1] >> ((j & 1) << 4)) & 0xffffu;
          if (i + j < cols) atomicAdd(&cnt[count_word(r)], 1u << ((r & 1u) << 4));
        }
      }
    }
  }
  __syncthreads();

  // ---- which values occur: 64 keys = two bitmap words per thread, thread 0 the largest keys -------------------------
  // pair_rank[t] = number of distinct values above the 64 keys of thread t; `distinct` = number of distinct values
  {
    const uint32_t hi = SMP_KEYS - (uint32_t)tid * SMP_KEYS_PER_THREAD, lo = hi - SMP_KEYS_PER_THREAD;
    // the 64 keys are 64 consecutive bit patterns: ascending with the key for positive values, descending for negative
    const bool negative = lo < 0x8000u;
    const uint32_t rb = negative ? (0xffffu - lo - 63u) : (lo & 0x7fffu);
    uint32_t c0 = 0u, c1 = 0u;                             // presence of patterns rb .. rb+31 / rb+32 .. rb+63
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {                     // 8 patterns = 4 counter words per load
      const uint4 ql = *reinterpret_cast<const uint4*>(&cnt[count_word(rb + 8 * j)]);
      const uint4 qh = *reinterpret_cast<const uint4*>(&cnt[count_word(rb + 32 + 8 * j)]);
      c0 |= (present2(ql.x) | present2(ql.y) << 2 | present2(ql.z) << 4 | present2(ql.w) << 6) << (8 * j);
      c1 |= (present2(qh.x) | present2(qh.y) << 2 | present2(qh.z) << 4 | present2(qh.w) << 6) << (8 * j);
    }
    uint32_t b0 = negative ? __brev(c1) : c0;              // keys lo .. lo+31
    uint32_t b1 = negative ? __brev(c0) : c1;              // keys lo+32 .. lo+63
    // NaN patterns take no part: keys above +inf (threads 0 and 1) and below -inf (the last two threads)
    if (tid == 0 || tid == SMP_THREADS - 1) { b0 = 0u; b1 = 0u; }
    if (tid == 1) { b0 &= 1u; b1 = 0u; }                   // keeps +inf, key 0xff80
    if (tid == SMP_THREADS - 2) { b0 = 0u; b1 &= 0x80000000u; }   // keeps -inf, key 0x007f
    const uint32_t wa = lo >> 5;
    bm[wa] = b0;
    bm[wa + 1] = b1;
    // the warp's 64 bitmap words are two words of sm: lanes 0-15 hold the upper one's 32 words, lanes 16-31 the lower's
    const uint32_t nz = (b0 ? 1u : 0u) | (b1 ? 2u : 0u);
    const uint32_t s_up = __reduce_or_sync(0xffffffffu, lane < 16 ? nz << (30 - 2 * lane) : 0u);
    const uint32_t s_lo = __reduce_or_sync(0xffffffffu, lane >= 16 ? nz << (62 - 2 * lane) : 0u);
    if (lane == 0) {
      const int su = 63 - 2 * wid;                         // = (wa + 1) >> 5 of lane 0
      sm[su] = s_up;
      sm[su - 1] = s_lo;
      if (s_up) atomicOr(&top2[su >> 5], 1u << (su & 31));
      if (s_lo) atomicOr(&top2[(su - 1) >> 5], 1u << ((su - 1) & 31));
    }
    uint32_t distinct_all;
    const uint32_t above = block_exclusive_scan<uint32_t>(__popc(b0) + __popc(b1), scratch32, distinct_all);
    pair_rank[tid] = above;
    sh_n = distinct_all;                                   // same value from every thread
  }
  __syncthreads();
  const uint32_t distinct = sh_n;
  if (distinct == 0u) {                                    // nothing but NaNs in the row
    if (tid == 0) out[blockIdx.x] = 0;
    return;
  }
  const unsigned long long top = (unsigned long long)top2[0] | ((unsigned long long)top2[1] << 32);
  // thread t walks the values of rank [t * per, t * per + mine) in descending order
  const uint32_t per = (distinct + SMP_THREADS - 1) / SMP_THREADS;
  const uint32_t rank0 = (uint32_t)tid * per;
  const int mine = rank0 < distinct ? (int)min(per, distinct - rank0) : 0;
  KeyCursor start{0, 0u};
  if (mine) {
    int a = 0, b = SMP_THREADS - 1;                        // last pair whose rank is <= rank0
    while (a < b) {
      const int mid = (a + b + 1) >> 1;
      if (pair_rank[mid] <= rank0) a = mid; else b = mid - 1;
    }
    uint32_t skip = rank0 - pair_rank[a];                  // < 64: ranks inside this pair of words
    start.w = (int)((SMP_KEYS - (uint32_t)a * SMP_KEYS_PER_THREAD) >> 5) - 1;
    start.m = bm[start.w];
    const uint32_t n_hi = __popc(start.m);
    if (skip >= n_hi) { skip -= n_hi; --start.w; start.m = bm[start.w]; }
    while (skip) { start.m &= ~(1u << (31 - __clz(start.m))); --skip; }
  }
  if (tid == 0) { KeyCursor c = start; sh_key = c.next(bm, sm, top); }   // the largest value
  __syncthreads();
  const uint32_t kmax = sh_key;
  __syncthreads();

  uint32_t draw_key = kmax, draw_rank = 0u;       // greedy unless a distribution is sampled below
  const bool greedy = !(temperature > 0.0f) || top_k == 1;
  if (!greedy) {
    const float inv_t = 1.0f / temperature;
    const float vmax = order_key_value(kmax);
    // ---- one scan: tokens and softmax mass above each thread's values ------------------------------------------
    uint32_t c_mine = 0u;
    unsigned long long w_mine = 0ull;
    {
      KeyCursor cur = start;
      for (int i = 0; i < mine; ++i) {
        const uint32_t k = cur.next(bm, sm, top);
        const uint32_t c = count_of(cnt, k);
        c_mine += c;
        w_mine += (unsigned long long)c * mass_of(k, kmax, vmax, inv_t);
      }
    }
    // tokens (< 2^16) ride in the top 16 bits of the mass (< 2^48): one scan for both
    unsigned long long packed_total;
    const unsigned long long packed_before =
        block_exclusive_scan<unsigned long long>(w_mine | ((unsigned long long)c_mine << 48), scratch64, packed_total);
    const uint32_t c_before = (uint32_t)(packed_before >> 48);
    const unsigned long long w_before = packed_before & 0xffffffffffffull;
    unsigned long long z = packed_total & 0xffffffffffffull;
    const uint32_t c_total = (uint32_t)(packed_total >> 48);                  // tokens that are not NaN
    // ---- top-k: smallest key that stays, and the mass down to it ------------------------------------------------
    uint32_t keep_from = 0u;
    if (top_k > 0 && (uint32_t)top_k < c_total) {
      if (c_before < (uint32_t)top_k && c_before + c_mine >= (uint32_t)top_k) {
        uint32_t cum = c_before;
        unsigned long long wcum = w_before;
        KeyCursor cur = start;
        for (int i = 0; i < mine; ++i) {
          const uint32_t k = cur.next(bm, sm, top);
          const uint32_t c = count_of(cnt, k);
          cum += c;
          wcum += (unsigned long long)c * mass_of(k, kmax, vmax, inv_t);
          if (cum >= (uint32_t)top_k) { sh_key = k; sh_mass = wcum; break; }
        }
      }
      __syncthreads();
      keep_from = sh_key;
      z = sh_mass;
      __syncthreads();
    }
    // ---- top-p: last key that stays and how many of its tokens --------------------------------------------------
    uint32_t cut_key = keep_from, cut_n = 0xffffffffu;      // default: nothing more is removed
    unsigned long long z_kept = z;
    if (top_p < 1.0f) {
      const unsigned long long limit = (unsigned long long)((double)fmaxf(top_p, 0.0f) * (double)z);
      if (limit < z) {                                       // the cut lies above keep_from: one thread holds it
        if (w_before <= limit && w_before + w_mine > limit) {
          unsigned long long cum = w_before;
          KeyCursor cur = start;
          for (int i = 0; i < mine; ++i) {
            const uint32_t k = cur.next(bm, sm, top);
            const uint32_t c = count_of(cnt, k);
            const unsigned long long q = mass_of(k, kmax, vmax, inv_t);
            const unsigned long long g = (unsigned long long)c * q;
            if (cum + g > limit) {                           // token i of this value stays iff cum + i*q <= limit
              const unsigned long long n = min((unsigned long long)c, (limit - cum) / q + 1ull);
              sh_key = k; sh_n = (uint32_t)n; sh_mass = cum + n * q;
              break;
            }
            cum += g;
          }
        }
        __syncthreads();
        cut_key = sh_key; cut_n = sh_n; z_kept = sh_mass;
        __syncthreads();
      }
    }
    // ---- the draw: first kept token whose cumulative mass exceeds u * (kept mass); it lies above the cut ----------
    float u = uniforms[blockIdx.x];
    u = fminf(fmaxf(u, 0.0f), 0.99999994f);
    unsigned long long target = (unsigned long long)((double)u * (double)z_kept);
    if (target >= z_kept) target = z_kept - 1ull;            // z_kept >= 2^32
    if (w_before <= target && w_before + w_mine > target) {
      unsigned long long cum = w_before;
      KeyCursor cur = start;
      for (int i = 0; i < mine; ++i) {
        const uint32_t k = cur.next(bm, sm, top);
        uint32_t c = count_of(cnt, k);
        if (k == cut_key) c = min(c, cut_n);
        const unsigned long long q = mass_of(k, kmax, vmax, inv_t);
        const unsigned long long g = (unsigned long long)c * q;
        if (cum + g > target) { sh_key = k; sh_n = (uint32_t)((target - cum) / q); break; }
        cum += g;
      }
    }
    __syncthreads();
    draw_key = sh_key; draw_rank = sh_n;
    __syncthreads();
  }

  // ---- pass 2 over the row: the draw_rank-th token (ascending id) whose value is draw_key ----------------------------
  // each warp takes one contiguous segment of at most 8 x 256 elements, 8 consecutive elements per lane and step
  const int seg = (((cols + 31) / 32) + 255) & ~255;
  const int w0 = min(cols, wid * seg), w1 = min(cols, w0 + seg);
  const uint32_t draw_raw = key_to_raw(draw_key), pat2 = draw_raw | (draw_raw << 16);
  uint32_t step_count = 0u;                                  // matches per step, 4 bits each (a lane sees <= 8 per step)
  {
    uint4 q[8];
    if (vec && w0 + seg <= w1) {                             // a full segment inside the row: nothing between the loads
#pragma unroll
      for (int b = 0; b < 8; ++b)
        q[b] = (b * 256 < seg) ? canon_zero(__ldcg(reinterpret_cast<const uint4*>(bits + w0 + b * 256 + lane * 8)))
                               : make_uint4(0u, 0u, 0u, 0u);
    } else {
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        const int i = w0 + b * 256 + lane * 8;
        q[b] = (i < w1) ? load_raw8(bits, i, cols, vec) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const int i = w0 + b * 256 + lane * 8;
      const uint32_t c = (i < w1) ? count_equal8(q[b], i, cols, draw_raw, pat2) : 0u;
      step_count |= c << (4 * b);
    }
  }
  uint32_t in_seg = 0u;
#pragma unroll
  for (int b = 0; b < 8; ++b) in_seg += (step_count >> (4 * b)) & 15u;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) in_seg += __shfl_xor_sync(0xffffffffu, in_seg, o);   // matches in this warp's segment
  uint32_t tot;
  uint32_t first = block_exclusive_scan<uint32_t>(lane == 0 ? in_seg : 0u, scratch32, tot);
  first = __shfl_sync(0xffffffffu, first, 0);                                           // matches in earlier segments
  if (draw_rank >= tot) draw_rank = tot ? tot - 1u : 0u;     // cannot happen for counts taken from the same row
  if (first <= draw_rank && first + in_seg > draw_rank) {    // warp-uniform: the drawn token is in this segment
    uint32_t seen = first;
    for (int b = 0; b < 8; ++b) {
      const uint32_t c = (step_count >> (4 * b)) & 15u;
      uint32_t inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
      }
      const uint32_t step_total = __shfl_sync(0xffffffffu, inc, 31);
      if (seen + step_total > draw_rank) {                   // the token is in this step: one lane reads its 8 again
        uint32_t at = seen + inc - c;                        // matches before this lane's elements
        if (at <= draw_rank && at + c > draw_rank) {
          const int i = w0 + b * 256 + lane * 8;
          const uint4 q = load_raw8(bits, i, cols, vec);
          const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (i + j < cols && ((w[j >> 1] >> ((j & 1) << 4)) & 0xffffu) == draw_raw) {
              if (at == draw_rank) out[blockIdx.x] = (int64_t)(i + j);
              ++at;
            }
          }
        }
        break;
      }
      seen += step_total;
    }
  }
}

}  // namespace hb200

using namespace hb200;

extern "C" int hb200_sample_rows(const void* logits, int64_t rows, int cols, int64_t ld, float temperature, int top_k,
                                 float top_p, const float* uniforms, int64_t* out, void* stream) {
  HB_REQUIRE(logits && out, HB200_ERR_INVALID, "sample_rows: null pointer");
  HB_REQUIRE(rows >= 0 && cols >= 1 && ld >= cols, HB200_ERR_INVALID, "sample_rows: bad shape");
  HB_REQUIRE(cols <= 65535, HB200_ERR_UNSUPPORTED, "sample_rows: at most 65535 columns (16-bit value counters), got %d", cols);
  HB_REQUIRE(top_k >= 0, HB200_ERR_INVALID, "sample_rows: top_k must be >= 0 (0 = off)");
  const bool greedy = !(temperature > 0.0f) || top_k == 1;
  HB_REQUIRE(greedy || uniforms, HB200_ERR_INVALID, "sample_rows: uniforms are required unless the choice is greedy");
  if (rows == 0) return HB200_OK;
  HB_PROPAGATE(ensure_dynamic_smem((const void*)sample_rows_kernel, SMP_SMEM));
  sample_rows_kernel<<<(unsigned)rows, SMP_THREADS, SMP_SMEM, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)logits, cols, ld, temperature, top_k, top_p, uniforms, out);
  HB_CUDA(cudaGetLastError());
  return HB200_OK;
}
