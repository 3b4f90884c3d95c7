// Cached decode: one new token per sequence through every block against the latent-space KV cache.
//
// The reference has no decode path; this executor adds a latent-space KV cache for autoregressive decode.
// Per block and step (B sequences in lockstep, position p = *state.pos read from device memory by every kernel, so
// the same launch sequence - and a CUDA graph of it - serves every step):
//
//   a    = AdaRMSNorm(x)                                       (exit norm of the previous block / embed_norm)
//   qkv  = a Wqkv^T                                            skinny tcgen05 GEMM (gemm_skinny.cu), M = B
//   conv prep: window of q|k rows p-4..p (halo + new row), grouped conv1 on its last three rows, written as the
//              im2col rows [y1(p-2) | y1(p-1) | y1(p)] of the dense conv; value row [v_curr(p) | v_shift(p-1)] appended
//              to the value cache; halo and v_shift advanced                         decode_conv_prep_kernel
//   c2q  = im2col_q W2q^T                                      skinny GEMM (the repacked conv2 weights ARE the
//                                                              [C_out, 3*C_in] matrices these products need)
//   c2k  = im2col_k W2k^T (small: on the CUDA cores), QK-mean, L2 norm, temperature, RoPE(p); key appended to the
//          key cache                                                                 decode_qk_finish_kernel
//   o    = softmax(q K^T / sqrt(hd)) V over the p+1 cached positions                 decode_attention_kernel
//   cur  = x + 0.5 * o Wo^T                                    skinny GEMM, residual epilogue
//   per recursion: MoR depth (first recursion), MoD score; "selected" iff fewer than k cached scores are >= the new
//   score (k = int((p+1) * capacity), the newest position loses ties); gather-norm of the selected & active rows
//                                                                                    decode_route_kernel
//   gate_up / down skinny GEMMs with the device-side row count
//   x'   = RMSNorm(cur) (+ next block's input norm)                                  decode_dual_norm_kernel
// then the final norm, the output projection for the B rows, the greedy choice, and p += 1.
//
// The step is a chain of ~19 small launches per block, each a programmatic-dependent-launch link.  What bounds it is
// the number of dependent memory round trips per kernel, not bytes or launches, so every kernel here requests its
// static weights before the wait on its predecessor and everything else in one batch right after it; and because a
// chained kernel starts before its predecessor ends, everything the chain writes is read through L2 only.
#include <cmath>
#include <utility>

#include "gemm_epilogue.cuh"
#include "row_kernels.cuh"
#include "tcgen05.cuh"
#include "tma_host.cuh"

namespace hb200 {

int launch_argmax_rows(const void* x, int64_t rows, int cols, int64_t ld, int64_t* out, cudaStream_t st, bool chained);

struct DecodeWs {
  __nv_bfloat16 *sout, *x0, *x1, *a, *qkv, *aq, *ak, *c2q, *qnew, *o, *cur, *ug, *act, *hid, *logits;
  float *qm, *km, *score, *rlogit;
  int32_t *depth, *rows, *counts, *hints;
  size_t bytes;
};

static size_t dalign(size_t v) { return (v + 255) / 256 * 256; }

static DecodeWs carve_decode(const hb200_model* m, int B, void* base) {
  const size_t D = m->dim, lat = (size_t)m->n_heads * m->head_dim, kvd = (size_t)m->n_kv_heads * m->head_dim,
               F = m->ffn_hidden, hd = m->head_dim, ld = ((size_t)m->vocab + 7) / 8 * 8;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    void* p = base ? (void*)((char*)base + off) : nullptr;
    off += dalign(bytes);
    return p;
  };
  DecodeWs w{};
  w.sout = (__nv_bfloat16*)take(m->static_routing ? B * D * 2 : 0);   // static routing: weighted sum of the recursion states
  w.x0 = (__nv_bfloat16*)take(B * D * 2);
  w.x1 = (__nv_bfloat16*)take(B * D * 2);
  w.a = (__nv_bfloat16*)take(B * D * 2);
  w.qkv = (__nv_bfloat16*)take(B * (lat + 2 * kvd) * 2);
  w.aq = (__nv_bfloat16*)take(B * 3 * lat * 2);
  w.ak = (__nv_bfloat16*)take(B * 3 * kvd * 2);
  w.c2q = (__nv_bfloat16*)take(B * lat * 2);
  w.qnew = (__nv_bfloat16*)take(B * lat * 2);
  w.o = (__nv_bfloat16*)take(B * lat * 2);
  w.cur = (__nv_bfloat16*)take(B * D * 2);
  w.ug = (__nv_bfloat16*)take(B * D * 2);
  w.act = (__nv_bfloat16*)take(B * F * 2);
  w.hid = (__nv_bfloat16*)take(B * D * 2);
  w.logits = (__nv_bfloat16*)take(B * ld * 2);
  w.qm = (float*)take(B * hd * 4);
  w.km = (float*)take(B * hd * 4);
  w.score = (float*)take(B * 4);
  w.rlogit = (float*)take(B * 4);
  w.depth = (int32_t*)take(B * 4);
  w.rows = (int32_t*)take(B * 4);
  w.counts = (int32_t*)take((size_t)m->n_blocks * m->n_rec * 4);
  w.hints = (int32_t*)take((size_t)m->n_blocks * m->n_rec * 2 * 4);   // row counts of the previous step, per GEMM site
  w.bytes = off;
  return w;
}

// ---- conv prep: one CTA per sequence ---------------------------------------------------------------------------
// dynamic smem: win[5][C] + y1[3][C] floats.  Laid out for latency: the conv1 weight rows of this thread's (up to
// three) output channels are static and are requested before the wait on the predecessor (head_dim <= 32: they fit in
// registers); the position, the halo, the new q|k row and the value pieces are requested together right after it.
constexpr int CONV_CPT = 3;       // output channels per thread held in registers: latent + kv width <= 768
template <int HD>
__global__ void __launch_bounds__(256) decode_conv_prep_kernel(
    const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ w1, __nv_bfloat16* __restrict__ halo,
    __nv_bfloat16* __restrict__ vshift, __nv_bfloat16* __restrict__ vcache, __nv_bfloat16* __restrict__ aq,
    __nv_bfloat16* __restrict__ ak, float* __restrict__ qm, float* __restrict__ km, int32_t* __restrict__ first_count,
    const int32_t* __restrict__ pos_ptr, int B, int H, int KV, int capacity) {
  extern __shared__ float smem_f[];
  constexpr int hd = HD;
  constexpr int WV = 3 * HD / 8;                  // 16-byte pieces of one weight row
  constexpr bool PRE = HD <= 32;
  const int lat = H * hd, kvd = KV * hd, C = lat + kvd, qkv_ld = lat + 2 * kvd, half = kvd / 2;
  const int b = blockIdx.x, tid = threadIdx.x;
  const bool in_regs = PRE && C <= CONV_CPT * 256;
  chain_release();
  uint4 wreg[PRE ? CONV_CPT : 1][PRE ? WV : 1];
  if (in_regs) {
#pragma unroll
    for (int k = 0; k < CONV_CPT; ++k) {
      const int c = tid + k * 256;
      if (c < C) {
#pragma unroll
        for (int e = 0; e < WV; ++e) wreg[k][e] = *reinterpret_cast<const uint4*>(w1 + (size_t)c * 3 * hd + e * 8);
      }
    }
  }
  chain_wait();
  float* win = smem_f;            // [5][C]: positions p-4 .. p
  float* y1 = smem_f + 5 * C;     // [3][C]: positions p-2 .. p
  if (b == 0 && tid == 0) *first_count = 0;   // row counter of this block's first recursion (see decode_route_kernel)
  const int pos = __ldcg(pos_ptr);
  __nv_bfloat16* hb = halo + (size_t)b * 4 * C;
  const __nv_bfloat16* row = qkv + (size_t)b * qkv_ld;
  // (everything other kernels of the chain write is read through L2, see load_bf16x8_cg)
  for (int i = tid * 8; i < 5 * C; i += 256 * 8) {        // C % 8 == 0: a piece never straddles halo and new row
    float f[8];
    load_bf16x8_cg(i < 4 * C ? hb + i : row + (i - 4 * C), f);
#pragma unroll
    for (int q = 0; q < 8; ++q) win[i + q] = f[q];
  }
  // this thread's value channel: current half from the new row, shifted half from the previous position
  float vval = 0.f, vnext = 0.f;
  if (tid < kvd) vval = (tid < half) ? ldcg_bf16(row + C + tid) : ldcg_bf16(vshift + (size_t)b * half + (tid - half));
  if (tid < half) vnext = ldcg_bf16(row + C + half + tid);
  if (pos >= capacity) return;    // cache full: the step is a no-op (the host checks capacity before launching)
  __syncthreads();
  // grouped conv1 (kernel 3, causal) on rows 2..4 of the window; rounded to bf16 like the prefill's y1 tile.
  // One thread per output channel: its weight row (3 taps x hd inputs) serves all three positions.
  auto conv_channel = [&](int c, auto&& weight_piece) {
    const int hb0 = (c / hd) * hd;
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f;
#pragma unroll
    for (int e = 0; e < WV; ++e) {
      const uint4 raw = weight_piece(e);
      const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
      float wv[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        wv[2 * q] = __uint_as_float(w4[q] << 16);
        wv[2 * q + 1] = __uint_as_float(w4[q] & 0xffff0000u);
      }
      const int j = (e * 8) / hd, ci0 = e * 8 - j * hd;        // hd % 8 == 0: the 8 weights share a tap
      const float* x0 = win + j * C + hb0 + ci0;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        acc0 += wv[q] * x0[q];
        acc1 += wv[q] * x0[C + q];
        acc2 += wv[q] * x0[2 * C + q];
      }
    }
    y1[c] = __bfloat162float(__float2bfloat16_rn(acc0));
    y1[C + c] = __bfloat162float(__float2bfloat16_rn(acc1));
    y1[2 * C + c] = __bfloat162float(__float2bfloat16_rn(acc2));
  };
  if (in_regs) {
#pragma unroll
    for (int k = 0; k < CONV_CPT; ++k) {
      const int c = tid + k * 256;
      if (c < C) conv_channel(c, [&](int e) { return wreg[k][e]; });
    }
  } else {
    for (int c = tid; c < C; c += 256) {
      const __nv_bfloat16* wr = w1 + (size_t)c * 3 * hd;
      conv_channel(c, [&](int e) { return *reinterpret_cast<const uint4*>(wr + e * 8); });
    }
  }
  // QK-mean halves and the value row
  for (int d = tid; d < 2 * hd; d += 256) {
    if (d < hd) {
      float sacc = 0.f;
      for (int h = 0; h < H; ++h) sacc += win[4 * C + h * hd + d];
      qm[(size_t)b * hd + d] = sacc * (0.5f / (float)H);
    } else {
      const int dd = d - hd;
      float sacc = 0.f;
      for (int g = 0; g < KV; ++g) sacc += win[4 * C + lat + g * hd + dd];
      km[(size_t)b * hd + dd] = sacc * (0.5f / (float)KV);
    }
  }
  if (tid < kvd) vcache[(((size_t)b * KV + tid / hd) * capacity + pos) * hd + (tid % hd)] = __float2bfloat16_rn(vval);
  __syncthreads();
  // im2col rows of the dense conv: [tap 0 | tap 1 | tap 2], each tap = y1 of one position
  for (int i = tid; i < 3 * C; i += 256) {
    const int j = i / C, c = i % C;
    const __nv_bfloat16 v = __float2bfloat16_rn(y1[i]);
    if (c < lat) aq[(size_t)b * 3 * lat + j * lat + c] = v;
    else ak[(size_t)b * 3 * kvd + j * kvd + (c - lat)] = v;
  }
  // advance the halo (drop the oldest row) and the v_shift half
  for (int i = tid; i < 4 * C; i += 256) hb[i] = __float2bfloat16_rn(win[C + i]);
  if (tid < half) vshift[(size_t)b * half + tid] = __float2bfloat16_rn(vnext);
}

// ---- QK finish: one CTA per sequence, hd/2 lanes per head ---------------------------------------------------------
// Latency layout: the temperature and (when they fit in registers) this thread's share of the key conv weights are
// static and requested before the wait; the q / k finishing runs lph = hd/2 lanes per head (one RoPE pair per lane),
// i.e. up to four heads per warp side by side, so all heads of a sequence are done in one or two passes.
constexpr int QKF_WPT = 8;        // 16-byte weight pieces per thread held in registers
__global__ void __launch_bounds__(256) decode_qk_finish_kernel(
    const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ c2q, const __nv_bfloat16* __restrict__ ak,
    const __nv_bfloat16* __restrict__ w2k, const float* __restrict__ qm, const float* __restrict__ km, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, const float* __restrict__ temp, __nv_bfloat16* __restrict__ qnew,
    __nv_bfloat16* __restrict__ kcache, const int32_t* __restrict__ pos_ptr, int H, int KV, int hd, int capacity) {
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int lat = H * hd, kvd = KV * hd, qkv_ld = lat + 2 * kvd;
  const bool same_heads = (H == KV);
  extern __shared__ float smem_f[];
  float* a_row = smem_f;                 // [3 * kvd]
  float* c2k = smem_f + 3 * kvd;         // [kvd]
  // key conv: tpc threads per output channel, each a contiguous run of `per` 16-byte pieces of the channel's weight row
  const int pieces = 3 * kvd / 8;
  const int tpc = 256 / kvd;             // > 0: kvd <= 256
  const bool pow2 = tpc > 0 && (tpc & (tpc - 1)) == 0 && tpc <= 32;
  const int per = pow2 ? (pieces + tpc - 1) / tpc : 0;
  const bool in_regs = pow2 && per <= QKF_WPT;
  const int n_ch = in_regs ? tid / tpc : 0, part = in_regs ? tid % tpc : 0;
  chain_release();
  uint4 wreg[QKF_WPT];
  if (in_regs) {
#pragma unroll
    for (int q = 0; q < QKF_WPT; ++q) {
      const int e = part * per + q;
      if (q < per && e < pieces) wreg[q] = *reinterpret_cast<const uint4*>(w2k + (size_t)n_ch * 3 * kvd + e * 8);
    }
  }
  const float temperature = *temp;
  chain_wait();
  const int pos = __ldcg(pos_ptr);
  for (int i = tid; i < 3 * kvd; i += 256) a_row[i] = ldcg_bf16(ak + (size_t)b * 3 * kvd + i);
  if (pos >= capacity) return;
  __syncthreads();
  // the key side of the dense conv is small (kvd x 3 kvd): done here on the CUDA cores, result rounded to bf16 like a
  // stored GEMM output
  if (in_regs) {
    float acc = 0.f;
#pragma unroll
    for (int q = 0; q < QKF_WPT; ++q) {
      const int e = part * per + q;
      if (q < per && e < pieces) {
        const uint32_t w4[4] = {wreg[q].x, wreg[q].y, wreg[q].z, wreg[q].w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc += __uint_as_float(w4[j] << 16) * a_row[e * 8 + 2 * j] + __uint_as_float(w4[j] & 0xffff0000u) * a_row[e * 8 + 2 * j + 1];
      }
    }
    for (int off = tpc >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (part == 0 && n_ch < kvd) c2k[n_ch] = __bfloat162float(__float2bfloat16_rn(acc));
  } else {
    for (int n = tid; n < kvd; n += 256) {
      const __nv_bfloat16* wr = w2k + (size_t)n * 3 * kvd;
      float acc = 0.f;
      for (int e = 0; e < 3 * kvd; e += 8) {
        float wv[8];
        load_bf16x8(wr + e, wv);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc += wv[q] * a_row[e + q];
      }
      c2k[n] = __bfloat162float(__float2bfloat16_rn(acc));
    }
  }
  __syncthreads();
  // lph lanes per head, hpw heads per warp
  const int lph = hd / 2, hpw = 32 / lph, sub = lane / lph, l = lane % lph;
  const int d0 = 2 * l;
  const float cs = cos_t[(size_t)pos * lph + l], sn = sin_t[(size_t)pos * lph + l];
  for (int base_h = warp * hpw; base_h < H + KV; base_h += 8 * hpw) {     // warp-uniform trip count
    const int hh = base_h + sub;
    const bool valid = hh < H + KV;
    const bool is_k = hh >= H;
    const int h = is_k ? hh - H : hh;
    float v0 = 0.f, v1 = 0.f;
    if (valid) {
      float c0, c1;
      if (same_heads) {   // one query head per kv head: both sides couple with 0.5 * (q0 + k0) of that head
        const __nv_bfloat16* row = qkv + (size_t)b * qkv_ld;
        c0 = 0.5f * (ldcg_bf16(row + h * hd + d0) + ldcg_bf16(row + lat + h * hd + d0));
        c1 = 0.5f * (ldcg_bf16(row + h * hd + d0 + 1) + ldcg_bf16(row + lat + h * hd + d0 + 1));
      } else {            // otherwise with half the head-mean of the other side
        const float* mean = (is_k ? qm : km) + (size_t)b * hd;
        c0 = __ldcg(mean + d0);
        c1 = __ldcg(mean + d0 + 1);
      }
      const __nv_bfloat16* conv = c2q + (size_t)b * lat + h * hd;
      v0 = (is_k ? c2k[h * hd + d0] : ldcg_bf16(conv + d0)) + c0;
      v1 = (is_k ? c2k[h * hd + d0 + 1] : ldcg_bf16(conv + d0 + 1)) + c1;
    }
    float ss = v0 * v0 + v1 * v1;
    for (int off = lph >> 1; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (valid) {
      const float inv = (is_k ? temperature : 1.0f) / fmaxf(sqrtf(ss), 1e-12f);
      v0 *= inv;
      v1 *= inv;
      const __nv_bfloat162 out = __floats2bfloat162_rn(v0 * cs - v1 * sn, v0 * sn + v1 * cs);
      __nv_bfloat16* dst = is_k ? kcache + (((size_t)b * KV + h) * capacity + pos) * hd + d0
                                : qnew + (size_t)b * lat + h * hd + d0;
      *reinterpret_cast<__nv_bfloat162*>(dst) = out;
    }
  }
}

// ---- attention of one query per head against the cache: CTA = (kv head, sequence) -------------------------------
// Pass 1: one thread per cached key, logits of the G query heads of this kv head into shared memory, row maxima.
// Pass 2: exponentials and row sums.  Pass 3: P V with 16-byte loads of V (lane = 8-dim chunk, key slices across
// the rest of the CTA), reduced by shuffles and a small shared-memory table.  Exact softmax for any temperature.
// STAGED: the cached K rows of this (sequence, kv head) are first copied into shared memory with cp.async (one round
// trip with every 16-byte piece in flight at once, L1 bypassed); once the logits exist the same buffer receives the V
// rows while the exponentials are computed.  Used while all CTAs of the grid are resident at once.
constexpr int DATT_THREADS = 256;
constexpr int DATT_WARPS = DATT_THREADS / 32;
constexpr int DATT_GMAX = 8;      // query heads per kv head
template <int HD, bool STAGED>
__global__ void __launch_bounds__(DATT_THREADS) decode_attention_kernel(
    const __nv_bfloat16* __restrict__ qnew, const __nv_bfloat16* __restrict__ kcache,
    const __nv_bfloat16* __restrict__ vcache, __nv_bfloat16* __restrict__ o, const int32_t* __restrict__ pos_ptr, int H,
    int KV, int capacity, float scale_log2) {
  extern __shared__ float smem_f[];
  constexpr int CH = HD / 8;                 // 16-byte chunks per row
  const int kvh = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = H / KV, lat = H * HD;
  chain_release();
  chain_wait();
  const int n_keys = min(__ldcg(pos_ptr) + 1, capacity);
  float* qs = smem_f;                          // [G][HD], pre-scaled by scale * log2(e)
  float* red = qs + DATT_GMAX * HD;            // [DATT_WARPS][DATT_GMAX]
  float* part = red + DATT_WARPS * DATT_GMAX;  // [DATT_WARPS][DATT_GMAX][HD]
  float* sc = part + DATT_WARPS * DATT_GMAX * HD;   // [G][capacity]
  const __nv_bfloat16* kb = kcache + ((size_t)b * KV + kvh) * capacity * HD;
  const __nv_bfloat16* vb = vcache + ((size_t)b * KV + kvh) * capacity * HD;
  // staged copies of the cached rows (16-byte aligned: the tables before them are multiples of 4 floats)
  const uint32_t stage_k = s_addr(sc + (size_t)((G * capacity + 3) & ~3));
  const uint32_t stage_v = stage_k;              // V follows K in the same buffer (after pass 1)
  const int pieces = n_keys * CH;
  if (STAGED) {
    for (int i = tid; i < pieces; i += DATT_THREADS) cp_async16(stage_k + (uint32_t)i * 16u, kb + (size_t)i * 8);
    cp_async16_commit();
  }
  for (int i = tid; i < G * HD; i += DATT_THREADS)
    qs[i] = ldcg_bf16(qnew + (size_t)b * lat + (size_t)(kvh * G) * HD + i) * scale_log2;
  if (STAGED) cp_async16_wait_all();
  __syncthreads();
  auto row8 = [&](uint32_t stage, const __nv_bfloat16* gptr, int key, int c, float (&f)[8]) {
    if (STAGED) {
      const uint4 raw = ld_shared_v4(stage + (uint32_t)(key * HD + c * 8) * 2u);
      const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        f[2 * q] = __uint_as_float(w4[q] << 16);
        f[2 * q + 1] = __uint_as_float(w4[q] & 0xffff0000u);
      }
    } else {
      load_bf16x8_cg(gptr + (size_t)key * HD + c * 8, f);
    }
  };
  // pass 1
  float mx[DATT_GMAX];
#pragma unroll
  for (int g = 0; g < DATT_GMAX; ++g) mx[g] = -INFINITY;
#pragma unroll 2
  for (int key = tid; key < n_keys; key += DATT_THREADS) {
    float kf[HD];
#pragma unroll
    for (int c = 0; c < CH; ++c) row8(stage_k, kb, key, c, *reinterpret_cast<float(*)[8]>(&kf[c * 8]));
#pragma unroll
    for (int g = 0; g < DATT_GMAX; ++g) {
      if (g < G) {
        float s = 0.f;
#pragma unroll
        for (int d = 0; d < HD; ++d) s += qs[g * HD + d] * kf[d];
        sc[(size_t)g * capacity + key] = s;
        mx[g] = fmaxf(mx[g], s);
      }
    }
  }
#pragma unroll
  for (int g = 0; g < DATT_GMAX; ++g) {
    float v = mx[g];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    if (lane == 0) red[warp * DATT_GMAX + g] = v;
  }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < DATT_GMAX; ++g) {
    float v = -INFINITY;
#pragma unroll
    for (int wv = 0; wv < DATT_WARPS; ++wv) v = fmaxf(v, red[wv * DATT_GMAX + g]);
    mx[g] = v;
  }
  __syncthreads();
  if (STAGED) {   // every thread is past pass 1: the K rows are dead, V takes their place while pass 2 runs
    for (int i = tid; i < pieces; i += DATT_THREADS) cp_async16(stage_v + (uint32_t)i * 16u, vb + (size_t)i * 8);
    cp_async16_commit();
  }
  // pass 2 (each thread revisits the logits it wrote)
  float sum[DATT_GMAX];
#pragma unroll
  for (int g = 0; g < DATT_GMAX; ++g) sum[g] = 0.f;
  for (int key = tid; key < n_keys; key += DATT_THREADS) {
#pragma unroll
    for (int g = 0; g < DATT_GMAX; ++g) {
      if (g < G) {
        const float pr = exp2f(sc[(size_t)g * capacity + key] - mx[g]);
        sc[(size_t)g * capacity + key] = pr;
        sum[g] += pr;
      }
    }
  }
#pragma unroll
  for (int g = 0; g < DATT_GMAX; ++g) {
    const float v = warp_sum(sum[g]);
    if (lane == 0) red[warp * DATT_GMAX + g] = v;
  }
  if (STAGED) cp_async16_wait_all();
  __syncthreads();
#pragma unroll
  for (int g = 0; g < DATT_GMAX; ++g) {
    float v = 0.f;
#pragma unroll
    for (int wv = 0; wv < DATT_WARPS; ++wv) v += red[wv * DATT_GMAX + g];
    sum[g] = v;
  }
  // pass 3
  const int chunk = tid % CH, slice = tid / CH;
  constexpr int NSLICE = DATT_THREADS / CH;
  float acc[DATT_GMAX][8];
#pragma unroll
  for (int g = 0; g < DATT_GMAX; ++g)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[g][j] = 0.f;
#pragma unroll 4
  for (int key = slice; key < n_keys; key += NSLICE) {
    float vf[8];
    row8(stage_v, vb, key, chunk, vf);
#pragma unroll
    for (int g = 0; g < DATT_GMAX; ++g) {
      if (g < G) {
        const float pr = sc[(size_t)g * capacity + key];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] += pr * vf[j];
      }
    }
  }
#pragma unroll
  for (int g = 0; g < DATT_GMAX; ++g) {
    if (g < G) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float v = acc[g][j];
#pragma unroll
        for (int off = 16; off >= CH; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane < CH) part[(warp * DATT_GMAX + g) * HD + lane * 8 + j] = v;
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < G * HD; i += DATT_THREADS) {
    const int g = i / HD, d = i % HD;
    float v = 0.f;
#pragma unroll
    for (int wv = 0; wv < DATT_WARPS; ++wv) v += part[(wv * DATT_GMAX + g) * HD + d];
    o[(size_t)b * lat + (size_t)(kvh * G + g) * HD + d] = __float2bfloat16_rn(v / sum[g]);
  }
}

static size_t decode_attention_smem(int hd, int G, int capacity) {
  return ((size_t)DATT_GMAX * hd + DATT_WARPS * DATT_GMAX + (size_t)DATT_WARPS * DATT_GMAX * hd + (size_t)G * capacity) *
         sizeof(float);
}

template <int HD>
static int launch_decode_attention(const __nv_bfloat16* qnew, const __nv_bfloat16* kc, const __nv_bfloat16* vc,
                                   __nv_bfloat16* o, const int32_t* pos, int B, int H, int KV, int capacity, float scale,
                                   cudaStream_t st, bool chain) {
  const size_t base = decode_attention_smem(HD, H / KV, capacity) + 16;
  const size_t staged = base + (size_t)capacity * HD * 2;
  // staging is worth it while every CTA of the grid is resident at once (the kernel is then a latency chain); larger
  // grids keep the small footprint and stream from L2
  const long long resident = staged <= 200 * 1024 ? (long long)sm_count() * ((226 * 1024) / (staged + 1024)) : 0;
  if ((long long)KV * B <= resident) {
    HB_PROPAGATE(ensure_dynamic_smem((const void*)decode_attention_kernel<HD, true>, staged));
    return launch_chained(decode_attention_kernel<HD, true>, dim3(KV, B), dim3(DATT_THREADS), staged, st, chain, 1, qnew, kc,
                          vc, o, pos, H, KV, capacity, scale * 1.4426950408889634f);
  }
  HB_PROPAGATE(ensure_dynamic_smem((const void*)decode_attention_kernel<HD, false>, base));
  return launch_chained(decode_attention_kernel<HD, false>, dim3(KV, B), dim3(DATT_THREADS), base, st, chain, 1, qnew, kc, vc,
                        o, pos, H, KV, capacity, scale * 1.4426950408889634f);
}

// ---- routing of the newest position + gather-norm: one CTA per sequence -------------------------------------
// Per recursion r of a block, for every sequence b:
//   router (r == 0, adaptive): depth[b] from the raw row;
//   MoD: score s_b of AdaRMSNorm(cur_b + rec) (same formula as the prefill's score pass); "selected" iff fewer than
//        k cached scores of b are >= s_b, k = int((p+1) * capacity) clamped to [1, p+1] (the newest position loses
//        ties); s_b is appended to the score cache;
//   if selected(b) and depth[b] >= r: a compact slot j is taken from the counter, rows[j] = b and
//   ug[j] = AdaRMSNorm(cur_b + rec) straight from the registers that hold the row.
// Slots are handed out in arrival order: which slot a row gets does not change its result (rows of the two MLP
// contractions are independent), only where it sits in the compact buffers.  *count must be zero on entry; the
// kernel zeroes `next_count` (the counter of the following recursion) for its successor.
//
// The kernel is a latency chain, not a bandwidth problem (one 4 KB row per CTA), so it is laid out to need two
// memory round trips: every thread owns 8 columns; the per-column vectors (static weights) are requested before
// the wait on the predecessor, and the row piece, the position, the depth and this thread's slice of the score cache
// (read up to the cache capacity, masked by the position afterwards) are all requested together right after it.
constexpr int ROUTE_THREADS = 256;
constexpr int ROUTE_CACHE_PER_THREAD = 16;     // score-cache entries per thread requested up front (the first 4096)
template <bool HAS_MOD, bool HAS_ROUTER>
__global__ void __launch_bounds__(ROUTE_THREADS) decode_route_kernel(
    const __nv_bfloat16* __restrict__ cur, const float* __restrict__ rec, const float* __restrict__ norm2_w,
    const float* __restrict__ mod_wn, const float* __restrict__ mod_b, const float* __restrict__ mor_w,
    const float* __restrict__ mor_b, float* __restrict__ score_cache, int32_t* __restrict__ depth, int min_active,
    int32_t* __restrict__ rows, int32_t* __restrict__ count, int32_t* __restrict__ next_count,
    __nv_bfloat16* __restrict__ ug, const int32_t* __restrict__ pos_ptr, int B, int D, int capacity, float cap_ratio,
    float eps, int n_rec, int min_d, float* __restrict__ stat_q, float* __restrict__ stat_logit) {
  // stat_q != nullptr: static routing - every row is taken, the MoD probability sigmoid(clamp(score)) and (recursion 0)
  // the raw depth-router logit are left for decode_static_update_kernel
  __shared__ float red[ROUTE_THREADS / 32][4];
  __shared__ int bcast[2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = blockIdx.x;
  const int i = tid * 8;
  const bool have = i < D;
  chain_release();
  // ---- static per-column vectors: independent of the predecessor
  float rc[8], g2[8], wn[8], wr[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) rc[j] = g2[j] = wn[j] = wr[j] = 0.f;
  float bias_mod = 0.f, bias_mor = 0.f;
  if (have) {
    const float4 a0 = *reinterpret_cast<const float4*>(rec + i), a1 = *reinterpret_cast<const float4*>(rec + i + 4);
    const float4 b0 = *reinterpret_cast<const float4*>(norm2_w + i), b1 = *reinterpret_cast<const float4*>(norm2_w + i + 4);
    rc[0] = a0.x; rc[1] = a0.y; rc[2] = a0.z; rc[3] = a0.w; rc[4] = a1.x; rc[5] = a1.y; rc[6] = a1.z; rc[7] = a1.w;
    g2[0] = b0.x; g2[1] = b0.y; g2[2] = b0.z; g2[3] = b0.w; g2[4] = b1.x; g2[5] = b1.y; g2[6] = b1.z; g2[7] = b1.w;
    if (HAS_MOD) {
      const float4 c0 = *reinterpret_cast<const float4*>(mod_wn + i), c1 = *reinterpret_cast<const float4*>(mod_wn + i + 4);
      wn[0] = c0.x; wn[1] = c0.y; wn[2] = c0.z; wn[3] = c0.w; wn[4] = c1.x; wn[5] = c1.y; wn[6] = c1.z; wn[7] = c1.w;
    }
    if (HAS_ROUTER) {
      const float4 d0 = *reinterpret_cast<const float4*>(mor_w + i), d1 = *reinterpret_cast<const float4*>(mor_w + i + 4);
      wr[0] = d0.x; wr[1] = d0.y; wr[2] = d0.z; wr[3] = d0.w; wr[4] = d1.x; wr[5] = d1.y; wr[6] = d1.z; wr[7] = d1.w;
    }
  }
  if (HAS_MOD) bias_mod = mod_b[0];
  if (HAS_ROUTER) bias_mor = mor_b[0];
  chain_wait();
  // ---- everything that depends on earlier kernels, requested in one go
  if (next_count != nullptr && b == 0 && tid == 0) *next_count = 0;
  const int pos = __ldcg(pos_ptr);
  const uint4 raw = have ? __ldcg(reinterpret_cast<const uint4*>(cur + (size_t)b * D + i)) : make_uint4(0, 0, 0, 0);
  int dep = HAS_ROUTER ? 0 : __ldcg(depth + b);
  float cached[ROUTE_CACHE_PER_THREAD];
  float* sc = score_cache + (size_t)b * capacity;
  if (HAS_MOD) {
#pragma unroll
    for (int q = 0; q < ROUTE_CACHE_PER_THREAD; ++q) {
      const int idx = q * ROUTE_THREADS + tid;
      cached[q] = (idx < capacity) ? __ldcg(sc + idx) : 0.f;   // entries at or beyond the position are masked below
    }
  }
  // ---- row statistics
  float v[8], x[8];
  {
    const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      x[2 * j] = __uint_as_float(w4[j] << 16);
      x[2 * j + 1] = __uint_as_float(w4[j] & 0xffff0000u);
    }
  }
  float ss = 0.f, dm = 0.f, lm = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    v[j] = have ? x[j] + rc[j] : 0.f;
    ss += v[j] * v[j];
    if (HAS_MOD) dm += v[j] * wn[j];
    if (HAS_ROUTER) lm += x[j] * wr[j];
  }
  ss = warp_sum(ss);
  if (HAS_MOD) dm = warp_sum(dm);
  if (HAS_ROUTER) lm = warp_sum(lm);
  if (lane == 0) { red[warp][0] = ss; red[warp][1] = dm; red[warp][2] = lm; }
  __syncthreads();
  ss = dm = lm = 0.f;
#pragma unroll
  for (int w8 = 0; w8 < ROUTE_THREADS / 32; ++w8) { ss += red[w8][0]; dm += red[w8][1]; lm += red[w8][2]; }
  const float ri = rsqrtf(ss / (float)D + eps);
  if (HAS_ROUTER) dep = mor_depth_from_logit(lm + bias_mor, n_rec, min_d);
  const bool room = pos < capacity;
  bool sel = true;
  float s = 0.f;
  if (HAS_MOD) {
    double c = (double)cap_ratio;
    c = c < 1e-4 ? 1e-4 : (c > 1.0 ? 1.0 : c);
    int k = (int)((double)(pos + 1) * c);
    k = k < 1 ? 1 : (k > pos + 1 ? pos + 1 : k);
    s = ri * dm + bias_mod;
    const int n = min(pos, capacity);
    int cnt = 0;
#pragma unroll
    for (int q = 0; q < ROUTE_CACHE_PER_THREAD; ++q) {
      const int idx = q * ROUTE_THREADS + tid;
      cnt += (idx < n && cached[q] >= s) ? 1 : 0;
    }
    // positions beyond the register-resident slice (a cache longer than 4096 entries): read on demand
    for (int idx = ROUTE_CACHE_PER_THREAD * ROUTE_THREADS + tid; idx < n; idx += ROUTE_THREADS)
      cnt += (__ldcg(sc + idx) >= s) ? 1 : 0;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, off);
    if (lane == 0) red[warp][3] = __int_as_float(cnt);
    __syncthreads();
    int total = 0;
#pragma unroll
    for (int w8 = 0; w8 < ROUTE_THREADS / 32; ++w8) total += __float_as_int(red[w8][3]);
    sel = total < k;
  }
  const bool is_static = stat_q != nullptr;
  const bool take = room && (is_static || (sel && dep >= min_active));
  if (tid == 0) {
    if (HAS_ROUTER) depth[b] = dep;
    if (HAS_ROUTER && is_static) stat_logit[b] = lm + bias_mor;
    if (is_static) stat_q[b] = HAS_MOD ? 1.f / (1.f + expf(-fminf(fmaxf(s, -10.f), 10.f))) : 1.f;
    if (HAS_MOD && room) sc[pos] = s;
    int j = -1;
    if (take) {
      j = atomicAdd(count, 1);
      rows[j] = b;
    }
    bcast[0] = j;
  }
  __syncthreads();
  const int j = bcast[0];
  if (j < 0 || !have) return;
  float o[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) o[q] = v[q] * ri * g2[q];
  store_bf16x8(ug + (size_t)j * D + i, o);
}

// ---- static routing, one compact row per CTA (slot j holds sequence rows[j]):
//   cur[b] += q * mlp[j] + (1 - q) * u[j];   out[b] (+)= w_r * cur[b]   (static_update_kernel of the prefill, same formulas)
__global__ void __launch_bounds__(256) decode_static_update_kernel(
    __nv_bfloat16* __restrict__ cur, const __nv_bfloat16* __restrict__ mlp, const __nv_bfloat16* __restrict__ u,
    const int32_t* __restrict__ rows, const int32_t* __restrict__ count, const float* __restrict__ stat_q,
    const float* __restrict__ stat_logit, __nv_bfloat16* __restrict__ out, int D, int r, int R, int has_out) {
  chain_release();
  chain_wait();
  const int j = blockIdx.x;
  if (j >= __ldcg(count)) return;
  const int b = __ldcg(rows + j);
  const int i = threadIdx.x * 8;
  if (i >= D) return;
  const float q = __ldcg(stat_q + b);
  float wr = 0.f;
  if (has_out) {
    const float d = (float)(R - 1) / (1.f + expf(-3.f * tanhf(0.5f * __ldcg(stat_logit + b))));
    float sum = 0.f;
    for (int jj = 0; jj < R; ++jj) {
      const float e = expf(-(d - (float)jj) * (d - (float)jj));
      sum += e;
      if (jj == r) wr = e;
    }
    wr /= sum + 1e-8f;
  }
  float c[8], m[8], un[8], o[8];
  load_bf16x8_cg(cur + (size_t)b * D + i, c);
  load_bf16x8_cg(mlp + (size_t)j * D + i, m);
  load_bf16x8_cg(u + (size_t)j * D + i, un);
#pragma unroll
  for (int k = 0; k < 8; ++k) o[k] = 0.f;
  if (has_out && r > 0) load_bf16x8_cg(out + (size_t)b * D + i, o);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    c[k] += q * m[k] + (1.f - q) * un[k];
    o[k] += wr * c[k];
  }
  store_bf16x8(cur + (size_t)b * D + i, c);
  if (has_out) store_bf16x8(out + (size_t)b * D + i, o);
}

// ---- block exit for one row per CTA: y = RMSNorm(src; w1) (or src if w1 == nullptr), z = RMSNorm(y; w2) --------
// Same arithmetic as dual_norm_kernel (row kernels of the prefill), laid out for latency: every thread owns 8 columns,
// both gain vectors are requested before the wait on the predecessor, the row piece right after it.
__global__ void __launch_bounds__(256) decode_dual_norm_kernel(const __nv_bfloat16* __restrict__ src,
                                                               const float* __restrict__ w1, __nv_bfloat16* __restrict__ y,
                                                               const float* __restrict__ w2, __nv_bfloat16* __restrict__ z,
                                                               int D, float eps) {
  __shared__ float red[2][8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int i = tid * 8;
  const bool have = i < D;
  const size_t row = blockIdx.x;
  chain_release();
  float g1[8], g2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) g1[j] = g2[j] = 1.f;
  if (have) {
    if (w1 != nullptr) {
      const float4 a0 = *reinterpret_cast<const float4*>(w1 + i), a1 = *reinterpret_cast<const float4*>(w1 + i + 4);
      g1[0] = a0.x; g1[1] = a0.y; g1[2] = a0.z; g1[3] = a0.w; g1[4] = a1.x; g1[5] = a1.y; g1[6] = a1.z; g1[7] = a1.w;
    }
    const float4 b0 = *reinterpret_cast<const float4*>(w2 + i), b1 = *reinterpret_cast<const float4*>(w2 + i + 4);
    g2[0] = b0.x; g2[1] = b0.y; g2[2] = b0.z; g2[3] = b0.w; g2[4] = b1.x; g2[5] = b1.y; g2[6] = b1.z; g2[7] = b1.w;
  }
  chain_wait();
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = 0.f;
  if (have) load_bf16x8_cg(src + row * D + i, v);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
  ss = warp_sum(ss);
  if (lane == 0) red[0][warp] = ss;
  __syncthreads();
  ss = 0.f;
#pragma unroll
  for (int w8 = 0; w8 < 8; ++w8) ss += red[0][w8];
  if (w1 != nullptr) {
    const float r1 = rsqrtf(ss / (float)D + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(v[j] * r1 * g1[j]));
  }
  if (have) store_bf16x8(y + row * D + i, v);
  float ss2 = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss2 += v[j] * v[j];
  ss2 = warp_sum(ss2);
  if (lane == 0) red[1][warp] = ss2;
  __syncthreads();
  ss2 = 0.f;
#pragma unroll
  for (int w8 = 0; w8 < 8; ++w8) ss2 += red[1][w8];
  const float r2 = rsqrtf(ss2 / (float)D + eps);
  float o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = v[j] * r2 * g2[j];
  if (have) store_bf16x8(z + row * D + i, o);
}

__global__ void decode_fill_kernel(int32_t* p, int n, int32_t val) {
  chain_release();
  chain_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = val;
}

// greedy token bookkeeping at the end of a step
__global__ void decode_advance_kernel(int32_t* pos_ptr, const int64_t* __restrict__ tokens, int64_t* __restrict__ history,
                                      int B, int capacity) {
  chain_release();
  chain_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  const int pos = __ldcg(pos_ptr);
  if (pos >= capacity) return;
  if (b < B && history != nullptr && pos + 1 < capacity) history[(size_t)b * capacity + pos + 1] = __ldcg(tokens + b);
  __syncthreads();
  if (b == 0) *pos_ptr = pos + 1;
}

// Contractions of a decode step: up to 512 rows (four 128-row tiles) -> the cluster split-K weight-streaming kernel
// (gemm_impl 0); larger batches, or gemm_impl 1 (the mma.sync cross-check), take the general entry point.
static int dgemm(const hb200_model* m, const DecodeWs& w, const void* A, const void* W, void* C, int M, int N, int K,
                 int64_t ldc, int epi, const void* resid, float alpha, const int32_t* rows, const int32_t* m_dev,
                 int32_t* err, cudaStream_t st, bool chain, int32_t* m_hint = nullptr) {
  if (m->gemm_impl == 0 && M <= 512) {
    GemmParams p{(const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (__nv_bfloat16*)C, M, N, K, K, K, ldc, epi,
                 (const __nv_bfloat16*)resid, epi == EPI_SCATTER_ADD ? 1.0f : alpha, rows, m_dev, err, m_hint};
    return launch_gemm_skinny(p, st, chain);
  }
  return hb200_gemm_bf16(A, W, C, M, N, K, K, K, ldc, epi, resid, alpha, rows, m_dev, m->gemm_impl, err, st);
}

}  // namespace hb200

using namespace hb200;

extern "C" size_t hb200_decode_workspace_bytes(const hb200_model* m, int B) {
  if (m == nullptr || B < 1) return 0;
  return carve_decode(m, B, nullptr).bytes;
}

extern "C" int hb200_model_decode_step(const hb200_model* m, const hb200_decode_state* ds, void* workspace,
                                       size_t workspace_bytes, void* last_logits, int64_t ld_logits, int32_t* err,
                                       void* stream) {
  HB_REQUIRE(m && m->blocks && ds && workspace, HB200_ERR_INVALID, "decode_step: null pointer");
  HB_REQUIRE(m->attn_disable == 0 && (m->conv_ksize == 0 || m->conv_ksize == 3), HB200_ERR_UNSUPPORTED,
             "decode_step: attention stages switched off (attn_disable = %d) or conv kernel size %d are not built for the "
             "cached decode", m->attn_disable, m->conv_ksize);
  HB_REQUIRE(!(m->adaptive && m->mor_rampup > 0.f && m->mor_rampup < 1.f), HB200_ERR_UNSUPPORTED,
             "decode_step: the MoR ramp-up blend is built for the forward / prefill only");
  HB_REQUIRE(ds->kcache && ds->vcache && ds->halo && ds->vshift && ds->scores && ds->pos && ds->tokens,
             HB200_ERR_INVALID, "decode_step: incomplete decode state");
  const int B = ds->batch, cap = ds->capacity;
  HB_REQUIRE(B >= 1 && B <= 1024, HB200_ERR_UNSUPPORTED, "decode_step: batch %d outside 1..1024", B);
  HB_REQUIRE(cap >= 1 && cap <= m->max_seq_len, HB200_ERR_INVALID, "decode_step: capacity %d exceeds the RoPE table", cap);
  HB_REQUIRE(m->dim % 8 == 0 && m->dim <= 256 * ROW_NCH && m->ffn_hidden % 8 == 0, HB200_ERR_UNSUPPORTED,
             "decode_step: dim %d must be a multiple of 8 and at most %d, ffn hidden a multiple of 8", m->dim,
             256 * ROW_NCH);
  HB_REQUIRE(m->head_dim == 8 || m->head_dim == 16 || m->head_dim == 32 || m->head_dim == 64, HB200_ERR_UNSUPPORTED,
             "decode_step: head_dim %d (8, 16, 32 or 64 are built)", m->head_dim);
  HB_REQUIRE(m->n_kv_heads >= 1 && m->n_heads % m->n_kv_heads == 0 && m->n_heads / m->n_kv_heads <= DATT_GMAX,
             HB200_ERR_UNSUPPORTED, "decode_step: at most %d query heads per kv head", DATT_GMAX);
  HB_REQUIRE((size_t)8 * (m->n_heads + m->n_kv_heads) * m->head_dim * sizeof(float) <= 48 * 1024, HB200_ERR_UNSUPPORTED,
             "decode_step: latent + kv width too large for the conv window in shared memory");
  HB_REQUIRE(m->n_kv_heads * m->head_dim <= 256, HB200_ERR_UNSUPPORTED, "decode_step: kv width %d beyond 256",
             m->n_kv_heads * m->head_dim);
  HB_REQUIRE(decode_attention_smem(m->head_dim, m->n_heads / m->n_kv_heads, ds->capacity) <= 200 * 1024,
             HB200_ERR_UNSUPPORTED, "decode_step: capacity %d needs more shared memory than one CTA has", ds->capacity);
  HB_REQUIRE(last_logits == nullptr || (ld_logits >= m->vocab && ld_logits % 8 == 0), HB200_ERR_INVALID,
             "decode_step: ld_logits must be >= vocab and a multiple of 8");
  const size_t ld = last_logits ? (size_t)ld_logits : ((size_t)m->vocab + 7) / 8 * 8;
  DecodeWs w = carve_decode(m, B, workspace);
  HB_REQUIRE(workspace_bytes >= w.bytes, HB200_ERR_WORKSPACE, "workspace too small: %zu < %zu", workspace_bytes, w.bytes);
  cudaStream_t st = (cudaStream_t)stream;
  const int D = m->dim, H = m->n_heads, KV = m->n_kv_heads, hd = m->head_dim, F = m->ffn_hidden, R = m->n_rec;
  const int lat = H * hd, kvd = KV * hd, C = lat + kvd, nq = lat + 2 * kvd;
  const unsigned row_grid = (unsigned)ceil_div(B, 8);
  const size_t cache_block = (size_t)B * KV * cap * hd;
  const bool stat = m->static_routing != 0;   // dense compute, soft routing weights (cur is updated by a separate link)
  const float scale = 1.0f / sqrtf((float)hd);

  // Every launch of the step is a link of one programmatic-dependent-launch chain: a kernel's scheduling and
  // prologue overlap its predecessor's tail, and each kernel reads global memory only after chain_wait().
  static const bool chain = [] {
    const char* e = getenv("HB200_DECODE_CHAIN");
    return e == nullptr || e[0] != '0';
  }();
  // per-launch event recorder (only when the model carries a profile handle; the events serialise the chain)
#define PS(KIND, REC, N_, K_) ProfScope ps_(m->profile, st, KIND, bi_prof, REC, B, N_, K_)
  int bi_prof = 0;
#define HB_ROW_LAUNCH(KERNEL, GRID, ...) \
  HB_DISPATCH_NCH(D, HB_PROPAGATE(launch_chained(KERNEL<NCH>, dim3(GRID), dim3(256), 0, st, chain, 1, __VA_ARGS__)))
  {
  PS(HB200_K_EMBED, 0, D, 0);
  HB_ROW_LAUNCH(embed_norm_kernel, row_grid, (const int64_t*)ds->tokens, (const __nv_bfloat16*)m->tok_emb, w.x0,
                m->blocks[0].norm1_w, w.a, (int64_t)B, D, m->vocab, sqrtf((float)D), m->norm_eps);
  }
  __nv_bfloat16 *xin = w.x0, *xout = w.x1;
  for (int bi = 0; bi < m->n_blocks; ++bi) {
    const hb200_block_weights& bw = m->blocks[bi];
    const bool has_mod = bw.mod_wn != nullptr;
    const bool last = (bi == m->n_blocks - 1);
    __nv_bfloat16* kc = (__nv_bfloat16*)ds->kcache + (size_t)bi * cache_block;
    __nv_bfloat16* vc = (__nv_bfloat16*)ds->vcache + (size_t)bi * cache_block;
    // ---- attention half ----
    bi_prof = bi;
    { PS(HB200_K_GEMM_QKV, 0, nq, D);
    HB_PROPAGATE(dgemm(m, w, w.a, bw.w_qkv, w.qkv, B, nq, D, nq, EPI_STORE, nullptr, 1.0f, nullptr, nullptr, err, st, chain)); }
    { PS(HB200_K_PRE_ATTENTION, 0, C, 0);
#define HB_CONV_PREP(HD_)                                                                                               \
  HB_PROPAGATE(launch_chained(decode_conv_prep_kernel<HD_>, dim3(B), dim3(256), (size_t)8 * C * sizeof(float), st, chain, 1,  \
                              (const __nv_bfloat16*)w.qkv, (const __nv_bfloat16*)bw.w1_qk,                                     \
                              (__nv_bfloat16*)ds->halo + (size_t)bi * B * 4 * C,                                               \
                              (__nv_bfloat16*)ds->vshift + (size_t)bi * B * (kvd / 2), vc, w.aq, w.ak, w.qm, w.km,             \
                              w.counts + (size_t)bi * R, (const int32_t*)ds->pos, B, H, KV, cap))
    if (hd == 8) HB_CONV_PREP(8);
    else if (hd == 16) HB_CONV_PREP(16);
    else if (hd == 32) HB_CONV_PREP(32);
    else HB_CONV_PREP(64);
#undef HB_CONV_PREP
    }
    { PS(HB200_K_OTHER, 0, lat, 3 * lat);
    HB_PROPAGATE(dgemm(m, w, w.aq, bw.w2_q, w.c2q, B, lat, 3 * lat, lat, EPI_STORE, nullptr, 1.0f, nullptr, nullptr, err, st,
                       chain)); }
    { PS(HB200_K_PRE_ATTENTION, 1, lat, 0);
    HB_PROPAGATE(launch_chained(decode_qk_finish_kernel, dim3(B), dim3(256), (size_t)4 * kvd * sizeof(float), st, chain, 1,
                                w.qkv, w.c2q, w.ak, (const __nv_bfloat16*)bw.w2_k, w.qm, w.km, m->rope_cos, m->rope_sin,
                                bw.key_temperature, w.qnew, kc, (const int32_t*)ds->pos, H, KV, hd, cap)); }
    { PS(HB200_K_ATTENTION, 0, lat, cap);
    switch (hd) {
      case 8: HB_PROPAGATE(launch_decode_attention<8>(w.qnew, kc, vc, w.o, ds->pos, B, H, KV, cap, scale, st, chain)); break;
      case 16: HB_PROPAGATE(launch_decode_attention<16>(w.qnew, kc, vc, w.o, ds->pos, B, H, KV, cap, scale, st, chain)); break;
      case 32: HB_PROPAGATE(launch_decode_attention<32>(w.qnew, kc, vc, w.o, ds->pos, B, H, KV, cap, scale, st, chain)); break;
      default: HB_PROPAGATE(launch_decode_attention<64>(w.qnew, kc, vc, w.o, ds->pos, B, H, KV, cap, scale, st, chain)); break;
    } }
    { PS(HB200_K_GEMM_O, 0, D, lat);
    HB_PROPAGATE(dgemm(m, w, w.o, bw.w_o, w.cur, B, D, lat, D, EPI_RESID, xin, m->residual_scale * m->output_scale, nullptr,
                       nullptr, err, st, chain)); }
    // ---- MoR loop on the B new rows ----
    if (!m->adaptive)
      HB_PROPAGATE(launch_chained(decode_fill_kernel, dim3(ceil_div(B, 256)), dim3(256), 0, st, chain, 1, w.depth, B, R - 1));
    for (int r = 0; r < R; ++r) {
      const float* rec = bw.rec + (size_t)r * D;
      const bool need_router = (r == 0) && m->adaptive;
      int32_t* count = w.counts + (size_t)bi * R + r;
      float* cache = has_mod ? ds->scores + (((size_t)bi * R + r) * B) * cap : nullptr;
#define HB_DROUTE(MOD_, ROUTER_)                                                                                     \
  HB_PROPAGATE(launch_chained(decode_route_kernel<MOD_, ROUTER_>, dim3(B), dim3(ROUTE_THREADS), 0, st, chain, 1,         \
                              (const __nv_bfloat16*)w.cur, rec, bw.norm2_w, bw.mod_wn, bw.mod_b, bw.mor_w, bw.mor_b,     \
                              cache, w.depth, stat ? 0 : r, w.rows, count, (r + 1 < R) ? count + 1 : (int32_t*)nullptr, w.ug,       \
                              (const int32_t*)ds->pos, B, D, cap, m->mod_capacity, m->norm_eps, R, m->min_depth,          \
                              stat ? w.score : (float*)nullptr, stat ? w.rlogit : (float*)nullptr))
      { PS(HB200_K_SELECT, r, D, 0);
      if (has_mod && need_router) HB_DROUTE(true, true);
      else if (has_mod) HB_DROUTE(true, false);
      else if (need_router) HB_DROUTE(false, true);
      else HB_DROUTE(false, false); }
#undef HB_DROUTE
      { PS(HB200_K_GEMM_GATE_UP, r, 2 * F, D);
      int32_t* hint = (r > 0) ? w.hints + ((size_t)bi * R + r) * 2 : nullptr;   // recursion 0 always has rows
      HB_PROPAGATE(dgemm(m, w, w.ug, bw.w_gate_up, w.act, B, 2 * F, D, F, EPI_SWIGLU, nullptr, 1.0f, nullptr, count, err, st,
                         chain, hint)); }
      { PS(HB200_K_GEMM_DOWN, r, D, F);
      if (!stat) {
        HB_PROPAGATE(dgemm(m, w, w.act, bw.w_down, w.cur, B, D, F, D, EPI_SCATTER_ADD, nullptr, 1.0f, w.rows, count, err, st,
                           chain, (r > 0) ? w.hints + ((size_t)bi * R + r) * 2 + 1 : nullptr));
      } else {
        // static routing: the MLP result of every row (compact order) goes to w.a, free between the qkv projection and
        // the exit norm; one more link of the chain mixes it into cur and accumulates the weighted state
        HB_PROPAGATE(dgemm(m, w, w.act, bw.w_down, w.a, B, D, F, D, EPI_STORE, nullptr, 1.0f, nullptr, count, err, st, chain));
        HB_PROPAGATE(launch_chained(decode_static_update_kernel, dim3(B), dim3(256), 0, st, chain, 1, w.cur,
                                    (const __nv_bfloat16*)w.a, (const __nv_bfloat16*)w.ug, (const int32_t*)w.rows,
                                    (const int32_t*)count, (const float*)w.score, (const float*)w.rlogit, w.sout, D, r, R,
                                    m->adaptive ? 1 : 0));
      } }
    }
    const float* next_w = last ? m->norm_w : m->blocks[bi + 1].norm1_w;
    { PS(HB200_K_RMS_NORM, R, D, 0);
    HB_PROPAGATE(launch_chained(decode_dual_norm_kernel, dim3(B), dim3(256), 0, st, chain, 1,
                                (const __nv_bfloat16*)((stat && m->adaptive) ? w.sout : w.cur), bw.final_norm_w, xout, next_w,
                                last ? w.hid : w.a, D, m->norm_eps)); }
    std::swap(xin, xout);
  }
#undef HB_ROW_LAUNCH
  __nv_bfloat16* lg = last_logits ? (__nv_bfloat16*)last_logits : w.logits;
  bi_prof = m->n_blocks;
  { PS(HB200_K_GEMM_LM_HEAD, 0, m->vocab, D);
  HB_PROPAGATE(dgemm(m, w, w.hid, output_weight(m), lg, B, m->vocab, D, (int64_t)ld, EPI_STORE, nullptr, 1.0f, nullptr, nullptr, err,
                     st, chain)); }
  { PS(HB200_K_OTHER, 1, m->vocab, 0);
  HB_PROPAGATE(launch_argmax_rows(lg, B, m->vocab, (int64_t)ld, ds->tokens, st, chain)); }
  HB_PROPAGATE(launch_chained(decode_advance_kernel, dim3(ceil_div(B, 1024)), dim3(1024), 0, st, chain, 1, ds->pos,
                              (const int64_t*)ds->tokens, ds->history, B, cap));
#undef PS
  return 0;
}
