// Cached decode: one new token per sequence through every block against the latent-space KV cache.
//
// The reference has no decode path; this executor adds a latent-space KV cache for autoregressive decode.
// Per block and step (B sequences in lockstep, position p = *state.pos read from device memory by every kernel, so
// the same launch sequence - and a CUDA graph of it - serves every step):
//
//   a    = AdaRMSNorm(x)                                       (dual_norm of the previous block / embed_norm)
//   qkv  = a Wqkv^T                                            tcgen05 GEMM, M = B
//   conv prep: window of q|k rows p-4..p (halo + new row), grouped conv1 on its last three rows, written as the
//              im2col rows [y1(p-2) | y1(p-1) | y1(p)] of the dense conv; value row [v_curr(p) | v_shift(p-1)] appended
//              to the value cache; halo and v_shift advanced                         decode_conv_prep_kernel
//   c2q  = im2col_q W2q^T,  c2k = im2col_k W2k^T               tcgen05 GEMMs (the repacked conv2 weights ARE the
//                                                              [C_out, 3*C_in] matrices these products need)
//   QK-mean, L2 norm, temperature, RoPE(p); key appended to the key cache            decode_qk_finish_kernel
//   o    = softmax(q K^T / sqrt(hd)) V over the p+1 cached positions                 decode_attention_kernel
//   cur  = x + 0.5 * o Wo^T                                    tcgen05 GEMM, residual epilogue
//   MoR depth, then per recursion: MoD score; "selected" iff fewer than k cached scores are >= the new score
//   (k = int((p+1) * capacity), the newest position loses ties); norm-gather of the selected & active rows;
//   gate_up / down GEMMs with the device-side row count                              row kernels shared with prefill
//   x'   = RMSNorm(cur) (+ next block's input norm)
// then the final norm, the output projection for the B rows, the greedy choice, and p += 1.
#include <cmath>
#include <utility>

#include "gemm_epilogue.cuh"
#include "row_kernels.cuh"

namespace hb200 {

int launch_argmax_rows(const void* x, int64_t rows, int cols, int64_t ld, int64_t* out, cudaStream_t st, bool chained);

struct DecodeWs {
  __nv_bfloat16 *x0, *x1, *a, *qkv, *aq, *ak, *c2q, *qnew, *o, *cur, *ug, *act, *hid, *logits;
  float *qm, *km, *score, *rlogit;
  int32_t *depth, *rows, *counts;
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
  w.bytes = off;
  return w;
}

// ---- conv prep: one CTA per sequence ---------------------------------------------------------------------------
// dynamic smem: win[5][C] + y1[3][C] floats
__global__ void __launch_bounds__(256) decode_conv_prep_kernel(
    const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ w1, __nv_bfloat16* __restrict__ halo,
    __nv_bfloat16* __restrict__ vshift, __nv_bfloat16* __restrict__ vcache, __nv_bfloat16* __restrict__ aq,
    __nv_bfloat16* __restrict__ ak, float* __restrict__ qm, float* __restrict__ km, int32_t* __restrict__ first_count,
    const int32_t* __restrict__ pos_ptr, int B, int H, int KV, int hd, int capacity) {
  extern __shared__ float smem_f[];
  chain_release();
  chain_wait();
  const int lat = H * hd, kvd = KV * hd, C = lat + kvd, qkv_ld = lat + 2 * kvd, half = kvd / 2;
  float* win = smem_f;            // [5][C]: positions p-4 .. p
  float* y1 = smem_f + 5 * C;     // [3][C]: positions p-2 .. p
  const int b = blockIdx.x, tid = threadIdx.x;
  if (b == 0 && tid == 0) *first_count = 0;   // row counter of this block's first recursion (see decode_route_kernel)
  const int pos = *pos_ptr;
  if (pos >= capacity) return;    // cache full: the step is a no-op (the host checks capacity before launching)
  __nv_bfloat16* hb = halo + (size_t)b * 4 * C;
  const __nv_bfloat16* row = qkv + (size_t)b * qkv_ld;
  for (int i = tid; i < 4 * C; i += 256) win[i] = __bfloat162float(hb[i]);
  for (int c = tid; c < C; c += 256) win[4 * C + c] = __bfloat162float(row[c]);
  __syncthreads();
  // grouped conv1 (kernel 3, causal) on rows 2..4 of the window; rounded to bf16 like the prefill's y1 tile.
  // One thread per output channel: its weight row (3 taps x hd inputs, 16-byte loads) serves all three positions.
  for (int c = tid; c < C; c += 256) {
    const int hb0 = (c / hd) * hd;
    const __nv_bfloat16* wr = w1 + (size_t)c * 3 * hd;
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f;
    for (int e = 0; e < 3 * hd; e += 8) {
      float wv[8];
      load_bf16x8(wr + e, wv);
      const int j = e / hd, ci0 = e - j * hd;                 // hd % 8 == 0: the 8 weights share a tap
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
  for (int c = tid; c < kvd; c += 256) {
    const __nv_bfloat16 val = (c < half) ? row[C + c] : vshift[(size_t)b * half + (c - half)];
    vcache[(((size_t)b * KV + c / hd) * capacity + pos) * hd + (c % hd)] = val;
  }
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
  for (int c = tid; c < half; c += 256) vshift[(size_t)b * half + c] = row[C + half + c];
}

// ---- QK finish: one CTA per sequence, one warp per head ----------------------------------------------------------
__global__ void __launch_bounds__(256) decode_qk_finish_kernel(
    const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ c2q, const __nv_bfloat16* __restrict__ ak,
    const __nv_bfloat16* __restrict__ w2k, const float* __restrict__ qm, const float* __restrict__ km, const float* __restrict__ cos_t,
    const float* __restrict__ sin_t, const float* __restrict__ temp, __nv_bfloat16* __restrict__ qnew,
    __nv_bfloat16* __restrict__ kcache, const int32_t* __restrict__ pos_ptr, int H, int KV, int hd, int capacity) {
  const int b = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  chain_release();
  chain_wait();
  const int pos = *pos_ptr;
  if (pos >= capacity) return;
  const int lat = H * hd, kvd = KV * hd, qkv_ld = lat + 2 * kvd;
  const bool same_heads = (H == KV);
  // the key side of the dense conv is small (kvd x 3 kvd): done here on the CUDA cores, one thread per output
  // channel, im2col row in shared memory, result rounded to bf16 like a stored GEMM output
  extern __shared__ float smem_f[];
  float* a_row = smem_f;                 // [3 * kvd]
  float* c2k = smem_f + 3 * kvd;         // [kvd]
  for (int i = threadIdx.x; i < 3 * kvd; i += 256) a_row[i] = __bfloat162float(ak[(size_t)b * 3 * kvd + i]);
  __syncthreads();
  for (int n = threadIdx.x; n < kvd; n += 256) {
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
  __syncthreads();
  for (int hh = warp; hh < H + KV; hh += 8) {
    const bool is_k = hh >= H;
    const int h = is_k ? hh - H : hh;
    // hd <= 64: each lane owns elements 2*lane and 2*lane+1 (one RoPE pair)
    const int d0 = 2 * lane;
    float v0 = 0.f, v1 = 0.f;
    if (d0 < hd) {
      const __nv_bfloat16* conv = c2q + (size_t)b * lat + h * hd;
      float c0, c1;
      if (same_heads) {   // one query head per kv head: both sides couple with 0.5 * (q0 + k0) of that head
        const __nv_bfloat16* row = qkv + (size_t)b * qkv_ld;
        c0 = 0.5f * (__bfloat162float(row[h * hd + d0]) + __bfloat162float(row[lat + h * hd + d0]));
        c1 = 0.5f * (__bfloat162float(row[h * hd + d0 + 1]) + __bfloat162float(row[lat + h * hd + d0 + 1]));
      } else {            // otherwise with half the head-mean of the other side
        const float* mean = (is_k ? qm : km) + (size_t)b * hd;
        c0 = mean[d0];
        c1 = mean[d0 + 1];
      }
      v0 = (is_k ? c2k[h * hd + d0] : __bfloat162float(conv[d0])) + c0;
      v1 = (is_k ? c2k[h * hd + d0 + 1] : __bfloat162float(conv[d0 + 1])) + c1;
    }
    const float ss = warp_sum(v0 * v0 + v1 * v1);
    const float inv = (is_k ? *temp : 1.0f) / fmaxf(sqrtf(ss), 1e-12f);
    if (d0 < hd) {
      v0 *= inv;
      v1 *= inv;
      const float cs = cos_t[(size_t)pos * (hd / 2) + lane], sn = sin_t[(size_t)pos * (hd / 2) + lane];
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
constexpr int DATT_THREADS = 256;
constexpr int DATT_WARPS = DATT_THREADS / 32;
constexpr int DATT_GMAX = 8;      // query heads per kv head
template <int HD>
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
  const int n_keys = min(*pos_ptr + 1, capacity);
  float* qs = smem_f;                          // [G][HD], pre-scaled by scale * log2(e)
  float* red = qs + DATT_GMAX * HD;            // [DATT_WARPS][DATT_GMAX]
  float* part = red + DATT_WARPS * DATT_GMAX;  // [DATT_WARPS][DATT_GMAX][HD]
  float* sc = part + DATT_WARPS * DATT_GMAX * HD;   // [G][capacity]
  for (int i = tid; i < G * HD; i += DATT_THREADS)
    qs[i] = __bfloat162float(qnew[(size_t)b * lat + (size_t)(kvh * G) * HD + i]) * scale_log2;
  __syncthreads();
  const __nv_bfloat16* kb = kcache + ((size_t)b * KV + kvh) * capacity * HD;
  const __nv_bfloat16* vb = vcache + ((size_t)b * KV + kvh) * capacity * HD;
  // pass 1
  float mx[DATT_GMAX];
#pragma unroll
  for (int g = 0; g < DATT_GMAX; ++g) mx[g] = -INFINITY;
#pragma unroll 2
  for (int key = tid; key < n_keys; key += DATT_THREADS) {
    float kf[HD];
#pragma unroll
    for (int c = 0; c < CH; ++c) load_bf16x8(kb + (size_t)key * HD + c * 8, *reinterpret_cast<float(*)[8]>(&kf[c * 8]));
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
    load_bf16x8(vb + (size_t)key * HD + chunk * 8, vf);
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
  const size_t smem = decode_attention_smem(HD, H / KV, capacity);
  HB_PROPAGATE(ensure_dynamic_smem((const void*)decode_attention_kernel<HD>, smem));
  return launch_chained(decode_attention_kernel<HD>, dim3(KV, B), dim3(DATT_THREADS), smem, st, chain, 1, qnew, kc, vc, o,
                        pos, H, KV, capacity, scale * 1.4426950408889634f);
}

// ---- routing of the newest position + gather-norm: one warp per sequence ------------------------------------
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
template <int NCH, bool HAS_MOD, bool HAS_ROUTER>
__global__ void __launch_bounds__(256) decode_route_kernel(
    const __nv_bfloat16* __restrict__ cur, const float* __restrict__ rec, const float* __restrict__ norm2_w,
    const float* __restrict__ mod_wn, const float* __restrict__ mod_b, const float* __restrict__ mor_w,
    const float* __restrict__ mor_b, float* __restrict__ score_cache, int32_t* __restrict__ depth, int min_active,
    int32_t* __restrict__ rows, int32_t* __restrict__ count, int32_t* __restrict__ next_count,
    __nv_bfloat16* __restrict__ ug, const int32_t* __restrict__ pos_ptr, int B, int D, int capacity, float cap_ratio,
    float eps, int n_rec, int min_d) {
  const int lane = threadIdx.x & 31;
  const int b = blockIdx.x * 8 + (threadIdx.x >> 5);
  chain_release();
  chain_wait();
  if (next_count != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *next_count = 0;
  if (b >= B) return;
  const int pos = *pos_ptr;
  const bool room = pos < capacity;
  // one pass over the row: every load (row pieces, then the per-column vectors) is issued before it is needed
  uint4 raw[NCH];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * 8;
    raw[c] = (i < D) ? *reinterpret_cast<const uint4*>(cur + (size_t)b * D + i) : make_uint4(0, 0, 0, 0);
  }
  float v[NCH][8];
  float ss = 0.f, dm = 0.f, lm = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * 8;
    if (i < D) {
      const float4 r0 = *reinterpret_cast<const float4*>(rec + i), r1 = *reinterpret_cast<const float4*>(rec + i + 4);
      const float rc[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
      const uint32_t w4[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
      float x[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        x[2 * j] = __uint_as_float(w4[j] << 16);
        x[2 * j + 1] = __uint_as_float(w4[j] & 0xffff0000u);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[c][j] = x[j] + rc[j];
        ss += v[c][j] * v[c][j];
      }
      if (HAS_MOD) {
        const float4 a0 = *reinterpret_cast<const float4*>(mod_wn + i), a1 = *reinterpret_cast<const float4*>(mod_wn + i + 4);
        dm += v[c][0] * a0.x + v[c][1] * a0.y + v[c][2] * a0.z + v[c][3] * a0.w + v[c][4] * a1.x + v[c][5] * a1.y +
              v[c][6] * a1.z + v[c][7] * a1.w;
      }
      if (HAS_ROUTER) {   // the depth router sees the raw row (no recursion offset)
        const float4 a0 = *reinterpret_cast<const float4*>(mor_w + i), a1 = *reinterpret_cast<const float4*>(mor_w + i + 4);
        lm += x[0] * a0.x + x[1] * a0.y + x[2] * a0.z + x[3] * a0.w + x[4] * a1.x + x[5] * a1.y + x[6] * a1.z + x[7] * a1.w;
      }
    }
  }
  ss = warp_sum(ss);
  const float ri = rsqrtf(ss / (float)D + eps);
  int dep;
  if (HAS_ROUTER) {
    lm = warp_sum(lm);
    dep = mor_depth_from_logit(lm + mor_b[0], n_rec, min_d);
    if (lane == 0) depth[b] = dep;
  } else {
    dep = depth[b];
  }
  bool sel = true;
  if (HAS_MOD) {
    double c = (double)cap_ratio;
    c = c < 1e-4 ? 1e-4 : (c > 1.0 ? 1.0 : c);
    int k = (int)((double)(pos + 1) * c);
    k = k < 1 ? 1 : (k > pos + 1 ? pos + 1 : k);
    dm = warp_sum(dm);
    const float s = ri * dm + mod_b[0];
    float* sc = score_cache + (size_t)b * capacity;
    int cnt = 0;
    const int n = min(pos, capacity);
    if ((capacity & 3) == 0) {
      // 16-byte pieces of the cached scores, several in flight per lane; entries at or beyond n do not count
      const float4* sc4 = reinterpret_cast<const float4*>(sc);
      const int n4 = (n + 3) >> 2;
#pragma unroll 4
      for (int i = lane; i < n4; i += 32) {
        const float4 q = sc4[i];
        const int i0 = i * 4;
        cnt += (q.x >= s) ? 1 : 0;
        cnt += (i0 + 1 < n && q.y >= s) ? 1 : 0;
        cnt += (i0 + 2 < n && q.z >= s) ? 1 : 0;
        cnt += (i0 + 3 < n && q.w >= s) ? 1 : 0;
      }
    } else {
#pragma unroll 4
      for (int i = lane; i < n; i += 32) cnt += (sc[i] >= s) ? 1 : 0;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, off);
    sel = cnt < k;
    if (lane == 0 && room) sc[pos] = s;
  }
  if (!(room && sel && dep >= min_active)) return;      // warp-uniform
  int j = 0;
  if (lane == 0) {
    j = atomicAdd(count, 1);
    rows[j] = b;
  }
  j = __shfl_sync(0xffffffffu, j, 0);
  scale_row<NCH>(norm2_w, ri, D, lane, v);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * 32 + lane) * 8;
    if (i < D) store_bf16x8(ug + (size_t)j * D + i, v[c]);
  }
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
  const int pos = *pos_ptr;
  if (pos >= capacity) return;
  if (b < B && history != nullptr && pos + 1 < capacity) history[(size_t)b * capacity + pos + 1] = tokens[b];
  __syncthreads();
  if (b == 0) *pos_ptr = pos + 1;
}

// Contractions of a decode step: at most 128 rows -> the cluster split-K weight-streaming kernel (gemm_impl 0); larger
// batches, or gemm_impl 1 (the mma.sync cross-check), take the general entry point.
static int dgemm(const hb200_model* m, const DecodeWs& w, const void* A, const void* W, void* C, int M, int N, int K,
                 int64_t ldc, int epi, const void* resid, float alpha, const int32_t* rows, const int32_t* m_dev,
                 int32_t* err, cudaStream_t st, bool chain) {
  if (m->gemm_impl == 0 && M <= 128) {
    GemmParams p{(const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (__nv_bfloat16*)C, M, N, K, K, K, ldc, epi,
                 (const __nv_bfloat16*)resid, epi == EPI_SCATTER_ADD ? 1.0f : alpha, rows, m_dev, err};
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
  HB_REQUIRE(ds->kcache && ds->vcache && ds->halo && ds->vshift && ds->scores && ds->pos && ds->tokens,
             HB200_ERR_INVALID, "decode_step: incomplete decode state");
  const int B = ds->batch, cap = ds->capacity;
  HB_REQUIRE(B >= 1 && B <= 1024, HB200_ERR_UNSUPPORTED, "decode_step: batch %d outside 1..1024", B);
  HB_REQUIRE(cap >= 1 && cap <= m->max_seq_len, HB200_ERR_INVALID, "decode_step: capacity %d exceeds the RoPE table", cap);
  HB_REQUIRE(m->dim % 8 == 0 && m->dim <= 256 * ROW_NCH && m->ffn_hidden % 8 == 0, HB200_ERR_UNSUPPORTED,
             "decode_step: dim %d must be a multiple of 8 and at most %d, ffn hidden a multiple of 8", m->dim,
             256 * ROW_NCH);
  HB_REQUIRE(m->head_dim == 16 || m->head_dim == 32 || m->head_dim == 64, HB200_ERR_UNSUPPORTED,
             "decode_step: head_dim %d (16, 32 or 64 are built)", m->head_dim);
  HB_REQUIRE(m->n_kv_heads >= 1 && m->n_heads % m->n_kv_heads == 0 && m->n_heads / m->n_kv_heads <= DATT_GMAX,
             HB200_ERR_UNSUPPORTED, "decode_step: at most %d query heads per kv head", DATT_GMAX);
  HB_REQUIRE((size_t)8 * (m->n_heads + m->n_kv_heads) * m->head_dim * sizeof(float) <= 48 * 1024, HB200_ERR_UNSUPPORTED,
             "decode_step: latent + kv width too large for the conv window in shared memory");
  HB_REQUIRE(decode_attention_smem(m->head_dim, m->n_heads / m->n_kv_heads, ds->capacity) <= 200 * 1024,
             HB200_ERR_UNSUPPORTED, "decode_step: capacity %d needs more shared memory than one CTA has", ds->capacity);
  const size_t ld = ((size_t)m->vocab + 7) / 8 * 8;
  HB_REQUIRE(last_logits == nullptr || (size_t)ld_logits == ld, HB200_ERR_INVALID, "decode_step: ld_logits must be %zu", ld);
  DecodeWs w = carve_decode(m, B, workspace);
  HB_REQUIRE(workspace_bytes >= w.bytes, HB200_ERR_WORKSPACE, "workspace too small: %zu < %zu", workspace_bytes, w.bytes);
  cudaStream_t st = (cudaStream_t)stream;
  const int D = m->dim, H = m->n_heads, KV = m->n_kv_heads, hd = m->head_dim, F = m->ffn_hidden, R = m->n_rec;
  const int lat = H * hd, kvd = KV * hd, C = lat + kvd, nq = lat + 2 * kvd;
  const unsigned row_grid = (unsigned)ceil_div(B, 8);
  const size_t cache_block = (size_t)B * KV * cap * hd;
  const float scale = 1.0f / sqrtf((float)hd);

  // Every launch of the step is a link of one programmatic-dependent-launch chain: a kernel's scheduling and
  // prologue overlap its predecessor's tail, and each kernel reads global memory only after chain_wait().
  static const bool chain = [] {
    const char* e = getenv("HB200_DECODE_CHAIN");
    return e == nullptr || e[0] != '0';
  }();
#define HB_ROW_LAUNCH(KERNEL, GRID, ...) \
  HB_DISPATCH_NCH(D, HB_PROPAGATE(launch_chained(KERNEL<NCH>, dim3(GRID), dim3(256), 0, st, chain, 1, __VA_ARGS__)))
  HB_ROW_LAUNCH(embed_norm_kernel, row_grid, (const int64_t*)ds->tokens, (const __nv_bfloat16*)m->tok_emb, w.x0,
                m->blocks[0].norm1_w, w.a, (int64_t)B, D, m->vocab, sqrtf((float)D), m->norm_eps);
  __nv_bfloat16 *xin = w.x0, *xout = w.x1;
  for (int bi = 0; bi < m->n_blocks; ++bi) {
    const hb200_block_weights& bw = m->blocks[bi];
    const bool has_mod = bw.mod_wn != nullptr;
    const bool last = (bi == m->n_blocks - 1);
    __nv_bfloat16* kc = (__nv_bfloat16*)ds->kcache + (size_t)bi * cache_block;
    __nv_bfloat16* vc = (__nv_bfloat16*)ds->vcache + (size_t)bi * cache_block;
    // ---- attention half ----
    HB_PROPAGATE(dgemm(m, w, w.a, bw.w_qkv, w.qkv, B, nq, D, nq, EPI_STORE, nullptr, 1.0f, nullptr, nullptr, err, st, chain));
    HB_PROPAGATE(launch_chained(decode_conv_prep_kernel, dim3(B), dim3(256), (size_t)8 * C * sizeof(float), st, chain, 1,
                                w.qkv, (const __nv_bfloat16*)bw.w1_qk, (__nv_bfloat16*)ds->halo + (size_t)bi * B * 4 * C,
                                (__nv_bfloat16*)ds->vshift + (size_t)bi * B * (kvd / 2), vc, w.aq, w.ak, w.qm, w.km,
                                w.counts + (size_t)bi * R, (const int32_t*)ds->pos, B, H, KV, hd, cap));
    HB_PROPAGATE(dgemm(m, w, w.aq, bw.w2_q, w.c2q, B, lat, 3 * lat, lat, EPI_STORE, nullptr, 1.0f, nullptr, nullptr, err, st,
                       chain));
    HB_PROPAGATE(launch_chained(decode_qk_finish_kernel, dim3(B), dim3(256), (size_t)4 * kvd * sizeof(float), st, chain, 1,
                                w.qkv, w.c2q, w.ak, (const __nv_bfloat16*)bw.w2_k, w.qm, w.km, m->rope_cos, m->rope_sin,
                                bw.key_temperature, w.qnew, kc, (const int32_t*)ds->pos, H, KV, hd, cap));
    switch (hd) {
      case 16: HB_PROPAGATE(launch_decode_attention<16>(w.qnew, kc, vc, w.o, ds->pos, B, H, KV, cap, scale, st, chain)); break;
      case 32: HB_PROPAGATE(launch_decode_attention<32>(w.qnew, kc, vc, w.o, ds->pos, B, H, KV, cap, scale, st, chain)); break;
      default: HB_PROPAGATE(launch_decode_attention<64>(w.qnew, kc, vc, w.o, ds->pos, B, H, KV, cap, scale, st, chain)); break;
    }
    HB_PROPAGATE(dgemm(m, w, w.o, bw.w_o, w.cur, B, D, lat, D, EPI_RESID, xin, m->residual_scale * m->output_scale, nullptr,
                       nullptr, err, st, chain));
    // ---- MoR loop on the B new rows ----
    if (!m->adaptive)
      HB_PROPAGATE(launch_chained(decode_fill_kernel, dim3(ceil_div(B, 256)), dim3(256), 0, st, chain, 1, w.depth, B, R - 1));
    for (int r = 0; r < R; ++r) {
      const float* rec = bw.rec + (size_t)r * D;
      const bool need_router = (r == 0) && m->adaptive;
      int32_t* count = w.counts + (size_t)bi * R + r;
      float* cache = has_mod ? ds->scores + (((size_t)bi * R + r) * B) * cap : nullptr;
#define HB_DROUTE(MOD_, ROUTER_)                                                                                       \
  HB_DISPATCH_NCH(D, HB_PROPAGATE(launch_chained(decode_route_kernel<NCH, MOD_, ROUTER_>, dim3(row_grid), dim3(256), 0,   \
                                                 st, chain, 1, (const __nv_bfloat16*)w.cur, rec, bw.norm2_w, bw.mod_wn,  \
                                                 bw.mod_b, bw.mor_w, bw.mor_b, cache, w.depth, r, w.rows, count,         \
                                                 (r + 1 < R) ? count + 1 : (int32_t*)nullptr, w.ug,                      \
                                                 (const int32_t*)ds->pos, B, D, cap, m->mod_capacity, m->norm_eps, R,    \
                                                 m->min_depth)))
      if (has_mod && need_router) HB_DROUTE(true, true);
      else if (has_mod) HB_DROUTE(true, false);
      else if (need_router) HB_DROUTE(false, true);
      else HB_DROUTE(false, false);
#undef HB_DROUTE
      HB_PROPAGATE(dgemm(m, w, w.ug, bw.w_gate_up, w.act, B, 2 * F, D, F, EPI_SWIGLU, nullptr, 1.0f, nullptr, count, err, st,
                         chain));
      HB_PROPAGATE(dgemm(m, w, w.act, bw.w_down, w.cur, B, D, F, D, EPI_SCATTER_ADD, nullptr, 1.0f, w.rows, count, err, st,
                         chain));
    }
    const float* next_w = last ? m->norm_w : m->blocks[bi + 1].norm1_w;
    HB_ROW_LAUNCH(dual_norm_kernel, row_grid, (const __nv_bfloat16*)w.cur, bw.final_norm_w, xout, next_w,
                  last ? w.hid : w.a, (int64_t)B, D, m->norm_eps);
    std::swap(xin, xout);
  }
#undef HB_ROW_LAUNCH
  __nv_bfloat16* lg = last_logits ? (__nv_bfloat16*)last_logits : w.logits;
  HB_PROPAGATE(dgemm(m, w, w.hid, m->tok_emb, lg, B, m->vocab, D, (int64_t)ld, EPI_STORE, nullptr, 1.0f, nullptr, nullptr, err,
                     st, chain));
  HB_PROPAGATE(launch_argmax_rows(lg, B, m->vocab, (int64_t)ld, ds->tokens, st, chain));
  HB_PROPAGATE(launch_chained(decode_advance_kernel, dim3(ceil_div(B, 1024)), dim3(1024), 0, st, chain, 1, ds->pos,
                              (const int64_t*)ds->tokens, ds->history, B, cap));
  return 0;
}
