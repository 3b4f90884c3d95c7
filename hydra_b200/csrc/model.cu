// Host-side executor of the HYDRA block / model forward (eval, dynamic MoR + hard MoD routing) and the small
// row kernels that sit between the GEMMs.  Everything is enqueued on one stream; routing decisions stay on
// the device (row lists + device-side counts feed the GEMMs), so a forward never synchronises with the host.
//
// Per block:
//   a   = AdaRMSNorm(x)                                   rms_norm kernel
//   qkv = a Wqkv^T                                        tcgen05 GEMM
//   q,k,v = fused pre-attention(qkv)                      ccgqa_pre kernel
//   o   = causal GQA attention                            attention kernel
//   cur = x + 0.5*scale * o Wo^T                          tcgen05 GEMM, residual epilogue
//   depth = MoR router(cur)                               mor_score kernel (recursion 0)
//   for r < R:
//     s    = MoD router(AdaRMSNorm(cur + rec_r))          mor_score kernel (all tokens, streaming, nothing written
//                                                         but the scores)
//     rows = topk(s) AND depth >= r   (or depth >= r)     mod_select / compact_active kernel -> device row list
//     act  = silu(u Wg^T) * (u Wu^T), u = AdaRMSNorm(cur[rows] + rec_r):  tcgen05 GEMM over the routed rows of cur
//                                                         themselves (gathered by the kernel), norm folded in as
//                                                         inv_rms[row] * (cur W'^T + rec_r W'^T) in the SwiGLU epilogue;
//                                                         inv_rms comes from the score pass (or a rows-only pass)
//        (without the folded weights, static routing, cross-check GEMM: ug = norm_gather(...) then the plain GEMM)
//     cur[rows] += act Wd^T                               tcgen05 GEMM, scatter-add epilogue
//   y = RMSNorm(cur)        (the executor's output accumulator equals the final `cur`: a token stops
//                            changing after its exit recursion, and it exits exactly once)
#include <cmath>
#include <mutex>
#include <new>
#include <utility>
#include <vector>

#include "gemm_epilogue.cuh"
#include <nvtx3/nvToolsExt.h>

#include "row_kernels.cuh"
#include "row_stream.cuh"
#include "tma_host.cuh"

namespace hb200 {

__global__ void fill_i32_kernel(int32_t* p, int64_t n, int32_t val) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = val;
}

// Row list of every token in order (static routing: the dense MLP result is read back by token index, so the list has
// to be the identity; the compacting kernel orders its 4096-token chunks by atomic reservation)
__global__ void all_rows_kernel(int32_t* __restrict__ rows, int64_t n, int32_t* __restrict__ count) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) rows[i] = (int32_t)i;
  if (i == 0) *count = (int32_t)n;
}

// gate_up [2F,K] -> rows interleaved in groups of 8 (8 gate rows, 8 up rows, ...)
__global__ void interleave_gate_up_kernel(const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ o, int F,
                                          int K) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // one 16-byte piece
  const int ppr = K / 8;
  if (idx >= (int64_t)2 * F * ppr) return;
  const int orow = (int)(idx / ppr), piece = (int)(idx % ppr);
  const int grp = orow / 16, r = orow % 16;
  const int srow = (r < 8) ? grp * 8 + r : F + grp * 8 + (r - 8);
  *reinterpret_cast<uint4*>(o + (size_t)orow * K + piece * 8) =
      *reinterpret_cast<const uint4*>(w + (size_t)srow * K + piece * 8);
}

// Conv1d weight [Cout, Cin, K] -> [Cout, K*Cin] with (co, j*Cin + ci) = w[co, ci, j]
__global__ void repack_conv_kernel(const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ o, int cout,
                                   int cin, int ks) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)cout * cin * ks) return;
  const int co = (int)(idx / (ks * cin)), rem = (int)(idx % (ks * cin));
  const int j = rem / cin, ci = rem % cin;
  o[idx] = w[((size_t)co * cin + ci) * ks + j];
}

// Named host-side ranges around the stages of a forward (block, attention half, each MLP recursion, output projection)
// for timeline tools that read NVTX; without such a tool attached the calls return at once.
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  NvtxRange(const char* fmt, int a) {
    char buf[48];
    snprintf(buf, sizeof(buf), fmt, a);
    nvtxRangePushA(buf);
  }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

// ---- workspace ----------------------------------------------------------------------------------------------
struct Workspace {
  __nv_bfloat16 *x0, *x1, *a, *qkv, *q, *k, *v, *o, *cur, *ug, *act, *blend;
  float *scores, *logits, *inv_rms;
  int32_t *depth, *rows, *sel_idx, *counts, *counts2;
  size_t bytes;
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// MoR curriculum in the middle of its ramp: the block output is a blend of the adaptive and the fixed-depth path
static bool mor_blend_active(const hb200_model* m) { return m->adaptive && m->mor_rampup > 0.f && m->mor_rampup < 1.f; }

static Workspace carve(const hb200_model* m, int B, int S, void* base) {
  const size_t T = (size_t)B * S, D = m->dim, lat = (size_t)m->n_heads * m->head_dim,
               kvd = (size_t)m->n_kv_heads * m->head_dim, F = m->ffn_hidden;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    void* p = base ? (void*)((char*)base + off) : nullptr;
    off += align_up(bytes, 1024);
    return p;
  };
  Workspace w{};
  w.x0 = (__nv_bfloat16*)take(T * D * 2);
  w.x1 = (__nv_bfloat16*)take(T * D * 2);
  w.a = (__nv_bfloat16*)take(T * D * 2);
  w.qkv = (__nv_bfloat16*)take(T * (lat + 2 * kvd) * 2);
  w.q = (__nv_bfloat16*)take(T * lat * 2);
  w.k = (__nv_bfloat16*)take(T * kvd * 2);
  w.v = (__nv_bfloat16*)take(T * kvd * 2);
  w.o = (__nv_bfloat16*)take(T * lat * 2);
  w.cur = (__nv_bfloat16*)take(T * D * 2);
  w.ug = (__nv_bfloat16*)take(T * D * 2);
  w.act = (__nv_bfloat16*)take(T * F * 2);
  w.scores = (float*)take(T * 4);
  w.logits = (float*)take(T * 4);
  w.inv_rms = (float*)take(T * 4);
  w.depth = (int32_t*)take(T * 4);
  w.rows = (int32_t*)take(T * 4);
  w.sel_idx = (int32_t*)take(T * 4);
  w.counts = (int32_t*)take((size_t)m->n_blocks * m->n_rec * 4);
  const bool blend = mor_blend_active(m);                   // second block output + second set of row counters
  w.blend = (__nv_bfloat16*)take(blend ? T * D * 2 : 0);
  w.counts2 = (int32_t*)take(blend ? (size_t)m->n_blocks * m->n_rec * 4 : 0);
  w.bytes = off;
  return w;
}

static int mod_k(int L, float cap) {
  // k = max(1, min(L, int(L * clamp(cap, 1e-4, 1)))) evaluated in double like the reference's Python floats
  double c = (double)cap;
  c = c < 1e-4 ? 1e-4 : (c > 1.0 ? 1.0 : c);
  int k = (int)((double)L * c);
  return k < 1 ? 1 : (k > L ? L : k);
}

static int check_model(const hb200_model* m, int B, int S) {
  HB_REQUIRE(m != nullptr && m->blocks != nullptr, HB200_ERR_INVALID, "model: null model or block table");
  HB_REQUIRE(B >= 1 && S >= 1, HB200_ERR_INVALID, "model: batch and sequence length must be positive (B=%d S=%d)", B, S);
  HB_REQUIRE(S <= m->max_seq_len, HB200_ERR_INVALID, "model: sequence length %d exceeds the RoPE table (%d)", S,
             m->max_seq_len);
  HB_REQUIRE(m->dim % 8 == 0 && m->dim <= 256 * ROW_NCH, HB200_ERR_UNSUPPORTED,
             "model: dim %d must be a multiple of 8 and at most %d", m->dim, 256 * ROW_NCH);
  HB_REQUIRE(m->ffn_hidden % 8 == 0, HB200_ERR_UNSUPPORTED, "model: ffn hidden %d must be a multiple of 8", m->ffn_hidden);
  HB_REQUIRE(m->n_heads % m->n_kv_heads == 0, HB200_ERR_INVALID, "model: n_heads must be a multiple of n_kv_heads");
  HB_REQUIRE(m->n_rec >= 1 && m->min_depth >= 0 && m->min_depth <= m->n_rec - 1, HB200_ERR_INVALID,
             "model: bad recursion settings");
  HB_REQUIRE((int64_t)B * S < (1ll << 31), HB200_ERR_UNSUPPORTED, "model: too many tokens");
  return 0;
}

static int gemm(const hb200_model* m, int kind, int bi, int r, const void* A, const void* W, void* C, int M, int N,
                int K, int64_t lda, int64_t ldw, int64_t ldc, int epi, const void* resid, float alpha,
                const int32_t* rows, const int32_t* m_dev, int32_t* err, cudaStream_t st) {
  ProfScope ps(m->profile, st, kind, bi, r, M, N, K);
  return hb200_gemm_bf16(A, W, C, M, N, K, lda, ldw, ldc, epi, resid, alpha, rows, m_dev, m->gemm_impl, err, st);
}

// attention sub-block: y_out = epilogue(o Wo^T); resid == nullptr -> plain store scaled by alpha
static int attention_part(const hb200_model* m, int bi, const hb200_block_weights& bw, const Workspace& w, const void* a_in,
                          const void* resid, float alpha, void* out, int B, int S, int32_t* err, cudaStream_t st,
                          const uint8_t* key_valid = nullptr, int mask_mode = 0) {
  const int T = B * S, D = m->dim, H = m->n_heads, KV = m->n_kv_heads, hd = m->head_dim;
  const int lat = H * hd, kvd = KV * hd, nq = lat + 2 * kvd;
  HB_PROPAGATE(gemm(m, HB200_K_GEMM_QKV, bi, 0, a_in, bw.w_qkv, w.qkv, T, nq, D, D, D, nq, EPI_STORE, nullptr, 1.0f,
                    nullptr, nullptr, err, st));
  {
    ProfScope ps(m->profile, st, HB200_K_PRE_ATTENTION, bi, 0, T, nq, 0);
    HB_PROPAGATE(hb200_ccgqa_pre_attention_ablated(w.qkv, bw.w1_qk, bw.w2_q, bw.w2_k, m->rope_cos, m->rope_sin,
                                                   bw.key_temperature, w.q, w.k, w.v, B, S, H, KV, hd, m->attn_disable,
                                                   m->conv_ksize ? m->conv_ksize : 3, err, st));
  }
  {
    ProfScope ps(m->profile, st, HB200_K_ATTENTION, bi, 0, T, lat, S);
    if (key_valid != nullptr)
      HB_PROPAGATE(hb200_attention_masked_gqa(w.q, w.k, w.v, w.o, key_valid, mask_mode, B, S, H, KV, hd,
                                              1.0f / sqrtf((float)hd), st));
    else
      // without the QK norm nothing bounds the logits: the online-softmax kernel
      HB_PROPAGATE(hb200_attention_causal_gqa(w.q, w.k, w.v, w.o, B, S, H, KV, hd, 1.0f / sqrtf((float)hd),
                                              (m->attn_disable & HB200_ATTN_NO_QK_NORM) ? 0.f : bw.attn_logit_bound,
                                              err, st));
  }
  HB_PROPAGATE(gemm(m, HB200_K_GEMM_O, bi, 0, w.o, bw.w_o, out, T, D, lat, lat, lat, D, resid ? EPI_RESID : EPI_STORE, resid, alpha, nullptr,
                    nullptr, err, st));
  return 0;
}

// q|k rows of the last four positions and the last v_shift half of every sequence -> decode state
__global__ void save_halo_kernel(const __nv_bfloat16* __restrict__ qkv, int S, int qkv_ld, int C, int kvd_half,
                                 __nv_bfloat16* __restrict__ halo, __nv_bfloat16* __restrict__ vshift) {
  const int b = blockIdx.x;
  for (int i = threadIdx.x; i < 4 * C; i += blockDim.x) {
    const int slot = i / C, c = i % C;
    const int tok = S - 4 + slot;
    halo[((size_t)b * 4 + slot) * C + c] = tok >= 0 ? qkv[((size_t)b * S + tok) * qkv_ld + c] : __float2bfloat16(0.f);
  }
  for (int c = threadIdx.x; c < kvd_half; c += blockDim.x)
    vshift[(size_t)b * kvd_half + c] = qkv[((size_t)b * S + S - 1) * qkv_ld + C + kvd_half + c];
}

// After the attention half of block `bi` in a prefill: keys / values into the caches (row stride = capacity), conv
// halo and v_shift from the qkv buffer.
static int capture_attention_state(const hb200_model* m, int bi, const Workspace& w, int B, int S,
                                   const hb200_decode_state* ds, cudaStream_t st) {
  const int H = m->n_heads, KV = m->n_kv_heads, hd = m->head_dim;
  const int lat = H * hd, kvd = KV * hd, C = lat + kvd;
  const size_t cache_block = (size_t)B * KV * ds->capacity * hd;
  __nv_bfloat16* kc = (__nv_bfloat16*)ds->kcache + (size_t)bi * cache_block;
  __nv_bfloat16* vc = (__nv_bfloat16*)ds->vcache + (size_t)bi * cache_block;
  HB_CUDA(cudaMemcpy2DAsync(kc, (size_t)ds->capacity * hd * 2, w.k, (size_t)S * hd * 2, (size_t)S * hd * 2,
                            (size_t)B * KV, cudaMemcpyDeviceToDevice, st));
  HB_CUDA(cudaMemcpy2DAsync(vc, (size_t)ds->capacity * hd * 2, w.v, (size_t)S * hd * 2, (size_t)S * hd * 2,
                            (size_t)B * KV, cudaMemcpyDeviceToDevice, st));
  save_halo_kernel<<<B, 256, 0, st>>>(w.qkv, S, lat + 2 * kvd, C, kvd / 2,
                                      (__nv_bfloat16*)ds->halo + (size_t)bi * B * 4 * C,
                                      (__nv_bfloat16*)ds->vshift + (size_t)bi * B * (kvd / 2));
  HB_LAUNCH_CHECK();
  return 0;
}

// x: block input; a_in: AdaRMSNorm(x; norm1) if the caller already has it (else computed here);
// y: block output; next_w / a_next: optional gain and destination of the norm that consumes y next.
// Static routing (dense compute, soft weights), one thread per 8 columns of a row:
//   cur += q * mlp + (1 - q) * u   with q = sigmoid(clamp(score, -10, 10)) in a MoD block (blocks.py:190-241), else q = 1;
//   out (+)= w_r * cur             with the soft depth weight w_r = exp(-(d - r)^2) / (sum_j exp(-(d - j)^2) + 1e-8),
//                                  d = sigmoid(3 tanh(l / 2)) * (R - 1)  (mixture_of_recursions.py:482-558).
template <bool HAS_MOD, bool HAS_OUT>
__global__ void __launch_bounds__(256) static_update_kernel(__nv_bfloat16* __restrict__ cur,
                                                            const __nv_bfloat16* __restrict__ mlp,
                                                            const __nv_bfloat16* __restrict__ u,
                                                            const float* __restrict__ scores,
                                                            const float* __restrict__ logits,
                                                            __nv_bfloat16* __restrict__ out, int64_t T, int D, int r, int R) {
  const int per_row = D / 8;
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (idx >= T * per_row) return;
  const int64_t t = idx / per_row;
  const int64_t at = t * D + (idx - t * per_row) * 8;
  float q = 1.f, wr = 0.f;
  if (HAS_MOD) q = 1.f / (1.f + expf(-fminf(fmaxf(scores[t], -10.f), 10.f)));
  if (HAS_OUT) {
    const float d = (float)(R - 1) / (1.f + expf(-3.f * tanhf(0.5f * logits[t])));
    float sum = 0.f;
    for (int j = 0; j < R; ++j) {
      const float e = expf(-(d - (float)j) * (d - (float)j));
      sum += e;
      if (j == r) wr = e;
    }
    wr /= sum + 1e-8f;
  }
  float c[8], m[8], un[8], o[8];
  load_bf16x8(cur + at, c);
  load_bf16x8(mlp + at, m);
  if (HAS_MOD) load_bf16x8(u + at, un);
  if (HAS_OUT && r > 0) load_bf16x8(out + at, o);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    c[j] += HAS_MOD ? q * m[j] + (1.f - q) * un[j] : m[j];
    if (HAS_OUT) o[j] = (r > 0 ? o[j] : 0.f) + wr * c[j];
  }
  store_bf16x8(cur + at, c);
  if (HAS_OUT) store_bf16x8(out + at, o);
}

static int block_forward(const hb200_model* m, int bi, const __nv_bfloat16* x, const __nv_bfloat16* a_in,
                         __nv_bfloat16* y, const float* next_w, __nv_bfloat16* a_next, int B, int S,
                         const Workspace& w, const hb200_taps* taps, int32_t* counts, int32_t* err, cudaStream_t st,
                         const hb200_decode_state* ds = nullptr) {
  const hb200_block_weights& bw = m->blocks[bi];
  const int T = B * S, D = m->dim, F = m->ffn_hidden, R = m->n_rec;
  const bool force = taps && taps->force_routing;
  const bool has_mod = bw.mod_wn != nullptr;
  const int k = mod_k(S, m->mod_capacity);
  const unsigned row_grid = (unsigned)ceil_div(T, 8);
  // pre-MLP norm folded into the first MLP contraction (needs the folded weights; not for static routing, whose mixing
  // step reads the normalised rows, nor for the cross-check GEMM)
  const bool fold = bw.w_gate_up_n != nullptr && bw.gate_up_bias != nullptr && m->static_routing == 0 && m->gemm_impl == 0;
  // row kernels in their streaming form (rows staged through shared memory by bulk copies) unless switched off
  static const bool stream_on = [] {
    const char* e = getenv("HB200_ROW_STREAM");
    return e == nullptr || e[0] != '0';
  }();

  NvtxRange block_range("hb200 block %d", bi);
  // attention half
  if (a_in == nullptr) {
    ProfScope ps(m->profile, st, HB200_K_RMS_NORM, bi, 0, T, D, 0);
    HB_PROPAGATE(hb200_rms_norm(x, bw.norm1_w, w.a, T, D, m->norm_eps, HB200_BF16, HB200_F32, st));
    a_in = w.a;
  }
  {
    NvtxRange r("hb200 attention");
    HB_PROPAGATE(attention_part(m, bi, bw, w, a_in, x, m->residual_scale * m->output_scale, w.cur, B, S, err, st));
  }

  if (ds != nullptr) HB_PROPAGATE(capture_attention_state(m, bi, w, B, S, ds, st));

  // routing buffers: the taps slots double as the working buffers when present
  int32_t* depth = (taps && taps->depths) ? taps->depths + (size_t)bi * T : w.depth;
  float* logits = (taps && taps->router_logits) ? taps->router_logits + (size_t)bi * T : w.logits;
  if (force) HB_REQUIRE(taps->depths != nullptr, HB200_ERR_INVALID, "forced routing needs taps.depths");
  if (force && has_mod) HB_REQUIRE(taps->mod_idx != nullptr, HB200_ERR_INVALID, "forced routing needs taps.mod_idx");
  const bool stat = m->static_routing != 0;
  if (stat) {
    HB_REQUIRE(!force, HB200_ERR_INVALID, "static routing makes no routing decisions to replay");
  }
  if ((!m->adaptive || stat) && !force) {                  // static routing: every token runs every recursion
    ProfScope ps(m->profile, st, HB200_K_OTHER, bi, 0, T, 0, 0);
    fill_i32_kernel<<<(unsigned)ceil_div(T, 256), 256, 0, st>>>(depth, T, R - 1);
    HB_LAUNCH_CHECK();
  }

  for (int r = 0; r < R; ++r) {
    NvtxRange rec_range("hb200 mlp recursion %d", r);
    const float* rec = bw.rec + (size_t)r * D;
    const bool need_router = (r == 0) && m->adaptive;
    float* scores = (taps && taps->mod_scores) ? taps->mod_scores + ((size_t)bi * R + r) * T : w.scores;
    if (need_router || has_mod) {
      ProfScope ps(m->profile, st, HB200_K_MOR_SCORE, bi, r, T, D, 0);
#define HB_SCORE(MOD_, ROUTER_, SS_)                                                                                   \
  HB_DISPATCH_NCH(D, {                                                                                                 \
    if (stream_on) {                                                                                                   \
      using SCfg = StreamCfg<NCH, 3>;                                                                                  \
      auto kern = mor_score_stream_kernel<NCH, MOD_, ROUTER_, SS_>;                                                    \
      HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, (size_t)SCfg::SMEM_BYTES));                                  \
      const int64_t n_tiles = ceil_div64(T, SCfg::TILE_ROWS);                                                          \
      const unsigned sgrid = (unsigned)std::min<int64_t>(n_tiles, sm_count());                                         \
      kern<<<sgrid, STREAM_THREADS, SCfg::SMEM_BYTES, st>>>(                                                           \
          w.cur, rec, bw.mod_wn, bw.mod_b, bw.mor_w, bw.mor_b, scores, logits, (force || stat) ? nullptr : depth, T, D, \
          m->norm_eps, R, m->min_depth, w.inv_rms, err);                                                               \
    } else {                                                                                                           \
      mor_score_kernel<NCH, MOD_, ROUTER_, SS_><<<(unsigned)ceil_div(T, 8 * SCORE_ROWS), 256, 0, st>>>(                \
          w.cur, rec, bw.mod_wn, bw.mod_b, bw.mor_w, bw.mor_b, scores, logits, (force || stat) ? nullptr : depth, T, D, \
          m->norm_eps, R, m->min_depth, w.inv_rms);                                                                    \
    }                                                                                                                  \
  })
      if (fold) {                                   // the pass over every row also leaves its norm scale
        if (has_mod && need_router) HB_SCORE(true, true, true);
        else if (has_mod) HB_SCORE(true, false, true);
        else HB_SCORE(false, true, true);
      } else {
        if (has_mod && need_router) HB_SCORE(true, true, false);
        else if (has_mod) HB_SCORE(true, false, false);
        else HB_SCORE(false, true, false);
      }
#undef HB_SCORE
      HB_LAUNCH_CHECK();
    }
    const bool have_scale = fold && (need_router || has_mod);
    if (ds != nullptr && has_mod)   // decode cache: the score of every prompt position, row stride = capacity
      HB_CUDA(cudaMemcpy2DAsync(ds->scores + (((size_t)bi * R + r) * B) * ds->capacity, (size_t)ds->capacity * 4, scores,
                                (size_t)S * 4, (size_t)S * 4, B, cudaMemcpyDeviceToDevice, st));
    int32_t* count = counts + (size_t)bi * R + r;
    {
    ProfScope ps(m->profile, st, HB200_K_SELECT, bi, r, T, 0, 0);
    if (has_mod && !stat) {
      int32_t* slot = (taps && taps->mod_idx) ? taps->mod_idx + ((size_t)bi * R + r) * B * k : w.sel_idx;
      HB_PROPAGATE(launch_mod_select(scores, B, S, k, force ? nullptr : slot, depth, r, w.rows, count,
                                     force ? slot : nullptr, st));
    } else if (stat) {
      all_rows_kernel<<<(unsigned)ceil_div(T, 256), 256, 0, st>>>(w.rows, T, count);
      HB_LAUNCH_CHECK();
    } else {
      HB_PROPAGATE(launch_compact_active(depth, T, r, w.rows, count, st));
    }
    }
    if (fold) {
      if (!have_scale) {                          // no score pass touched the rows: norm scale of the routed rows only
        ProfScope ps(m->profile, st, HB200_K_NORM_GATHER, bi, r, T, D, 0);
        HB_DISPATCH_NCH(D, rows_inv_rms_kernel<NCH><<<row_grid, 256, 0, st>>>(w.cur, rec, w.rows, count, w.inv_rms, D,
                                                                              m->norm_eps));
        HB_LAUNCH_CHECK();
      }
      ProfScope ps(m->profile, st, HB200_K_GEMM_GATE_UP, bi, r, T, 2 * F, D);
      GemmParams gp{w.cur, (const __nv_bfloat16*)bw.w_gate_up_n, w.act, T, 2 * F, D, D, D, F, EPI_SWIGLU, nullptr, 1.0f,
                    nullptr, count, err};
      gp.a_rows = w.rows;
      gp.row_scale = w.inv_rms;
      gp.col_bias = bw.gate_up_bias + (size_t)r * 2 * F;
      HB_PROPAGATE(launch_gemm_tcgen05(gp, st));
    } else {
      {
        ProfScope ps(m->profile, st, HB200_K_NORM_GATHER, bi, r, T, D, 0);
        HB_DISPATCH_NCH(D, {
          if (stream_on) {
            using SCfg = StreamCfg<NCH, 2>;
            auto kern = norm_gather_stream_kernel<NCH>;
            HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, (size_t)SCfg::SMEM_BYTES));
            const unsigned sgrid = (unsigned)std::min<int64_t>(ceil_div64(T, SCfg::TILE_ROWS), sm_count());
            kern<<<sgrid, STREAM_THREADS, SCfg::SMEM_BYTES, st>>>(w.cur, rec, bw.norm2_w, w.rows, count, w.ug, D, m->norm_eps, err);
          } else {
            norm_gather_kernel<NCH><<<row_grid, 256, 0, st>>>(w.cur, rec, bw.norm2_w, w.rows, count, w.ug, D, m->norm_eps);
          }
        });
        HB_LAUNCH_CHECK();
      }
      HB_PROPAGATE(gemm(m, HB200_K_GEMM_GATE_UP, bi, r, w.ug, bw.w_gate_up, w.act, T, 2 * F, D, D, D, F, EPI_SWIGLU, nullptr, 1.0f, nullptr, count,
                        err, st));
    }
    if (!stat) {
      HB_PROPAGATE(gemm(m, HB200_K_GEMM_DOWN, bi, r, w.act, bw.w_down, w.cur, T, D, F, F, F, D, EPI_SCATTER_ADD, nullptr, 1.0f, w.rows, count,
                        err, st));
      continue;
    }
    // static routing: the MLP result of every row goes to w.a (free between the attention half and the exit norm),
    // then one pass mixes it into cur and, with the depth router, accumulates the weighted state in y
    HB_PROPAGATE(gemm(m, HB200_K_GEMM_DOWN, bi, r, w.act, bw.w_down, w.a, T, D, F, F, F, D, EPI_STORE, nullptr, 1.0f, nullptr, nullptr,
                      err, st));
    {
      ProfScope ps(m->profile, st, HB200_K_OTHER, bi, r, T, D, 0);
      const unsigned grid = (unsigned)ceil_div64((int64_t)T * (D / 8), 256);
#define HB_STATIC(MOD_, OUT_)                                                                                         \
  static_update_kernel<MOD_, OUT_><<<grid, 256, 0, st>>>(w.cur, w.a, w.ug, scores, logits, y, (int64_t)T, D, r, R)
      if (has_mod && m->adaptive) HB_STATIC(true, true);
      else if (has_mod) HB_STATIC(true, false);
      else if (m->adaptive) HB_STATIC(false, true);
      else HB_STATIC(false, false);
#undef HB_STATIC
      HB_LAUNCH_CHECK();
    }
  }
  {
    ProfScope ps(m->profile, st, HB200_K_RMS_NORM, bi, R, T, D, 0);
    const __nv_bfloat16* exit_src = (stat && m->adaptive) ? y : w.cur;      // static + depth router: the weighted sum
    HB_DISPATCH_NCH(D, {
      if (stream_on) {
        using SCfg = StreamCfg<NCH, 2>;
        auto kern = dual_norm_stream_kernel<NCH>;
        HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, (size_t)SCfg::SMEM_BYTES));
        const unsigned sgrid = (unsigned)std::min<int64_t>(ceil_div64(T, SCfg::TILE_ROWS), sm_count());
        kern<<<sgrid, STREAM_THREADS, SCfg::SMEM_BYTES, st>>>(exit_src, bw.final_norm_w, y, next_w, next_w ? a_next : nullptr,
                                                             (int64_t)T, D, m->norm_eps, err);
      } else {
        dual_norm_kernel<NCH><<<row_grid, 256, 0, st>>>(exit_src, bw.final_norm_w, y, next_w, next_w ? a_next : nullptr, T, D,
                                                        m->norm_eps);
      }
    });
    HB_LAUNCH_CHECK();
  }
  if (taps && taps->block_out)
    HB_CUDA(cudaMemcpyAsync((__nv_bfloat16*)taps->block_out + (size_t)bi * T * D, y, (size_t)T * D * 2,
                            cudaMemcpyDeviceToDevice, st));
  return 0;
}

// y = s * y + (1 - s) * other, 8 columns per thread
__global__ void __launch_bounds__(256) blend_rows_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ other,
                                                         int64_t n8, float s) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n8) return;
  float a[8], b[8];
  load_bf16x8(y + i * 8, a);
  load_bf16x8(other + i * 8, b);
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = s * a[j] + (1.f - s) * b[j];
  store_bf16x8(y + i * 8, a);
}

// HydraMoRBlock.forward (blocks.py:645-657): with the MoR ramp-up scale strictly between 0 and 1 the block is run twice
// from the same input - fixed depth, then adaptive (whose routing the taps record) - and the two outputs are blended;
// the next consumer's input norm is then taken from the blend.
static int block_forward_or_blend(const hb200_model* m, int bi, const __nv_bfloat16* x, const __nv_bfloat16* a_in,
                                  __nv_bfloat16* y, const float* next_w, __nv_bfloat16* a_next, int B, int S,
                                  const Workspace& w, const hb200_taps* taps, int32_t* counts, int32_t* err, cudaStream_t st,
                                  const hb200_decode_state* ds) {
  if (!mor_blend_active(m)) return block_forward(m, bi, x, a_in, y, next_w, a_next, B, S, w, taps, counts, err, st, ds);
  HB_REQUIRE(ds == nullptr, HB200_ERR_UNSUPPORTED, "MoR ramp-up blend: cached decode is not built (forward / prefill only)");
  HB_REQUIRE(!(taps && taps->force_routing), HB200_ERR_UNSUPPORTED, "MoR ramp-up blend: forced routing is not built");
  const int64_t T = (int64_t)B * S;
  const int D = m->dim, R = m->n_rec;
  hb200_model fixed = *m, adaptive = *m;
  fixed.adaptive = 0;
  fixed.mor_rampup = adaptive.mor_rampup = 0.f;
  HB_CUDA(cudaMemsetAsync(w.counts2 + (size_t)bi * R, 0, (size_t)R * 4, st));
  // both passes take their own input norm (a_in = nullptr): the static-routing path uses w.a as scratch
  HB_PROPAGATE(block_forward(&fixed, bi, x, nullptr, w.blend, nullptr, nullptr, B, S, w, nullptr, w.counts2, err, st, nullptr));
  HB_PROPAGATE(block_forward(&adaptive, bi, x, nullptr, y, nullptr, nullptr, B, S, w, taps, counts, err, st, nullptr));
  {
    ProfScope ps(m->profile, st, HB200_K_OTHER, bi, R, (int)T, D, 0);
    blend_rows_kernel<<<(unsigned)ceil_div64(T * (D / 8), 256), 256, 0, st>>>(y, w.blend, T * (D / 8), m->mor_rampup);
    HB_LAUNCH_CHECK();
  }
  if (next_w != nullptr && a_next != nullptr) {
    ProfScope ps(m->profile, st, HB200_K_RMS_NORM, bi, R, (int)T, D, 0);
    HB_PROPAGATE(hb200_rms_norm(y, next_w, a_next, T, D, m->norm_eps, HB200_BF16, HB200_F32, st));
  }
  if (taps && taps->block_out)
    HB_CUDA(cudaMemcpyAsync((__nv_bfloat16*)taps->block_out + (size_t)bi * T * D, y, (size_t)T * D * 2,
                            cudaMemcpyDeviceToDevice, st));
  return 0;
}

}  // namespace hb200

using namespace hb200;

static int check_gemm_args(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw,
                           int64_t ldc, int epilogue, const void* resid, const int32_t* rows) {
  HB_REQUIRE(A && W && C, HB200_ERR_INVALID, "gemm: null pointer");
  HB_REQUIRE(M >= 0 && N >= 1 && K >= 1, HB200_ERR_INVALID, "gemm: bad shape M=%d N=%d K=%d", M, N, K);
  HB_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && ldc % 8 == 0 && lda >= K && ldw >= K, HB200_ERR_INVALID,
             "gemm: K and leading dimensions must be multiples of 8 (K=%d lda=%lld ldw=%lld ldc=%lld)", K,
             (long long)lda, (long long)ldw, (long long)ldc);
  HB_REQUIRE(aligned16(A) && aligned16(W) && aligned16(C) && (resid == nullptr || aligned16(resid)), HB200_ERR_INVALID,
             "gemm: pointers must be 16-byte aligned");
  HB_REQUIRE(epilogue >= EPI_STORE && epilogue <= EPI_SCATTER_ADD, HB200_ERR_INVALID, "gemm: unknown epilogue %d", epilogue);
  HB_REQUIRE(epilogue != EPI_RESID || resid != nullptr, HB200_ERR_INVALID, "gemm: residual epilogue needs resid");
  HB_REQUIRE(epilogue != EPI_SCATTER_ADD || rows != nullptr, HB200_ERR_INVALID, "gemm: scatter-add epilogue needs rows");
  HB_REQUIRE(epilogue != EPI_SWIGLU || N % 16 == 0, HB200_ERR_INVALID, "gemm: SwiGLU epilogue needs N %% 16 == 0");
  HB_REQUIRE(epilogue == EPI_SWIGLU ? ldc >= N / 2 : ldc >= N, HB200_ERR_INVALID, "gemm: ldc too small");
  return 0;
}

extern "C" int hb200_gemm_bf16(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw,
                               int64_t ldc, int epilogue, const void* resid, float alpha, const int32_t* rows,
                               const int32_t* m_dev, int impl, int32_t* err_flag, void* stream) {
  HB_PROPAGATE(check_gemm_args(A, W, C, M, N, K, lda, ldw, ldc, epilogue, resid, rows));
  HB_REQUIRE(impl == 0 || impl == 1, HB200_ERR_INVALID, "gemm: impl must be 0 (tcgen05) or 1 (mma.sync cross-check)");
  if (M == 0) return 0;
  GemmParams p{(const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (__nv_bfloat16*)C, M, N, K, lda, ldw, ldc, epilogue,
               (const __nv_bfloat16*)resid, epilogue == EPI_SCATTER_ADD ? 1.0f : alpha, rows, m_dev, err_flag};
  return impl == 0 ? launch_gemm_tcgen05(p, (cudaStream_t)stream) : launch_gemm_mma(p, (cudaStream_t)stream);
}

extern "C" int hb200_gemm_skinny_bf16(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw,
                                      int64_t ldc, int epilogue, const void* resid, float alpha, const int32_t* rows,
                                      const int32_t* m_dev, int32_t* err_flag, void* stream) {
  HB_PROPAGATE(check_gemm_args(A, W, C, M, N, K, lda, ldw, ldc, epilogue, resid, rows));
  if (M == 0) return 0;
  GemmParams p{(const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (__nv_bfloat16*)C, M, N, K, lda, ldw, ldc, epilogue,
               (const __nv_bfloat16*)resid, epilogue == EPI_SCATTER_ADD ? 1.0f : alpha, rows, m_dev, err_flag};
  return launch_gemm_skinny(p, (cudaStream_t)stream);
}

extern "C" int hb200_interleave_gate_up(const void* w_gate_up, void* w_out, int F, int K, void* stream) {
  HB_REQUIRE(w_gate_up && w_out && w_gate_up != w_out, HB200_ERR_INVALID, "interleave_gate_up: bad pointers");
  HB_REQUIRE(F >= 8 && F % 8 == 0 && K % 8 == 0, HB200_ERR_INVALID, "interleave_gate_up: F and K must be multiples of 8");
  const int64_t n = (int64_t)2 * F * (K / 8);
  interleave_gate_up_kernel<<<(unsigned)ceil_div64(n, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)w_gate_up, (__nv_bfloat16*)w_out, F, K);
  HB_LAUNCH_CHECK();
  return 0;
}

extern "C" int hb200_repack_conv_weight_k(const void* w, void* w_out, int c_out, int c_in, int ksize, void* stream) {
  HB_REQUIRE(w && w_out && w != w_out && c_out > 0 && c_in > 0 && ksize >= 1, HB200_ERR_INVALID,
             "repack_conv_weight: bad arguments");
  const int64_t n = (int64_t)c_out * c_in * ksize;
  repack_conv_kernel<<<(unsigned)ceil_div64(n, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)w, (__nv_bfloat16*)w_out, c_out, c_in, ksize);
  HB_LAUNCH_CHECK();
  return 0;
}

extern "C" int hb200_repack_conv_weight(const void* w, void* w_out, int c_out, int c_in, void* stream) {
  return hb200_repack_conv_weight_k(w, w_out, c_out, c_in, 3, stream);
}

extern "C" size_t hb200_model_workspace_bytes(const hb200_model* m, int B, int S) {
  if (m == nullptr || B < 1 || S < 1) return 0;
  return carve(m, B, S, nullptr).bytes;
}

extern "C" int hb200_ccgqa_forward(const hb200_model* m, int block_index, const void* x, void* y, int B, int S,
                                   void* workspace, size_t workspace_bytes, int32_t* err_flag, void* stream) {
  HB_PROPAGATE(check_model(m, B, S));
  HB_REQUIRE(x && y && workspace, HB200_ERR_INVALID, "ccgqa_forward: null pointer");
  HB_REQUIRE(block_index >= 0 && block_index < m->n_blocks, HB200_ERR_INVALID, "ccgqa_forward: bad block index");
  Workspace w = carve(m, B, S, workspace);
  HB_REQUIRE(workspace_bytes >= w.bytes, HB200_ERR_WORKSPACE, "workspace too small: %zu < %zu", workspace_bytes, w.bytes);
  return attention_part(m, block_index, m->blocks[block_index], w, x, nullptr, m->output_scale, y, B, S, err_flag,
                        (cudaStream_t)stream);
}

extern "C" int hb200_ccgqa_forward_masked(const hb200_model* m, int block_index, const void* x, void* y,
                                          const uint8_t* key_valid, int mask_mode, int B, int S, void* workspace,
                                          size_t workspace_bytes, int32_t* err_flag, void* stream) {
  HB_PROPAGATE(check_model(m, B, S));
  HB_REQUIRE(x && y && workspace && key_valid, HB200_ERR_INVALID, "ccgqa_forward_masked: null pointer");
  HB_REQUIRE(block_index >= 0 && block_index < m->n_blocks, HB200_ERR_INVALID, "ccgqa_forward_masked: bad block index");
  Workspace w = carve(m, B, S, workspace);
  HB_REQUIRE(workspace_bytes >= w.bytes, HB200_ERR_WORKSPACE, "workspace too small: %zu < %zu", workspace_bytes, w.bytes);
  return attention_part(m, block_index, m->blocks[block_index], w, x, nullptr, m->output_scale, y, B, S, err_flag,
                        (cudaStream_t)stream, key_valid, mask_mode);
}

// ---- attention forward on library-owned scratch (no allocation anywhere on the call path) -------------------
// The intermediates of the attention sub-block (qkv, q, k, v, o) live in this file-scope device array instead of a
// caller-provided workspace.  Its name is only a host-side handle: the device address is obtained once per device
// with cudaGetSymbolAddress (below) and that pointer is what the kernels receive.
constexpr size_t STATIC_SCRATCH_BYTES = (size_t)8 << 20;   // 8 MiB per GPU that loads the library
static __device__ __align__(256) unsigned char g_attn_scratch[STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
static void* g_attn_scratch_ptr[MAX_DEVICES] = {};
static std::mutex g_attn_scratch_mutex;

static size_t attention_scratch_bytes(const hb200_model* m, int64_t T, Workspace* w, void* base) {
  const size_t lat = (size_t)m->n_heads * m->head_dim, kvd = (size_t)m->n_kv_heads * m->head_dim;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    void* p = base ? (void*)((char*)base + off) : nullptr;
    off += align_up(bytes, 256);
    return p;
  };
  __nv_bfloat16* qkv = (__nv_bfloat16*)take((size_t)T * (lat + 2 * kvd) * 2);
  __nv_bfloat16* q = (__nv_bfloat16*)take((size_t)T * lat * 2);
  __nv_bfloat16* k = (__nv_bfloat16*)take((size_t)T * kvd * 2);
  __nv_bfloat16* v = (__nv_bfloat16*)take((size_t)T * kvd * 2);
  __nv_bfloat16* o = (__nv_bfloat16*)take((size_t)T * lat * 2);
  if (w != nullptr) {
    *w = Workspace{};
    w->qkv = qkv; w->q = q; w->k = k; w->v = v; w->o = o;
    w->bytes = off;
  }
  return off;
}

extern "C" size_t hb200_ccgqa_forward_static_max_bytes(void) { return STATIC_SCRATCH_BYTES; }

extern "C" int hb200_ccgqa_forward_static(const hb200_model* m, int block_index, const void* x, void* y, int B, int S,
                                          int32_t* err_flag, void* stream) {
  HB_PROPAGATE(check_model(m, B, S));
  HB_REQUIRE(x && y, HB200_ERR_INVALID, "ccgqa_forward_static: null pointer");
  HB_REQUIRE(block_index >= 0 && block_index < m->n_blocks, HB200_ERR_INVALID, "ccgqa_forward_static: bad block index");
  const size_t need = attention_scratch_bytes(m, (int64_t)B * S, nullptr, nullptr);
  HB_REQUIRE(need <= STATIC_SCRATCH_BYTES, HB200_ERR_WORKSPACE,
             "ccgqa_forward_static: %d x %d tokens need %zu bytes of scratch, the built-in array holds %zu; "
             "use hb200_ccgqa_forward with a caller-provided workspace for larger batches",
             B, S, need, STATIC_SCRATCH_BYTES);
  int dev = -1;
  HB_CUDA(cudaGetDevice(&dev));
  HB_REQUIRE(dev >= 0 && dev < MAX_DEVICES, HB200_ERR_UNSUPPORTED, "ccgqa_forward_static: device index %d out of range", dev);
  void* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_attn_scratch_mutex);
    if (g_attn_scratch_ptr[dev] == nullptr) {
      // once per device, with that device current: resolve the symbol to this device's copy of the array
      void* ptr = nullptr;
      HB_CUDA(cudaGetSymbolAddress(&ptr, g_attn_scratch));
      HB_REQUIRE(ptr != nullptr, HB200_ERR_CUDA, "ccgqa_forward_static: cudaGetSymbolAddress returned a null address");
      g_attn_scratch_ptr[dev] = ptr;
    }
    base = g_attn_scratch_ptr[dev];
  }
  Workspace w;
  attention_scratch_bytes(m, (int64_t)B * S, &w, base);
  return attention_part(m, block_index, m->blocks[block_index], w, x, nullptr, m->output_scale, y, B, S, err_flag,
                        (cudaStream_t)stream);
}

extern "C" int hb200_block_forward(const hb200_model* m, int block_index, const void* x, void* y, int B, int S,
                                   void* workspace, size_t workspace_bytes, const hb200_taps* taps, int32_t* err_flag,
                                   void* stream) {
  HB_PROPAGATE(check_model(m, B, S));
  HB_REQUIRE(x && y && workspace, HB200_ERR_INVALID, "block_forward: null pointer");
  HB_REQUIRE(block_index >= 0 && block_index < m->n_blocks, HB200_ERR_INVALID, "block_forward: bad block index");
  Workspace w = carve(m, B, S, workspace);
  HB_REQUIRE(workspace_bytes >= w.bytes, HB200_ERR_WORKSPACE, "workspace too small: %zu < %zu", workspace_bytes, w.bytes);
  cudaStream_t st = (cudaStream_t)stream;
  int32_t* counts = (taps && taps->mlp_rows) ? taps->mlp_rows : w.counts;
  HB_CUDA(cudaMemsetAsync(counts + (size_t)block_index * m->n_rec, 0, (size_t)m->n_rec * 4, st));
  return block_forward_or_blend(m, block_index, (const __nv_bfloat16*)x, nullptr, (__nv_bfloat16*)y, nullptr, nullptr, B, S,
                                w, taps, counts, err_flag, st, nullptr);
}

static int run_model(const hb200_model* m, const int64_t* ids, int B, int S, const Workspace& w, void* logits,
                     int64_t ld_logits, __nv_bfloat16* hid, const hb200_taps* taps, int32_t* err_flag, cudaStream_t st,
                     const hb200_decode_state* ds) {
  const int T = B * S, D = m->dim;
  int32_t* counts = (taps && taps->mlp_rows) ? taps->mlp_rows : w.counts;
  HB_CUDA(cudaMemsetAsync(counts, 0, (size_t)m->n_blocks * m->n_rec * 4, st));
  HB_REQUIRE(aligned16(m->tok_emb) && aligned16(m->lm_head) && m->norm_w != nullptr, HB200_ERR_INVALID,
             "model_forward: bad embedding / output projection / norm pointer");
  {
    // embedding fused with the first block's pre-attention norm
    ProfScope ps(m->profile, st, HB200_K_EMBED, -1, 0, T, D, 0);
    HB_DISPATCH_NCH(D, embed_norm_kernel<NCH><<<(unsigned)ceil_div(T, 8), 256, 0, st>>>(
                           ids, (const __nv_bfloat16*)m->tok_emb, w.x0, m->blocks[0].norm1_w, w.a, T, D, m->vocab,
                           sqrtf((float)D), m->norm_eps));
    HB_LAUNCH_CHECK();
  }
  // each block's exit norm also produces the next consumer's input norm: the next block's norm1 into w.a, or the
  // model's final norm into the hidden-state buffer after the last block
  __nv_bfloat16 *xin = w.x0, *xout = w.x1;
  for (int bi = 0; bi < m->n_blocks; ++bi) {
    const bool last = (bi == m->n_blocks - 1);
    const float* next_w = last ? m->norm_w : m->blocks[bi + 1].norm1_w;
    // w.a is read by this block's qkv GEMM long before its exit norm overwrites it with the next block's input
    HB_PROPAGATE(block_forward_or_blend(m, bi, xin, w.a, xout, next_w, last ? hid : w.a, B, S, w, taps, counts, err_flag, st,
                                        ds));
    std::swap(xin, xout);
  }
  if (logits != nullptr) {
    NvtxRange r("hb200 output projection");
    HB_PROPAGATE(gemm(m, HB200_K_GEMM_LM_HEAD, m->n_blocks, 0, hid, output_weight(m), logits, T, m->vocab, D, D, D, ld_logits,
                      EPI_STORE, nullptr, 1.0f, nullptr, nullptr, err_flag, st));
  }
  return 0;
}

extern "C" int hb200_model_forward(const hb200_model* m, const int64_t* ids, int B, int S, void* workspace,
                                   size_t workspace_bytes, void* logits, int64_t ld_logits, void* hidden_out,
                                   const hb200_taps* taps, int32_t* err_flag, void* stream) {
  HB_PROPAGATE(check_model(m, B, S));
  HB_REQUIRE(ids && workspace, HB200_ERR_INVALID, "model_forward: null pointer");
  HB_REQUIRE(logits == nullptr || (ld_logits >= m->vocab && ld_logits % 8 == 0), HB200_ERR_INVALID,
             "model_forward: ld_logits must be >= vocab and a multiple of 8");
  Workspace w = carve(m, B, S, workspace);
  HB_REQUIRE(workspace_bytes >= w.bytes, HB200_ERR_WORKSPACE, "workspace too small: %zu < %zu", workspace_bytes, w.bytes);
  __nv_bfloat16* hid = hidden_out ? (__nv_bfloat16*)hidden_out : w.ug;   // ug is free once the last block is done
  return run_model(m, ids, B, S, w, logits, ld_logits, hid, taps, err_flag, (cudaStream_t)stream, nullptr);
}

// last hidden row of every sequence -> compact [B, D]; prompt tokens -> history
__global__ void prefill_tail_kernel(const __nv_bfloat16* __restrict__ hid, int S, int D, __nv_bfloat16* __restrict__ last,
                                    const int64_t* __restrict__ ids, int64_t* __restrict__ history, int capacity) {
  const int b = blockIdx.x;
  for (int i = threadIdx.x * 8; i < D; i += blockDim.x * 8)
    *reinterpret_cast<uint4*>(last + (size_t)b * D + i) =
        *reinterpret_cast<const uint4*>(hid + ((size_t)b * S + S - 1) * D + i);
  if (history != nullptr)
    for (int t = threadIdx.x; t < S; t += blockDim.x) history[(size_t)b * capacity + t] = ids[(size_t)b * S + t];
}

__global__ void set_pos_kernel(int32_t* pos, int value, const int64_t* __restrict__ tokens, int64_t* __restrict__ history,
                               int capacity, int B) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B && history != nullptr && value < capacity) history[(size_t)b * capacity + value] = tokens[b];
  if (b == 0) *pos = value;
}

extern "C" int hb200_model_prefill_cached(const hb200_model* m, const int64_t* ids, int B, int S, void* workspace,
                                          size_t workspace_bytes, const hb200_decode_state* state, void* last_logits,
                                          int64_t ld_logits, int32_t* err_flag, void* stream) {
  HB_PROPAGATE(check_model(m, B, S));
  HB_REQUIRE(ids && workspace && state, HB200_ERR_INVALID, "prefill_cached: null pointer");
  HB_REQUIRE(state->kcache && state->vcache && state->halo && state->vshift && state->scores && state->pos &&
                 state->tokens,
             HB200_ERR_INVALID, "prefill_cached: incomplete decode state");
  HB_REQUIRE(state->batch == B && state->capacity >= S && state->capacity <= m->max_seq_len, HB200_ERR_INVALID,
             "prefill_cached: state is for batch %d / capacity %d (need batch %d, %d <= capacity <= %d)", state->batch,
             state->capacity, B, S, m->max_seq_len);
  HB_REQUIRE(m->attn_disable == 0 && (m->conv_ksize == 0 || m->conv_ksize == 3), HB200_ERR_UNSUPPORTED,
             "prefill_cached: attention stages switched off (attn_disable = %d) or conv kernel size %d are not built for "
             "the cached decode", m->attn_disable, m->conv_ksize);
  HB_REQUIRE(ld_logits >= m->vocab && ld_logits % 8 == 0, HB200_ERR_INVALID, "prefill_cached: bad ld_logits");
  HB_REQUIRE(m->dim % 8 == 0, HB200_ERR_UNSUPPORTED, "prefill_cached: dim must be a multiple of 8");
  Workspace w = carve(m, B, S, workspace);
  HB_REQUIRE(workspace_bytes >= w.bytes, HB200_ERR_WORKSPACE, "workspace too small: %zu < %zu", workspace_bytes, w.bytes);
  cudaStream_t st = (cudaStream_t)stream;
  const int D = m->dim;
  HB_PROPAGATE(run_model(m, ids, B, S, w, nullptr, 0, w.ug, nullptr, err_flag, st, state));
  // last position of every sequence -> logits -> greedy token; w.a / w.act are free now
  __nv_bfloat16* last = w.a;
  __nv_bfloat16* lg = last_logits ? (__nv_bfloat16*)last_logits : w.act;
  HB_REQUIRE(last_logits != nullptr || (size_t)m->ffn_hidden * B * S >= (size_t)B * ld_logits, HB200_ERR_WORKSPACE,
             "prefill_cached: pass last_logits (the workspace cannot hold them for this shape)");
  prefill_tail_kernel<<<B, 128, 0, st>>>(w.ug, S, D, last, ids, state->history, state->capacity);
  HB_LAUNCH_CHECK();
  HB_PROPAGATE(gemm(m, HB200_K_GEMM_LM_HEAD, m->n_blocks, 0, last, output_weight(m), lg, B, m->vocab, D, D, D, ld_logits,
                    EPI_STORE, nullptr, 1.0f, nullptr, nullptr, err_flag, st));
  HB_PROPAGATE(hb200_argmax_rows(lg, B, m->vocab, ld_logits, state->tokens, st));
  set_pos_kernel<<<ceil_div(B, 128), 128, 0, st>>>(state->pos, S, state->tokens, state->history, state->capacity, B);
  HB_LAUNCH_CHECK();
  return 0;
}

extern "C" void* hb200_profile_create(int capacity) {
  if (capacity <= 0) return nullptr;
  Profile* p = new (std::nothrow) Profile();
  if (p == nullptr) return nullptr;
  p->capacity = capacity;
  p->rec.resize(capacity);
  p->ev.resize(2 * (size_t)capacity, nullptr);
  for (auto& e : p->ev) {
    if (cudaEventCreate(&e) != cudaSuccess) {
      for (auto& d : p->ev)
        if (d) cudaEventDestroy(d);
      delete p;
      set_error("profile_create: cudaEventCreate failed");
      return nullptr;
    }
  }
  return p;
}

extern "C" void hb200_profile_destroy(void* profile) {
  Profile* p = static_cast<Profile*>(profile);
  if (p == nullptr) return;
  for (auto& e : p->ev)
    if (e) cudaEventDestroy(e);
  delete p;
}

extern "C" int hb200_profile_reset(void* profile) {
  HB_REQUIRE(profile != nullptr, HB200_ERR_INVALID, "profile_reset: null handle");
  static_cast<Profile*>(profile)->count = 0;
  static_cast<Profile*>(profile)->dropped = 0;
  return 0;
}

extern "C" int hb200_profile_read(void* profile, hb200_launch_record* records, float* ms, int max_records) {
  HB_REQUIRE(profile != nullptr && records != nullptr && ms != nullptr, HB200_ERR_INVALID, "profile_read: null pointer");
  Profile* p = static_cast<Profile*>(profile);
  const int n = p->count < max_records ? p->count : max_records;
  for (int i = 0; i < n; ++i) {
    records[i] = p->rec[i];
    HB_CUDA(cudaEventElapsedTime(&ms[i], p->ev[2 * i], p->ev[2 * i + 1]));
  }
  return p->count + p->dropped;
}
