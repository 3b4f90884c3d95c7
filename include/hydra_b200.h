/*
 * hydra_b200 — C ABI of the B200 (sm_100a) implementation of HYDRA's inference
 * forward hot path.
 *
 * The reference (mcpirate17/HYDRA) is pure Python + Triton and has no FFI of its
 * own: its replaceable boundary is a set of Python-level names.  Each entry point
 * below names the reference interface it stands behind (file:line relative to
 * the reference project root).  The Python package `hydra_b200` binds these
 * symbols with ctypes and re-exposes them under the reference's own function
 * signatures (`hydra.kernels.fused_*`, `hydra.attention.build_hybrid_attention_module`).
 *
 * Conventions
 *   - every function returns 0 on success or a negative hb200_status;
 *     hb200_last_error() returns a thread-local description of the last failure;
 *   - all data pointers are DEVICE pointers, 16-byte aligned, owned by the caller;
 *     no entry point allocates or frees device memory, synchronises the device,
 *     or traps; work is enqueued on `stream` (a cudaStream_t passed as void*);
 *   - tensors are row-major; "bf16" is the 16-bit brain float bit pattern;
 *   - entry points are re-entrant per stream.
 */
#ifndef HYDRA_B200_H
#define HYDRA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum hb200_status {
  HB200_OK = 0,
  HB200_ERR_INVALID = -1,      /* bad argument (null pointer, unsupported shape, misalignment) */
  HB200_ERR_CUDA = -2,         /* a CUDA runtime / driver call failed */
  HB200_ERR_WORKSPACE = -3,    /* workspace too small */
  HB200_ERR_UNSUPPORTED = -4,  /* shape outside what the kernels are built for */
  HB200_ERR_DEVICE_WAIT = -5   /* a bounded in-kernel wait ran out (see hb200_gemm_bf16) */
} hb200_status;

typedef enum hb200_dtype { HB200_F32 = 0, HB200_BF16 = 1, HB200_F16 = 2 } hb200_dtype;

/* Library version (major*10000 + minor*100 + patch). */
int hb200_version(void);
/* Thread-local text for the most recent non-zero status returned on this thread. */
const char* hb200_last_error(void);

/* ---------------------------------------------------------------------------
 * Exported fused-op semantics  (hydra/kernels/__init__.py:13-38)
 * ------------------------------------------------------------------------- */

/* fused_rms_norm(x, weight, eps): y = x * rsqrt(mean(x^2) + eps) * w, row-wise.
 * Replaces hydra/kernels/fused_ops.py:1114-1132 (and RMSNorm / AdaRMSNorm forward,
 * hydra/layers/common.py:90-118,153-160).  x,y: [rows, dim] of `dtype`; w: [dim] of `w_dtype`. */
int hb200_rms_norm(const void* x, const void* w, void* y, int64_t rows, int dim, float eps,
                   int dtype, int w_dtype, void* stream);

/* fused_rope(x, cos, sin): interleaved-pair rotary embedding.
 * Replaces hydra/kernels/fused_ops.py:240-306.  x: [B,H,S,hd] with element strides
 * (sb, sh, ss) and unit stride on hd (may be a transposed view); y: contiguous [B,H,S,hd];
 * cos/sin: fp32 tables, row t at cos + t*table_ld, hd/2 entries per row. */
int hb200_rope(const void* x, const float* cos_t, const float* sin_t, void* y,
               int B, int H, int S, int hd, int64_t sb, int64_t sh, int64_t ss,
               int table_ld, int dtype, void* stream);

/* fused_qk_norm(q, k, scale, temperature): per-head-vector L2 normalisation.
 * Replaces hydra/kernels/fused_ops.py:474-493.  mode 0: x / max(||x||, 1e-12) * s
 * (the PyTorch path, fused_ops.py:587-596, also attention.py:260-262);
 * mode 1: x * rsqrt(sum x^2 + 1e-8) * s (the reference's device kernel, fused_ops.py:350-369).
 * q: [rows_q, hd], k: [rows_k, hd] contiguous; K is additionally multiplied by temperature. */
int hb200_qk_norm(const void* q, const void* k, void* q_out, void* k_out, int64_t rows_q,
                  int64_t rows_k, int hd, float scale, float temperature, int mode, int dtype,
                  void* stream);

/* fused_swiglu(gate, up) = silu(gate) * up.  Replaces hydra/kernels/fused_ops.py:808-883.
 * gate/up: [rows, cols] with leading dimensions ld_gate / ld_up (chunk views of one
 * [rows, 2*cols] buffer are the usual case); out contiguous [rows, cols]. */
int hb200_swiglu(const void* gate, const void* up, void* out, int64_t rows, int cols,
                 int64_t ld_gate, int64_t ld_up, int dtype, void* stream);

/* ---------------------------------------------------------------------------
 * CCGQA attention block pieces  (hydra/attention/backends/ccgqa/attention.py:201-331)
 * ------------------------------------------------------------------------- */

/* Dense contraction C = epilogue(A @ W^T) on the tcgen05 tensor cores; A [M,K], W [N,K] bf16.
 * Stands for every nn.Linear on the path (attention.py:122-124,205,330;
 * hydra/layers/common.py:221-230; hydra/model/framework/model.py:343,506).
 *   epilogue 0  STORE        C[m,n]        = acc                       (C bf16 [M,N], ld ldc)
 *   epilogue 1  RESID        C[m,n]        = resid[m,n] + alpha*acc    (resid bf16, ld ldc)
 *   epilogue 2  SWIGLU       C[m,j]        = silu(g)*u, W rows interleaved in groups of 8:
 *                            row 16*i+r is gate row 8*i+r (r<8) or up row 8*i+r-8 (r>=8);
 *                            C is [M, N/2]
 *   epilogue 3  SCATTER_ADD  C[rows[m], n] += acc  (rows int32 [M], each target row once)
 * m_dev, when non-null, is a device int32 holding the live row count (<= M); tiles beyond it are
 * skipped and `rows` is not read beyond it.  Epilogues 1 and 3 never touch rows of C beyond the live
 * count; epilogues 0 and 2 write whole 32-row boxes, so rows [live, M) of C may be overwritten.
 * impl 0 = tcgen05/TMEM/TMA kernel (product path); impl 1 = plain mma.sync kernel kept as an
 * independent cross-check for tests.
 * err_flag: optional device int32; set non-zero if a bounded in-kernel wait ran out (the kernel
 * then returns without hanging; outputs are undefined). */
int hb200_gemm_bf16(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda,
                    int64_t ldw, int64_t ldc, int epilogue, const void* resid, float alpha,
                    const int32_t* rows, const int32_t* m_dev, int impl, int32_t* err_flag,
                    void* stream);

/* The same contraction for M <= 512 rows (decode; one 128-row tile per grid.y), where streaming W from HBM once is the
 * bound: one CTA per (128 weight rows, slice of K) so that all SMs stream, tcgen05/TMEM/TMA inside a CTA, and the K slices of a row tile
 * reduced in fixed order through the distributed shared memory of a thread-block cluster (deterministic; no global
 * scratch, no atomics).  No counterpart in the reference (which has no decode path); arguments as hb200_gemm_bf16. */
int hb200_gemm_skinny_bf16(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda,
                           int64_t ldw, int64_t ldc, int epilogue, const void* resid, float alpha,
                           const int32_t* rows, const int32_t* m_dev, int32_t* err_flag, void* stream);

/* Interleave a [2F, K] gate_up weight (gate rows then up rows, hydra/layers/common.py:225-226)
 * into the row order epilogue 2 expects. */
int hb200_interleave_gate_up(const void* w_gate_up, void* w_out, int F, int K, void* stream);

/* Repack Conv1d weights [C, C/groups, 3] (kernels/fused_conv.py:22-37) to [C, 3*(C/groups)]
 * with element (c_out, j*cin + c_in) = w[c_out, c_in, j], bf16 -> bf16. */
int hb200_repack_conv_weight(const void* w, void* w_out, int c_out, int c_in, void* stream);
/* The same for kernel size ksize: [C, C/groups, ksize] -> [C, ksize*(C/groups)]. */
int hb200_repack_conv_weight_k(const void* w, void* w_out, int c_out, int c_in, int ksize, void* stream);

/* Everything between qkv_proj and SDPA in one kernel (attention.py:208-266,
 * kernels/fused_conv.py:39-62): value shift, grouped k=3 causal conv, dense k=3 causal conv,
 * QK-mean coupling, L2 norm with key temperature, RoPE.
 * qkv [B,S,lat+2*kvd] bf16 -> q [B,H,S,hd], k [B,KV,S,hd], v [B,KV,S,hd] bf16.
 * w1_qk: repacked conv1 weights, q rows then k rows: [lat+kvd, 3*hd];
 * w2_q [lat, 3*lat], w2_k [kvd, 3*kvd] repacked conv2 weights; cos/sin fp32 [>=S, hd/2];
 * key_temperature: device fp32 scalar.
 * For latent 256 / kv_dim 64 with head_dim 16 or 32 the dense conv runs on tcgen05 with TMEM accumulators and a
 * TMA-fed weight ring; other shapes use the mma.sync kernel.  err_flag: optional device int32, set non-zero if a
 * bounded in-kernel wait ran out. */
int hb200_ccgqa_pre_attention(const void* qkv, const void* w1_qk, const void* w2_q, const void* w2_k,
                              const float* cos_t, const float* sin_t, const float* key_temperature,
                              void* q, void* k, void* v, int B, int S, int H, int KV, int hd,
                              int32_t* err_flag, void* stream);

/* The same with some of the reference module's stages switched off (CCGQAAttention(use_rope=, use_qk_norm=, use_convs=,
 * use_qk_mean=, use_value_shift=), attention.py:74-160, 211-266): `disable` is a mask of the bits below; 0 is
 * hb200_ccgqa_pre_attention.  Without convolutions q and k go on as projected (conv weights may be NULL); without the
 * QK norm neither the L2 normalisation nor the key temperature is applied (key_temperature may be NULL); without RoPE
 * the tables may be NULL; without the value shift v is the last kv_dim columns of qkv.  conv_ksize is the module's
 * conv_kernel_size (1 .. 8; weights repacked with hb200_repack_conv_weight_k: w1_qk [lat+kvd, ksize*hd], w2_q
 * [lat, ksize*lat], w2_k [kvd, ksize*kvd]; each conv pads ksize-1 zeros on the left).  Any switched-off stage, and any
 * kernel size other than 3, selects the CUDA-core kernel (the reference's models never do either: these are its
 * ablation switches). */
enum {
  HB200_ATTN_NO_ROPE = 1, HB200_ATTN_NO_QK_NORM = 2, HB200_ATTN_NO_CONVS = 4, HB200_ATTN_NO_QK_MEAN = 8,
  HB200_ATTN_NO_VALUE_SHIFT = 16, HB200_ATTN_NO_ALL = 31
};
int hb200_ccgqa_pre_attention_ablated(const void* qkv, const void* w1_qk, const void* w2_q, const void* w2_k,
                                      const float* cos_t, const float* sin_t, const float* key_temperature,
                                      void* q, void* k, void* v, int B, int S, int H, int KV, int hd, int disable,
                                      int conv_ksize, int32_t* err_flag, void* stream);

/* Causal grouped-query attention in the latent space (attention.py:288-327):
 * o[b,t,h,:] = softmax_causal(q[b,h] k[b,h/(H/KV)]^T * scale) v[b,h/(H/KV)].
 * q [B,H,S,hd], k/v [B,KV,S,hd] bf16; o token-major [B,S,H*hd] bf16.
 * logit_bound > 0 is the caller's guarantee that |q.k| * scale <= logit_bound for every pair (CCGQA: q is a unit
 * vector and |k| is the key temperature, so temperature * scale, plus rounding slack): the tcgen05/TMEM kernel then
 * runs, which subtracts the bound instead of a running row maximum.  logit_bound <= 0 (unknown), or a bound above
 * 27 (2^-80 would underflow the probabilities), selects the online-softmax mma.sync kernel.
 * err_flag: optional device int32, set non-zero if a bounded in-kernel wait ran out. */
int hb200_attention_causal_gqa(const void* q, const void* k, const void* v, void* o, int B, int S,
                               int H, int KV, int hd, float scale, float logit_bound, int32_t* err_flag,
                               void* stream);

/* Attention with a padding mask: CCGQAAttention.forward(x, mask), mask [B,S] with 1 = valid token, 0 = padding
 * (attention.py:269-283).  key_valid: device uint8 [B*S], non-zero = valid.  Query i uses key j where
 *   HB200_MASK_AS_REFERENCE: j > i or key j is padding.  This is what the reference computes: its boolean mask is True
 *     for future and padded keys, and F.scaled_dot_product_attention reads True as "takes part";
 *   HB200_MASK_INTENDED:     j <= i and key j is valid - what the comments at that place describe.
 * A query with no usable key gives zeros (SDPA's result for a fully masked row).  Same layouts as
 * hb200_attention_causal_gqa.  One CUDA-core kernel (a thread per query): the reference's models never reach this
 * path - both block types drop the mask - so it is built for the module contract, not for speed. */
enum { HB200_MASK_AS_REFERENCE = 0, HB200_MASK_INTENDED = 1 };
int hb200_attention_masked_gqa(const void* q, const void* k, const void* v, void* o, const uint8_t* key_valid,
                               int mode, int B, int S, int H, int KV, int hd, float scale, void* stream);

/* ---------------------------------------------------------------------------
 * Routing  (hydra/routing/mixture_of_depths.py:159-216, mixture_of_recursions.py:251-291,
 *           hydra/model/framework/blocks.py:243-269)
 * ------------------------------------------------------------------------- */

/* MoD selection: for each of B rows of fp32 scores [B,L], the ascending indices of the k
 * largest (torch.topk + torch.sort, mixture_of_depths.py:187, blocks.py:261).  Among scores
 * equal to the k-th largest the lowest indices are taken; NaN ranks above +inf.
 * idx_out int32 [B,k].  If depth (int32 [B,L]) and rows_out are given, the flat token ids
 * b*L+pos of the selected positions with depth >= min_active_depth are appended to rows_out
 * and counted in *count (device int32, must be zero on entry). */
int hb200_mod_topk_select(const float* scores, int B, int L, int k, int32_t* idx_out,
                          const int32_t* depth, int min_active_depth, int32_t* rows_out,
                          int32_t* count, void* stream);

/* MoR depth assignment from raw router logits (mixture_of_recursions.py:268-289):
 * depth = clamp(round_half_even(min_d + sigmoid(3*tanh(l/2))*(R-1-min_d)), min_d, R-1). */
int hb200_mor_depths(const float* logits, int32_t* depth, int64_t n, int n_rec, int min_depth,
                     void* stream);

/* Token embedding (hydra/model/framework/model.py:51-73,427): ids clamped into [0,V),
 * rows gathered and scaled.  ids int64 [T]; table bf16 [V,D]; out bf16 [T,D]. */
int hb200_embed(const int64_t* ids, const void* table, void* out, int64_t T, int D, int V,
                float scale, void* stream);

/* Greedy next-token choice: out[r] = argmax over the first `cols` entries of bf16 row r (rows are `ld` elements
 * apart; lowest index among equal maxima).  Stands for the sampling step of the reference's generation helper
 * (diagnostics/eval_checkpoint.py:112-166) in its deterministic, temperature-free form. */
int hb200_argmax_rows(const void* x, int64_t rows, int cols, int64_t ld, int64_t* out, void* stream);

/* Token-level cross-entropy of bf16 logit rows, the loss of the reference's evaluation helper
 * (diagnostics/eval_checkpoint.py:168-193: F.cross_entropy of the logits against the next tokens):
 * nll[r] = logsumexp(row r over the first `cols` entries) - row[targets[r]], fp32; 0 where targets[r] == ignore_index
 * (F.cross_entropy's default -100).  Other targets must lie in [0, cols).  The caller reduces (sum / mean). */
int hb200_cross_entropy_rows(const void* logits, const int64_t* targets, int64_t rows, int cols, int64_t ld,
                             int64_t ignore_index, float* nll, void* stream);

/* The sampling step of the reference's generation helper (diagnostics/eval_checkpoint.py:133-155) for bf16 rows:
 * logits / temperature; top_k > 0: values below the k-th largest are removed (ties with it stay); top_p < 1: in
 * descending order a token is removed iff the probability mass before it exceeds top_p (the first always stays),
 * probabilities being the softmax of what top-k left; then one draw from the renormalised rest.  The reference draws
 * with torch.multinomial; here out[r] is the inverse CDF, in descending-logit order with equal logits by ascending
 * index, at uniforms[r] in [0,1) (device fp32 [rows]) - a function of (row, uniform), reproducible on any stream.
 * temperature <= 0 or top_k == 1 gives the argmax (uniforms may then be NULL).  cols <= 65535.  NaN logits take no
 * part; -0 and +0 are one value.  Arithmetic: fp32 exponentials of the bf16 logits, masses accumulated exactly in
 * 64-bit fixed point. */
int hb200_sample_rows(const void* logits, int64_t rows, int cols, int64_t ld, float temperature, int top_k,
                      float top_p, const float* uniforms, int64_t* out, void* stream);

/* ---------------------------------------------------------------------------
 * Whole block / whole model  (hydra/model/framework/blocks.py:608-632,
 *                             hydra/model/framework/model.py:408-506)
 * ------------------------------------------------------------------------- */

typedef struct hb200_block_weights {
  const float* norm1_w;          /* [D] AdaRMSNorm gain before attention */
  const float* norm2_w;          /* [D] AdaRMSNorm gain before the MLP   */
  const float* final_norm_w;     /* [D] RMSNorm gain at block exit, or NULL: no exit norm (HydraBlock, blocks.py:33-70) */
  const void* w_qkv;             /* bf16 [lat+2*kvd, D]                  */
  const void* w_o;               /* bf16 [D, lat]                        */
  const void* w1_qk;             /* bf16 repacked conv1 (q rows, k rows) */
  const void* w2_q;              /* bf16 repacked conv2 for q            */
  const void* w2_k;              /* bf16 repacked conv2 for k            */
  const float* key_temperature;  /* device fp32 [1]                      */
  const void* w_gate_up;         /* bf16 [2F, D], interleaved            */
  const void* w_down;            /* bf16 [D, F]                          */
  const float* mor_w;            /* fp32 [D] depth-router weight         */
  const float* mor_b;            /* fp32 [1] depth-router bias           */
  const float* rec;              /* fp32 [R, D] recursion_bias + recursion_embed */
  const float* mod_wn;           /* fp32 [D] MoD router weight times the norm2 gain (elementwise), or NULL */
  const float* mod_b;            /* fp32 [1] MoD router bias, or NULL    */
  float attn_logit_bound;        /* HOST value: |key_temperature| / sqrt(head_dim) * 1.02, or 0 if unknown */
  /* Optional pair that folds the pre-MLP norm into the first MLP contraction (both or neither):
   *   AdaRMSNorm(x + rec_r; g) W^T  =  inv_rms(x + rec_r) * ( x W'^T + rec_r W'^T ),   W' = W diag(g).
   * With them the executor contracts the routed rows of the hidden state directly (no normalised copy is written
   * or re-read) and applies the row scale and the per-recursion column bias in the SwiGLU epilogue. */
  const void* w_gate_up_n;       /* bf16 [2F, D]: gate_up.weight * norm2 gain (per input column), interleaved as w_gate_up; or NULL */
  const float* gate_up_bias;     /* fp32 [R, 2F]: rec[r] . w_gate_up_n rows (fp32 sums over the bf16 values), same interleaving; or NULL */
} hb200_block_weights;

typedef struct hb200_model {
  int32_t vocab, dim, n_blocks, n_rec, n_heads, n_kv_heads, head_dim, ffn_hidden;
  int32_t min_depth, adaptive, max_seq_len, gemm_impl;
  float mod_capacity, norm_eps, residual_scale, output_scale;
  const void* tok_emb;            /* bf16 [V, D] (also the output projection when lm_head is NULL) */
  const float* norm_w;            /* fp32 [D] */
  const float* rope_cos;          /* fp32 [max_seq_len, hd/2] */
  const float* rope_sin;
  const hb200_block_weights* blocks;   /* HOST array of n_blocks entries */
  void* profile;                  /* optional hb200_profile handle (see below), or NULL */
  const void* lm_head;            /* bf16 [V, D] untied output projection (tie_weights=False, model.py:343-349),
                                     or NULL: the output projection is tok_emb */
  int32_t static_routing;         /* 1: the model was built with static_routing_mode (model.py:202, honoured in eval
                                     too): every token runs every recursion; MoD mixes mlp(u) with u by the router
                                     probability (blocks.py:190-241), MoR weights each recursion's state by soft depth
                                     weights (mixture_of_recursions.py:482-558).  Honoured by the forward, the cached prefill
                                     and the decode step. */
  float mor_rampup;               /* MoR curriculum scale (blocks.py:645-657, 731-745).  Strictly between 0 and 1 (with
                                     adaptive = 1): every block returns scale * adaptive + (1 - scale) * fixed-depth, both
                                     computed in full - forward / prefill only.  Any other value (0 included): no blend,
                                     `adaptive` alone decides. */
  int32_t attn_disable;           /* HB200_ATTN_NO_* bits: stages of the attention module that are switched off (the
                                     reference's ablation switches).  0 for every model the reference builds; non-zero is
                                     honoured by hb200_ccgqa_forward[_masked] / hb200_block_forward / hb200_model_forward
                                     and refused by the cached decode. */
  int32_t conv_ksize;             /* conv kernel size of the attention modules (conv_kernel_size, attention.py:86); 0 means 3,
                                     the value of every model the reference builds.  Other sizes (1 .. 8) run the CUDA-core
                                     pre-attention kernel and are refused by the cached decode. */
} hb200_model;

/* Optional routing taps / forced routing for one forward (device pointers or NULL). */
typedef struct hb200_taps {
  int32_t* depths;        /* int32 [NB, B*S]: written; read instead if force_routing */
  int32_t* mod_idx;       /* int32 [NB, R, B, k]: ascending MoD indices; read if force_routing */
  float* mod_scores;      /* fp32 [NB, R, B*S] (written only) */
  float* router_logits;   /* fp32 [NB, B*S] raw depth-router logits (written only) */
  int32_t* mlp_rows;      /* int32 [NB, R]: rows whose MLP result was used (always written) */
  void* block_out;        /* bf16 [NB, B*S, D] block outputs (written only) */
  int32_t force_routing;  /* 1: take depths and mod_idx from the buffers above */
} hb200_taps;

/* Bytes of workspace hb200_model_forward needs for a [B,S] batch. */
size_t hb200_model_workspace_bytes(const hb200_model* m, int B, int S);

/* HydraModel.forward in eval (model.py:408-506): ids int64 [B,S] -> logits bf16 [B*S, ld_logits]
 * (ld_logits >= vocab, multiple of 8; a multiple of 64 - rows on 128-byte boundaries - lets the output projection
 * store whole memory sectors and is what the Python layer uses).  `hidden_out` (bf16 [B*S, D], optional) receives the
 * post-norm hidden state (forward_hidden).  If logits is NULL the output projection is skipped.
 * err_flag: device int32, set non-zero if a bounded in-kernel wait ran out. */
int hb200_model_forward(const hb200_model* m, const int64_t* ids, int B, int S, void* workspace,
                        size_t workspace_bytes, void* logits, int64_t ld_logits, void* hidden_out,
                        const hb200_taps* taps, int32_t* err_flag, void* stream);

/* One HydraMoRBlock forward (blocks.py:608-632) on x bf16 [B*S, D] -> y bf16 [B*S, D];
 * `block_index` selects the taps slot. Same workspace as the model. */
int hb200_block_forward(const hb200_model* m, int block_index, const void* x, void* y, int B, int S,
                        void* workspace, size_t workspace_bytes, const hb200_taps* taps,
                        int32_t* err_flag, void* stream);

/* CCGQAAttention.forward (attention.py:201-331) on x bf16 [B*S, D] -> y bf16 [B*S, D]
 * (y = o_proj(attn) * output_scale; no residual). Uses blocks[block_index] weights. */
int hb200_ccgqa_forward(const hb200_model* m, int block_index, const void* x, void* y, int B, int S,
                        void* workspace, size_t workspace_bytes, int32_t* err_flag, void* stream);
/* The same with a padding mask (key_valid, mask_mode: see hb200_attention_masked_gqa).  Projections, convolutions and
 * the value shift run over padded positions unchanged, as in the reference; only the attention core reads the mask. */
int hb200_ccgqa_forward_masked(const hb200_model* m, int block_index, const void* x, void* y, const uint8_t* key_valid,
                               int mask_mode, int B, int S, void* workspace, size_t workspace_bytes, int32_t* err_flag,
                               void* stream);

/* ---------------------------------------------------------------------------
 * Cached (incremental) decode.  The reference has no KV cache and no decode path: its generation helper
 * re-runs the whole forward for every token (diagnostics/eval_checkpoint.py:127-160).  These entry points add a
 * latent-space KV cache for autoregressive decode.  With MoD capacity 1.0 a cached step
 * computes exactly what a re-forward computes for the newest position; with capacity < 1 a past token's MoD
 * selection stays frozen at what it was when the token was newest (MoD's top-k over the sequence is not causal).
 * ------------------------------------------------------------------------- */
typedef struct hb200_decode_state {
  int32_t batch, capacity;   /* B sequences advancing in lockstep; room for `capacity` positions            */
  void* kcache;              /* bf16 [NB, B, KV, capacity, hd]  post-RoPE keys                               */
  void* vcache;              /* bf16 [NB, B, KV, capacity, hd]  value-shifted values                         */
  void* halo;                /* bf16 [NB, B, 4, lat+kvd]  pre-conv q|k rows of the last four positions       */
  void* vshift;              /* bf16 [NB, B, kvd/2]  v_shift half of the last position                       */
  float* scores;             /* fp32 [NB, R, B, capacity]  MoD router score of every cached position         */
  int32_t* pos;              /* device int32: number of cached positions                                     */
  int64_t* tokens;           /* device int64 [B]: token processed by the next step; each step overwrites it
                                with its greedy choice                                                       */
  int64_t* history;          /* device int64 [B, capacity] or NULL: token of every position (prompt + generated) */
} hb200_decode_state;

/* Bytes of workspace one decode step needs for B sequences. */
size_t hb200_decode_workspace_bytes(const hb200_model* m, int B);

/* Prefill with cache capture: the eval forward of ids [B,S] (workspace as hb200_model_forward) that also fills
 * `state` (caches, halos, scores, pos = S) and leaves the greedy choice after the last prompt position in
 * state->tokens (and history[:, S]).  last_logits: optional bf16 [B, ld_logits] output of the last position. */
int hb200_model_prefill_cached(const hb200_model* m, const int64_t* ids, int B, int S, void* workspace,
                               size_t workspace_bytes, const hb200_decode_state* state, void* last_logits,
                               int64_t ld_logits, int32_t* err_flag, void* stream);

/* One decode step: processes state->tokens at position *state->pos through every block against the caches,
 * appends to the caches, writes the greedy next token back to state->tokens (and history), advances *pos.
 * Everything position-dependent is read from device memory, so the identical launch sequence serves every step.
 * last_logits: optional bf16 [B, ld_logits]. */
int hb200_model_decode_step(const hb200_model* m, const hb200_decode_state* state, void* workspace,
                            size_t workspace_bytes, void* last_logits, int64_t ld_logits, int32_t* err_flag,
                            void* stream);

/* CCGQAAttention.forward for callers that must not allocate.  This entry point has no counterpart in the
 * reference; it is hb200_ccgqa_forward with the workspace argument removed.
 *
 * Who needs it: code that runs where device memory cannot be requested at call time - a serving process that has
 * handed all of its HBM to a pool owned by someone else (a KV-cache arena, another framework's caching allocator),
 * a plugin running on threads of a host runtime that forbids allocation calls there, or a latency-critical loop
 * that cannot afford cudaMalloc's implicit device synchronisation and unbounded duration.  Such callers cannot
 * create the workspace that hb200_ccgqa_forward asks for.
 *
 * How: the intermediates (qkv, q, k, v, attention output) are kept in an 8 MiB device array that is part of the
 * library image (every GPU that loads the library carries it until the process exits).  The call performs no
 * cudaMalloc / cudaFree and calls no allocating library routine.  x and y are still the caller's buffers
 * (bf16 [B*S, dim] each, 16-byte aligned).
 *
 * Limits and rules:
 *   - B*S tokens must fit: qkv (latent + 2*kv_dim) + q (latent) + k (kv_dim) + v (kv_dim) + o (latent) columns of
 *     bf16 per token, i.e. B*S*2*(3*latent + 4*kv_dim) bytes (each of the five buffers rounded up to 256) <= 8 MiB:
 *     4096 tokens at dim 1024 with 8q/2kv heads (latent 256, kv_dim 64: 2048 B per token); larger requests return
 *     HB200_ERR_WORKSPACE and launch nothing (hb200_ccgqa_forward_static_max_bytes() reports the capacity);
 *   - the first call on each device is the set-up call: it resolves the array's device address
 *     (cudaGetSymbolAddress, with that device current), and with CUDA's default lazy module loading that is also the
 *     moment the driver loads the part of the library that holds the array, so THAT call can take the 8 MiB (plus the
 *     kernels' code) from the device and can fail with HB200_ERR_CUDA if the device has nothing left.  Only the calls
 *     after it are allocation-free.  Make the set-up call once at start-up, while memory can still be had, and
 *     outside any stream capture;
 *   - the resolved address is remembered per device for the life of the process; cudaDeviceReset invalidates it, so
 *     a process that resets a device must not use this entry point on that device afterwards;
 *   - all calls on one device share the one array and it keeps the previous call's contents.  Every byte a call
 *     reads it has written first, so nothing needs clearing, but two calls that overlap on the GPU (different
 *     streams) race on it: serialise them. */
size_t hb200_ccgqa_forward_static_max_bytes(void);
int hb200_ccgqa_forward_static(const hb200_model* m, int block_index, const void* x, void* y, int B, int S,
                               int32_t* err_flag, void* stream);

/* ---------------------------------------------------------------------------
 * Measurement aid (no counterpart in the reference): per-launch CUDA-event timing of the kernels that
 * hb200_model_forward / hb200_block_forward / hb200_ccgqa_forward enqueue.  When hb200_model.profile holds a
 * handle, every kernel launch of the executor is bracketed by two events recorded on the launching stream.
 * ------------------------------------------------------------------------- */
typedef enum hb200_kernel_kind {
  HB200_K_GEMM_QKV = 0, HB200_K_GEMM_O = 1, HB200_K_GEMM_GATE_UP = 2, HB200_K_GEMM_DOWN = 3,
  HB200_K_GEMM_LM_HEAD = 4, HB200_K_RMS_NORM = 5, HB200_K_PRE_ATTENTION = 6, HB200_K_ATTENTION = 7,
  HB200_K_MOR_SCORE = 8, HB200_K_SELECT = 9, HB200_K_NORM_GATHER = 10, HB200_K_EMBED = 11, HB200_K_OTHER = 12
} hb200_kernel_kind;

/* One record per launch: kind, block, recursion, M (upper bound for device-counted launches), N, K. */
typedef struct hb200_launch_record { int32_t kind, block, rec, m, n, k; } hb200_launch_record;

/* Create a recorder able to hold `capacity` launches (events are created here, once). NULL on failure. */
void* hb200_profile_create(int capacity);
void hb200_profile_destroy(void* profile);
/* Forget the recorded launches (call between measured steps, after reading). */
int hb200_profile_reset(void* profile);
/* After the stream has been synchronised: copies up to `max_records` records and their durations in
 * milliseconds; returns the number of launches the executor made since the last reset (negative on error).  A
 * return value above the recorder's capacity means that many launches found it full and were not recorded: size
 * the recorder for the launches between two reads. */
int hb200_profile_read(void* profile, hb200_launch_record* records, float* ms, int max_records);

#ifdef __cplusplus
}
#endif
#endif /* HYDRA_B200_H */
