// Causal grouped-query attention in the CCGQA latent space (head_dim 16 / 32 / 64; 8 on a CUDA-core kernel).
//
// One CTA = 64 query rows of one (batch, q-head): 4 warps x 16 rows.  K/V tiles of 64 keys are staged in
// shared memory; S = QK^T and O += PV run on the tensor cores (mma.sync m16n8k16, bf16 in / fp32 acc),
// with a base-2 online softmax in registers.  Heavy (late) query tiles are scheduled first so the causal
// triangle balances across the SMs.  Output is token-major [B,S,H*hd], the A operand of the o_proj GEMM.
#include "common.cuh"
#include "mma.cuh"

namespace hb200 {

constexpr int ATT_BM = 64;   // query rows per CTA
constexpr int ATT_BN = 64;   // keys per tile

template <int HD>
__global__ void __launch_bounds__(128) attention_causal_gqa_kernel(const __nv_bfloat16* __restrict__ q,
                                                                   const __nv_bfloat16* __restrict__ k,
                                                                   const __nv_bfloat16* __restrict__ v,
                                                                   __nv_bfloat16* __restrict__ o, int S, int H,
                                                                   int KV, float scale_log2) {
  constexpr int LDS = HD + 8;                 // padded smem row (bf16 elements)
  constexpr int KSTEPS = HD / 16;             // k-steps of QK^T
  constexpr int NT_O = HD / 8;                // n-tiles of the output
  __shared__ __align__(16) __nv_bfloat16 Ks[2][ATT_BN][LDS];
  __shared__ __align__(16) __nv_bfloat16 Vs[2][ATT_BN][LDS];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n_qt = (S + ATT_BM - 1) / ATT_BM;
  const int qt = n_qt - 1 - (int)blockIdx.x;   // late tiles (most keys) first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (H / KV);
  const int q0 = qt * ATT_BM;
  const __nv_bfloat16* qp = q + ((size_t)b * H + h) * S * HD;
  const __nv_bfloat16* kp = k + ((size_t)b * KV + kvh) * S * HD;
  const __nv_bfloat16* vp = v + ((size_t)b * KV + kvh) * S * HD;

  // Q fragments for this warp's 16 rows (rows beyond S read as zero)
  const int r_lo = q0 + warp * 16 + g, r_hi = r_lo + 8;
  uint32_t qa[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    const int c = ks * 16 + 2 * t;
    qa[ks][0] = r_lo < S ? *reinterpret_cast<const uint32_t*>(qp + (size_t)r_lo * HD + c) : 0u;
    qa[ks][1] = r_hi < S ? *reinterpret_cast<const uint32_t*>(qp + (size_t)r_hi * HD + c) : 0u;
    qa[ks][2] = r_lo < S ? *reinterpret_cast<const uint32_t*>(qp + (size_t)r_lo * HD + c + 8) : 0u;
    qa[ks][3] = r_hi < S ? *reinterpret_cast<const uint32_t*>(qp + (size_t)r_hi * HD + c + 8) : 0u;
  }

  float oacc[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) oacc[i][c] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  const int n_kt = qt + 1;   // causal: key tiles 0..qt (ATT_BM == ATT_BN)
  auto load_tile = [&](int kt, int buf) {
    const int k0 = kt * ATT_BN;
    constexpr int PIECES = HD / 8;
    for (int idx = tid; idx < ATT_BN * PIECES; idx += 128) {
      const int r = idx / PIECES, pc = idx % PIECES;
      const int key = k0 + r;
      if (key < S) {
        cp_async_16(&Ks[buf][r][pc * 8], kp + (size_t)key * HD + pc * 8);
        cp_async_16(&Vs[buf][r][pc * 8], vp + (size_t)key * HD + pc * 8);
      } else {
        *reinterpret_cast<uint4*>(&Ks[buf][r][pc * 8]) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(&Vs[buf][r][pc * 8]) = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_commit();
  };

  load_tile(0, 0);
  for (int kt = 0; kt < n_kt; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < n_kt) {
      load_tile(kt + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    // S = Q K^T  (16 x 64 per warp)
    float s[ATT_BN / 8][4];
#pragma unroll
    for (int nt = 0; nt < ATT_BN / 8; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const __nv_bfloat16* kr = &Ks[buf][nt * 8 + g][ks * 16 + 2 * t];
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kr);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kr + 8);
        mma_bf16_16816(s[nt], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
      }
    }
    // scale to base-2 logits, causal mask on the diagonal tile
    const int k0 = kt * ATT_BN;
    const bool diag = (kt == qt);
#pragma unroll
    for (int nt = 0; nt < ATT_BN / 8; ++nt) {
      const int c = k0 + nt * 8 + 2 * t;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = c + (e & 1);
        const int row = (e < 2) ? r_lo : r_hi;
        float val = s[nt][e] * scale_log2;
        if (diag && key > row) val = -INFINITY;
        s[nt][e] = val;
      }
    }
    // online softmax (each row lives in the 4 lanes of a quad)
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < ATT_BN / 8; ++nt) {
      mx_lo = fmaxf(mx_lo, fmaxf(s[nt][0], s[nt][1]));
      mx_hi = fmaxf(mx_hi, fmaxf(s[nt][2], s[nt][3]));
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    // key 0 is visible to every row, so the running maximum is finite from the first tile on
    const float a_lo = exp2f(m_lo - mn_lo), a_hi = exp2f(m_hi - mn_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    float rs_lo = 0.f, rs_hi = 0.f;
    uint32_t pa[ATT_BN / 16][4];
#pragma unroll
    for (int nt = 0; nt < ATT_BN / 8; ++nt) {
      const float p0 = exp2f(s[nt][0] - mn_lo), p1 = exp2f(s[nt][1] - mn_lo);
      const float p2 = exp2f(s[nt][2] - mn_hi), p3 = exp2f(s[nt][3] - mn_hi);
      rs_lo += p0 + p1;
      rs_hi += p2 + p3;
      // C fragments of two adjacent n-tiles form the A fragment of one k16 step of P V
      pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(p0, p1);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(p2, p3);
    }
    l_lo = l_lo * a_lo + rs_lo;
    l_hi = l_hi * a_hi + rs_hi;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      oacc[i][0] *= a_lo;
      oacc[i][1] *= a_lo;
      oacc[i][2] *= a_hi;
      oacc[i][3] *= a_hi;
    }
    // O += P V  (k = key index inside the tile)
#pragma unroll
    for (int kk = 0; kk < ATT_BN / 16; ++kk) {
#pragma unroll
      for (int nt = 0; nt < NT_O; ++nt) {
        uint32_t b0, b1;
        ldmatrix_x2_trans(b0, b1, &Vs[buf][kk * 16 + (lane & 15)][nt * 8]);
        mma_bf16_16816(oacc[nt], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
      }
    }
    __syncthreads();
  }

  // finish: row sums across the quad, normalise, token-major bf16 store
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float i_lo = 1.0f / l_lo, i_hi = 1.0f / l_hi;
  const size_t ld_o = (size_t)H * HD;
  __nv_bfloat16* ob = o + (size_t)b * S * ld_o + (size_t)h * HD;
#pragma unroll
  for (int nt = 0; nt < NT_O; ++nt) {
    const int c = nt * 8 + 2 * t;
    if (r_lo < S) *reinterpret_cast<uint32_t*>(ob + (size_t)r_lo * ld_o + c) = pack_bf16x2(oacc[nt][0] * i_lo, oacc[nt][1] * i_lo);
    if (r_hi < S) *reinterpret_cast<uint32_t*>(ob + (size_t)r_hi * ld_o + c) = pack_bf16x2(oacc[nt][2] * i_hi, oacc[nt][3] * i_hi);
  }
}

// Heads narrower than a tensor-core k-step (head_dim 8: the reference's small test models, dim 128 with four heads):
// one thread per query row, online softmax in registers, K / V rows read as 16-byte pieces (every thread of a warp asks
// for the same key, so each piece is one broadcast).  Built for coverage, not speed.
template <int HD>
__global__ void __launch_bounds__(128) attention_small_head_kernel(const __nv_bfloat16* __restrict__ q,
                                                                   const __nv_bfloat16* __restrict__ k,
                                                                   const __nv_bfloat16* __restrict__ v,
                                                                   __nv_bfloat16* __restrict__ o, int S, int H, int KV,
                                                                   float scale_log2) {
  const int i = blockIdx.x * 128 + threadIdx.x;       // query position
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (H / KV);
  const __nv_bfloat16* kp = k + ((size_t)b * KV + kvh) * S * HD;
  const __nv_bfloat16* vp = v + ((size_t)b * KV + kvh) * S * HD;
  float qv[HD], acc[HD];
#pragma unroll
  for (int d = 0; d < HD; ++d) { qv[d] = 0.f; acc[d] = 0.f; }
  if (i < S) {
#pragma unroll
    for (int c = 0; c < HD / 8; ++c) {
      float t[8];
      load_bf16x8(q + (((size_t)b * H + h) * S + i) * HD + c * 8, t);
#pragma unroll
      for (int d = 0; d < 8; ++d) qv[c * 8 + d] = t[d] * scale_log2;
    }
  }
  float mx = -INFINITY, l = 0.f;
  const int last = min(S - 1, blockIdx.x * 128 + 127);  // keys any row of this CTA may need
  for (int j = 0; j <= last; ++j) {
    float kr[HD], vr[HD];
#pragma unroll
    for (int c = 0; c < HD / 8; ++c) {
      float tk[8], tv[8];
      load_bf16x8(kp + (size_t)j * HD + c * 8, tk);
      load_bf16x8(vp + (size_t)j * HD + c * 8, tv);
#pragma unroll
      for (int d = 0; d < 8; ++d) { kr[c * 8 + d] = tk[d]; vr[c * 8 + d] = tv[d]; }
    }
    if (j > i || i >= S) continue;
    float sc = 0.f;
#pragma unroll
    for (int d = 0; d < HD; ++d) sc += qv[d] * kr[d];
    const float nm = fmaxf(mx, sc);
    const float corr = exp2f(mx - nm), pj = exp2f(sc - nm);   // exp2f(-inf) = 0 on the first key
    l = l * corr + pj;
#pragma unroll
    for (int d = 0; d < HD; ++d) acc[d] = acc[d] * corr + pj * vr[d];
    mx = nm;
  }
  if (i >= S) return;
  const float inv = 1.0f / l;
  __nv_bfloat16* dst = o + ((size_t)b * S + i) * ((size_t)H * HD) + (size_t)h * HD;
#pragma unroll
  for (int c = 0; c < HD / 8; ++c) {
    float t[8];
#pragma unroll
    for (int d = 0; d < 8; ++d) t[d] = acc[c * 8 + d] * inv;
    store_bf16x8(dst + c * 8, t);
  }
}

// Attention with a padding mask (key_valid[b, j] != 0 <=> token j of sequence b is not padding), one thread per query row,
// online softmax in registers, K and V rows read in 16-byte pieces (all threads of a warp ask for the same key: one
// broadcast each).  Which keys query i may use:
//   mode HB200_MASK_AS_REFERENCE: j > i or key j is padding - what the reference module computes when it is handed a
//     mask: it marks future and padded keys True in a boolean mask (attention.py:269-283), which SDPA reads as "takes part";
//   mode HB200_MASK_INTENDED:     j <= i and key j is valid - what its comments describe.
// A query with no usable key gives zeros.  The reference's models never reach this path (their blocks drop the mask);
// it is built for the module contract, not for speed.
template <int HD>
__global__ void __launch_bounds__(128) attention_masked_kernel(const __nv_bfloat16* __restrict__ q,
                                                               const __nv_bfloat16* __restrict__ k,
                                                               const __nv_bfloat16* __restrict__ v,
                                                               const uint8_t* __restrict__ key_valid,
                                                               __nv_bfloat16* __restrict__ o, int S, int H, int KV,
                                                               float scale_log2, int mode) {
  const int i = blockIdx.x * 128 + threadIdx.x;       // query position
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (H / KV);
  const __nv_bfloat16* kp = k + ((size_t)b * KV + kvh) * S * HD;
  const __nv_bfloat16* vp = v + ((size_t)b * KV + kvh) * S * HD;
  const uint8_t* valid = key_valid + (size_t)b * S;
  float qv[HD], acc[HD];
#pragma unroll
  for (int d = 0; d < HD; ++d) { qv[d] = 0.f; acc[d] = 0.f; }
  if (i < S) {
#pragma unroll
    for (int c = 0; c < HD / 8; ++c) {
      float t[8];
      load_bf16x8(q + (((size_t)b * H + h) * S + i) * HD + c * 8, t);
#pragma unroll
      for (int d = 0; d < 8; ++d) qv[c * 8 + d] = t[d] * scale_log2;
    }
  }
  float mx = -INFINITY, l = 0.f;
  for (int j = 0; j < S; ++j) {
    const bool ok = valid[j] != 0;                                           // uniform over the CTA
    const bool use = i < S && (mode == HB200_MASK_AS_REFERENCE ? (j > i || !ok) : (j <= i && ok));
    if (!__syncthreads_or(use)) continue;                                    // no row of this CTA wants key j
    float sc = 0.f;
#pragma unroll
    for (int c = 0; c < HD / 8; ++c) {
      float tk[8];
      load_bf16x8(kp + (size_t)j * HD + c * 8, tk);
#pragma unroll
      for (int d = 0; d < 8; ++d) sc += qv[c * 8 + d] * tk[d];
    }
    if (!use) continue;
    const float nm = fmaxf(mx, sc);
    const float corr = exp2f(mx - nm), pj = exp2f(sc - nm);                  // exp2f(-inf) = 0 on the first key
    l = l * corr + pj;
#pragma unroll
    for (int c = 0; c < HD / 8; ++c) {
      float tv[8];
      load_bf16x8(vp + (size_t)j * HD + c * 8, tv);
#pragma unroll
      for (int d = 0; d < 8; ++d) acc[c * 8 + d] = acc[c * 8 + d] * corr + pj * tv[d];
    }
    mx = nm;
  }
  if (i >= S) return;
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  __nv_bfloat16* dst = o + ((size_t)b * S + i) * ((size_t)H * HD) + (size_t)h * HD;
#pragma unroll
  for (int c = 0; c < HD / 8; ++c) {
    float t[8];
#pragma unroll
    for (int d = 0; d < 8; ++d) t[d] = acc[c * 8 + d] * inv;
    store_bf16x8(dst + c * 8, t);
  }
}

int launch_attention_tcgen05(const void* q, const void* k, const void* v, void* o, int B, int S, int H, int KV, int hd,
                             float scale, float logit_bound, int32_t* err_flag, cudaStream_t st);

}  // namespace hb200

using namespace hb200;

extern "C" int hb200_attention_causal_gqa(const void* q, const void* k, const void* v, void* o, int B, int S, int H,
                                          int KV, int hd, float scale, float logit_bound, int32_t* err_flag,
                                          void* stream) {
  HB_REQUIRE(q && k && v && o, HB200_ERR_INVALID, "attention: null pointer");
  HB_REQUIRE(B >= 0 && S >= 0 && H >= 1 && KV >= 1 && H % KV == 0, HB200_ERR_INVALID, "attention: bad shape");
  HB_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o), HB200_ERR_INVALID,
             "attention: pointers must be 16-byte aligned");
  HB_REQUIRE(B <= 65535 && H <= 65535, HB200_ERR_UNSUPPORTED, "attention: batch/head count beyond grid limits");
  if ((int64_t)B * S == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (logit_bound > 0.f && logit_bound <= 27.f && (hd == 16 || hd == 32 || hd == 64) &&
      (int64_t)B * H * S < (1ll << 31))
    return launch_attention_tcgen05(q, k, v, o, B, S, H, KV, hd, scale, logit_bound, err_flag, st);
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid((S + ATT_BM - 1) / ATT_BM, H, B);
  const __nv_bfloat16 *qp = (const __nv_bfloat16*)q, *kp = (const __nv_bfloat16*)k, *vp = (const __nv_bfloat16*)v;
  if (hd == 16)
    attention_causal_gqa_kernel<16><<<grid, 128, 0, st>>>(qp, kp, vp, (__nv_bfloat16*)o, S, H, KV, scale_log2);
  else if (hd == 32)
    attention_causal_gqa_kernel<32><<<grid, 128, 0, st>>>(qp, kp, vp, (__nv_bfloat16*)o, S, H, KV, scale_log2);
  else if (hd == 64)
    attention_causal_gqa_kernel<64><<<grid, 128, 0, st>>>(qp, kp, vp, (__nv_bfloat16*)o, S, H, KV, scale_log2);
  else if (hd == 8)
    attention_small_head_kernel<8><<<dim3((S + 127) / 128, H, B), 128, 0, st>>>(qp, kp, vp, (__nv_bfloat16*)o, S, H, KV,
                                                                              scale_log2);
  else {
    set_error("attention: head_dim %d not built (8, 16, 32, 64)", hd);
    return HB200_ERR_UNSUPPORTED;
  }
  HB_LAUNCH_CHECK();
  return 0;
}

extern "C" int hb200_attention_masked_gqa(const void* q, const void* k, const void* v, void* o, const uint8_t* key_valid,
                                          int mode, int B, int S, int H, int KV, int hd, float scale, void* stream) {
  HB_REQUIRE(q && k && v && o && key_valid, HB200_ERR_INVALID, "masked attention: null pointer");
  HB_REQUIRE(B >= 0 && S >= 0 && H >= 1 && KV >= 1 && H % KV == 0, HB200_ERR_INVALID, "masked attention: bad shape");
  HB_REQUIRE(mode == HB200_MASK_AS_REFERENCE || mode == HB200_MASK_INTENDED, HB200_ERR_INVALID,
             "masked attention: unknown mask mode %d", mode);
  HB_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o), HB200_ERR_INVALID,
             "masked attention: pointers must be 16-byte aligned");
  HB_REQUIRE(B <= 65535 && H <= 65535, HB200_ERR_UNSUPPORTED, "masked attention: batch/head count beyond grid limits");
  if ((int64_t)B * S == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const float scale_log2 = scale * 1.4426950408889634f;
  const dim3 grid((S + 127) / 128, H, B);
  const __nv_bfloat16 *qp = (const __nv_bfloat16*)q, *kp = (const __nv_bfloat16*)k, *vp = (const __nv_bfloat16*)v;
#define HB_MASKED(HD_)                                                                                          \
  attention_masked_kernel<HD_><<<grid, 128, 0, st>>>(qp, kp, vp, key_valid, (__nv_bfloat16*)o, S, H, KV, scale_log2, mode)
  if (hd == 8) HB_MASKED(8);
  else if (hd == 16) HB_MASKED(16);
  else if (hd == 32) HB_MASKED(32);
  else if (hd == 64) HB_MASKED(64);
  else {
    set_error("masked attention: head_dim %d not built (8, 16, 32, 64)", hd);
    return HB200_ERR_UNSUPPORTED;
  }
#undef HB_MASKED
  HB_LAUNCH_CHECK();
  return 0;
}
