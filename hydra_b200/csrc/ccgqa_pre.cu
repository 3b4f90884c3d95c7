// Fused CCGQA pre-attention kernel: everything between the qkv projection and the attention core.
//
//   qkv [B,S,lat+2kvd] (read once)  ->  q [B,H,S,hd], k [B,KV,S,hd], v [B,KV,S,hd]  (written once)
//
// Per CTA: one tile of 64 tokens of one sequence (plus an 18-token causal halo re-read from L2).
//   1. the q|k columns of the tile go to shared memory (zero rows before the sequence start);
//   2. conv1 (grouped, k=3, causal) as per-head [rows,3*hd]x[3*hd,hd] mma.sync contractions, result
//      kept in shared memory as bf16;
//   3. conv2 (dense, k=3, causal) as a [64, 3*C]x[3*C, C] contraction; its weight is streamed from
//      L2 through a double-buffered cp.async ring in 64-wide K chunks; fp32 accumulators in registers;
//   4. epilogue, one warp per token: QK-mean coupling, L2 norm (warp-shuffle reductions over the lanes of
//      a head), key temperature, RoPE, head-major bf16x2 stores; value shift straight from global.
//
// Nominally HBM-bound (1536 B/token at lat 256, kvd 64) but the dense conv2 carries ~0.48 MFLOP/token,
// which puts the kernel on the ridge between the HBM and tensor rooflines.
#include "common.cuh"
#include "mma.cuh"

namespace hb200 {

// Tile geometry (template parameters of the kernel): TT tokens per tile, XR = TT + 18 input rows held
// (t0-18 .. t0+TT-1), YR = TT + 16 conv1 rows held (t0-16 .. t0+TT-1), KC = conv2 K chunk, WLD = KC + 8 padded
// weight-chunk row (conflict-free fragment loads).  64/64 is the default; latent 512 uses 32/32 to fit.

struct PreParams {
  const __nv_bfloat16* qkv;
  const __nv_bfloat16* w1;   // [lat+kvd][3*hd]
  const __nv_bfloat16* w2q;  // [lat][3*lat]
  const __nv_bfloat16* w2k;  // [kvd][3*kvd]
  const float* cos_t;
  const float* sin_t;
  const float* temp;
  __nv_bfloat16* q;
  __nv_bfloat16* k;
  __nv_bfloat16* v;
  int B, S, H, KV;
  int disable;               // HB200_ATTN_NO_* bits (generic kernel only; the tiled kernels run the full sequence)
  int ksize;                 // conv kernel size (generic kernel only; the tiled kernels are built for 3)
};

// out[m][n] (fp32 regs) = sum_{j<3} sum_{c<Cin} Y1[m + 14 + j][col_off + c] * W[n][j*Cin + c]
template <int WM, int WN, int MT, int NT, int KC>
__device__ __forceinline__ void conv2_tile(const __nv_bfloat16* __restrict__ Y1, int ldx, int col_off, int Cin,
                                           const __nv_bfloat16* __restrict__ Wg, __nv_bfloat16* wbuf,
                                           float (&acc)[MT][NT][4]) {
  static_assert(WM * WN == 8, "8 warps");
  constexpr int WLD = KC + 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int warp_m = warp / WN, warp_n = warp % WN;
  const int m0 = warp_m * MT * 16;
  const int n0 = warp_n * NT * 8;
  const int N = WN * NT * 8;
  const int K = 3 * Cin;
  const int nchunks = (K + KC - 1) / KC;
#pragma unroll
  for (int a = 0; a < MT; ++a)
#pragma unroll
    for (int b = 0; b < NT; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;

  auto load_chunk = [&](int ch, int buf) {
    __nv_bfloat16* dst = wbuf + buf * N * WLD;
    const int k0 = ch * KC;
    for (int idx = tid; idx < N * (KC / 8); idx += 256) {
      const int n = idx / (KC / 8), piece = idx % (KC / 8);
      if (k0 + piece * 8 < K) cp_async_16(dst + n * WLD + piece * 8, Wg + (size_t)n * K + k0 + piece * 8);
    }
    cp_async_commit();
  };

  load_chunk(0, 0);
  for (int ch = 0; ch < nchunks; ++ch) {
    const int buf = ch & 1;
    if (ch + 1 < nchunks) {
      load_chunk(ch + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* wb = wbuf + buf * N * WLD;
    const int ksteps = min(KC / 16, (K - ch * KC) / 16);
    for (int ks = 0; ks < ksteps; ++ks) {
      const int kk0 = ch * KC + ks * 16;
      const int j = kk0 / Cin, c0 = kk0 - j * Cin;
      uint32_t a[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const __nv_bfloat16* r0 = Y1 + (m0 + mt * 16 + g + 14 + j) * ldx + col_off + c0 + 2 * t;
        const __nv_bfloat16* r1 = r0 + 8 * ldx;
        a[mt][0] = *reinterpret_cast<const uint32_t*>(r0);
        a[mt][1] = *reinterpret_cast<const uint32_t*>(r1);
        a[mt][2] = *reinterpret_cast<const uint32_t*>(r0 + 8);
        a[mt][3] = *reinterpret_cast<const uint32_t*>(r1 + 8);
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const __nv_bfloat16* wr = wb + (n0 + nt * 8 + g) * WLD + ks * 16 + 2 * t;
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(wr);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(wr + 8);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) mma_bf16_16816(acc[mt][nt], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
      }
    }
    __syncthreads();
  }
}

template <int WM, int WN, int MT, int NT>
__device__ __forceinline__ void store_acc(float* out, int ldo, const float (&acc)[MT][NT][4]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int m0 = (warp / WN) * MT * 16, n0 = (warp % WN) * NT * 8;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float* p = out + (m0 + mt * 16 + g) * ldo + n0 + nt * 8 + 2 * t;
      *reinterpret_cast<float2*>(p) = make_float2(acc[mt][nt][0], acc[mt][nt][1]);
      *reinterpret_cast<float2*>(p + 8 * ldo) = make_float2(acc[mt][nt][2], acc[mt][nt][3]);
    }
}

// HD: head dim; NTQ = lat/32; NTK = kvd/16; TT tokens per tile (64 or 32); KC conv2 K chunk
template <int HD, int NTQ, int NTK, int TT, int KC>
__global__ void __launch_bounds__(256, 1) ccgqa_pre_kernel(const PreParams p) {
  constexpr int XR = TT + 18, YR = TT + 16, WLD = KC + 8;
  constexpr int MTQ = TT / 32, MTK = TT / 64;   // m16 tiles per warp in the q (2 m-warps) and k (4 m-warps) conv2
  constexpr int LAT = NTQ * 32, KVD = NTK * 16, C = LAT + KVD;
  constexpr int LDX = C + 8;        // bf16 elements; 16-byte multiple, bank-staggered rows
  constexpr int LDQ = LAT + 4, LDK = KVD + 4;
  constexpr int WROWS = (LAT > KVD ? LAT : KVD);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* X = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [XR][LDX]
  __nv_bfloat16* Y1 = X + XR * LDX;                                          // [YR][LDX]
  __nv_bfloat16* Wb = Y1 + YR * LDX;                                         // [2][WROWS][WLD]
  float* OutK = reinterpret_cast<float*>(Wb + 2 * WROWS * WLD);              // [TT][LDK]
  float* OutQ = reinterpret_cast<float*>(Y1);                                // [TT][LDQ], aliases Y1|Wb after conv2
  static_assert((size_t)TT * LDQ * 4 <= (size_t)(YR * LDX + 2 * WROWS * WLD) * 2, "OutQ alias does not fit");

  const int H = p.H, KV = p.KV, S = p.S;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tiles_per_seq = (S + TT - 1) / TT;
  const int b = blockIdx.x / tiles_per_seq;
  const int t0 = (blockIdx.x % tiles_per_seq) * TT;
  const int QKV_LD = LAT + 2 * KVD;
  const __nv_bfloat16* qkv_b = p.qkv + (size_t)b * S * QKV_LD;

  // ---- 1. q|k columns of the tile -> shared memory ------------------------------------------
  for (int idx = tid; idx < XR * (C / 8); idx += 256) {
    const int r = idx / (C / 8), piece = idx % (C / 8);
    const int tok = t0 - 18 + r;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (tok >= 0 && tok < S) val = *reinterpret_cast<const uint4*>(qkv_b + (size_t)tok * QKV_LD + piece * 8);
    *reinterpret_cast<uint4*>(X + r * LDX + piece * 8) = val;
  }
  __syncthreads();

  // ---- 2. conv1 (grouped): Y1[r][c], r <-> token t0-16+r ------------------------------------
  {
    constexpr int NT1 = HD / 8, KS1 = 3 * HD / 16;
    const int units = (YR / 16) * (H + KV);
    for (int u = warp; u < units; u += 8) {
      const int mt = u % (YR / 16), hg = u / (YR / 16);
      const int cb = hg * HD;
      float acc[NT1][4];
#pragma unroll
      for (int i = 0; i < NT1; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS1; ++ks) {
        const int kk0 = ks * 16;
        const int j = kk0 / HD, c0 = kk0 % HD;
        const __nv_bfloat16* r0 = X + (mt * 16 + g + j) * LDX + cb + c0 + 2 * t;
        const __nv_bfloat16* r1 = r0 + 8 * LDX;
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(r0);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(r1);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(r0 + 8);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(r1 + 8);
#pragma unroll
        for (int nt = 0; nt < NT1; ++nt) {
          const __nv_bfloat16* wr = p.w1 + (size_t)(cb + nt * 8 + g) * (3 * HD) + kk0 + 2 * t;
          const uint32_t b0 = __ldg(reinterpret_cast<const unsigned int*>(wr));
          const uint32_t b1 = __ldg(reinterpret_cast<const unsigned int*>(wr + 8));
          mma_bf16_16816(acc[nt], a0, a1, a2, a3, b0, b1);
        }
      }
#pragma unroll
      for (int nt = 0; nt < NT1; ++nt) {
        __nv_bfloat16* y = Y1 + (mt * 16 + g) * LDX + cb + nt * 8 + 2 * t;
        *reinterpret_cast<uint32_t*>(y) = pack_bf16x2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<uint32_t*>(y + 8 * LDX) = pack_bf16x2(acc[nt][2], acc[nt][3]);
      }
    }
  }
  __syncthreads();

  // ---- 3. conv2 (dense): K first (small), then Q ---------------------------------------------
  {
    if constexpr (MTK >= 1) {
      float acck[MTK][NTK][4];
      conv2_tile<4, 2, MTK, NTK, KC>(Y1, LDX, LAT, KVD, p.w2k, Wb, acck);
      store_acc<4, 2, MTK, NTK>(OutK, LDK, acck);
    } else {   // 32-token tile: two m-warps of 16 rows, four n-warps
      static_assert(TT == 32 && NTK % 2 == 0, "32-token tiles need kv_dim divisible by 32");
      float acck[1][NTK / 2][4];
      conv2_tile<2, 4, 1, NTK / 2, KC>(Y1, LDX, LAT, KVD, p.w2k, Wb, acck);
      store_acc<2, 4, 1, NTK / 2>(OutK, LDK, acck);
    }
  }
  {
    float accq[MTQ][NTQ][4];
    conv2_tile<2, 4, MTQ, NTQ, KC>(Y1, LDX, 0, LAT, p.w2q, Wb, accq);   // ends with __syncthreads(): Y1/Wb are dead
    store_acc<2, 4, MTQ, NTQ>(OutQ, LDQ, accq);
  }
  __syncthreads();

  // ---- 4. epilogue: one warp per token ---------------------------------------------------------
  constexpr int PH = HD / 2;              // lanes per head (one rotary pair each)
  constexpr int HPI = (32 / PH) > 0 ? (32 / PH) : 1;   // heads per warp iteration
  static_assert(PH <= 32, "head_dim up to 64");
  const int i = lane % PH, hsub = lane / PH;
  const float temp = *p.temp;
  const bool mha = (H == KV);
  for (int tt = warp; tt < TT; tt += 8) {
    const int tok = t0 + tt;
    if (tok >= S) break;   // warp-uniform
    const __nv_bfloat16* xr = X + (tt + 18) * LDX;
    float qm0 = 0.f, qm1 = 0.f, km0 = 0.f, km1 = 0.f;
    if (!mha) {
      for (int h = 0; h < H; ++h) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + h * HD + 2 * i));
        qm0 += f.x;
        qm1 += f.y;
      }
      for (int h = 0; h < KV; ++h) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + LAT + h * HD + 2 * i));
        km0 += f.x;
        km1 += f.y;
      }
      qm0 *= 0.5f / (float)H;  qm1 *= 0.5f / (float)H;
      km0 *= 0.5f / (float)KV; km1 *= 0.5f / (float)KV;
    }
    const float cs = p.cos_t[(size_t)tok * PH + i], sn = p.sin_t[(size_t)tok * PH + i];
    // queries
    for (int hb = 0; hb < H; hb += HPI) {
      const int h = min(hb + hsub, H - 1);
      const bool valid = (hb + hsub) < H;
      float2 vq = *reinterpret_cast<const float2*>(OutQ + tt * LDQ + h * HD + 2 * i);
      if (mha) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + h * HD + 2 * i));
        const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + LAT + h * HD + 2 * i));
        vq.x += 0.5f * (a.x + c.x);
        vq.y += 0.5f * (a.y + c.y);
      } else {
        vq.x += km0;
        vq.y += km1;
      }
      float ss = vq.x * vq.x + vq.y * vq.y;
#pragma unroll
      for (int o = PH >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float inv = 1.0f / fmaxf(sqrtf(ss), 1e-12f);
      const float x0 = vq.x * inv, x1 = vq.y * inv;
      if (valid)
        *reinterpret_cast<uint32_t*>(p.q + (((size_t)b * H + h) * S + tok) * HD + 2 * i) =
            pack_bf16x2(x0 * cs - x1 * sn, x0 * sn + x1 * cs);
    }
    // keys
    for (int hb = 0; hb < KV; hb += HPI) {
      const int h = min(hb + hsub, KV - 1);
      const bool valid = (hb + hsub) < KV;
      float2 vk = *reinterpret_cast<const float2*>(OutK + tt * LDK + h * HD + 2 * i);
      if (mha) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + h * HD + 2 * i));
        const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + LAT + h * HD + 2 * i));
        vk.x += 0.5f * (a.x + c.x);
        vk.y += 0.5f * (a.y + c.y);
      } else {
        vk.x += qm0;
        vk.y += qm1;
      }
      float ss = vk.x * vk.x + vk.y * vk.y;
#pragma unroll
      for (int o = PH >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float inv = temp / fmaxf(sqrtf(ss), 1e-12f);
      const float x0 = vk.x * inv, x1 = vk.y * inv;
      if (valid)
        *reinterpret_cast<uint32_t*>(p.k + (((size_t)b * KV + h) * S + tok) * HD + 2 * i) =
            pack_bf16x2(x0 * cs - x1 * sn, x0 * sn + x1 * cs);
    }
    // values: first half of the channels from this token, second half from the previous one
    for (int cp = lane; cp < KVD / 2; cp += 32) {
      const int c = 2 * cp;
      const int src_tok = (c < KVD / 2) ? tok : tok - 1;
      uint32_t val = 0;
      if (src_tok >= 0)
        val = *reinterpret_cast<const uint32_t*>(qkv_b + (size_t)src_tok * QKV_LD + LAT + KVD + c);
      *reinterpret_cast<uint32_t*>(p.v + (((size_t)b * KV + c / HD) * S + tok) * HD + (c % HD)) = val;
    }
  }
}

template <int HD, int NTQ, int NTK, int TT = 64, int KC = 64>
static int launch_pre(const PreParams& p, cudaStream_t st) {
  constexpr int XR = TT + 18, YR = TT + 16, WLD = KC + 8;
  constexpr int LAT = NTQ * 32, KVD = NTK * 16, C = LAT + KVD, LDX = C + 8;
  constexpr int WROWS = (LAT > KVD ? LAT : KVD);
  constexpr size_t smem = (size_t)(XR + YR) * LDX * 2 + (size_t)2 * WROWS * WLD * 2 + (size_t)TT * (KVD + 4) * 4;
  static_assert(smem <= 227 * 1024, "tile does not fit in shared memory");
  auto kern = ccgqa_pre_kernel<HD, NTQ, NTK, TT, KC>;
  HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, (size_t)((int)smem)));
  const int tiles = p.B * ((p.S + TT - 1) / TT);
  kern<<<tiles, 256, smem, st>>>(p);
  HB_LAUNCH_CHECK();
  return 0;
}

// ---- any other shape: CUDA-core kernel ---------------------------------------------------------------------------
// Head counts the tiled kernels above are not instantiated for (H and KV are run-time values here; head_dim 16, 32 or
// 64).  Same arithmetic: the grouped conv's result is rounded to bf16 before the dense conv (as the tensor-core
// kernels round their operand), everything after it stays in fp32 until the final store.  One CTA = TT tokens of one
// sequence; thread = output channel in both convs (its weight row is read once and used for all TT tokens, the
// activations come from shared memory as broadcasts).  Built for coverage, not speed.
constexpr int PRE_GENERIC_MAX_K = 8;       // largest conv kernel size of the generic kernel (register rows per thread)
template <int HD, int TT>
__global__ void __launch_bounds__(256) ccgqa_pre_generic_kernel(const PreParams p) {
  extern __shared__ __align__(16) float gsm[];
  const int H = p.H, KV = p.KV, S = p.S;
  const int LAT = H * HD, KVD = KV * HD, C = LAT + KVD, QKV_LD = LAT + 2 * KVD;
  const int K = p.ksize, PAD = K - 1;     // causal convs of kernel size K look PAD tokens back (K = 3: the model's)
  float* xs = gsm;                        // [TT + 2 PAD][C]  q|k columns of tokens t0-2 PAD .. t0+TT-1 (0 before the sequence)
  float* y1 = xs + (TT + 2 * PAD) * C;    // [TT + PAD][C]    grouped-conv output of tokens t0-PAD .. (0 before the sequence)
  float* y2 = y1 + (TT + PAD) * C;        // [TT][C]          dense-conv output of tokens t0 ..
  float* mean = y2 + TT * C;              // [TT][2][HD]  0.5 * mean over heads of q0 / of k0 (H != KV only)
  const int tid = threadIdx.x;
  const int tiles_per_seq = (S + TT - 1) / TT;
  const int b = blockIdx.x / tiles_per_seq;
  const int t0 = (blockIdx.x % tiles_per_seq) * TT;
  const __nv_bfloat16* qkv_b = p.qkv + (size_t)b * S * QKV_LD;

  for (int idx = tid; idx < (TT + 2 * PAD) * C; idx += 256) {
    const int r = idx / C, c = idx - r * C, tok = t0 - 2 * PAD + r;
    xs[idx] = (tok >= 0 && tok < S) ? __bfloat162float(qkv_b[(size_t)tok * QKV_LD + c]) : 0.f;
  }
  __syncthreads();
  const bool convs = !(p.disable & HB200_ATTN_NO_CONVS), couple_on = !(p.disable & HB200_ATTN_NO_QK_MEAN);
  const bool norm_on = !(p.disable & HB200_ATTN_NO_QK_NORM), rope_on = !(p.disable & HB200_ATTN_NO_ROPE);
  const bool shift_on = !(p.disable & HB200_ATTN_NO_VALUE_SHIFT);

  // grouped conv: y1[t][c] = sum_j sum_i w1[c][j*HD + i] * x[t-2+j][head(c)*HD + i]
  for (int c = tid; convs && c < C; c += 256) {
    float acc[TT + PRE_GENERIC_MAX_K - 1];
#pragma unroll
    for (int r = 0; r < TT + PRE_GENERIC_MAX_K - 1; ++r) acc[r] = 0.f;
    const __nv_bfloat16* w = p.w1 + (size_t)c * K * HD;
    const int c0 = (c / HD) * HD;
    for (int j = 0; j < K; ++j)
      for (int i = 0; i < HD; ++i) {
        const float wv = __bfloat162float(w[j * HD + i]);
#pragma unroll
        for (int r = 0; r < TT + PRE_GENERIC_MAX_K - 1; ++r)
          if (r < TT + PAD) acc[r] += wv * xs[(r + j) * C + c0 + i];
      }
#pragma unroll
    for (int r = 0; r < TT + PRE_GENERIC_MAX_K - 1; ++r)
      if (r < TT + PAD)
        y1[r * C + c] = (t0 - PAD + r >= 0) ? __bfloat162float(__float2bfloat16(acc[r])) : 0.f;   // conv2 pads with zeros
  }
  __syncthreads();

  // dense conv: y2[t][c] = sum_j sum_ci w2[c][j*Cin + ci] * y1[t-2+j][off + ci]
  for (int c = tid; convs && c < C; c += 256) {
    float acc[TT];
#pragma unroll
    for (int r = 0; r < TT; ++r) acc[r] = 0.f;
    const bool is_q = c < LAT;
    const int cin = is_q ? LAT : KVD, off = is_q ? 0 : LAT;
    const __nv_bfloat16* w = is_q ? p.w2q + (size_t)c * K * LAT : p.w2k + (size_t)(c - LAT) * K * KVD;
    for (int j = 0; j < K; ++j)
      for (int ci = 0; ci < cin; ++ci) {
        const float wv = __bfloat162float(w[j * cin + ci]);
#pragma unroll
        for (int r = 0; r < TT; ++r) acc[r] += wv * y1[(r + j) * C + off + ci];
      }
#pragma unroll
    for (int r = 0; r < TT; ++r) y2[r * C + c] = acc[r];
  }
  if (!convs)                               // no convolutions: q and k go on as projected
    for (int idx = tid; idx < TT * C; idx += 256) y2[idx] = xs[2 * PAD * C + idx];
  // QK-mean vectors from the un-convolved q0 / k0 of each token
  if (H != KV && couple_on) {
    for (int idx = tid; idx < TT * 2 * HD; idx += 256) {
      const int r = idx / (2 * HD), which = (idx / HD) & 1, d = idx % HD;
      const float* row = xs + (r + 2 * PAD) * C;
      float sum = 0.f;
      if (which == 0) { for (int h = 0; h < H; ++h) sum += row[h * HD + d]; sum *= 0.5f / (float)H; }
      else            { for (int h = 0; h < KV; ++h) sum += row[LAT + h * HD + d]; sum *= 0.5f / (float)KV; }
      mean[idx] = sum;
    }
  }
  __syncthreads();

  // finish: coupling, L2 norm, temperature, RoPE; one thread per (token, head)
  const float temp = norm_on ? *p.temp : 1.0f;
  for (int idx = tid; idx < TT * (H + KV); idx += 256) {
    const int r = idx / (H + KV), hh = idx - r * (H + KV), tok = t0 + r;
    if (tok >= S) continue;
    const bool is_q = hh < H;
    const int h = is_q ? hh : hh - H;
    const int c0 = is_q ? h * HD : LAT + h * HD;
    const float* x0 = xs + (r + 2 * PAD) * C;
    float v[HD];
    float ss = 0.f;
#pragma unroll
    for (int d = 0; d < HD; ++d) {
      float couple = 0.f;
      if (!couple_on) {}
      else if (H == KV) couple = 0.5f * (x0[h * HD + d] + x0[LAT + h * HD + d]);   // m = 0.5 (q0 + k0), channel by channel
      else couple = is_q ? mean[(r * 2 + 1) * HD + d] : mean[(r * 2 + 0) * HD + d];
      v[d] = y2[r * C + c0 + d] + couple;
      ss += v[d] * v[d];
    }
    const float inv = norm_on ? (is_q ? 1.0f : temp) / fmaxf(sqrtf(ss), 1e-12f) : 1.0f;
    __nv_bfloat16* dst = is_q ? p.q + (((size_t)b * H + h) * S + tok) * HD : p.k + (((size_t)b * KV + h) * S + tok) * HD;
    const float* cs = p.cos_t + (size_t)tok * (HD / 2);
    const float* sn = p.sin_t + (size_t)tok * (HD / 2);
#pragma unroll
    for (int i = 0; i < HD / 2; ++i) {
      const float a0 = v[2 * i] * inv, a1 = v[2 * i + 1] * inv;
      const float c_ = rope_on ? cs[i] : 1.0f, s_ = rope_on ? sn[i] : 0.0f;
      dst[2 * i] = __float2bfloat16(a0 * c_ - a1 * s_);
      dst[2 * i + 1] = __float2bfloat16(a0 * s_ + a1 * c_);
    }
  }
  // value shift: first half of the channels from this token, second half from the previous one
  for (int idx = tid; idx < TT * KVD; idx += 256) {
    const int r = idx / KVD, c = idx - r * KVD, tok = t0 + r;
    if (tok >= S) continue;
    const int src = (c < KVD / 2 || !shift_on) ? tok : tok - 1;
    p.v[(((size_t)b * KV + c / HD) * S + tok) * HD + (c % HD)] =
        src >= 0 ? qkv_b[(size_t)src * QKV_LD + LAT + KVD + c] : __float2bfloat16(0.f);
  }
}

template <int HD>
static int launch_pre_generic(const PreParams& p, cudaStream_t st) {
  const size_t C = (size_t)(p.H + p.KV) * HD;
  const int pad = p.ksize - 1;
  auto bytes = [&](int tt) { return ((size_t)(3 * tt + 3 * pad) * C + (size_t)tt * 2 * HD) * sizeof(float); };
  if (bytes(16) <= 200 * 1024) {
    auto kern = ccgqa_pre_generic_kernel<HD, 16>;
    HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, bytes(16)));
    kern<<<p.B * ((p.S + 15) / 16), 256, bytes(16), st>>>(p);
  } else {
    HB_REQUIRE(bytes(4) <= 227 * 1024, HB200_ERR_UNSUPPORTED,
               "ccgqa_pre_attention: latent + kv width %d does not fit the generic kernel", (int)C);
    auto kern = ccgqa_pre_generic_kernel<HD, 4>;
    HB_PROPAGATE(ensure_dynamic_smem((const void*)kern, bytes(4)));
    kern<<<p.B * ((p.S + 3) / 4), 256, bytes(4), st>>>(p);
  }
  HB_LAUNCH_CHECK();
  return 0;
}

int launch_ccgqa_pre_tc(const void* qkv, const void* w1_qk, const void* w2_q, const void* w2_k, const float* cos_t,
                        const float* sin_t, const float* key_temperature, void* q, void* k, void* v, int B, int S, int H,
                        int KV, int hd, int32_t* err_flag, cudaStream_t st);

}  // namespace hb200

using namespace hb200;

static int pre_attention(const void* qkv, const void* w1_qk, const void* w2_q, const void* w2_k, const float* cos_t,
                         const float* sin_t, const float* key_temperature, void* q, void* k, void* v, int B, int S, int H,
                         int KV, int hd, int disable, int conv_ksize, int32_t* err_flag, void* stream) {
  HB_REQUIRE(qkv && q && k && v, HB200_ERR_INVALID, "ccgqa_pre_attention: null pointer");
  HB_REQUIRE(conv_ksize >= 1 && conv_ksize <= PRE_GENERIC_MAX_K, HB200_ERR_UNSUPPORTED,
             "ccgqa_pre_attention: conv kernel size %d not built (1 .. %d)", conv_ksize, PRE_GENERIC_MAX_K);
  HB_REQUIRE((disable & ~HB200_ATTN_NO_ALL) == 0, HB200_ERR_INVALID, "ccgqa_pre_attention: unknown switch bits %d", disable);
  HB_REQUIRE((disable & HB200_ATTN_NO_CONVS) || (w1_qk && w2_q && w2_k), HB200_ERR_INVALID,
             "ccgqa_pre_attention: null conv weights");
  HB_REQUIRE((disable & HB200_ATTN_NO_ROPE) || (cos_t && sin_t), HB200_ERR_INVALID, "ccgqa_pre_attention: null RoPE tables");
  HB_REQUIRE((disable & HB200_ATTN_NO_QK_NORM) || key_temperature, HB200_ERR_INVALID,
             "ccgqa_pre_attention: null key temperature");
  HB_REQUIRE(B >= 0 && S >= 0 && H >= 1 && KV >= 1 && H % KV == 0, HB200_ERR_INVALID,
             "ccgqa_pre_attention: bad shape B=%d S=%d H=%d KV=%d", B, S, H, KV);
  HB_REQUIRE(aligned16(qkv) && aligned16(w2_q) && aligned16(w2_k) && aligned16(q) && aligned16(k) && aligned16(v),
             HB200_ERR_INVALID, "ccgqa_pre_attention: pointers must be 16-byte aligned");
  HB_REQUIRE(hd % 2 == 0, HB200_ERR_INVALID, "ccgqa_pre_attention: head_dim must be even");
  if ((int64_t)B * S == 0) return 0;
  const int lat = H * hd, kvd = KV * hd;
  PreParams p{(const __nv_bfloat16*)qkv, (const __nv_bfloat16*)w1_qk, (const __nv_bfloat16*)w2_q,
              (const __nv_bfloat16*)w2_k, cos_t, sin_t, key_temperature, (__nv_bfloat16*)q, (__nv_bfloat16*)k,
              (__nv_bfloat16*)v, B, S, H, KV, disable, conv_ksize};
  cudaStream_t st = (cudaStream_t)stream;
  if (conv_ksize != 3) disable |= 1 << 30;     // any other kernel size: CUDA-core kernel (bit 30 only steers the dispatch below)
  if (disable == 0) {
    // tcgen05 kernel for the 250M-class shapes; HB200_ERR_UNSUPPORTED means "not this shape", anything else is final
    const int rc = launch_ccgqa_pre_tc(qkv, w1_qk, w2_q, w2_k, cos_t, sin_t, key_temperature, q, k, v, B, S, H, KV, hd,
                                       err_flag, st);
    if (rc != HB200_ERR_UNSUPPORTED) return rc;
  }
#define HB_PRE_CASE(HD_, NTQ_, NTK_) \
  if (disable == 0 && hd == HD_ && lat == NTQ_ * 32 && kvd == NTK_ * 16) return launch_pre<HD_, NTQ_, NTK_>(p, st);
  HB_PRE_CASE(32, 8, 4)    // dim 1024: 8q/2kv heads of 32
  HB_PRE_CASE(16, 8, 4)    // dim 1024: 16q/4kv heads of 16
  HB_PRE_CASE(16, 4, 2)    // dim 512: 8q/2kv heads of 16
  HB_PRE_CASE(16, 6, 3)    // dim 768: 12q/3kv heads of 16
  HB_PRE_CASE(32, 4, 4)    // dim 512: 4q/2kv heads of 32
  HB_PRE_CASE(16, 2, 2)    // dim 256: 4q/2kv heads of 16
  HB_PRE_CASE(32, 2, 2)    // dim 256: 2q/1kv heads of 32
  HB_PRE_CASE(16, 2, 4)    // dim 256: 4q/4kv heads of 16 (H == KV)
  HB_PRE_CASE(64, 4, 8)    // dim 512: 2q/2kv heads of 64
  HB_PRE_CASE(16, 3, 2)    // dim 384: 6q/2kv heads of 16
  HB_PRE_CASE(16, 9, 3)    // dim 1152: 18q/3kv heads of 16 (the reference's 300M preset)
#undef HB_PRE_CASE
  // latent 512 (dim 2048, 32q/4kv heads of 16: the 1.5B shape): 32-token tiles and 32-wide weight chunks to fit
  if (disable == 0 && hd == 16 && lat == 512 && kvd == 64) return launch_pre<16, 16, 4, 32, 32>(p, st);
  // the reference's other presets, same tile shape: dim 1792 (28q/4kv: 500M, 1B), dim 1536 (24q/4kv: 750M) and the
  // trainer's default dim 1280 (20q/5kv)
  if (disable == 0 && hd == 16 && lat == 448 && kvd == 64) return launch_pre<16, 14, 4, 32, 32>(p, st);
  if (disable == 0 && hd == 16 && lat == 384 && kvd == 64) return launch_pre<16, 12, 4, 32, 32>(p, st);
  if (disable == 0 && hd == 16 && lat == 320 && kvd == 80) return launch_pre<16, 10, 5, 64, 32>(p, st);
  // everything else with a head_dim the attention kernels are built for
  if (hd == 8) return launch_pre_generic<8>(p, st);
  if (hd == 16) return launch_pre_generic<16>(p, st);
  if (hd == 32) return launch_pre_generic<32>(p, st);
  if (hd == 64) return launch_pre_generic<64>(p, st);
  set_error("ccgqa_pre_attention: head_dim %d not built (8, 16, 32, 64)", hd);
  return HB200_ERR_UNSUPPORTED;
}

extern "C" int hb200_ccgqa_pre_attention(const void* qkv, const void* w1_qk, const void* w2_q, const void* w2_k,
                                         const float* cos_t, const float* sin_t, const float* key_temperature, void* q,
                                         void* k, void* v, int B, int S, int H, int KV, int hd, int32_t* err_flag,
                                         void* stream) {
  return pre_attention(qkv, w1_qk, w2_q, w2_k, cos_t, sin_t, key_temperature, q, k, v, B, S, H, KV, hd, 0, 3, err_flag,
                       stream);
}

extern "C" int hb200_ccgqa_pre_attention_ablated(const void* qkv, const void* w1_qk, const void* w2_q, const void* w2_k,
                                                 const float* cos_t, const float* sin_t, const float* key_temperature,
                                                 void* q, void* k, void* v, int B, int S, int H, int KV, int hd,
                                                 int disable, int conv_ksize, int32_t* err_flag, void* stream) {
  return pre_attention(qkv, w1_qk, w2_q, w2_k, cos_t, sin_t, key_temperature, q, k, v, B, S, H, KV, hd, disable,
                       conv_ksize, err_flag, stream);
}
