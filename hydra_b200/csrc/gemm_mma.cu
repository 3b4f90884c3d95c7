// Plain mma.sync GEMM (C = epilogue(A W^T), bf16 in, fp32 accumulate).  It is NOT the product path: it exists
// as an independent implementation of the same contraction + epilogues so that the tcgen05 kernel can be
// cross-checked on the device, tile by tile, in the test-suite.
#include "gemm_epilogue.cuh"
#include "mma.cuh"

namespace hb200 {

constexpr int LBM = 64, LBN = 128, LBK = 32, LLD = LBK + 8, LCLD = LBN + 4;

__global__ void __launch_bounds__(256) gemm_mma_kernel(const GemmParams p) {
  __shared__ __align__(16) unsigned char raw[LBM * LCLD * 4];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(raw);   // [LBM][LLD]
  __nv_bfloat16* Bs = As + LBM * LLD;                            // [LBN][LLD]
  float* Cs = reinterpret_cast<float*>(raw);                     // [LBM][LCLD], aliases As/Bs after the mainloop
  static_assert((LBM + LBN) * LLD * 2 <= LBM * LCLD * 4, "stage alias");

  const int M = p.m_dev ? min(*p.m_dev, p.M) : p.M;
  const int m0 = blockIdx.y * LBM, n0 = blockIdx.x * LBN;
  if (m0 >= M) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int wm = (warp >> 2) * 32, wn = (warp & 3) * 32;
  float acc[2][4][4] = {};

  for (int k0 = 0; k0 < p.K; k0 += LBK) {
    {  // A: 64 rows x 4 pieces
      const int r = tid >> 2, pc = tid & 3;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (m0 + r < M && k0 + pc * 8 < p.K)
        val = *reinterpret_cast<const uint4*>(p.A + (size_t)(m0 + r) * p.lda + k0 + pc * 8);
      *reinterpret_cast<uint4*>(As + r * LLD + pc * 8) = val;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {  // W: 128 rows x 4 pieces
      const int idx = tid + i * 256;
      const int r = idx >> 2, pc = idx & 3;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (n0 + r < p.N && k0 + pc * 8 < p.K)
        val = *reinterpret_cast<const uint4*>(p.W + (size_t)(n0 + r) * p.ldw + k0 + pc * 8);
      *reinterpret_cast<uint4*>(Bs + r * LLD + pc * 8) = val;
    }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < LBK / 16; ++ks) {
      uint32_t a[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const __nv_bfloat16* r0 = As + (wm + mt * 16 + g) * LLD + ks * 16 + 2 * t;
        a[mt][0] = *reinterpret_cast<const uint32_t*>(r0);
        a[mt][1] = *reinterpret_cast<const uint32_t*>(r0 + 8 * LLD);
        a[mt][2] = *reinterpret_cast<const uint32_t*>(r0 + 8);
        a[mt][3] = *reinterpret_cast<const uint32_t*>(r0 + 8 * LLD + 8);
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const __nv_bfloat16* wr = Bs + (wn + nt * 8 + g) * LLD + ks * 16 + 2 * t;
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(wr);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(wr + 8);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) mma_bf16_16816(acc[mt][nt], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float* c = Cs + (wm + mt * 16 + g) * LCLD + wn + nt * 8 + 2 * t;
      *reinterpret_cast<float2*>(c) = make_float2(acc[mt][nt][0], acc[mt][nt][1]);
      *reinterpret_cast<float2*>(c + 8 * LCLD) = make_float2(acc[mt][nt][2], acc[mt][nt][3]);
    }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int unit = tid + i * 256;
    const int r = unit >> 3, ch = unit & 7;
    const int m = m0 + r, col = n0 + ch * 16;
    if (m < M && col < p.N) {
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        const float4 f = *reinterpret_cast<const float4*>(Cs + r * LCLD + ch * 16 + j);
        v[j] = f.x; v[j + 1] = f.y; v[j + 2] = f.z; v[j + 3] = f.w;
      }
      epilogue_row_chunk<16>(p, m, col, v);
    }
  }
}

int launch_gemm_mma(const GemmParams& p, cudaStream_t st) {
  dim3 grid(ceil_div(p.N, LBN), ceil_div(p.M, LBM));
  HB_REQUIRE(grid.y <= 65535, HB200_ERR_UNSUPPORTED, "gemm(mma): M too large for this cross-check kernel");
  gemm_mma_kernel<<<grid, 256, 0, st>>>(p);
  HB_LAUNCH_CHECK();
  return 0;
}

}  // namespace hb200
