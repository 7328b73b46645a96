// CUDA-core GEMM engine with the fused bias/activation epilogue.
//
// Serves what the tcgen05 engine does not take: fp32 operands (the reference's
// 1e-6 operator fixtures need true fp32 products, not tf32), transposed A,
// leading dimensions that break TMA's 16-byte rule, and tiny shapes.
// 64x64 output tile, 16-deep k slices staged in shared memory, 4x4 outputs per
// thread, fp32 accumulation with k ascending.
#include "xb_common.cuh"

namespace xb {

struct SimtGemmParams {
  int M, N, K, trans_a, trans_b;
  float alpha, beta;
  const void* A; int64_t lda, stride_a;
  const void* B; int64_t ldb, stride_b;
  const void* bias; int64_t ldbias, stride_bias, bias_group; int bias_kind, bias_dtype;
  void* Y; int64_t ldy, stride_y;
  EpiParams epi; int64_t stride_ep;
};

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const __grid_constant__ SimtGemmParams p) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 1];
  __shared__ float Bs[BK][BN + 1];
  const int b = blockIdx.z;
  const TIn* __restrict__ A = reinterpret_cast<const TIn*>(p.A) + (int64_t)b * p.stride_a;
  const TIn* __restrict__ B = reinterpret_cast<const TIn*>(p.B) + (int64_t)b * p.stride_b;
  TOut* __restrict__ Y = reinterpret_cast<TOut*>(p.Y) + (int64_t)b * p.stride_y;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < p.K; k0 += BK) {
    // A tile: BM x BK
    for (int idx = threadIdx.x; idx < BM * BK; idx += 256) {
      int m, k;
      if (p.trans_a) { m = idx % BM; k = idx / BM; } else { k = idx % BK; m = idx / BK; }
      const int gm = m0 + m, gk = k0 + k;
      float v = 0.f;
      if (gm < p.M && gk < p.K)
        v = to_f32<TIn>(p.trans_a ? A[(int64_t)gk * p.lda + gm] : A[(int64_t)gm * p.lda + gk]);
      As[k][m] = v;
    }
    for (int idx = threadIdx.x; idx < BN * BK; idx += 256) {
      int n, k;
      if (p.trans_b) { k = idx % BK; n = idx / BK; } else { n = idx % BN; k = idx / BN; }
      const int gn = n0 + n, gk = k0 + k;
      float v = 0.f;
      if (gn < p.N && gk < p.K)
        v = to_f32<TIn>(p.trans_b ? B[(int64_t)gn * p.ldb + gk] : B[(int64_t)gk * p.ldb + gn]);
      Bs[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], bb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bb[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
    __syncthreads();
  }

  EpiParams epi = p.epi;
  if (epi.a) epi.a += (int64_t)b * p.stride_ep;
  if (epi.b) epi.b += (int64_t)b * p.stride_ep;
  if (epi.c) epi.c += (int64_t)b * p.stride_ep;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= p.N) continue;
      float v = p.alpha * acc[i][j];
      if (p.bias_kind == XB_BIAS_ROW)
        v += p.beta * load_as_f32(p.bias, (int64_t)b * p.stride_bias + gn, p.bias_dtype);
      else if (p.bias_kind == XB_BIAS_FULL)
        v += p.beta * load_as_f32(p.bias, (int64_t)b * p.stride_bias + (int64_t)(gm / p.bias_group) * p.ldbias + gn, p.bias_dtype);
      v = apply_epilogue(epi, v, gn);
      Y[(int64_t)gm * p.ldy + gn] = from_f32<TOut>(v);
    }
  }
}

template <typename TIn>
static int launch_simt_out(const SimtGemmParams& p, int y_dtype, dim3 grid, cudaStream_t s) {
  switch (y_dtype) {
    case XB_F32: gemm_simt_kernel<TIn, float><<<grid, 256, 0, s>>>(p); break;
    case XB_F16: gemm_simt_kernel<TIn, __half><<<grid, 256, 0, s>>>(p); break;
    case XB_BF16: gemm_simt_kernel<TIn, __nv_bfloat16><<<grid, 256, 0, s>>>(p); break;
    default: return fail(XB_ERR_UNSUPPORTED, "xb_gemm: output dtype %d", y_dtype);
  }
  return check_launch("gemm_simt_kernel");
}

int gemm_simt(const xb_gemm_args& a, cudaStream_t stream) {
  SimtGemmParams p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.trans_a = a.trans_a; p.trans_b = a.trans_b;
  p.alpha = a.alpha; p.beta = a.beta;
  p.A = a.A; p.lda = a.lda; p.stride_a = a.stride_a;
  p.B = a.B; p.ldb = a.ldb; p.stride_b = a.stride_b;
  p.bias = a.bias; p.ldbias = a.ldbias; p.stride_bias = a.stride_bias;
  p.bias_group = a.bias_row_group > 1 ? a.bias_row_group : 1;
  p.bias_kind = a.bias ? a.bias_kind : XB_BIAS_NONE; p.bias_dtype = a.bias_dtype;
  p.Y = a.Y; p.ldy = a.ldy; p.stride_y = a.stride_y;
  p.epi.kind = a.epilogue; p.epi.a = a.ep_a; p.epi.b = a.ep_b; p.epi.c = a.ep_c;
  p.epi.count = a.ep_count; p.epi.nosqrt = a.dice_nosqrt; p.stride_ep = a.stride_ep;
  dim3 grid((a.N + 63) / 64, (a.M + 63) / 64, a.batch);
  XB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, XB_ERR_LIMIT, "xb_gemm: M or batch too large for the SIMT engine");
  switch (a.ab_dtype) {
    case XB_F32: return launch_simt_out<float>(p, a.y_dtype, grid, stream);
    case XB_F16: return launch_simt_out<__half>(p, a.y_dtype, grid, stream);
    case XB_BF16: return launch_simt_out<__nv_bfloat16>(p, a.y_dtype, grid, stream);
    default: return fail(XB_ERR_UNSUPPORTED, "xb_gemm: operand dtype %d", a.ab_dtype);
  }
}

}  // namespace xb
