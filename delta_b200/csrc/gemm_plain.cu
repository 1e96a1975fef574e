// Plain matrix product  C[M,N] = A[M,K] * W[N,K]^T  on the FMA units, float
// accumulation, no reduced-precision matrix mode and no split over K: the sum of
// one output element runs over k in the same order whatever M is, so a token's
// result does not depend on what shares its batch.  This is the product of the
// 32-bit path and the plain twin of the tensor-core products.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) gemm_nt_kernel(const TI* __restrict__ A, const TI* __restrict__ W, TO* __restrict__ C,
                                                      int M, int N, int K, int lda, int ldw, int ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < (BM * BK) / 256; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int r = idx / BK, c = idx % BK;
      const int m = m0 + r, k = k0 + c;
      As[c][r] = (m < M && k < K) ? to_f32<TI>(A[(size_t)m * lda + k]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < (BN * BK) / 256; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int r = idx / BK, c = idx % BK;
      const int n = n0 + r, k = k0 + c;
      Ws[c][r] = (n < N && k < K) ? to_f32<TI>(W[(size_t)n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[(size_t)m * ldc + n] = from_f32<TO>(acc[i][j]);
    }
  }
}
}  // namespace

// in_dtype: type of A and W; out_dtype: type of C (float output from bfloat16
// operands is how logits are made).
extern "C" int dk_gemm_nt_plain(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
                                int in_dtype, int out_dtype, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  DK_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
  DK_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm: leading sizes %d %d %d too small", lda, ldw, ldc);
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  DK_REQUIRE(grid.y <= 65535, "gemm: M=%d is too large for this kernel", M);
#define LAUNCH(TI, TO) \
  gemm_nt_kernel<TI, TO><<<grid, 256, 0, stream>>>((const TI*)A, (const TI*)W, (TO*)C, M, N, K, lda, ldw, ldc)
  if (in_dtype == DK_F32 && out_dtype == DK_F32) LAUNCH(float, float);
  else if (in_dtype == DK_BF16 && out_dtype == DK_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == DK_BF16 && out_dtype == DK_F32) LAUNCH(__nv_bfloat16, float);
  else DK_REQUIRE(false, "gemm: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
#undef LAUNCH
  return dk_check_launch("gemm_nt_plain");
}
