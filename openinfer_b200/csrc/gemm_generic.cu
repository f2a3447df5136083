// C[M,N] = A[M,K] * W[N,K]^T with float32 accumulation on the ordinary (non-tensor) pipes.
//
// The product of the true 32-bit path (no reduced-precision matrix mode), and the fallback
// for operand types the tensor-core kernels do not take. Every output element is summed over k
// in ascending order by one thread, so a row's result does not depend on M or on the other rows.
// The sum is formed in two levels: 256 consecutive products are added up in a register of their
// own, and that partial sum is then added to the total. The rounding error of a float32 sum grows
// with the size of the running total; with partial sums that start at zero every 256 terms it
// grows like sqrt(256) + sqrt(K / 256) instead of sqrt(K) (at K = 12,288: 23 against 111), which
// keeps a model of real width inside the tolerance that the tiny ones meet.
// Same contract as the reference's library call: row-major weight [out, in], no bias,
// float32 accumulate (pegainfer-kernels/csrc/shared/linear.cu:312-362).
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
constexpr int TILES_PER_PARTIAL = 16;   // 16 tiles of BK = 256 terms per partial sum

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_generic_kernel(TC* __restrict__ C, const TA* __restrict__ A, const TW* __restrict__ W, int M, int N,
                    int K, long long lda, long long ldw, long long ldc) {
  pdl_start();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN], part[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = part[i][j] = 0.f;

  // each thread loads 4 consecutive k of one row of A and of W per tile
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  int tile = 0;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + e][lrow] = (am < M && k < K) ? to_f32(A[(size_t)am * lda + k]) : 0.f;
      Ws[lk + e][lrow] = (wn < N && k < K) ? to_f32(W[(size_t)wn * ldw + k]) : 0.f;
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
        for (int j = 0; j < TN; ++j) part[i][j] = fmaf(a[i], w[j], part[i][j]);
    }
    if (++tile == TILES_PER_PARTIAL || k0 + BK >= K) {
      tile = 0;
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[i][j] += part[i][j];
          part[i][j] = 0.f;
        }
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
      if (n < N) C[(size_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
    }
  }
}

template <typename TA, typename TW, typename TC>
int launch(void* C, const void* A, const void* W, int M, int N, int K, long long lda, long long ldw,
           long long ldc, cudaStream_t s) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  oi_launch(gemm_generic_kernel<TA, TW, TC>, grid, 256, 0, s, (TC*)C, (const TA*)A, (const TW*)W, M, N, K, lda, ldw, ldc);
  OI_CHECK_LAUNCH();
  return OI_OK;
}
}  // namespace

// Leading dimensions are in elements; rows of A, W and C are contiguous in k / n.
OI_API int oi_gemm_generic(void* C, int c_dtype, const void* A, int a_dtype, const void* W, int w_dtype,
                           int M, int N, int K, long long lda, long long ldw, long long ldc, void* stream) {
  OI_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
  OI_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm: leading dimension smaller than the row");
  if (M == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int code = (a_dtype << 2) | (w_dtype << 1) | c_dtype;
  switch (code) {
    case 0b000: return launch<float, float, float>(C, A, W, M, N, K, lda, ldw, ldc, s);
    case 0b001: return launch<float, float, bf16>(C, A, W, M, N, K, lda, ldw, ldc, s);
    case 0b010: return launch<float, bf16, float>(C, A, W, M, N, K, lda, ldw, ldc, s);
    case 0b011: return launch<float, bf16, bf16>(C, A, W, M, N, K, lda, ldw, ldc, s);
    case 0b100: return launch<bf16, float, float>(C, A, W, M, N, K, lda, ldw, ldc, s);
    case 0b101: return launch<bf16, float, bf16>(C, A, W, M, N, K, lda, ldw, ldc, s);
    case 0b110: return launch<bf16, bf16, float>(C, A, W, M, N, K, lda, ldw, ldc, s);
    case 0b111: return launch<bf16, bf16, bf16>(C, A, W, M, N, K, lda, ldw, ldc, s);
  }
  OI_REQUIRE(false, "gemm: unknown dtype codes %d/%d/%d", a_dtype, w_dtype, c_dtype);
}
