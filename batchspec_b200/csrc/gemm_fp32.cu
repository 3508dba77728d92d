// True float32 matrix product on the CUDA cores (plain FFMA, no tensor-core or
// reduced-precision mode):  C[M,N] = A[M,K] * W[N,K]^T, all row-major, K contiguous.
// Each output element is summed over k = 0..K-1 in that order by one thread, so its
// value does not depend on M or on which other rows are in the batch.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256)
sgemm_tn_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C, int M, int N, int K,
                long long lda, long long ldw, long long ldc) {
  bspec::pdl_prologue(10);
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;           // 16 x 16 threads, each a 4 x 4 tile
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
  // loader mapping: 64 rows x 16 k per tile = 1024 elements, 4 per thread
  const int lr = tid / 4;            // row within the tile, 0..63
  const int lk = (tid % 4) * 4;      // k offset 0,4,8,12
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lk + u;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + u][lr] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
      Ws[lk + u][lr] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
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
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}
}  // namespace

BSPEC_API int bspec_sgemm_tn(const float* A, const float* W, float* C, int M, int N, int K, long long lda,
                             long long ldw, long long ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return (int)cudaErrorInvalidConfiguration;
  BSPEC_LAUNCH((sgemm_tn_kernel), grid, 256, 0, stream, A, W, C, M, N, K, lda, ldw, ldc);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_gemm_fp32)
