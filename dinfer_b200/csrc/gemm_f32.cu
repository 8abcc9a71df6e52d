// C[M, N] = A[M, K] * W[N, K]^T with plain 32-bit multiply-adds on the CUDA cores: the matrix
// product of the true 32-bit model (no tensor cores, no reduced-precision matrix mode), and of a
// bfloat16 model whose file stores a matrix in 32-bit.  A, W and C may each be f32 or bf16 in
// memory; every product and sum is f32.  Any M, N, K.
//
// Two kernels: a 128x128x8 register-tiled one for prompts, and a warp-per-output-column one for
// the few rows of a decode step.  The reference has no 32-bit path (its weights are bf16 and its
// products cuBLASLt: crates/kernels/src/gemm.rs:649-690).
#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int BM = 128, BN = 128, BK = 8;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_tile_kernel(const TA* __restrict__ A, int64_t lda, const TW* __restrict__ W, int64_t ldw,
                 TC* __restrict__ C, int64_t ldc, int M, int N, int K) {
  __shared__ float As[BK][BM];
  __shared__ float Ws[BK][BN];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  const int lr = tid >> 1, lk = (tid & 1) * 4;   // this thread loads row lr, k = lk..lk+3 of both tiles
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lk + u;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + u][lr] = (am < M && k < K) ? to_f32<TA>(A[(int64_t)am * lda + k]) : 0.f;
      Ws[lk + u][lr] = (wn < N && k < K) ? to_f32<TW>(W[(int64_t)wn * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[8], b[8];
      *reinterpret_cast<float4*>(a) = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      *reinterpret_cast<float4*>(a + 4) = *reinterpret_cast<const float4*>(&As[k][64 + ty * 4]);
      *reinterpret_cast<float4*>(b) = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      *reinterpret_cast<float4*>(b + 4) = *reinterpret_cast<const float4*>(&Ws[k][64 + tx * 4]);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (n < N) C[(int64_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
    }
  }
}

// M <= ROWS rows: one warp per output column n; lanes stride over K, the weight row is read once.
template <typename TA, typename TW, typename TC, int ROWS>
__global__ void __launch_bounds__(256)
gemm_rows_kernel(const TA* __restrict__ A, int64_t lda, const TW* __restrict__ W, int64_t ldw,
                 TC* __restrict__ C, int64_t ldc, int M, int N, int K) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const TW* w = W + (int64_t)n * ldw;
  float acc[ROWS];
#pragma unroll
  for (int m = 0; m < ROWS; ++m) acc[m] = 0.f;
  for (int k = lane; k < K; k += 32) {
    const float wv = to_f32<TW>(w[k]);
#pragma unroll
    for (int m = 0; m < ROWS; ++m)
      if (m < M) acc[m] = fmaf(to_f32<TA>(A[(int64_t)m * lda + k]), wv, acc[m]);
  }
#pragma unroll
  for (int m = 0; m < ROWS; ++m) {
    const float s = warp_sum(acc[m]);
    if (lane == 0 && m < M) C[(int64_t)m * ldc + n] = from_f32<TC>(s);
  }
}

template <typename TA, typename TW, typename TC>
int launch(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc, int M, int N,
           int K, cudaStream_t stream) {
  if (M <= 8) {
    gemm_rows_kernel<TA, TW, TC, 8><<<(N + 7) / 8, 256, 0, stream>>>(
        (const TA*)A, lda, (const TW*)W, ldw, (TC*)C, ldc, M, N, K);
  } else {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return refuse(DINFER_BAD_ARGUMENT, "gemm_f32: M=%d too large", M);
    gemm_tile_kernel<TA, TW, TC><<<grid, 256, 0, stream>>>(
        (const TA*)A, lda, (const TW*)W, ldw, (TC*)C, ldc, M, N, K);
  }
  return cuda_status("gemm_f32");
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// A [M, K] row stride lda; W [N, K] row stride ldw; C [M, N] row stride ldc (strides in elements).
DINFER_API int dinfer_gemm_f32(const void* A, int64_t lda, int a_dtype, const void* W, int64_t ldw,
                               int w_dtype, void* C, int64_t ldc, int c_dtype, int M, int N, int K,
                               cudaStream_t stream) {
  if (M < 0 || N <= 0 || K <= 0 || lda < K || ldw < K || ldc < N)
    return refuse(DINFER_BAD_ARGUMENT, "gemm_f32: bad sizes M=%d N=%d K=%d lda=%lld ldw=%lld ldc=%lld", M, N, K,
                  (long long)lda, (long long)ldw, (long long)ldc);
  if (M == 0) return 0;
  DINFER_DISPATCH_DTYPE(a_dtype, TA,
    DINFER_DISPATCH_DTYPE(w_dtype, TW,
      DINFER_DISPATCH_DTYPE(c_dtype, TC,
        return launch<TA, TW, TC>(A, lda, W, ldw, C, ldc, M, N, K, stream))));
  return 0;
}
