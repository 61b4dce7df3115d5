// C[M, N] = A[M, K] * W[N, K]^T on the CUDA cores (FFMA, float32 accumulate).
//
// This is the true 32-bit matrix product of the engine and the fallback of the
// bfloat16 path for shapes the tensor-core kernel refuses.  One thread block
// owns one 64x64 output tile and walks K in ascending order with one
// accumulator per element, so an output element's value does not depend on M
// (the batch) or on where its row lies in the batch.  There is no split-K.
//
// Epilogues:
//   0 store        C[m, n]  = acc                       (C of type TC)
//   1 residual     C[m, n] += acc                       (C float32, in place)
//   2 silu-mul     C[m, n]  = silu(acc_gate) * acc_up   (W holds gate rows [0, N)
//                                                        and up rows [N, 2N))
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

template <typename TA, typename TW, typename TC, int EPI>
__global__ void __launch_bounds__(256)
gemm_nt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C, int M,
               int N, int K, int64_t lda, int64_t ldw, int64_t ldc) {
  ls_dependency_sync();
  __shared__ float As[BK][BM + PAD];
  __shared__ float Ws[BK][BN + PAD];
  __shared__ float Us[EPI == 2 ? BK : 1][BN + PAD];

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float acc[4][4] = {};
  float acu[4][4] = {};

  // each thread stages 4 consecutive k of one row of A and of W
  const int lrow = tid >> 2;        // 0..63
  const int lk = (tid & 3) * 4;     // 0,4,8,12

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int m = m0 + lrow, n = n0 + lrow;
      As[lk + j][lrow] = (m < M && k < K) ? ls_to_float<TA>(A[(int64_t)m * lda + k]) : 0.f;
      Ws[lk + j][lrow] = (n < N && k < K) ? ls_to_float<TW>(W[(int64_t)n * ldw + k]) : 0.f;
      if (EPI == 2)
        Us[lk + j][lrow] = (n < N && k < K) ? ls_to_float<TW>(W[(int64_t)(n + N) * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], w[4], u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
      if (EPI == 2) {
#pragma unroll
        for (int j = 0; j < 4; ++j) u[j] = Us[k][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
          if (EPI == 2) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
        }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      TC* c = C + (int64_t)m * ldc + n;
      if (EPI == 0) {
        *c = ls_from_float<TC>(acc[i][j]);
      } else if (EPI == 1) {
        *c = ls_from_float<TC>(ls_to_float<TC>(*c) + acc[i][j]);
      } else {
        const float g = acc[i][j];
        *c = ls_from_float<TC>(g / (1.0f + expf(-g)) * acu[i][j]);
      }
    }
  }
}

template <typename TA, typename TW, typename TC>
int launch(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw,
           int64_t ldc, int epilogue, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return LS_E_SIZE;
  switch (epilogue) {
    case 0:
      LS_COUNT(LS_K_GEMM_SIMT), ls_launch(gemm_nt_kernel<TA, TW, TC, 0>, grid, 256, 0, stream, (const TA*)A, (const TW*)W, (TC*)C, M, N, K, lda, ldw, ldc);
      break;
    case 1:
      LS_COUNT(LS_K_GEMM_SIMT), ls_launch(gemm_nt_kernel<TA, TW, TC, 1>, grid, 256, 0, stream, (const TA*)A, (const TW*)W, (TC*)C, M, N, K, lda, ldw, ldc);
      break;
    case 2:
      LS_COUNT(LS_K_GEMM_SIMT), ls_launch(gemm_nt_kernel<TA, TW, TC, 2>, grid, 256, 0, stream, (const TA*)A, (const TW*)W, (TC*)C, M, N, K, lda, ldw, ldc);
      break;
    default:
      return LS_E_SIZE;
  }
  return ls_launch_status();
}

}  // namespace

// a_dtype is also the type of W; c_dtype is the type of C (float32 for the
// residual epilogue and for logits).
LS_API int ls_gemm_nt_simt(const void* A, const void* W, void* C, int a_dtype, int c_dtype, int M,
                           int N, int K, int64_t lda, int64_t ldw, int64_t ldc, int epilogue,
                           cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return LS_E_SIZE;
  if (epilogue == 1 && c_dtype != LS_F32) return LS_E_DTYPE;
  typedef __nv_bfloat16 bf16;
  if (a_dtype == LS_F32 && c_dtype == LS_F32)
    return launch<float, float, float>(A, W, C, M, N, K, lda, ldw, ldc, epilogue, stream);
  if (a_dtype == LS_BF16 && c_dtype == LS_BF16)
    return launch<bf16, bf16, bf16>(A, W, C, M, N, K, lda, ldw, ldc, epilogue, stream);
  if (a_dtype == LS_BF16 && c_dtype == LS_F32)
    return launch<bf16, bf16, float>(A, W, C, M, N, K, lda, ldw, ldc, epilogue, stream);
  return LS_E_DTYPE;
}

LS_API const char* ls_constants_gemm_simt() {
  static char buf[256];
  static const LsConstant c[] = {{"gemm_simt.tile_m", BM}, {"gemm_simt.tile_n", BN}, {"gemm_simt.tile_k", BK}};
  return ls_format_constants(buf, sizeof buf, c, (int)(sizeof c / sizeof c[0]));
}
