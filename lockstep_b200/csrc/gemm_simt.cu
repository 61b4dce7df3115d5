// C[M, N] = A[M, K] * W[N, K]^T on the CUDA cores (FFMA, float32 accumulate).
//
// This is the true 32-bit matrix product of the engine and the fallback of the
// bfloat16 path for shapes the tensor-core kernel refuses.  An output element is
// one accumulator and one chain of FMAs over K in ascending order, so its value
// does not depend on M (the batch) or on where its row lies in the batch.  There
// is no split-K.  Three kernels make that same chain: the general one below (a
// block owns a 64x64 tile; any element type, any depth), one for up to 32
// float32 tokens and one for many float32 tokens.
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

// ---------------------------------------------------------------------------
// Few tokens (up to 32), float32: the decode step's products on the true 32-bit path.
// The tile kernel above would run a handful of blocks with most of their rows empty.  Here a
// block takes 16 rows of W (16 more for silu-mul: the up rows of the same features) and all
// the tokens; a thread owns one feature and the tokens m, m + 8, m + 16, m + 24, each with the
// accumulator and the ascending chain of FMAs it has in the tile kernel (fmaf(a, w, acc) from
// k = 0 up), so the two kernels give the same bits.  W and the token rows stream through a
// ring of shared-memory stages by 16-byte cp.async; the weights of the first stages are asked
// for before the wait on the kernel before.
// ---------------------------------------------------------------------------
constexpr int SK_BN = 16;        // features per block
constexpr int SK_BK = 128;       // depth of a stage
constexpr int SK_PITCH = SK_BK + 4;
constexpr int SK_STAGES = 6;     // five stages on their way while one is multiplied: a block of 16 rows has
                                 // 40 KB of weights in flight, and the blocks of a narrow weight are few
constexpr int SK_MAX_M = 32;

__device__ __forceinline__ void cp_async_16(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// MT: tokens per thread (1, 2 or 4: up to 8, 16 or 32 tokens)
template <typename TC, int EPI, int MT>
__global__ void __launch_bounds__(128)
gemm_nt_skinny_kernel(const float* __restrict__ A, const float* __restrict__ W, TC* __restrict__ C, int M, int N,
                      int K, int64_t lda, int64_t ldw, int64_t ldc) {
  constexpr int W_ROWS = EPI == 2 ? 2 * SK_BN : SK_BN;
  constexpr int X_ROWS = 8 * MT;
  constexpr int STAGE = (W_ROWS + X_ROWS) * SK_PITCH;       // floats
  ls_dependency_trigger();
  extern __shared__ __align__(16) float sk_smem[];
  const int tid = threadIdx.x;
  const int nl = tid >> 3, ml = tid & 7;
  const int n0 = blockIdx.x * SK_BN;
  const int stages_total = (K + SK_BK - 1) / SK_BK;

  // pieces of 16 bytes this thread fetches per stage: W rows, then token rows.  Rows past N or
  // M and pieces past K are not fetched: what lies there is never stored (rows) or never
  // multiplied (the loops below stop at K)
  auto load_w = [&](int st) {
    float* ws = sk_smem + (st % SK_STAGES) * STAGE;
    const int k0 = st * SK_BK;
    for (int i = tid; i < W_ROWS * (SK_BK / 4); i += 128) {
      const int r = i / (SK_BK / 4), ch = i - r * (SK_BK / 4);
      const int n = n0 + (r % SK_BN) + (r >= SK_BN ? N : 0);          // up rows follow the gate rows at N
      if (n0 + (r % SK_BN) < N && k0 + ch * 4 < K) cp_async_16(ws + r * SK_PITCH + ch * 4, W + (int64_t)n * ldw + k0 + ch * 4);
    }
  };
  auto load_x = [&](int st) {
    float* xs = sk_smem + (st % SK_STAGES) * STAGE + W_ROWS * SK_PITCH;
    const int k0 = st * SK_BK;
    for (int i = tid; i < X_ROWS * (SK_BK / 4); i += 128) {
      const int r = i / (SK_BK / 4), ch = i - r * (SK_BK / 4);
      if (r < M && k0 + ch * 4 < K) cp_async_16(xs + r * SK_PITCH + ch * 4, A + (int64_t)r * lda + k0 + ch * 4);
    }
  };

  const int ahead = stages_total < SK_STAGES - 1 ? stages_total : SK_STAGES - 1;
  for (int st = 0; st < ahead; ++st) load_w(st);          // weights do not depend on the kernel before
  ls_dependency_wait();
  for (int st = 0; st < SK_STAGES - 1; ++st) {            // one group per stage, empty ones included
    if (st < ahead) load_x(st);
    cp_async_commit();
  }

  float acc[MT], acu[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i) acc[i] = acu[i] = 0.f;

  for (int st = 0; st < stages_total; ++st) {
    cp_async_wait<SK_STAGES - 2>();                       // stage st has landed (for this thread)
    __syncthreads();                                      // ... for every thread; and stage st - 1 is read
    if (st + SK_STAGES - 1 < stages_total) {
      load_w(st + SK_STAGES - 1);
      load_x(st + SK_STAGES - 1);
    }
    cp_async_commit();
    const float* ws = sk_smem + (st % SK_STAGES) * STAGE;
    const float* xs = ws + W_ROWS * SK_PITCH;
    const int left = K - st * SK_BK;
    const int groups = left >= SK_BK ? SK_BK / 4 : left / 4;
    for (int g = 0; g < groups; ++g) {
      const float4 w4 = *reinterpret_cast<const float4*>(ws + nl * SK_PITCH + 4 * g);
      float4 u4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (EPI == 2) u4 = *reinterpret_cast<const float4*>(ws + (SK_BN + nl) * SK_PITCH + 4 * g);
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const float4 x4 = *reinterpret_cast<const float4*>(xs + (ml + 8 * i) * SK_PITCH + 4 * g);
        acc[i] = fmaf(x4.x, w4.x, acc[i]);
        acc[i] = fmaf(x4.y, w4.y, acc[i]);
        acc[i] = fmaf(x4.z, w4.z, acc[i]);
        acc[i] = fmaf(x4.w, w4.w, acc[i]);
        if (EPI == 2) {
          acu[i] = fmaf(x4.x, u4.x, acu[i]);
          acu[i] = fmaf(x4.y, u4.y, acu[i]);
          acu[i] = fmaf(x4.z, u4.z, acu[i]);
          acu[i] = fmaf(x4.w, u4.w, acu[i]);
        }
      }
    }
  }
  cp_async_wait<0>();

  const int n = n0 + nl;
  if (n < N) {
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      const int m = ml + 8 * i;
      if (m >= M) continue;
      TC* c = C + (int64_t)m * ldc + n;
      if (EPI == 0) {
        *c = ls_from_float<TC>(acc[i]);
      } else if (EPI == 1) {
        *c = ls_from_float<TC>(ls_to_float<TC>(*c) + acc[i]);
      } else {
        const float g = acc[i];
        *c = ls_from_float<TC>(g / (1.0f + expf(-g)) * acu[i]);
      }
    }
  }
}

template <typename TC, int EPI, int MT>
int launch_skinny_as(const float* A, const float* W, TC* C, int M, int N, int K, int64_t lda, int64_t ldw,
                     int64_t ldc, cudaStream_t stream) {
  constexpr int W_ROWS = EPI == 2 ? 2 * SK_BN : SK_BN;
  constexpr size_t smem = (size_t)SK_STAGES * (W_ROWS + 8 * MT) * SK_PITCH * sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_nt_skinny_kernel<TC, EPI, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return LS_E_SMEM;
    configured = true;
  }
  LS_COUNT(LS_K_GEMM_SIMT_FEW);
  ls_launch(gemm_nt_skinny_kernel<TC, EPI, MT>, dim3((N + SK_BN - 1) / SK_BN), 128, smem, stream, A, W, C, M, N, K,
            lda, ldw, ldc);
  return ls_launch_status();
}

template <int EPI>
int launch_skinny(const float* A, const float* W, float* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                  cudaStream_t stream) {
  if (M <= 8) return launch_skinny_as<float, EPI, 1>(A, W, C, M, N, K, lda, ldw, ldc, stream);
  if (M <= 16) return launch_skinny_as<float, EPI, 2>(A, W, C, M, N, K, lda, ldw, ldc, stream);
  return launch_skinny_as<float, EPI, 4>(A, W, C, M, N, K, lda, ldw, ldc, stream);
}

// float32 operands of up to 32 tokens whose rows can be fetched 16 bytes at a time
bool skinny_applies(const void* A, const void* W, int a_dtype, int c_dtype, int M, int K, int64_t lda, int64_t ldw) {
  return a_dtype == LS_F32 && c_dtype == LS_F32 && M <= SK_MAX_M && K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 &&
         ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0;
}

// ---------------------------------------------------------------------------
// Many tokens, float32: the prompt's products on the true 32-bit path.  A block owns 128 tokens
// x 128 features (silu-mul: 128 x 64, the other 64 columns of its tile being the up rows of the
// same features), a thread 8 x 8 of them as four 4 x 4 corners, so that what it reads from
// shared memory per step of k are four 16-byte pieces for 64 FMAs.  The next k-block is on its
// way from memory to registers while this one is multiplied.  Every element is still one
// accumulator and one ascending chain fmaf(a, w, acc), so the bits are those of the two
// kernels above.
// ---------------------------------------------------------------------------
constexpr int LM = 128, LN = 128, LK = 16, LPITCH = LM + 4;

// WR: rows of W in a tile: 128, or 64 where 128 would leave SMs without a tile (a narrow weight).
// The features of a tile are WR, or WR / 2 for silu-mul (gate rows, then the up rows of the same).
template <int EPI, int WR>
__global__ void __launch_bounds__(256, 2)
gemm_nt_large_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C, int M, int N,
                     int K, int64_t lda, int64_t ldw, int64_t ldc) {
  static_assert(WR == 128 || (WR == 64 && EPI != 2), "tile widths");
  constexpr int FN = EPI == 2 ? WR / 2 : WR;           // features of the tile
  constexpr int HALVES = WR / 64;                      // 64-row halves of W a thread fetches and multiplies
  constexpr int WC = 4 * HALVES;                       // columns of a thread
  ls_dependency_sync();
  __shared__ __align__(16) float As[2][LK][LPITCH];
  __shared__ __align__(16) float Ws[2][LK][WR + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * LM, n0 = blockIdx.x * FN;
  // staging: a thread fetches 4 consecutive k of rows lr and lr + 64 of both operands
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  // row of W behind column c of the tile: silu-mul tiles hold gate rows, then the up rows
  auto w_row = [&](int c) -> int64_t {
    if (EPI == 2) return c < FN ? (n0 + c < N ? n0 + c : -1) : (n0 + c - FN < N ? (int64_t)N + n0 + c - FN : -1);
    return n0 + c < N ? n0 + c : -1;
  };
  float4 ra[2], rw[HALVES];
  auto fetch = [&](int k0) {
    const bool k_ok = k0 + lk < K;                      // K is a multiple of 4: a piece is whole or absent
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = m0 + lr + 64 * half;
      ra[half] = (m < M && k_ok) ? *reinterpret_cast<const float4*>(A + (int64_t)m * lda + k0 + lk)
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int half = 0; half < HALVES; ++half) {
      const int64_t wr = w_row(lr + 64 * half);
      rw[half] = (wr >= 0 && k_ok) ? *reinterpret_cast<const float4*>(W + wr * ldw + k0 + lk)
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  auto stage = [&](int buf) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = lr + 64 * half;
      As[buf][lk + 0][r] = ra[half].x; As[buf][lk + 1][r] = ra[half].y;
      As[buf][lk + 2][r] = ra[half].z; As[buf][lk + 3][r] = ra[half].w;
    }
#pragma unroll
    for (int half = 0; half < HALVES; ++half) {
      const int r = lr + 64 * half;
      Ws[buf][lk + 0][r] = rw[half].x; Ws[buf][lk + 1][r] = rw[half].y;
      Ws[buf][lk + 2][r] = rw[half].z; Ws[buf][lk + 3][r] = rw[half].w;
    }
  };

  float acc[8][WC];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < WC; ++j) acc[i][j] = 0.f;

  fetch(0);
  stage(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += LK) {
    const bool more = k0 + LK < K;
    if (more) fetch(k0 + LK);
#pragma unroll
    for (int k = 0; k < LK; ++k) {
      const float4 a_lo = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a_hi = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      const float a[8] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w, a_hi.x, a_hi.y, a_hi.z, a_hi.w};
      float w[WC];
#pragma unroll
      for (int half = 0; half < HALVES; ++half) {
        const float4 w4 = *reinterpret_cast<const float4*>(&Ws[buf][k][64 * half + tx * 4]);
        w[4 * half + 0] = w4.x; w[4 * half + 1] = w4.y; w[4 * half + 2] = w4.z; w[4 * half + 3] = w4.w;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < WC; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    if (more) {
      stage(buf ^ 1);
      __syncthreads();
      buf ^= 1;
    }
  }

  // rows ty * 4 + i and 64 + ty * 4 + i; columns tx * 4 + j and (128 rows of W) 64 + tx * 4 + j
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
    if (m >= M) continue;
    float* crow = C + (int64_t)m * ldc;
    if (EPI == 2) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + tx * 4 + j;
        const float g = acc[i][j];
        if (n < N) crow[n] = g / (1.0f + expf(-g)) * acc[i][WC - 4 + j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < WC; ++j) {
        const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
        if (n < N) crow[n] = EPI == 1 ? crow[n] + acc[i][j] : acc[i][j];
      }
    }
  }
}

int large_sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  return sms;
}

template <int EPI, int WR>
int launch_large_as(const float* A, const float* W, float* C, int M, int N, int K, int64_t lda, int64_t ldw,
                    int64_t ldc, cudaStream_t stream) {
  constexpr int FN = EPI == 2 ? WR / 2 : WR;
  dim3 grid((N + FN - 1) / FN, (M + LM - 1) / LM);
  if (grid.y > 65535) return LS_E_SIZE;
  LS_COUNT(LS_K_GEMM_SIMT_MANY);
  ls_launch(gemm_nt_large_kernel<EPI, WR>, grid, 256, 0, stream, A, W, C, M, N, K, lda, ldw, ldc);
  return ls_launch_status();
}

template <int EPI>
int launch_large(const float* A, const float* W, float* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                 cudaStream_t stream) {
  if constexpr (EPI != 2) {
    // two blocks an SM: tiles of 64 features where 128 would not give every slot one (the tile's
    // width changes no sum)
    const long long wide = (long long)((N + 127) / 128) * ((M + LM - 1) / LM);
    if (wide < 2LL * large_sm_count()) return launch_large_as<EPI, 64>(A, W, C, M, N, K, lda, ldw, ldc, stream);
  }
  return launch_large_as<EPI, 128>(A, W, C, M, N, K, lda, ldw, ldc, stream);
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
  if (skinny_applies(A, W, a_dtype, c_dtype, M, K, lda, ldw)) {
    const float* a = (const float*)A;
    const float* w = (const float*)W;
    if (epilogue == 0) return launch_skinny<0>(a, w, (float*)C, M, N, K, lda, ldw, ldc, stream);
    if (epilogue == 1) return launch_skinny<1>(a, w, (float*)C, M, N, K, lda, ldw, ldc, stream);
    if (epilogue == 2) return launch_skinny<2>(a, w, (float*)C, M, N, K, lda, ldw, ldc, stream);
    return LS_E_SIZE;
  }
  // float32 rows that can be fetched 16 bytes at a time, more than a few of them
  if (a_dtype == LS_F32 && c_dtype == LS_F32 && M > SK_MAX_M && K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 &&
      ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0) {
    const float* a = (const float*)A;
    const float* w = (const float*)W;
    if (epilogue == 0) return launch_large<0>(a, w, (float*)C, M, N, K, lda, ldw, ldc, stream);
    if (epilogue == 1) return launch_large<1>(a, w, (float*)C, M, N, K, lda, ldw, ldc, stream);
    if (epilogue == 2) return launch_large<2>(a, w, (float*)C, M, N, K, lda, ldw, ldc, stream);
    return LS_E_SIZE;
  }
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
  static const LsConstant c[] = {{"gemm_simt.tile_m", BM}, {"gemm_simt.tile_n", BN}, {"gemm_simt.tile_k", BK},
                                 {"gemm_simt.few_tokens", SK_MAX_M}, {"gemm_simt.few_tokens_features", SK_BN},
                                 {"gemm_simt.many_tokens_tile", LM}};
  return ls_format_constants(buf, sizeof buf, c, (int)(sizeof c / sizeof c[0]));
}
