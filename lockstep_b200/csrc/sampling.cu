// Sampling on the device from float32 logits [rows, vocab].
//
// greedy:      argmax, ties to the lowest token id.
// temperature / nucleus: p = softmax(logits / T); tokens are ranked by
// (-p, id); the head is the shortest prefix of that ranking whose mass reaches
// top_p; the draw u * mass(head) picks the first rank whose cumulative mass
// reaches it.  u is word 0 of Philox-4x32-10 with counter (pos_lo, pos_hi, 0, 0)
// and the request's 64-bit key, times 2^-32.  No sort is done: the rank that a
// target mass falls on is found by bisection on the bit pattern of p (32 block
// sums in a fixed order), then ties of that value are counted in id order.
// Every sum is taken in an order fixed by the vocabulary size alone.
#include <math_constants.h>

#include "common.cuh"

namespace {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ void philox_round(uint32_t& c0, uint32_t& c1, uint32_t& c2, uint32_t& c3,
                                             uint32_t k0, uint32_t k1) {
  const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
  const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
  const uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
  const uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
  const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
  c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
}

__device__ __forceinline__ uint32_t philox_word0(uint32_t pos_lo, uint32_t pos_hi, uint32_t k0,
                                                 uint32_t k1) {
  uint32_t c0 = pos_lo, c1 = pos_hi, c2 = 0u, c3 = 0u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c0, c1, c2, c3, k0, k1);
    if (r < 9) { k0 += 0x9E3779B9u; k1 += 0xBB67AE85u; }
  }
  return c0;
}

struct ArgMax {
  float v;
  int i;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ ArgMax block_argmax(const float* row, int vocab, float* sval, int* sidx) {
  ArgMax best{-CUDART_INF_F, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    // NaN never wins; an all-NaN row gives token 0
    if (v > best.v || (v == best.v && i < best.i)) best = ArgMax{v, i};
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) { sval[warp] = best.v; sidx[warp] = best.i; }
  __syncthreads();
  ArgMax r{sval[0], sidx[0]};
  for (int w = 1; w < nwarps; ++w) r = better(r, ArgMax{sval[w], sidx[w]});
  if (r.i == 0x7fffffff) r.i = 0;
  return r;
}

__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
  ls_dependency_sync();
  __shared__ float sval[32];
  __shared__ int sidx[32];
  const ArgMax r = block_argmax(logits + (int64_t)blockIdx.x * vocab, vocab, sval, sidx);
  if (threadIdx.x == 0) out[blockIdx.x] = r.i;
}

// mass of the tokens with p >= the value whose bits are `bits` (p >= 0, so the
// unsigned bit pattern orders like the value)
__device__ float mass_at_least(const float* p, int vocab, uint32_t bits, float* scratch) {
  float s = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = p[i];
    if (__float_as_uint(v) >= bits) s += v;
  }
  return ls_block_sum(s, scratch);
}

// The rank that `target` falls on: the token x with before(x) < target <=
// before(x) + p_x in the (-p, id) order.  Also returns the mass up to and
// including x.  If target exceeds the whole mass, the last rank is returned.
__device__ int select_rank(const float* p, int vocab, float target, float* mass_through,
                           float* scratch, int* iscratch) {
  // largest value v (as bits) with mass_at_least(v) >= target
  target = fmaxf(target, 1e-37f);  // a draw of exactly 0 falls on the first rank
  uint32_t lo = 0u, hi = 0x7f800000u;  // invariant: mass(lo) >= target or lo == 0
  for (int it = 0; it < 32 && lo < hi; ++it) {
    const uint32_t mid = lo + (hi - lo + 1u) / 2u;
    const float mass = mass_at_least(p, vocab, mid, scratch);
    if (mass >= target) lo = mid; else hi = mid - 1u;
  }
  // lo may lie between two values that occur: snap it to the smallest p >= lo
  float vmin = CUDART_INF_F;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = p[i];
    if (__float_as_uint(v) >= lo) vmin = fminf(vmin, v);
  }
  vmin = -ls_warp_max(-vmin);
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = vmin;
    __syncthreads();
    vmin = scratch[0];
    for (int w = 1; w < nwarps; ++w) vmin = fminf(vmin, scratch[w]);
  }
  const uint32_t vbits = __float_as_uint(vmin);
  const float above = mass_at_least(p, vocab, vbits + 1u, scratch);  // mass of p > v
  // ties of value v in ascending id: the j-th (0-based) is the rank wanted
  int j = 0;
  if (vmin > 0.f) {
    const float need = target - above;
    j = (int)ceilf(need / vmin) - 1;
    if (j < 0) j = 0;
  }
  // count ties per thread over contiguous id ranges, then walk
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = threadIdx.x * chunk;
  const int end = begin + chunk < vocab ? begin + chunk : vocab;
  int count = 0;
  for (int i = begin; i < end; ++i) count += (__float_as_uint(p[i]) == vbits);
  __syncthreads();
  iscratch[threadIdx.x] = count;
  __syncthreads();
  __shared__ int s_token, s_j;
  if (threadIdx.x == 0) {
    int total = 0;
    for (int t = 0; t < blockDim.x; ++t) total += iscratch[t];
    if (j >= total) j = total - 1;
    if (j < 0) j = 0;
    s_j = j;
    s_token = -1;
  }
  __syncthreads();
  j = s_j;
  // exclusive prefix of this thread
  int before = 0;
  for (int t = 0; t < (int)threadIdx.x; ++t) before += iscratch[t];
  if (j >= before && j < before + count) {
    int k = before;
    for (int i = begin; i < end; ++i) {
      if (__float_as_uint(p[i]) == vbits) {
        if (k == j) { s_token = i; break; }
        ++k;
      }
    }
  }
  __syncthreads();
  *mass_through = above + (float)(j + 1) * vmin;
  return s_token < 0 ? 0 : s_token;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, float* __restrict__ probs,
              const float* __restrict__ temperature, const float* __restrict__ top_p,
              const uint32_t* __restrict__ keys, const uint32_t* __restrict__ positions,
              int* __restrict__ out, int vocab) {
  ls_dependency_sync();
  __shared__ float scratch[32];
  __shared__ int sidx[32];
  __shared__ int iscratch[SAMPLE_THREADS];
  const int r = blockIdx.x;
  const float* row = logits + (int64_t)r * vocab;
  float* p = probs + (int64_t)r * vocab;
  const float temp = temperature[r];
  const ArgMax top = block_argmax(row, vocab, scratch, sidx);
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) out[r] = top.i;
    return;
  }
  const float vmax = __fdiv_rn(top.v, temp);
  float s = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float e = expf(__fdiv_rn(row[i], temp) - vmax);
    p[i] = e;
    s += e;
  }
  const float z = ls_block_sum(s, scratch);
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) p[i] = __fdiv_rn(p[i], z);
  __syncthreads();

  const float u = (float)((double)philox_word0(positions[2 * r], positions[2 * r + 1], keys[2 * r],
                                               keys[2 * r + 1]) * 2.3283064365386963e-10);
  float head = 1.0f;
  const float tp = top_p[r];
  float through;
  if (tp < 1.0f) {
    select_rank(p, vocab, tp, &through, scratch, iscratch);
    head = through;
  } else {
    // the whole mass, summed in the order the bisection sums use
    head = mass_at_least(p, vocab, 0u, scratch);
  }
  const float draw = u * head;
  const int token = select_rank(p, vocab, draw, &through, scratch, iscratch);
  if (threadIdx.x == 0) out[r] = token;
}

// argmax in two stages, so that a few rows of a wide vocabulary fill the device:
// stage 1 reduces contiguous chunks of a row, stage 2 the chunks' winners.
constexpr int ARGMAX_CHUNKS = 64;

__global__ void argmax_chunk_kernel(const float* __restrict__ logits, float* __restrict__ cval,
                                    int* __restrict__ cidx, int vocab) {
  ls_dependency_sync();
  __shared__ float sval[32];
  __shared__ int sidx[32];
  const int r = blockIdx.x, c = blockIdx.y;
  const int per = (vocab + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
  const int lo = c * per, hi = lo + per < vocab ? lo + per : vocab;
  ArgMax best{-CUDART_INF_F, 0x7fffffff};
  if (lo < hi) {
    const ArgMax local = block_argmax(logits + (int64_t)r * vocab + lo, hi - lo, sval, sidx);
    best.v = local.v;
    best.i = local.i + lo;
    // a chunk of NaN only: block_argmax reports index 0 with value -inf; keep it out of the way
    if (!(local.v > -CUDART_INF_F)) best.i = 0x7fffffff;
  }
  if (threadIdx.x == 0) {
    cval[r * ARGMAX_CHUNKS + c] = best.v;
    cidx[r * ARGMAX_CHUNKS + c] = best.i;
  }
}

__global__ void argmax_final_kernel(const float* __restrict__ cval, const int* __restrict__ cidx,
                                    int* __restrict__ out) {
  ls_dependency_sync();
  const int r = blockIdx.x;
  ArgMax best{cval[r * ARGMAX_CHUNKS + threadIdx.x], cidx[r * ARGMAX_CHUNKS + threadIdx.x]};
  // 64 candidates: two per lane of one warp
  if (threadIdx.x < 32) {
    ArgMax second{cval[r * ARGMAX_CHUNKS + 32 + threadIdx.x], cidx[r * ARGMAX_CHUNKS + 32 + threadIdx.x]};
    best = better(best, second);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax peer{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = better(best, peer);
    }
    if (threadIdx.x == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
  }
}

}  // namespace

// scratch: rows * 64 floats followed by rows * 64 ints (the caller's; rows * 512 bytes)
LS_API int ls_argmax(const float* logits, int* out, void* scratch, int rows, int vocab,
                     cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (scratch == nullptr || vocab < 4 * ARGMAX_CHUNKS) {
    LS_COUNT(LS_K_ARGMAX), ls_launch(argmax_kernel, rows, 512, 0, stream, logits, out, vocab);
    return ls_launch_status();
  }
  float* cval = (float*)scratch;
  int* cidx = (int*)(cval + (size_t)rows * ARGMAX_CHUNKS);
  LS_COUNT(LS_K_ARGMAX), ls_launch(argmax_chunk_kernel, dim3(rows, ARGMAX_CHUNKS), 256, 0, stream, logits, cval, cidx, vocab);
  ls_launch(argmax_final_kernel, rows, 32, 0, stream, cval, cidx, out);
  return ls_launch_status();
}

// probs: scratch [rows, vocab] float32.  keys, positions: [rows, 2] uint32 (low, high).
LS_API int ls_sample(const float* logits, float* probs, const float* temperature,
                     const float* top_p, const uint32_t* keys, const uint32_t* positions, int* out,
                     int rows, int vocab, cudaStream_t stream) {
  if (rows <= 0) return 0;
  LS_COUNT(LS_K_SAMPLE), ls_launch(sample_kernel, rows, SAMPLE_THREADS, 0, stream, logits, probs, temperature, top_p, keys,
                                                     positions, out, vocab);
  return ls_launch_status();
}

LS_API const char* ls_constants_sampling() {
  static char buf[256];
  static const LsConstant c[] = {{"argmax.chunks", ARGMAX_CHUNKS}, {"sample.threads", SAMPLE_THREADS}};
  return ls_format_constants(buf, sizeof buf, c, (int)(sizeof c / sizeof c[0]));
}
