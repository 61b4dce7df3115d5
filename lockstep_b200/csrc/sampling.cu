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

// --------------------------------------------------------------------------
// The same sampling with a row spread over the eight blocks of a cluster: a thread keeps its
// tokens' probabilities in registers (ids gthread * per .. + per - 1, contiguous, so that ties
// are met in id order), every pass of the bisection is a compare-and-add over those registers,
// a block sum and one exchange of the eight blocks' partials through distributed shared
// memory, summed in rank order.  One block a row walked the row's 152 k probabilities from
// memory 31 times a selection (≈ 1 ms a call, 1.8 ms with top-p, whatever the number of rows).
// Sums are taken in an order fixed by the vocabulary size alone; all blocks of a cluster see the
// same totals and take the same decisions.
// --------------------------------------------------------------------------
constexpr int SAMPLE_CLUSTER = 8;
constexpr int SAMPLE_PER = 20;        // probabilities a thread keeps: vocabularies up to 8 x 1024 x 20 = 163,840

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_addr(const void* mine, int rank) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(mine), r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  return r;
}
__device__ __forceinline__ float ld_peer_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ int ld_peer_s32(uint32_t addr) {
  int v;
  asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

// What the blocks of a cluster exchange: two sets of slots used in turn, so that a block may
// write its next partial while a slow peer still reads the last one.
struct ClusterShare {
  float f[2][4];
  int i[2][2];
  float all_f[SAMPLE_CLUSTER][4];
  int all_i[SAMPLE_CLUSTER][2];
  float warp_f[3][32];
  int warp_i[32];
};

// Every block gives (a, b); every thread gets the eight blocks' pairs in rank order in sh.all_f.
// `turn` (every thread's own copy, the same in all) says which set of slots this exchange uses.
__device__ void cluster_gather_f(ClusterShare& sh, int& turn, float a, float b = 0.f, float c = 0.f) {
  const int t = turn;
  turn ^= 1;
  if (threadIdx.x == 0) { sh.f[t][0] = a; sh.f[t][1] = b; sh.f[t][2] = c; }
  cluster_sync_all();
  if (threadIdx.x < SAMPLE_CLUSTER * 4) {
    const int rank = threadIdx.x >> 2, which = threadIdx.x & 3;
    sh.all_f[rank][which] = ld_peer_f32(peer_addr(&sh.f[t][which], rank));
  }
  __syncthreads();
}
__device__ void cluster_gather_i(ClusterShare& sh, int& turn, int a, int b) {
  const int t = turn;
  turn ^= 1;
  if (threadIdx.x == 0) { sh.i[t][0] = a; sh.i[t][1] = b; }
  cluster_sync_all();
  if (threadIdx.x < SAMPLE_CLUSTER * 2) {
    const int rank = threadIdx.x >> 1, which = threadIdx.x & 1;
    sh.all_i[rank][which] = ld_peer_s32(peer_addr(&sh.i[t][which], rank));
  }
  __syncthreads();
}

// sum over the cluster: a thread's value, lanes by xor tree, warps ascending, blocks in rank order
__device__ float cluster_sum(ClusterShare& sh, int& turn, float v) {
  const float block = ls_block_sum(v, sh.warp_f[0]);
  cluster_gather_f(sh, turn, block);
  float total = 0.f;
#pragma unroll
  for (int r = 0; r < SAMPLE_CLUSTER; ++r) total += sh.all_f[r][0];
  __syncthreads();          // all have read before the next gather writes
  return total;
}

// three sums over the cluster at once (each in the order of cluster_sum): one exchange for all
__device__ void cluster_sum3(ClusterShare& sh, int& turn, float& a, float& b, float& c) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  a = ls_warp_sum(a);
  b = ls_warp_sum(b);
  c = ls_warp_sum(c);
  __syncthreads();
  if (lane == 0) { sh.warp_f[0][warp] = a; sh.warp_f[1][warp] = b; sh.warp_f[2][warp] = c; }
  __syncthreads();
  float ta = 0.f, tb = 0.f, tc = 0.f;
  for (int w = 0; w < 32; ++w) { ta += sh.warp_f[0][w]; tb += sh.warp_f[1][w]; tc += sh.warp_f[2][w]; }
  cluster_gather_f(sh, turn, ta, tb, tc);
  a = b = c = 0.f;
#pragma unroll
  for (int r = 0; r < SAMPLE_CLUSTER; ++r) { a += sh.all_f[r][0]; b += sh.all_f[r][1]; c += sh.all_f[r][2]; }
  __syncthreads();
}

// mass of this cluster's row with p >= the value whose bits are `bits`
__device__ float mass_at_least_regs(ClusterShare& sh, int& turn, const float* p, int per, uint32_t bits) {
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < SAMPLE_PER; ++j)
    if (j < per && __float_as_uint(p[j]) >= bits) s += p[j];
  return cluster_sum(sh, turn, s);
}

// select_rank over the registers of a cluster: the token on which `target` falls in the
// (-p, id) order, written to *token_out by the one thread that holds it; returns the mass up to
// and including that token.
__device__ float select_rank_regs(ClusterShare& sh, int& turn, const float* p, int per, int begin, float target,
                                  int* token_out) {
  target = fmaxf(target, 1e-37f);
  // the largest bit pattern lo with mass(lo) >= target, the interval cut in four a pass (three
  // thresholds' masses from one sweep over the registers and one exchange)
  uint32_t lo = 0u, hi = 0x7f800000u;
  for (int it = 0; it < 32 && lo < hi; ++it) {
    const uint32_t span = hi - lo;
    const uint32_t q1 = span >> 2, q2 = span >> 1, q3 = span - (span >> 2);
    const uint32_t t1 = lo + (q1 ? q1 : 1u), t2 = lo + (q2 ? q2 : 1u), t3 = lo + (q3 ? q3 : 1u);
    float m1 = 0.f, m2 = 0.f, m3 = 0.f;
#pragma unroll
    for (int j = 0; j < SAMPLE_PER; ++j) {
      if (j < per) {
        const uint32_t b = __float_as_uint(p[j]);
        if (b >= t1) m1 += p[j];
        if (b >= t2) m2 += p[j];
        if (b >= t3) m3 += p[j];
      }
    }
    cluster_sum3(sh, turn, m1, m2, m3);
    if (m3 >= target) lo = t3;
    else if (m2 >= target) { lo = t2; hi = t3 - 1u; }
    else if (m1 >= target) { lo = t1; hi = t2 - 1u; }
    else hi = t1 - 1u;
  }
  // snap lo to the smallest probability that occurs at or above it
  float vmin = CUDART_INF_F;
#pragma unroll
  for (int j = 0; j < SAMPLE_PER; ++j)
    if (j < per && __float_as_uint(p[j]) >= lo) vmin = fminf(vmin, p[j]);
  vmin = -ls_warp_max(-vmin);
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh.warp_f[0][warp] = vmin;
    __syncthreads();
    vmin = sh.warp_f[0][0];
    for (int w = 1; w < 32; ++w) vmin = fminf(vmin, sh.warp_f[0][w]);
    __syncthreads();
  }
  cluster_gather_f(sh, turn, vmin);
#pragma unroll
  for (int r = 0; r < SAMPLE_CLUSTER; ++r) vmin = fminf(vmin, sh.all_f[r][0]);
  __syncthreads();
  const uint32_t vbits = __float_as_uint(vmin);
  const float above = mass_at_least_regs(sh, turn, p, per, vbits + 1u);
  int j = 0;
  if (vmin > 0.f && vmin < CUDART_INF_F) {
    j = (int)ceilf((target - above) / vmin) - 1;
    if (j < 0) j = 0;
  }
  // ties of value vmin in ascending id: a thread's ids are contiguous and ascend with the thread
  int count = 0;
#pragma unroll
  for (int q = 0; q < SAMPLE_PER; ++q) count += (q < per && __float_as_uint(p[q]) == vbits);
  // exclusive prefix over the block: lanes by a scan, warps ascending
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = count;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  if (lane == 31) sh.warp_i[warp] = incl;
  __syncthreads();
  int before = incl - count, block_total = 0;
  for (int w = 0; w < 32; ++w) {
    if (w < warp) before += sh.warp_i[w];
    block_total += sh.warp_i[w];
  }
  __syncthreads();
  cluster_gather_i(sh, turn, block_total, 0);
  const int rank = (int)cluster_rank();
  int total = 0;
#pragma unroll
  for (int r = 0; r < SAMPLE_CLUSTER; ++r) {
    if (r < rank) before += sh.all_i[r][0];
    total += sh.all_i[r][0];
  }
  __syncthreads();
  if (j >= total) j = total - 1;
  if (j < 0) j = 0;
  if (total <= 0 && rank == 0 && threadIdx.x == 0) *token_out = 0;      // nothing to choose from (a row of NaN)
  if (j >= before && j < before + count) {
    int k = before;
#pragma unroll
    for (int q = 0; q < SAMPLE_PER; ++q) {
      if (q < per && __float_as_uint(p[q]) == vbits) {
        if (k == j) *token_out = begin + q;
        ++k;
      }
    }
  }
  return above + (float)(j + 1) * vmin;
}

__global__ void __cluster_dims__(SAMPLE_CLUSTER, 1, 1) __launch_bounds__(SAMPLE_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                      const float* __restrict__ top_p, const uint32_t* __restrict__ keys,
                      const uint32_t* __restrict__ positions, int* __restrict__ out, int vocab) {
  ls_dependency_sync();
  __shared__ ClusterShare sh;
  const int r = blockIdx.x / SAMPLE_CLUSTER;
  const int rank = (int)cluster_rank();
  const float* row = logits + (int64_t)r * vocab;
  const int per = (vocab + SAMPLE_CLUSTER * SAMPLE_THREADS - 1) / (SAMPLE_CLUSTER * SAMPLE_THREADS);
  const int begin = (rank * SAMPLE_THREADS + (int)threadIdx.x) * per;
  int turn = 0;
  // this thread's logits; the row's argmax (ties to the lowest id; NaN never wins)
  float p[SAMPLE_PER];
  ArgMax best{-CUDART_INF_F, 0x7fffffff};
#pragma unroll
  for (int j = 0; j < SAMPLE_PER; ++j) {
    p[j] = -CUDART_INF_F;
    if (j < per && begin + j < vocab) {
      p[j] = row[begin + j];
      if (p[j] > best.v || (p[j] == best.v && begin + j < best.i)) best = ArgMax{p[j], begin + j};
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sh.warp_f[0][warp] = best.v; sh.warp_i[warp] = best.i; }
    __syncthreads();
    best = ArgMax{sh.warp_f[0][0], sh.warp_i[0]};
    for (int w = 1; w < 32; ++w) best = better(best, ArgMax{sh.warp_f[0][w], sh.warp_i[w]});
    __syncthreads();
  }
  cluster_gather_f(sh, turn, best.v);
  cluster_gather_i(sh, turn, best.i, 0);
  ArgMax top{sh.all_f[0][0], sh.all_i[0][0]};
#pragma unroll
  for (int q = 1; q < SAMPLE_CLUSTER; ++q) top = better(top, ArgMax{sh.all_f[q][0], sh.all_i[q][0]});
  __syncthreads();
  if (top.i == 0x7fffffff) top.i = 0;
  const float temp = temperature[r];
  if (!(temp > 0.f)) {                       // the same branch in every block of the cluster
    if (rank == 0 && threadIdx.x == 0) out[r] = top.i;
    cluster_sync_all();                      // no block leaves while a peer may still read its shared memory
    return;
  }
  // p = exp(l / T - max) / sum, as the one-block kernel takes it
  const float vmax = __fdiv_rn(top.v, temp);
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < SAMPLE_PER; ++j) {
    if (j < per && begin + j < vocab) {
      p[j] = expf(__fdiv_rn(p[j], temp) - vmax);
      s += p[j];
    } else {
      p[j] = 0.f;
    }
  }
  const float z = cluster_sum(sh, turn, s);
#pragma unroll
  for (int j = 0; j < SAMPLE_PER; ++j) p[j] = __fdiv_rn(p[j], z);
  // tokens past the vocabulary hold 0: they never count as ties of a positive value, and a
  // selection never lands on them since `vmin` is taken over values at or above a mass that exists
  const int live = begin < vocab ? (vocab - begin < per ? vocab - begin : per) : 0;

  const float u = (float)((double)philox_word0(positions[2 * r], positions[2 * r + 1], keys[2 * r],
                                               keys[2 * r + 1]) * 2.3283064365386963e-10);
  const float tp = top_p[r];
  int token = -1;
  float head;
  if (tp < 1.0f) {
    int unused = -1;
    head = select_rank_regs(sh, turn, p, live, begin, tp, &unused);
  } else {
    head = mass_at_least_regs(sh, turn, p, live, 0u);
  }
  select_rank_regs(sh, turn, p, live, begin, u * head, &token);
  if (token >= 0) out[r] = token;            // exactly one thread of the cluster holds it
  cluster_sync_all();                        // no block leaves while a peer may still read its shared memory
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

// How many floats of scratch ls_sample needs for its probabilities: none where a row fits the
// registers of a cluster (vocabularies up to 163,840), else rows x vocab.
LS_API long long ls_sample_scratch_floats(int rows, int vocab) {
  return vocab <= SAMPLE_CLUSTER * SAMPLE_THREADS * SAMPLE_PER ? 0LL : (long long)rows * vocab;
}

// probs: scratch of ls_sample_scratch_floats(rows, vocab) floats (may be null when that is 0).
// keys, positions: [rows, 2] uint32 (low, high).
LS_API int ls_sample(const float* logits, float* probs, const float* temperature,
                     const float* top_p, const uint32_t* keys, const uint32_t* positions, int* out,
                     int rows, int vocab, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= SAMPLE_CLUSTER * SAMPLE_THREADS * SAMPLE_PER) {
    // a row over the eight blocks of a cluster, its probabilities in registers
    LS_COUNT(LS_K_SAMPLE), ls_launch(sample_cluster_kernel, rows * SAMPLE_CLUSTER, SAMPLE_THREADS, 0, stream, logits, temperature,
                                     top_p, keys, positions, out, vocab);
    return ls_launch_status();
  }
  if (probs == nullptr) return LS_E_SIZE;
  LS_COUNT(LS_K_SAMPLE), ls_launch(sample_kernel, rows, SAMPLE_THREADS, 0, stream, logits, probs, temperature, top_p, keys,
                                                     positions, out, vocab);
  return ls_launch_status();
}

LS_API const char* ls_constants_sampling() {
  static char buf[256];
  static const LsConstant c[] = {{"argmax.chunks", ARGMAX_CHUNKS}, {"sample.threads", SAMPLE_THREADS},
                                 {"sample.cluster_blocks", SAMPLE_CLUSTER}, {"sample.kept_per_thread", SAMPLE_PER}};
  return ls_format_constants(buf, sizeof buf, c, (int)(sizeof c / sizeof c[0]));
}
