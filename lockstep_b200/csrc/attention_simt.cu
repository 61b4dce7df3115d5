// Causal attention over the paged cache on the CUDA cores, for any head size
// that is a multiple of 16 (up to 256), any number of heads and groups, any
// page size that divides the key tile, float32 or bfloat16 storage, with an
// optional window.
//
// Keys are cut into splits of LS_SPLIT tokens at fixed absolute positions.  A
// split is reduced by an online softmax over ascending key tiles; the splits of
// a row are folded in ascending order by ls_fold().  A split's bounds and the
// fold order depend only on the row's own position, so a row's result does not
// depend on the portion or batch it came in.  Two ways of running the splits
// give the same arithmetic:
//   serial:   one block walks all splits of its rows and folds as it goes
//             (portions of prompts: many rows, no scratch memory);
//   parallel: one block per split writes a partial (acc, m, l) to scratch and
//             ls_attention_combine folds them (decoded tokens: few rows).
//
// pages: [num_pages, 2, nkv, page_size, d]; q, out: [tokens, nq, d].
// work item (8 ints): request row in the block table, first token (packed
// index), number of tokens, position of the first token, first split, end
// split, first scratch slot (-1: serial, write `out`), unused.
#include <math_constants.h>

#include "attention_fold.cuh"
#include "common.cuh"

namespace {

constexpr int TILE_M = 16;   // query tokens of a tile kernel block
constexpr int TILE_N = 32;   // keys per tile of the tile kernel
constexpr int MAX_D = 256;

template <typename T>
__device__ __forceinline__ const T* page_ptr(const T* pages, const int* table_row, int key,
                                             int which, int kvh, int nkv, int page_size, int d,
                                             int num_pages, int* err) {
  const int page = table_row[key / page_size];
  if (page < 0 || page >= num_pages) {
    ls_record_fault(err, LS_DEV_PAGE_RANGE, key);
    return nullptr;
  }
  return pages + ((((int64_t)page * 2 + which) * nkv + kvh) * page_size + (key % page_size)) * d;
}

// --------------------------------------------------------------------------
// tile kernel: up to 16 rows: query tokens of one request x query heads of one key head.
// A block has `hb` heads (a divisor of the group size): row m is token m / hb and head
// blockIdx.y * hb + m % hb, so that a single decoded token fills the tile's rows with the heads
// that share its keys and values, which are then loaded once for all of them.  An item with more
// tokens than fit beside `hb` heads takes its heads one after the other.  A row's arithmetic
// does not depend on what the other rows of its tile are.
// --------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128, 4)
attention_tile_kernel(const T* __restrict__ q, const T* __restrict__ pages, T* __restrict__ out,
                      float* __restrict__ part_acc, float* __restrict__ part_ml,
                      const int* __restrict__ work, const int* __restrict__ block_table,
                      int table_stride, int nq, int nkv, int d, int page_size, int num_pages,
                      int window, float scale, const float* __restrict__ slopes, int hb, int* err) {
  ls_dependency_sync();
  extern __shared__ __align__(16) float smem[];
  // rows of Q and K are d + 4 floats apart: 16-byte pieces stay aligned, and the eight key rows a
  // quarter of a warp reads together (keys sub, sub + 8, ...) fall into different banks
  const int dp = d + 4;
  constexpr int PP = TILE_N + 4;       // pitch of a row of P
  float* Qs = smem;                    // [TILE_M][d+4]
  float* Ks = Qs + TILE_M * dp;        // [TILE_N][d+4]
  float* Vs = Ks + TILE_N * dp;        // [TILE_N][d]
  float* Ps = Vs + TILE_N * d;         // [TILE_M][TILE_N+4]

  const int* w = work + (int64_t)blockIdx.x * 8;
  const int req_row = w[0], tok0 = w[1], ntok = w[2], pos0 = w[3];
  if (ntok == 0) return;                     // padding item of a recorded launch
  const int split_begin = w[4], split_end = w[5], slot_base = w[6];
  const int kvh = ((int)blockIdx.y * hb) / (nq / nkv);
  const int heads_at_once = ntok * hb <= TILE_M ? hb : 1;      // heads that share the tile's rows
  const int tid = threadIdx.x;
  const int m = tid >> 3, sub = tid & 7;
  const int m_tok = m / heads_at_once;                         // this row's token of the item
  // Outputs of a thread: dimensions sub * 4 + e + 32 * jj (e < 4) that lie below d.  Which thread
  // holds which key's score or which output changes no sum: a score is one chain over the head's
  // elements in ascending order, an output one chain over the tile's keys in ascending order, the
  // sum of a tile's weights is taken over groups of four neighbouring keys and then a tree.
  const int ngroup = (d + 31) >> 5;
  constexpr int VEC = 16 / (int)sizeof(T);   // elements of a 16-byte piece (a head size is a multiple of 16)
  constexpr int LOADS = 4;                   // pieces of keys (and of values) a thread has in flight
  const int pieces = d / VEC;
  const int* table_row = block_table + (int64_t)req_row * table_stride;

  const int pos_last = pos0 + ntok - 1;
  const int key_lo_tile = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int qpos = pos0 + m_tok;
  const bool row_valid = m < ntok * heads_at_once;
  const int row_lo = (window > 0 && qpos - window + 1 > 0) ? qpos - window + 1 : 0;

  for (int h_first = (int)blockIdx.y * hb; h_first < ((int)blockIdx.y + 1) * hb; h_first += heads_at_once) {
  const int h = h_first + m - m_tok * heads_at_once;           // this row's head
  // slopes (or null): a score gets slopes[head] x (key position - query position) added,
  // a position encoding that biases the scores instead of rotating queries and keys
  const float slope = slopes != nullptr && row_valid ? slopes[h] : 0.f;
  __syncthreads();                                             // the heads before are done with Q
  for (int i = tid; i < TILE_M * d; i += 128) {
    const int r = i / d, c = i - r * d;
    const int r_tok = r / heads_at_once;
    Qs[r * dp + c] = r < ntok * heads_at_once
                         ? ls_to_float<T>(q[((int64_t)(tok0 + r_tok) * nq + h_first + r - r_tok * heads_at_once) * d + c])
                         : 0.f;
  }

  float acc_run[MAX_D / 8], acc_s[MAX_D / 8];
#pragma unroll
  for (int j = 0; j < MAX_D / 8; ++j) acc_run[j] = 0.f;
  float m_run = -CUDART_INF_F, l_run = 0.f;

  for (int split = split_begin; split < split_end; ++split) {
    const int s_lo = split * LS_SPLIT;
    int s_hi = s_lo + LS_SPLIT;                 // exclusive
    if (s_hi > pos_last + 1) s_hi = pos_last + 1;
#pragma unroll
    for (int j = 0; j < MAX_D / 8; ++j) acc_s[j] = 0.f;
    float m_s = -CUDART_INF_F, l_s = 0.f;

    // tiles lie at fixed offsets from the split's start; those wholly before
    // the first row's window change nothing and are skipped
    int t_first = s_lo;
    if (key_lo_tile > s_lo) t_first = s_lo + ((key_lo_tile - s_lo) / TILE_N) * TILE_N;
    for (int n0 = t_first; n0 < s_hi; n0 += TILE_N) {
      __syncthreads();
      // the tile's keys and values, 16 bytes a load: four threads share a key (its page is looked
      // up once per thread and tile) and take its pieces in turn, LOADS pieces of each kind in
      // flight at a time
      {
        const int n = tid >> 2, key = n0 + n;
        const T* kp = nullptr;
        if (key < s_hi && key >= key_lo_tile)
          kp = page_ptr<T>(pages, table_row, key, 0, kvh, nkv, page_size, d, num_pages, err);
        const int64_t to_v = (int64_t)nkv * page_size * d;
        for (int ch0 = tid & 3; ch0 < pieces; ch0 += 4 * LOADS) {
          uint4 kraw[LOADS], vraw[LOADS];
#pragma unroll
          for (int b = 0; b < LOADS; ++b) {
            const int ch = ch0 + 4 * b;
            kraw[b] = vraw[b] = make_uint4(0u, 0u, 0u, 0u);        // zero bits are 0.0 in either type
            if (kp != nullptr && ch < pieces) {
              kraw[b] = *reinterpret_cast<const uint4*>(kp + ch * VEC);
              vraw[b] = *reinterpret_cast<const uint4*>(kp + to_v + ch * VEC);
            }
          }
#pragma unroll
          for (int b = 0; b < LOADS; ++b) {
            const int ch = ch0 + 4 * b;
            if (ch < pieces) {
              const T* kt = reinterpret_cast<const T*>(&kraw[b]);
              const T* vt = reinterpret_cast<const T*>(&vraw[b]);
#pragma unroll
              for (int e = 0; e < VEC; e += 4) {
                *reinterpret_cast<float4*>(Ks + n * dp + ch * VEC + e) = make_float4(
                    ls_to_float<T>(kt[e]), ls_to_float<T>(kt[e + 1]), ls_to_float<T>(kt[e + 2]), ls_to_float<T>(kt[e + 3]));
                *reinterpret_cast<float4*>(Vs + n * d + ch * VEC + e) = make_float4(
                    ls_to_float<T>(vt[e]), ls_to_float<T>(vt[e + 1]), ls_to_float<T>(vt[e + 2]), ls_to_float<T>(vt[e + 3]));
              }
            }
          }
        }
      }
      __syncthreads();

      // scores of keys sub, sub + 8, sub + 16, sub + 24 of the tile: each one chain over the
      // head's elements in ascending order
      float s[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
      float tile_max = -CUDART_INF_F;
      if (row_valid) {
        float dot[4] = {0.f, 0.f, 0.f, 0.f};
        const float* qr = Qs + m * dp;
        const float* kr = Ks + sub * dp;
#pragma unroll 4
        for (int c = 0; c < d; c += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qr + c);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 k4 = *reinterpret_cast<const float4*>(kr + j * 8 * dp + c);
            dot[j] = fmaf(q4.x, k4.x, dot[j]);
            dot[j] = fmaf(q4.y, k4.y, dot[j]);
            dot[j] = fmaf(q4.z, k4.z, dot[j]);
            dot[j] = fmaf(q4.w, k4.w, dot[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int key = n0 + sub + 8 * j;
          const bool keep = key < s_hi && key <= qpos && key >= row_lo;
          s[j] = !keep ? -CUDART_INF_F
                 : slopes != nullptr ? fmaf(slope, (float)(key - qpos), dot[j] * scale) : dot[j] * scale;
          tile_max = fmaxf(tile_max, s[j]);
        }
      }
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 4));
      const float m_new = fmaxf(m_s, tile_max);
      float alpha = 1.f;
      float p[4] = {0.f, 0.f, 0.f, 0.f};
      if (m_new != -CUDART_INF_F) {
        alpha = (m_s == -CUDART_INF_F) ? 0.f : expf(m_s - m_new);
#pragma unroll
        for (int j = 0; j < 4; ++j) p[j] = (s[j] == -CUDART_INF_F) ? 0.f : expf(s[j] - m_new);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) Ps[m * PP + sub + 8 * j] = p[j];
      __syncwarp();
      // the sum of the tile's weights: four neighbouring keys in order, then a tree over the
      // eight groups
      const float4 g4 = *reinterpret_cast<const float4*>(Ps + m * PP + sub * 4);
      float psum = 0.f;
      psum += g4.x;
      psum += g4.y;
      psum += g4.z;
      psum += g4.w;
      psum += __shfl_xor_sync(0xffffffffu, psum, 1);
      psum += __shfl_xor_sync(0xffffffffu, psum, 2);
      psum += __shfl_xor_sync(0xffffffffu, psum, 4);
      l_s = __fmaf_rn(l_s, alpha, psum);
      m_s = m_new;
      if (row_valid) {
#pragma unroll
        for (int jj = 0; jj < MAX_D / 32; ++jj) {
          if (jj < ngroup && sub * 4 + 32 * jj < d) {
            float a0 = __fmul_rn(acc_s[jj * 4 + 0], alpha), a1 = __fmul_rn(acc_s[jj * 4 + 1], alpha);
            float a2 = __fmul_rn(acc_s[jj * 4 + 2], alpha), a3 = __fmul_rn(acc_s[jj * 4 + 3], alpha);
            const float* pr = Ps + m * PP;
            const float* vc = Vs + sub * 4 + 32 * jj;
            for (int n = 0; n < TILE_N; n += 4) {
              const float4 p4 = *reinterpret_cast<const float4*>(pr + n);
              const float pn[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float4 v4 = *reinterpret_cast<const float4*>(vc + (n + e) * d);
                a0 = fmaf(pn[e], v4.x, a0);
                a1 = fmaf(pn[e], v4.y, a1);
                a2 = fmaf(pn[e], v4.z, a2);
                a3 = fmaf(pn[e], v4.w, a3);
              }
            }
            acc_s[jj * 4 + 0] = a0;
            acc_s[jj * 4 + 1] = a1;
            acc_s[jj * 4 + 2] = a2;
            acc_s[jj * 4 + 3] = a3;
          }
        }
      }
      __syncwarp();
    }

    if (slot_base >= 0) {
      // parallel mode: this block covers one split; write the partial
      if (row_valid) {
        const int64_t slot = (int64_t)slot_base + m_tok;
#pragma unroll
        for (int jj = 0; jj < MAX_D / 32; ++jj)
          if (jj < ngroup && sub * 4 + 32 * jj < d)
            *reinterpret_cast<float4*>(part_acc + (slot * nq + h) * d + sub * 4 + 32 * jj) =
                make_float4(acc_s[jj * 4], acc_s[jj * 4 + 1], acc_s[jj * 4 + 2], acc_s[jj * 4 + 3]);
        if (sub == 0) {
          part_ml[(slot * nq + h) * 2 + 0] = m_s;
          part_ml[(slot * nq + h) * 2 + 1] = l_s;
        }
      }
    } else {
      float alpha, beta, m_new;
      ls_fold_scales(m_run, m_s, alpha, beta, m_new);
      if (m_s != -CUDART_INF_F) {
#pragma unroll
        for (int j = 0; j < MAX_D / 8; ++j) acc_run[j] = ls_fold_value(acc_run[j], alpha, acc_s[j], beta);
        l_run = ls_fold_value(l_run, alpha, l_s, beta);
        m_run = m_new;
      }
    }
  }

  if (slot_base < 0 && row_valid) {
    T* o = out + ((int64_t)(tok0 + m_tok) * nq + h) * d;
#pragma unroll
    for (int jj = 0; jj < MAX_D / 32; ++jj)
      if (jj < ngroup && sub * 4 + 32 * jj < d) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          o[sub * 4 + 32 * jj + e] = ls_from_float<T>(l_run > 0.f ? __fdiv_rn(acc_run[jj * 4 + e], l_run) : 0.f);
      }
  }
  }   // heads of this block
}

// --------------------------------------------------------------------------
// decode kernel: one query token, one split, one kv head with its whole group
// of query heads (they share the loaded keys and values).  Writes a partial.
// --------------------------------------------------------------------------
constexpr int DEC_TILE = 64;
constexpr int DEC_ACC = 8;     // outputs per thread: group * d <= 128 * DEC_ACC

template <typename T>
__global__ void __launch_bounds__(128)
attention_decode_kernel(const T* __restrict__ q, const T* __restrict__ pages,
                        float* __restrict__ part_acc, float* __restrict__ part_ml,
                        const int* __restrict__ work, const int* __restrict__ block_table,
                        int table_stride, int nq, int nkv, int d, int page_size, int num_pages,
                        int window, float scale, const float* __restrict__ slopes, int slot_limit, int* err) {
  ls_dependency_sync();
  extern __shared__ __align__(16) unsigned char dsm[];
  constexpr int VEC = 16 / sizeof(T);        // elements per 16-byte chunk
  const int group = nq / nkv;
  const int kstride = d + VEC;               // padded row of K in elements
  T* Ks = reinterpret_cast<T*>(dsm);                       // [DEC_TILE][d+VEC]
  T* Vs = Ks + DEC_TILE * kstride;                         // [DEC_TILE][d]
  float* Qs = reinterpret_cast<float*>(Vs + DEC_TILE * d); // [group][d]
  float* Ss = Qs + group * d;                              // [group][DEC_TILE]
  float* St = Ss + group * DEC_TILE;                       // [group][3]: m, l, alpha

  const int* w = work + (int64_t)blockIdx.x * 8;
  if (w[2] == 0) return;                     // padding item of a recorded launch
  const int req_row = w[0], tok = w[1], pos = w[3], split = w[4], slot = w[6];
  // slot_limit > 0: the partials live in an array of that many slots that this kernel does not
  // own (the fixed scratch of the entry point that allocates nothing): a work item that names
  // a slot outside it is recorded and skipped, not written
  if (slot_limit > 0 && (slot < 0 || slot >= slot_limit)) {
    if (threadIdx.x == 0) ls_record_fault(err, LS_DEV_ROW_RANGE, slot);
    return;
  }
  const int kvh = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* table_row = block_table + (int64_t)req_row * table_stride;

  const int row_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int s_lo = split * LS_SPLIT;
  int s_hi = s_lo + LS_SPLIT;
  if (s_hi > pos + 1) s_hi = pos + 1;

  for (int i = tid; i < group * d; i += 128) {
    const int g = i / d, c = i - g * d;
    Qs[i] = ls_to_float<T>(q[((int64_t)tok * nq + kvh * group + g) * d + c]);
  }
  for (int g = tid; g < group; g += 128) {
    St[g * 3 + 0] = -CUDART_INF_F;
    St[g * 3 + 1] = 0.f;
    St[g * 3 + 2] = 1.f;
  }
  float acc[DEC_ACC];
#pragma unroll
  for (int j = 0; j < DEC_ACC; ++j) acc[j] = 0.f;

  const int cpr = d / VEC;                   // 16-byte chunks per row
  int t_first = s_lo;
  if (row_lo > s_lo) t_first = s_lo + ((row_lo - s_lo) / DEC_TILE) * DEC_TILE;

  for (int n0 = t_first; n0 < s_hi; n0 += DEC_TILE) {
    __syncthreads();
    for (int i = tid; i < DEC_TILE * cpr; i += 128) {
      const int n = i / cpr, c = i - n * cpr;
      const int key = n0 + n;
      uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
      if (key < s_hi && key >= row_lo) {
        const T* kp = page_ptr<T>(pages, table_row, key, 0, kvh, nkv, page_size, d, num_pages, err);
        if (kp != nullptr) {
          kv = *reinterpret_cast<const uint4*>(kp + c * VEC);
          vv = *reinterpret_cast<const uint4*>(kp + (int64_t)nkv * page_size * d + c * VEC);
        }
      }
      *reinterpret_cast<uint4*>(Ks + n * kstride + c * VEC) = kv;
      *reinterpret_cast<uint4*>(Vs + n * d + c * VEC) = vv;
    }
    __syncthreads();

    for (int u = tid; u < group * DEC_TILE; u += 128) {
      const int g = u / DEC_TILE, n = u - g * DEC_TILE;
      const int key = n0 + n;
      const T* kr = Ks + n * kstride;
      const float* qr = Qs + g * d;
      float dot = 0.f;
      for (int c = 0; c < d; c += VEC) {
        const uint4 raw = *reinterpret_cast<const uint4*>(kr + c);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int x = 0; x < VEC; ++x) dot = fmaf(qr[c + x], ls_to_float<T>(e[x]), dot);
      }
      const bool keep = key < s_hi && key >= row_lo;
      Ss[u] = !keep ? -CUDART_INF_F
              : slopes != nullptr ? fmaf(slopes[kvh * group + g], (float)(key - pos), dot * scale) : dot * scale;
    }
    __syncthreads();

    for (int g = warp; g < group; g += 4) {
      const float s0 = Ss[g * DEC_TILE + lane], s1 = Ss[g * DEC_TILE + lane + 32];
      const float tile_max = ls_warp_max(fmaxf(s0, s1));
      const float m_old = St[g * 3 + 0];
      const float m_new = fmaxf(m_old, tile_max);
      float alpha = 1.f, p0 = 0.f, p1 = 0.f;
      if (m_new != -CUDART_INF_F) {
        alpha = (m_old == -CUDART_INF_F) ? 0.f : expf(m_old - m_new);
        p0 = (s0 == -CUDART_INF_F) ? 0.f : expf(s0 - m_new);
        p1 = (s1 == -CUDART_INF_F) ? 0.f : expf(s1 - m_new);
      }
      const float psum = ls_warp_sum(p0 + p1);
      Ss[g * DEC_TILE + lane] = p0;
      Ss[g * DEC_TILE + lane + 32] = p1;
      if (lane == 0) {
        St[g * 3 + 0] = m_new;
        St[g * 3 + 1] = fmaf(St[g * 3 + 1], alpha, psum);
        St[g * 3 + 2] = alpha;
      }
    }
    __syncthreads();

#pragma unroll
    for (int j = 0; j < DEC_ACC; ++j) {
      const int u = tid + 128 * j;
      if (u < group * d) {
        const int g = u / d, c = u - g * d;
        float a = acc[j] * St[g * 3 + 2];
        const float* pr = Ss + g * DEC_TILE;
        const T* vc = Vs + c;
        for (int n = 0; n < DEC_TILE; ++n) a = fmaf(pr[n], ls_to_float<T>(vc[n * d]), a);
        acc[j] = a;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < DEC_ACC; ++j) {
    const int u = tid + 128 * j;
    if (u < group * d) {
      const int g = u / d, c = u - g * d;
      part_acc[((int64_t)slot * nq + kvh * group + g) * d + c] = acc[j];
    }
  }
  for (int g = tid; g < group; g += 128) {
    part_ml[((int64_t)slot * nq + kvh * group + g) * 2 + 0] = St[g * 3 + 0];
    part_ml[((int64_t)slot * nq + kvh * group + g) * 2 + 1] = St[g * 3 + 1];
  }
}

// --------------------------------------------------------------------------
// combine: fold the partials of a row in ascending split order
// combine item (4 ints): token (packed index), first slot, slot stride, splits
// --------------------------------------------------------------------------
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part_acc,
                                         const float* __restrict__ part_ml, T* __restrict__ out,
                                         const int* __restrict__ items, int nq, int d, int slot_limit,
                                         int* err) {
  ls_dependency_sync();
  const int* it = items + (int64_t)blockIdx.x * 4;
  const int tok = it[0], first = it[1], stride = it[2], n = it[3];
  if (n == 0) return;                        // padding item of a recorded launch
  if (slot_limit > 0) {                      // see attention_decode_kernel
    const long long last = (long long)first + (long long)stride * (n - 1);
    if (first < 0 || first >= slot_limit || last < 0 || last >= slot_limit) {
      if (threadIdx.x == 0) ls_record_fault(err, LS_DEV_ROW_RANGE, first);
      return;
    }
  }
  const int h = blockIdx.y;
  for (int c = threadIdx.x; c < d; c += blockDim.x)
    out[((int64_t)tok * nq + h) * d + c] = ls_from_float<T>(ls_fold_row(part_acc, part_ml, first, stride, n, nq, h, d, c));
}

size_t tile_smem_bytes(int d) {
  return sizeof(float) * ((size_t)TILE_M * (d + 4) + (size_t)TILE_N * (d + 4) + (size_t)TILE_N * d +
                          (size_t)TILE_M * (TILE_N + 4));
}

size_t decode_smem_bytes(int d, int group, int elem) {
  const int vec = 16 / elem;
  return (size_t)elem * ((size_t)DEC_TILE * (d + vec) + (size_t)DEC_TILE * d) +
         sizeof(float) * ((size_t)group * d + (size_t)group * DEC_TILE + (size_t)group * 3);
}

bool shape_ok(int nq, int nkv, int d, int page_size, int tile) {
  return nq > 0 && nkv > 0 && nq % nkv == 0 && d >= 16 && d <= MAX_D && d % 16 == 0 &&
         page_size > 0 && tile % page_size == 0;
}

}  // namespace

LS_API int ls_attention_split_size() { return LS_SPLIT; }

LS_API int ls_attention_tile(const void* q, const void* pages, void* out, float* part_acc,
                             float* part_ml, int dtype, const int* work, int n_work,
                             const int* block_table, int table_stride, int nq, int nkv, int d,
                             int page_size, int num_pages, int window, float scale,
                             const float* slopes, int* err, cudaStream_t stream) {
  if (n_work <= 0) return 0;
  if (!shape_ok(nq, nkv, d, page_size, LS_SPLIT)) return LS_E_SIZE;
  if (nq > 65535) return LS_E_SIZE;
  if ((uintptr_t)pages & 15) return LS_E_ALIGN;      // keys and values are read 16 bytes at a time
  const size_t smem = tile_smem_bytes(d);
  // split partials (decoded tokens: one row an item): the heads of a key head share a block,
  // as many of them as divide the group and fit the tile's rows
  int hb = 1;
  if (part_acc != nullptr)
    for (int c = 2; c <= TILE_M && c <= nq / nkv; ++c)
      if ((nq / nkv) % c == 0) hb = c;
  dim3 grid(n_work, nq / hb);
  cudaError_t e;
  static size_t set_f32 = 0, set_bf16 = 0;     // largest size configured so far
  if (dtype == LS_F32) {
    e = smem <= set_f32 ? cudaSuccess
                        : cudaFuncSetAttribute(attention_tile_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return LS_E_SMEM;
    if (smem > set_f32) set_f32 = smem;
    LS_COUNT(LS_K_ATTENTION_TILE), ls_launch(attention_tile_kernel<float>, grid, 128, smem, stream, 
        (const float*)q, (const float*)pages, (float*)out, part_acc, part_ml, work, block_table,
        table_stride, nq, nkv, d, page_size, num_pages, window, scale, slopes, hb, err);
  } else if (dtype == LS_BF16) {
    e = smem <= set_bf16 ? cudaSuccess
                         : cudaFuncSetAttribute(attention_tile_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return LS_E_SMEM;
    if (smem > set_bf16) set_bf16 = smem;
    LS_COUNT(LS_K_ATTENTION_TILE), ls_launch(attention_tile_kernel<__nv_bfloat16>, grid, 128, smem, stream, 
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)pages, (__nv_bfloat16*)out, part_acc,
        part_ml, work, block_table, table_stride, nq, nkv, d, page_size, num_pages, window, scale,
        slopes, hb, err);
  } else {
    return LS_E_DTYPE;
  }
  return ls_launch_status();
}

namespace {

// slot_limit: 0, or the number of slots the partial arrays hold (checked on the device)
int launch_attention_decode(const void* q, const void* pages, float* part_acc, float* part_ml,
                            int dtype, const int* work, int n_work, const int* block_table,
                            int table_stride, int nq, int nkv, int d, int page_size,
                            int num_pages, int window, float scale, const float* slopes, int slot_limit,
                            int* err, cudaStream_t stream) {
  if (n_work <= 0) return 0;
  if (!shape_ok(nq, nkv, d, page_size, DEC_TILE)) return LS_E_SIZE;
  const int group = nq / nkv;
  if (group * d > 128 * DEC_ACC || nkv > 65535) return LS_E_SIZE;
  dim3 grid(n_work, nkv);
  cudaError_t e;
  static size_t set_f32 = 0, set_bf16 = 0;     // largest size configured so far
  if (dtype == LS_F32) {
    const size_t smem = decode_smem_bytes(d, group, 4);
    e = smem <= set_f32 ? cudaSuccess
                        : cudaFuncSetAttribute(attention_decode_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return LS_E_SMEM;
    if (smem > set_f32) set_f32 = smem;
    LS_COUNT(LS_K_ATTENTION_DECODE), ls_launch(attention_decode_kernel<float>, grid, 128, smem, stream, 
        (const float*)q, (const float*)pages, part_acc, part_ml, work, block_table, table_stride,
        nq, nkv, d, page_size, num_pages, window, scale, slopes, slot_limit, err);
  } else if (dtype == LS_BF16) {
    const size_t smem = decode_smem_bytes(d, group, 2);
    e = smem <= set_bf16 ? cudaSuccess
                         : cudaFuncSetAttribute(attention_decode_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return LS_E_SMEM;
    if (smem > set_bf16) set_bf16 = smem;
    LS_COUNT(LS_K_ATTENTION_DECODE), ls_launch(attention_decode_kernel<__nv_bfloat16>, grid, 128, smem, stream, 
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)pages, part_acc, part_ml, work,
        block_table, table_stride, nq, nkv, d, page_size, num_pages, window, scale, slopes, slot_limit, err);
  } else {
    return LS_E_DTYPE;
  }
  return ls_launch_status();
}

int launch_attention_combine(const float* part_acc, const float* part_ml, void* out, int dtype,
                             const int* items, int n_items, int nq, int d, int slot_limit, int* err,
                             cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (nq > 65535) return LS_E_SIZE;
  dim3 grid(n_items, nq);
  const int threads = d >= 128 ? 128 : (d >= 64 ? 64 : 32);
  if (dtype == LS_F32)
    LS_COUNT(LS_K_ATTENTION_COMBINE), ls_launch(attention_combine_kernel<float>, grid, threads, 0, stream, part_acc, part_ml, (float*)out, items, nq, d, slot_limit, err);
  else if (dtype == LS_BF16)
    LS_COUNT(LS_K_ATTENTION_COMBINE), ls_launch(attention_combine_kernel<__nv_bfloat16>, grid, threads, 0, stream, part_acc, part_ml, (__nv_bfloat16*)out, items, nq, d, slot_limit, err);
  else
    return LS_E_DTYPE;
  return ls_launch_status();
}

}  // namespace

// Returns LS_E_SIZE for shapes it does not take (group * d > 1024); the caller
// then uses ls_attention_tile in parallel mode, which takes them all.
LS_API int ls_attention_decode(const void* q, const void* pages, float* part_acc, float* part_ml,
                               int dtype, const int* work, int n_work, const int* block_table,
                               int table_stride, int nq, int nkv, int d, int page_size,
                               int num_pages, int window, float scale, const float* slopes, int* err,
                               cudaStream_t stream) {
  return launch_attention_decode(q, pages, part_acc, part_ml, dtype, work, n_work, block_table, table_stride, nq,
                                 nkv, d, page_size, num_pages, window, scale, slopes, 0, err, stream);
}

LS_API int ls_attention_combine(const float* part_acc, const float* part_ml, void* out, int dtype,
                                const int* items, int n_items, int nq, int d,
                                cudaStream_t stream) {
  return launch_attention_combine(part_acc, part_ml, out, dtype, items, n_items, nq, d, 0, nullptr, stream);
}

// --------------------------------------------------------------------------
// The entry point that allocates nothing (see no_alloc.h).
// --------------------------------------------------------------------------
#include <mutex>

#include "no_alloc.h"

namespace {

// Partial results of ls_attention_decode_noalloc.  In host code this name is
// only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float ls_noalloc_scratch[LS_NOALLOC_SCRATCH_FLOATS];

constexpr int NOALLOC_MAX_DEVICES = 64;
float* noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
std::mutex noalloc_mutex;

// Device address of the scratch on the current device, looked up once per device.
int noalloc_scratch(float** ptr) {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= NOALLOC_MAX_DEVICES)
    return LS_E_NOALLOC_SETUP;
  std::lock_guard<std::mutex> guard(noalloc_mutex);
  if (noalloc_ptr[device] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, ls_noalloc_scratch) != cudaSuccess || p == nullptr)
      return LS_E_NOALLOC_SETUP;
    noalloc_ptr[device] = p;
  }
  *ptr = noalloc_ptr[device];
  return 0;
}

}  // namespace

LS_API int ls_attention_decode_noalloc(const void* q, const void* pages, void* out, int dtype,
                                       const int* work, int n_work, const int* combine,
                                       int n_combine, int n_slots, const int* block_table,
                                       int table_stride, int nq, int nkv, int d, int page_size,
                                       int num_pages, int window, float scale, int* err,
                                       cudaStream_t stream) {
  if (n_work <= 0 || n_combine <= 0) return 0;
  if (n_slots <= 0 || nq <= 0 || d <= 0) return LS_E_SIZE;
  const long long need = (long long)n_slots * nq * (d + 2);
  if (need > (long long)LS_NOALLOC_SCRATCH_FLOATS) return LS_E_NOALLOC_TOO_LARGE;
  float* scratch = nullptr;
  const int setup = noalloc_scratch(&scratch);
  if (setup != 0) return setup;
  float* part_acc = scratch;                                   // [n_slots, nq, d]
  float* part_ml = scratch + (size_t)n_slots * nq * d;         // [n_slots, nq, 2]
  // the kernels check every slot a work item names against n_slots: a wrong item is recorded
  // in the error word (LS_DEV_ROW_RANGE) and skipped, it cannot write outside the array
  const int status = launch_attention_decode(q, pages, part_acc, part_ml, dtype, work, n_work,
                                             block_table, table_stride, nq, nkv, d, page_size,
                                             num_pages, window, scale, nullptr, n_slots, err, stream);
  if (status != 0) return status;
  return launch_attention_combine(part_acc, part_ml, out, dtype, combine, n_combine, nq, d, n_slots, err, stream);
}

LS_API const char* ls_constants_attention_simt() {
  static char buf[256];
  static const LsConstant c[] = {{"attention.split_keys", LS_SPLIT}, {"attention_tile.queries", TILE_M},
                                 {"attention_tile.keys", TILE_N}, {"attention_decode.keys", DEC_TILE},
                                 {"attention.max_head_dim", MAX_D}};
  return ls_format_constants(buf, sizeof buf, c, (int)(sizeof c / sizeof c[0]));
}

// launches of this library's kernels so far, in the order of LS_KERNEL_NAMES
LS_API const char* ls_kernel_names_core() { return LS_KERNEL_NAMES; }
LS_API int ls_kernel_launches_core(unsigned long long* out, int n) {
  for (int i = 0; i < n && i < LS_K_COUNT; ++i) out[i] = ls_kernel_launches[i];
  return LS_K_COUNT;
}
