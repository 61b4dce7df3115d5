// Per-head RMSNorm (optional) and rotary position encoding of one head by one
// warp, shared by every kernel that does it, so that all of them produce the
// same bits.  Pair i < h = rot_dim / 2 of a head is (x[i], x[i+h]) in the half layout and
// (x[2i], x[2i+1]) in the interleaved one; with (lo, hi) the pair, out_lo = lo c_i - hi s_i
// and out_hi = hi c_i + lo s_i, written back where they came from.  Dimensions past
// rot_dim are only normed.
// Products and sums are rounded one by one (no fused multiply-add), so the
// result does not depend on how a compiler contracts the expression.
#pragma once

#include "common.cuh"

// store(i, value) receives every element of the head exactly once.
template <typename T, typename TG, typename Store>
__device__ __forceinline__ void ls_norm_rope_head(const T* __restrict__ src, const TG* __restrict__ gain,
                                                  const float* __restrict__ cs, const float* __restrict__ sn,
                                                  int d, int rot_dim, float eps, int lane, Store store,
                                                  bool interleaved = false) {
  float rstd = 1.f;
  if (gain != nullptr) {
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float v = ls_to_float<T>(src[i]);
      ss = fmaf(v, v, ss);
    }
    ss = ls_warp_sum(ss);
    rstd = 1.0f / sqrtf(ss / (float)d + eps);
  }
  const int half = rot_dim >> 1;
  for (int i = lane; i < half; i += 32) {
    const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
    float lo = __fmul_rn(ls_to_float<T>(src[a]), rstd);
    float hi = __fmul_rn(ls_to_float<T>(src[b]), rstd);
    if (gain != nullptr) {
      lo = __fmul_rn(lo, ls_to_float<TG>(gain[a]));
      hi = __fmul_rn(hi, ls_to_float<TG>(gain[b]));
    }
    const float c = cs[i], s = sn[i];
    store(a, __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, s)));
    store(b, __fadd_rn(__fmul_rn(hi, c), __fmul_rn(lo, s)));
  }
  for (int i = rot_dim + lane; i < d; i += 32) {
    float v = __fmul_rn(ls_to_float<T>(src[i]), rstd);
    if (gain != nullptr) v = __fmul_rn(v, ls_to_float<TG>(gain[i]));
    store(i, v);
  }
}

// Where the heads of a q/k/v projection go, shared by the kernel that reads the projection
// from memory and the product that makes it in its epilogue.
//   q_out: [tokens, nq * d];  pages: [num_pages, 2, nkv, page_size, d], one layer of one group.
// The page of token t is block_table[token_req[t] * table_stride + positions[t] / page_size].
struct LsQkvStore {
  void* q_out;
  void* pages;
  const void* q_gain;       // [d] each, or both null: no per-head norm
  const void* k_gain;
  const float* cos_table;   // [max_positions, rot_dim / 2]
  const float* sin_table;
  const int* positions;
  const int* token_req;
  const int* block_table;
  int gain_bf16;            // element type of the gains: 1 bfloat16, 0 float32
  int table_stride, nq, nkv, d, rot_dim, page_size, num_pages, max_positions, write_cache;
  float eps;
  int interleaved;          // 1: a rotated pair is two neighbouring elements; 0: halves of the rotated part
};

// Where head `head` (q heads, then k heads, then v heads) of token t goes.  It depends on the
// step's inputs alone (positions, block table), so a kernel may work it out before the values
// of the head exist.
struct LsHeadTarget {
  void* dst;        // null: nothing to write (v or k of a layer that does not write its cache, or a fault)
  int pos;
  int kind;         // 0 q, 1 k, 2 v
};

__device__ __forceinline__ LsHeadTarget ls_qkv_head_target(const LsQkvStore& a, int t, int head, int elem_bytes,
                                                           int lane, int* err) {
  LsHeadTarget target;
  target.kind = head < a.nq ? 0 : (head < a.nq + a.nkv ? 1 : 2);
  target.dst = nullptr;
  target.pos = 0;
  if (target.kind != 0 && !a.write_cache) return target;
  const int pos = a.positions[t];
  target.pos = pos;
  int64_t offset;
  char* base;
  if (target.kind == 0) {
    base = reinterpret_cast<char*>(a.q_out);
    offset = ((int64_t)t * a.nq + head) * a.d;
  } else {
    const int kvh = target.kind == 1 ? head - a.nq : head - a.nq - a.nkv;
    const int row = a.token_req[t];
    const int page = a.block_table[(int64_t)row * a.table_stride + pos / a.page_size];
    if (page < 0 || page >= a.num_pages) {
      if (lane == 0) ls_record_fault(err, LS_DEV_PAGE_RANGE, t);
      return target;
    }
    base = reinterpret_cast<char*>(a.pages);
    offset = ((((int64_t)page * 2 + (target.kind == 1 ? 0 : 1)) * a.nkv + kvh) * a.page_size + (pos % a.page_size)) * a.d;
  }
  if (target.kind != 2 && (a.rot_dim >> 1) > 0 && (pos < 0 || pos >= a.max_positions)) {
    if (lane == 0) ls_record_fault(err, LS_DEV_POSITION_RANGE, t);
    return target;
  }
  target.dst = base + offset * elem_bytes;
  return target;
}

// The head's values src[0 .. d) written to their target by one warp: q normed and rotated,
// k normed and rotated, v copied.
template <typename T, typename TG>
__device__ __forceinline__ void ls_qkv_head_write_as(const LsQkvStore& a, const T* src, const LsHeadTarget& target,
                                                     int lane) {
  if (target.dst == nullptr) return;
  T* dst = reinterpret_cast<T*>(target.dst);
  const int d = a.d;
  if (target.kind == 2) {
    for (int i = lane; i < d; i += 32) dst[i] = src[i];
    return;
  }
  const TG* gain = reinterpret_cast<const TG*>(target.kind == 0 ? a.q_gain : a.k_gain);
  const int half = a.rot_dim >> 1;
  ls_norm_rope_head<T, TG>(src, gain, a.cos_table + (int64_t)target.pos * half,
                           a.sin_table + (int64_t)target.pos * half, d, a.rot_dim, a.eps, lane,
                           [&](int i, float v) { dst[i] = ls_from_float<T>(v); }, a.interleaved != 0);
}

template <typename T>
__device__ __forceinline__ void ls_qkv_head_write(const LsQkvStore& a, const T* src, const LsHeadTarget& target,
                                                  int lane) {
  if (a.gain_bf16) ls_qkv_head_write_as<T, __nv_bfloat16>(a, src, target, lane);
  else ls_qkv_head_write_as<T, float>(a, src, target, lane);
}

template <typename T>
__device__ __forceinline__ void ls_qkv_head_store(const LsQkvStore& a, const T* src, int t, int head, int lane,
                                                  int* err) {
  ls_qkv_head_write<T>(a, src, ls_qkv_head_target(a, t, head, (int)sizeof(T), lane, err), lane);
}
