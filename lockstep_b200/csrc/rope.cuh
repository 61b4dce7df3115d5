// Per-head RMSNorm (optional) and rotary position encoding of one head by one
// warp, shared by every kernel that does it, so that all of them produce the
// same bits.  Half rotation: out[i] = x[i] c_i - x[i+h] s_i, out[i+h] = x[i+h] c_i
// + x[i] s_i for i < h = rot_dim / 2; dimensions past rot_dim are only normed.
// Products and sums are rounded one by one (no fused multiply-add), so the
// result does not depend on how a compiler contracts the expression.
#pragma once

#include "common.cuh"

// store(i, value) receives every element of the head exactly once.
template <typename T, typename TG, typename Store>
__device__ __forceinline__ void ls_norm_rope_head(const T* __restrict__ src, const TG* __restrict__ gain,
                                                  const float* __restrict__ cs, const float* __restrict__ sn,
                                                  int d, int rot_dim, float eps, int lane, Store store) {
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
    float lo = __fmul_rn(ls_to_float<T>(src[i]), rstd);
    float hi = __fmul_rn(ls_to_float<T>(src[i + half]), rstd);
    if (gain != nullptr) {
      lo = __fmul_rn(lo, ls_to_float<TG>(gain[i]));
      hi = __fmul_rn(hi, ls_to_float<TG>(gain[i + half]));
    }
    const float c = cs[i], s = sn[i];
    store(i, __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, s)));
    store(i + half, __fadd_rn(__fmul_rn(hi, c), __fmul_rn(lo, s)));
  }
  for (int i = rot_dim + lane; i < d; i += 32) {
    float v = __fmul_rn(ls_to_float<T>(src[i]), rstd);
    if (gain != nullptr) v = __fmul_rn(v, ls_to_float<TG>(gain[i]));
    store(i, v);
  }
}
