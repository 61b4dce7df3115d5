// The fold of attention partials (acc, m, l) of consecutive key ranges, shared by
// every kernel that folds, so that all of them produce the same bits.
#pragma once

#include <math_constants.h>

#include "common.cuh"

// scales of the running and the new partial for the fold  run <- run * alpha + part * beta
__device__ __forceinline__ void ls_fold_scales(float m_run, float m_s, float& alpha, float& beta,
                                               float& m_new) {
  m_new = fmaxf(m_run, m_s);
  alpha = (m_run == -CUDART_INF_F) ? 0.f : expf(m_run - m_new);
  beta = (m_s == -CUDART_INF_F) ? 0.f : expf(m_s - m_new);
}

__device__ __forceinline__ float ls_fold_value(float run, float alpha, float part, float beta) {
  return __fmaf_rn(part, beta, __fmul_rn(run, alpha));
}

// Element c of head h of a row whose partials lie in slots first, first + stride, ...
// (n of them), folded in ascending order; the partials of eight splits are fetched
// together (independent loads) before they are folded one after the other.
__device__ __forceinline__ float ls_fold_row(const float* __restrict__ part_acc,
                                             const float* __restrict__ part_ml, int64_t first,
                                             int64_t stride, int n, int nq, int h, int d, int c) {
  float acc = 0.f, m_run = -CUDART_INF_F, l_run = 0.f;
  for (int s0 = 0; s0 < n; s0 += 8) {
    float m_s[8], l_s[8], a_s[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (s0 + j < n) {
        const int64_t slot = first + (int64_t)(s0 + j) * stride;
        m_s[j] = part_ml[(slot * nq + h) * 2 + 0];
        l_s[j] = part_ml[(slot * nq + h) * 2 + 1];
        a_s[j] = part_acc[(slot * nq + h) * d + c];
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (s0 + j < n) {
        float alpha, beta, m_new;
        ls_fold_scales(m_run, m_s[j], alpha, beta, m_new);
        if (m_s[j] != -CUDART_INF_F) {
          acc = ls_fold_value(acc, alpha, a_s[j], beta);
          l_run = ls_fold_value(l_run, alpha, l_s[j], beta);
          m_run = m_new;
        }
      }
    }
  }
  return l_run > 0.f ? __fdiv_rn(acc, l_run) : 0.f;
}
