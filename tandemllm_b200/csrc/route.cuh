// The router's choice for one row, run by one full warp: scores (the sigmoid of each logit, or the softmax over all
// experts' logits), the top-k of score + bias (the bias for the choice only), weights = chosen scores, divided by
// (their sum + floor) when normalised, times scale.
// Ties go to the lower expert id; a NaN score is chosen only when nothing else is left.
// (engine/models/lfm2_moe/ref.py:185-197, engine/models/lfm2_moe/kernels.py:265-287 of the reference; the softmax
// scoring is what its other routed families use, engine/models/flashnext/ref.py:479-487)
//
// The launchers' `normalize` argument carries both choices: bit 0 = divide the chosen weights by their sum,
// bits 1.. = the scoring function (TL_SCORE_SIGMOID 0, TL_SCORE_SOFTMAX 1).
#pragma once

#include "common.cuh"

namespace tl {

#define TL_SCORE_SIGMOID 0
#define TL_SCORE_SOFTMAX 1
#define TL_SCORE_LAST 1

constexpr int MAX_EXPERTS = 1024;
constexpr int MAX_TOP_K = 32;

// `lg`: the row's E <= 32 PER logits (global or shared memory). Lanes 0..k-1 write ids[lane] and wts[lane], in the
// order of the choice (best first). PER: experts a lane holds.
template <int PER>
__device__ __forceinline__ void warp_route_sized(const float* lg, const float* __restrict__ bias, int E, int k,
                                                 int normalize, float floor_, float scale, int* ids, float* wts) {
  const int lane = threadIdx.x & 31;
  const int scoring = normalize >> 1;
  normalize &= 1;
  float score[PER], choice[PER];
  float top = -INFINITY, denom = 1.f;
  if (scoring == TL_SCORE_SOFTMAX) {        // the row's largest logit and the sum of exponentials, over the whole warp
#pragma unroll
    for (int t = 0; t < PER; ++t)
      if (lane + 32 * t < E) top = fmaxf(top, lg[lane + 32 * t]);
    top = warp_max(top);
    float part = 0.f;
#pragma unroll
    for (int t = 0; t < PER; ++t)
      if (lane + 32 * t < E) part += expf(lg[lane + 32 * t] - top);
    denom = warp_sum(part);
  }
#pragma unroll
  for (int t = 0; t < PER; ++t) {
    const int e = lane + 32 * t;
    if (e < E) {
      const float s = scoring == TL_SCORE_SOFTMAX ? expf(lg[e] - top) / denom : 1.f / (1.f + expf(-lg[e]));
      score[t] = s;
      choice[t] = bias ? s + bias[e] : s;
      if (!(choice[t] == choice[t])) choice[t] = -INFINITY;
    } else {
      score[t] = 0.f;
      choice[t] = -INFINITY;
    }
  }
  float sum = 0.f, my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    float best_s = 0.f;
#pragma unroll
    for (int t = 0; t < PER; ++t) {
      const int e = lane + 32 * t;
      if (e < E && choice[t] != -INFINITY && (choice[t] > best || (choice[t] == best && e < best_e))) {
        best = choice[t];
        best_e = e;
        best_s = score[t];
      }
    }
    if (best_e == 0x7fffffff) {     // nothing but -inf left in this lane: offer its lowest untaken id
#pragma unroll
      for (int t = 0; t < PER; ++t) {
        const int e = lane + 32 * t;
        if (e < E && score[t] != -1.f && e < best_e) {
          best_e = e;
          best_s = score[t];
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
        best_s = os;
      }
    }
    if ((best_e & 31) == lane) {    // the owner retires the winner
#pragma unroll
      for (int t = 0; t < PER; ++t)
        if (lane + 32 * t == best_e) {
          choice[t] = -INFINITY;
          score[t] = -1.f;
        }
    }
    sum += best_s;
    if (lane == j) {
      my_id = best_e;
      my_w = best_s;
    }
  }
  if (lane < k) {
    float w = my_w;
    if (normalize) w = w / (sum + floor_);
    ids[lane] = my_id;
    wts[lane] = w * scale;
  }
}

__device__ __forceinline__ void warp_route(const float* lg, const float* __restrict__ bias, int E, int k, int normalize,
                                           float floor_, float scale, int* ids, float* wts) {
  if (E <= 32) warp_route_sized<1>(lg, bias, E, k, normalize, floor_, scale, ids, wts);
  else if (E <= 128) warp_route_sized<4>(lg, bias, E, k, normalize, floor_, scale, ids, wts);
  else warp_route_sized<MAX_EXPERTS / 32>(lg, bias, E, k, normalize, floor_, scale, ids, wts);
}

}  // namespace tl
