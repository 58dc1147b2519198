// Scoring and (grouped) top-k selection of one token's gate logits by one warp; shared by the router kernels and the
// fused decode chain.
#pragma once
#include "api.h"
#include "common.cuh"

namespace mmb {

constexpr int kMaxExperts = 512;

// Scoring + (grouped) top-k of one token by one warp; `logit_s` holds the E gate logits on entry.
__device__ __forceinline__ void router_select(const MmbRouterParams& p, long long tk, float* logit_s, float* choice_s, float* group_s, int lane) {
  float mx = -INFINITY;
  for (int e = lane; e < p.E; e += 32) mx = fmaxf(mx, logit_s[e]);
  mx = warp_max(mx);
  if (p.scoring == 0) {
    float z = 0.f;
    for (int e = lane; e < p.E; e += 32) z += __expf(logit_s[e] - mx);
    z = warp_sum(z);
    for (int e = lane; e < p.E; e += 32) {
      const float pr = __expf(logit_s[e] - mx) / z;
      logit_s[e] = pr;       // weight source
      choice_s[e] = pr;      // selection score
    }
  } else {
    for (int e = lane; e < p.E; e += 32) {
      const float sg = 1.f / (1.f + __expf(-logit_s[e]));
      logit_s[e] = sg;
      choice_s[e] = sg + (p.bias ? p.bias[e] : 0.f);
    }
  }
  __syncwarp();
  // ---- grouped top-k: keep the topk_group groups with the largest (sum of top-2 choice scores)
  if (p.n_group > 1 && p.topk_group < p.n_group) {
    const int per = p.E / p.n_group;
    for (int gi = lane; gi < p.n_group; gi += 32) {
      float a = -INFINITY, b = -INFINITY;
      for (int j = 0; j < per; ++j) {
        const float v = choice_s[gi * per + j];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      group_s[gi] = a + b;
    }
    __syncwarp();
    for (int gi = lane; gi < p.n_group; gi += 32) {
      int rank = 0;
      const float v = group_s[gi];
      for (int j = 0; j < p.n_group; ++j) {
        const float u = group_s[j];
        rank += (u > v) || (u == v && j < gi);
      }
      if (rank >= p.topk_group)
        for (int j = 0; j < per; ++j) choice_s[gi * per + j] = -INFINITY;
    }
    __syncwarp();
  }
  // ---- iterative arg-max top-k (ties -> lowest index)
  float wsum = 0.f;
  float myw = 0.f;
  int myid = -1;
  for (int i = 0; i < p.topk; ++i) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < p.E; e += 32) {
      const float v = choice_s[e];
      if (v > bv) { bv = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi >= p.E) bi = 0;                  // all -inf (cannot happen with finite logits)
    const float w = logit_s[bi];
    wsum += w;
    if (lane == i) { myw = w; myid = bi; }
    if (lane == 0) choice_s[bi] = -INFINITY;
    __syncwarp();
  }
  if (lane < p.topk) {
    float w = myw;
    if (p.renorm) w = w / (wsum + 1e-20f);
    w *= p.routed_scale;
    p.ids[tk * p.topk + lane] = myid;
    p.weights[tk * p.topk + lane] = w;
    if (p.counts) atomicAdd(p.counts + myid, 1);
  }
}


}  // namespace mmb
