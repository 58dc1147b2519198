// MoE router: (residual add + RMSNorm) -> gate GEMV -> scoring -> (grouped) top-k -> renormalise,
// one CTA per token, everything on device so the expert kernels never wait for the host.
// Scoring 0: softmax over experts, top-k of the probabilities, optional renormalisation
// (Mixtral / Qwen3-MoE and the reference's MMFP4 layers).  Scoring 1: sigmoid scores, the choice
// uses score + e_score_correction_bias with grouped top-k, the weights use the unbiased scores
// (DeepSeek-V3 / GLM-4.x).
#include "api.h"
#include "common.cuh"

namespace mmb {

constexpr int kMaxExperts = 512;

__global__ void __launch_bounds__(256) moe_router_kernel(const MmbRouterParams p) {
  extern __shared__ float xs[];            // [K]
  __shared__ float red[32];
  __shared__ float logit_s[kMaxExperts];
  __shared__ float choice_s[kMaxExperts];
  __shared__ float group_s[64];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long tk = blockIdx.x;
  const bf16* x = reinterpret_cast<const bf16*>(p.x) + tk * p.K;
  const bf16* d = p.delta ? reinterpret_cast<const bf16*>(p.delta) + tk * p.K : nullptr;
  const bf16* nw = reinterpret_cast<const bf16*>(p.norm_w);
  bf16* ro = p.resid_out ? reinterpret_cast<bf16*>(p.resid_out) + tk * p.K : nullptr;
  float ss = 0.f;
  for (int k = tid; k < p.K; k += 256) {
    float v = __bfloat162float(x[k]);
    if (d) {
      const bf16 s = __float2bfloat16(v + __bfloat162float(d[k]));
      v = __bfloat162float(s);
      if (ro) ro[k] = s;
    }
    xs[k] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  if (nw) {
    const float rs = rsqrtf(ss / (float)p.K + p.eps);
    for (int k = tid; k < p.K; k += 256) xs[k] = __bfloat162float(__float2bfloat16(xs[k] * rs * __bfloat162float(nw[k])));
  }
  __syncthreads();
  const bf16* W = reinterpret_cast<const bf16*>(p.w);
  for (int e = warp; e < p.E; e += 8) {
    const bf16* wr = W + (long long)e * p.K;
    float acc = 0.f;
    for (int k = lane * 8; k < p.K; k += 256) {
      const uint4 wv = *reinterpret_cast<const uint4*>(wr + k);
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc = fmaf(__uint_as_float(ww[j] << 16), xs[k + 2 * j], acc);
        acc = fmaf(__uint_as_float(ww[j] & 0xffff0000u), xs[k + 2 * j + 1], acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      logit_s[e] = acc;
      if (p.logits_out) p.logits_out[tk * p.E + e] = acc;
    }
  }
  __syncthreads();
  if (warp != 0) return;

  // ---- scoring (warp 0)
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
    // each lane decides for its own groups whether they rank inside topk_group
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

MMB_API int mmb_moe_router(const MmbRouterParams* pp, cudaStream_t stream) {
  const MmbRouterParams& p = *pp;
  if (p.T <= 0) return 0;
  if (p.E > mmb::kMaxExperts || p.topk > 32 || p.K % 8 != 0 || p.n_group > 64) return (int)cudaErrorInvalidValue;
  if (p.n_group > 1 && p.E % p.n_group != 0) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)p.K * 4;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(mmb::moe_router_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  mmb::moe_router_kernel<<<p.T, 256, smem, stream>>>(p);
  return (int)cudaGetLastError();
}
