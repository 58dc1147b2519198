// MoE router: (residual add + RMSNorm) -> gate GEMV -> scoring -> (grouped) top-k -> renormalise, everything
// on device so the expert kernels never wait for the host.
//
// One thread-block CLUSTER per token: the gate matrix rows are split over the CTAs of the cluster (one expert
// per warp per round, each row requested with 16-byte loads that are all in flight before the activation is
// staged), the logits are written into the leader CTA's shared memory through distributed shared memory, and
// after a cluster barrier the leader's first warp scores and selects.  A decode-time router call is therefore
// one DRAM round trip deep instead of experts/warps round trips.
//
// Scoring 0: softmax over experts, top-k of the probabilities, optional renormalisation (Mixtral / Qwen3-MoE
// and the reference's MMFP4 layers).  Scoring 1: sigmoid scores, the choice uses score + e_score_correction_bias
// with grouped top-k, the weights use the unbiased scores (DeepSeek-V3 / GLM-4.x).
#include <cooperative_groups.h>

#include "api.h"
#include "common.cuh"
#include "launch.h"
#include "tp_comm.cuh"
#include "router_select.cuh"

namespace cg = cooperative_groups;

namespace mmb {

constexpr int kRouterMaxLoads = 8;     // 16-byte loads per lane per expert row held in registers (K <= 2048)

__global__ void __launch_bounds__(256) moe_router_kernel(const MmbRouterParams p, const int cluster_size) {
  extern __shared__ float xs[];            // [K]
  __shared__ float red[32];
  __shared__ float logit_s[kMaxExperts];   // complete only in the leader CTA
  __shared__ float choice_s[kMaxExperts];
  __shared__ float group_s[64];
  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (cluster_size > 1) ? (int)cluster.block_rank() : 0;
  if (cluster_size > 1) cluster_arrive();   // matched by cluster_wait() before the first store into the leader's table
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long tk = blockIdx.x / cluster_size;
  const bf16* W = reinterpret_cast<const bf16*>(p.w);

  // experts of this CTA: [e_lo, e_hi); warp w takes e_lo + w, e_lo + w + 8, ...
  const int per_cta = (p.E + cluster_size - 1) / cluster_size;
  const int e_lo = crank * per_cta, e_hi = min(p.E, e_lo + per_cta);
  const int n_loads = (p.K + 255) / 256;
  const bool in_regs = n_loads <= kRouterMaxLoads;
  uint4 wv[kRouterMaxLoads];
  const int e_first = e_lo + warp;
  if (in_regs && e_first < e_hi) {
#pragma unroll
    for (int u = 0; u < kRouterMaxLoads; ++u) {
      const int k = u * 256 + lane * 8;
      wv[u] = (k < p.K) ? ldg_stream(reinterpret_cast<const uint4*>(W + (long long)e_first * p.K + k)) : make_uint4(0, 0, 0, 0);
    }
  }

  // the RMSNorm weight is static too: this thread's slices (k = 2 * tid + 512 * j) are requested before the wait
  const bf16* nw = reinterpret_cast<const bf16*>(p.norm_w);
  constexpr int kNormCh = 16;            // K <= 16 * 512
  bf162 nwv[kNormCh];
  if (nw != nullptr) {
#pragma unroll
    for (int j = 0; j < kNormCh; ++j) {
      const int k = tid * 2 + j * 512;
      if (k < p.K) nwv[j] = *reinterpret_cast<const bf162*>(nw + k);
    }
  }
  pdl_launch_dependents();
  pdl_wait();
  // ---- stage the activation (every CTA of the cluster needs all of it)
  const bf16* x = reinterpret_cast<const bf16*>(p.x) + tk * p.K;
  const bf16* d = p.delta ? reinterpret_cast<const bf16*>(p.delta) + tk * p.K : nullptr;
  bf16* ro = (p.resid_out && crank == 0) ? reinterpret_cast<bf16*>(p.resid_out) + tk * p.K : nullptr;
  const bool has_tin = p.tpx.in_buf != nullptr;
  TpIn tin;
  tin.buf = p.tpx.in_buf;
  tin.flags = p.tpx.in_flags;
  tin.step = p.tpx.step;
  tin.status = p.tpx.status;
  tin.tp = p.tpx.tp;
  tin.slot_stride = p.tpx.in_slot_stride;
  if (has_tin) tp_wait(tin);
  float ss = 0.f;
  for (int k = tid * 2; k < p.K; k += 512) {
    float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(x + k));
    if (d || has_tin) {
      const float2 dv = has_tin ? tp_sum2(tin, tk * p.K + k) : __bfloat1622float2(*reinterpret_cast<const bf162*>(d + k));
      const bf162 s2 = __floats2bfloat162_rn(v.x + dv.x, v.y + dv.y);
      v = __bfloat1622float2(s2);
      if (ro) *reinterpret_cast<bf162*>(ro + k) = s2;
    }
    xs[k] = v.x;
    xs[k + 1] = v.y;
    ss += v.x * v.x + v.y * v.y;
  }
  ss = block_sum(ss, red);
  if (nw) {
    const float rs = rsqrtf(ss / (float)p.K + p.eps);
#pragma unroll
    for (int j = 0; j < kNormCh; ++j) {
      const int k = tid * 2 + j * 512;
      if (k < p.K) {
        const float2 w2 = __bfloat1622float2(nwv[j]);
        xs[k] = __bfloat162float(__float2bfloat16(xs[k] * rs * w2.x));
        xs[k + 1] = __bfloat162float(__float2bfloat16(xs[k + 1] * rs * w2.y));
      }
    }
  }
  __syncthreads();

  // ---- gate GEMV for this CTA's experts; results go to the leader's logit table
  if (cluster_size > 1) cluster_wait();
  float* leader_logits = (cluster_size > 1) ? cluster.map_shared_rank(logit_s, 0) : logit_s;
  for (int e = e_first; e < e_hi; e += 8) {
    float acc = 0.f;
    if (in_regs && e == e_first) {
#pragma unroll
      for (int u = 0; u < kRouterMaxLoads; ++u) {
        const int k = u * 256 + lane * 8;
        if (k < p.K) {
          const uint32_t ww[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc = fmaf(__uint_as_float(ww[j] << 16), xs[k + 2 * j], acc);
            acc = fmaf(__uint_as_float(ww[j] & 0xffff0000u), xs[k + 2 * j + 1], acc);
          }
        }
      }
    } else {
      const bf16* wr = W + (long long)e * p.K;
      for (int k = lane * 8; k < p.K; k += 256) {
        const uint4 w4 = ldg_stream(reinterpret_cast<const uint4*>(wr + k));
        const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc = fmaf(__uint_as_float(ww[j] << 16), xs[k + 2 * j], acc);
          acc = fmaf(__uint_as_float(ww[j] & 0xffff0000u), xs[k + 2 * j + 1], acc);
        }
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      leader_logits[e] = acc;
      if (p.logits_out) p.logits_out[tk * p.E + e] = acc;
    }
  }
  if (cluster_size > 1) cluster.sync();
  else __syncthreads();
  if (crank != 0 || warp != 0) return;

  router_select(p, tk, logit_s, choice_s, group_s, lane);
}

// Many tokens (prefill): the gate logits come from a tensor-core GEMM; one warp per token scores and selects.
__global__ void __launch_bounds__(256) moe_select_kernel(const MmbRouterParams p, const float* __restrict__ logits_in) {
  __shared__ float logit_w[8][kMaxExperts];
  __shared__ float choice_w[8][kMaxExperts];
  __shared__ float group_w[8][64];
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long tk = (long long)blockIdx.x * 8 + warp;
  if (tk >= p.T) return;
  for (int e = lane; e < p.E; e += 32) logit_w[warp][e] = logits_in[tk * p.E + e];
  __syncwarp();
  router_select(p, tk, logit_w[warp], choice_w[warp], group_w[warp], lane);
}

}  // namespace mmb

MMB_API int mmb_moe_select(const MmbRouterParams* pp, const float* logits_in, cudaStream_t stream) {
  const MmbRouterParams& p = *pp;
  if (p.T <= 0) return 0;
  if (p.E > mmb::kMaxExperts || p.topk > 32 || p.n_group > 64 || logits_in == nullptr) return (int)cudaErrorInvalidValue;
  if (p.n_group > 1 && p.E % p.n_group != 0) return (int)cudaErrorInvalidValue;
  return mmb::launch(mmb::moe_select_kernel, dim3((unsigned)((p.T + 7) / 8)), dim3(256), 0, stream, 1, p, logits_in);
}

MMB_API int mmb_moe_router(const MmbRouterParams* pp, cudaStream_t stream) {
  const MmbRouterParams& p = *pp;
  if (p.T <= 0) return 0;
  if (p.E > mmb::kMaxExperts || p.topk > 32 || p.K % 8 != 0 || p.n_group > 64 || p.K > 16 * 512)
    return (int)cudaErrorInvalidValue;
  if (p.n_group > 1 && p.E % p.n_group != 0) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)p.K * 4;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(mmb::moe_router_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  // one warp per expert per round: 8 experts per CTA; cluster of up to 8 CTAs (portable size) per token
  int cluster = 1;
  while (cluster < 8 && cluster * 8 < p.E) cluster *= 2;
  return mmb::launch(mmb::moe_router_kernel, dim3((unsigned)(p.T * cluster)), dim3(256), smem, stream, cluster, p, cluster);
}
