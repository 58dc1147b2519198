// Speculative-decoding verification on the device: sequential accept / reject of the K draft tokens of every
// sequence, the residual-distribution resample at the first rejection, or the bonus token when all are accepted.
// One CTA per sequence; the only serial part is the K-step accept chain (one thread), the resample is a block-wide
// reduction + scan over the vocabulary.
#include "api_ext.h"
#include "common.cuh"
#include "launch.h"

namespace mmb {

// Sample an index from the unnormalised non-negative weights w(i) = max(pt[i] - (pd ? pd[i] : 0), 0) with the uniform
// number u in [0, 1).  All 256 threads call it; every thread returns the same index.
__device__ int block_sample_residual(const float* __restrict__ pt, const float* __restrict__ pd_in, int V, float u, float* sh) {
  __shared__ int result;
  __shared__ float total_s;
  const int tid = threadIdx.x;
  const int per = (V + 255) / 256;
  const int lo = min(V, tid * per), hi = min(V, lo + per);
  const float* pd = pd_in;
  int r = -1;
  // second pass only when the residual is empty (p_target == p_draft): sample p_target itself
  for (int pass = 0; pass < 2; ++pass) {
    float part = 0.f;
    for (int i = lo; i < hi; ++i) part += fmaxf(pt[i] - (pd ? pd[i] : 0.f), 0.f);
    sh[tid] = part;
    __syncthreads();
    if (tid == 0) {
      float tot = 0.f;
      for (int t = 0; t < 256; ++t) tot += sh[t];
      total_s = tot;
      result = -1;
      if (tot > 0.f) {
        const float target = u * tot;
        float run = 0.f;
        int owner = 255;
        for (int t = 0; t < 256; ++t) {
          if (run + sh[t] > target) {
            owner = t;
            break;
          }
          run += sh[t];
        }
        const int olo = min(V, owner * per), ohi = min(V, olo + per);
        int pick = -1;
        for (int i = olo; i < ohi; ++i) {
          const float w = fmaxf(pt[i] - (pd ? pd[i] : 0.f), 0.f);
          if (w > 0.f) {
            pick = i;
            if (run + w > target) break;
          }
          run += w;
        }
        result = pick;
      }
    }
    __syncthreads();
    r = result;
    const float tot = total_s;
    __syncthreads();
    if (r >= 0 || tot > 0.f || pd == nullptr) break;
    pd = nullptr;
  }
  return r;
}

__global__ void __launch_bounds__(256) spec_verify_kernel(const float* __restrict__ p_target, const float* __restrict__ p_draft,
                                                          const int64_t* __restrict__ draft, const float* __restrict__ u,
                                                          const float* __restrict__ u_res, int64_t* __restrict__ out_tokens,
                                                          int* __restrict__ out_accepted, int K, int V) {
  __shared__ float sh[256];
  __shared__ int n_acc_s;
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, tid = threadIdx.x;
  const float* pt = p_target + (long long)b * (K + 1) * V;
  const float* pd = p_draft + (long long)b * K * V;
  if (tid == 0) {
    int n = 0;
    for (; n < K; ++n) {
      const long long tok = draft[(long long)b * K + n];
      const float q = pd[(long long)n * V + tok], p = pt[(long long)n * V + tok];
      const float ratio = (q > 0.f) ? fminf(1.f, p / q) : 1.f;
      if (!(u[(long long)b * K + n] < ratio)) break;
    }
    n_acc_s = n;
  }
  __syncthreads();
  const int n = n_acc_s;
  const int extra = block_sample_residual(pt + (long long)n * V, (n < K) ? pd + (long long)n * V : nullptr, V, u_res[b], sh);
  for (int j = tid; j <= K; j += 256) {
    long long v = -1;
    if (j < n) v = draft[(long long)b * K + j];
    else if (j == n) v = extra;
    out_tokens[(long long)b * (K + 1) + j] = v;
  }
  if (tid == 0) out_accepted[b] = n;
}

}  // namespace mmb

MMB_API int mmb_spec_verify(const float* p_target, const float* p_draft, const int64_t* draft, const float* u, const float* u_resample,
                            int64_t* out_tokens, int* out_accepted, int B, int K, int V, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (K < 1 || V < 1) return (int)cudaErrorInvalidValue;
  return mmb::launch(mmb::spec_verify_kernel, dim3((unsigned)B), dim3(256), 0, stream, 1, p_target, p_draft, draft, u, u_resample,
                     out_tokens, out_accepted, K, V);
}
