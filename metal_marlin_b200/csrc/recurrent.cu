// Decode-step state updates of the recurrent layer families: the gated delta rule (Gated DeltaNet layers of
// Qwen3.5 / 3.6 hybrids) and the Mamba selective-scan step.  Both keep an fp32 state resident in HBM and touch it
// exactly once per token (read-modify-write in one kernel), which is the whole cost of these layers at decode time.
#include "api_ext.h"
#include "common.cuh"
#include "launch.h"

namespace mmb {

// grid (H, B), 256 threads.  State S fp32 [B, H, dk, dv].  Per (b, h):
//   S <- S * exp(g);  m = S^T k;  d = (v - m) * beta;  S <- S + k d^T;  o = S^T q
// thread t owns value columns t, t + 256, ...: every column's update is independent, rows are walked serially.
__global__ void __launch_bounds__(256) gated_delta_step_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                               const bf16* __restrict__ v, const float* __restrict__ g,
                                                               const float* __restrict__ beta, float* __restrict__ state,
                                                               bf16* __restrict__ out, int H, int dk, int dv, float scale) {
  extern __shared__ float sh[];   // q [dk], k [dk]
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.x, b = blockIdx.y;
  const long long bh = (long long)b * H + h;
  float* qs = sh;
  float* ks = sh + dk;
  for (int i = threadIdx.x; i < dk; i += 256) {
    qs[i] = __bfloat162float(q[bh * dk + i]) * scale;
    ks[i] = __bfloat162float(k[bh * dk + i]);
  }
  __syncthreads();
  const float decay = __expf(g[bh]);
  const float bt = beta[bh];
  float* S = state + bh * dk * dv;
  for (int c = threadIdx.x; c < dv; c += 256) {
    float m = 0.f;
    for (int r = 0; r < dk; ++r) {
      const float s = S[(long long)r * dv + c] * decay;
      S[(long long)r * dv + c] = s;
      m = fmaf(s, ks[r], m);
    }
    const float d = (__bfloat162float(v[bh * dv + c]) - m) * bt;
    float o = 0.f;
    for (int r = 0; r < dk; ++r) {
      const float s = fmaf(ks[r], d, S[(long long)r * dv + c]);
      S[(long long)r * dv + c] = s;
      o = fmaf(s, qs[r], o);
    }
    out[bh * dv + c] = __float2bfloat16(o);
  }
}

// grid (ceil(D / 256), B).  State h fp32 [B, D, N].  Per channel d:
//   h <- exp(dt * A[d, :]) * h + dt * Bm[b, :] * x;  y = <h, C[b, :]> + Dskip[d] * x
__global__ void __launch_bounds__(256) selective_scan_step_kernel(const bf16* __restrict__ x, const float* __restrict__ dt,
                                                                  const float* __restrict__ A, const float* __restrict__ Bm,
                                                                  const float* __restrict__ Cm, const float* __restrict__ Dskip,
                                                                  float* __restrict__ state, bf16* __restrict__ y, int D, int N) {
  extern __shared__ float bc[];   // Bm [N], Cm [N]
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y;
  for (int i = threadIdx.x; i < N; i += 256) {
    bc[i] = Bm[(long long)b * N + i];
    bc[N + i] = Cm[(long long)b * N + i];
  }
  __syncthreads();
  const int d = blockIdx.x * 256 + threadIdx.x;
  if (d >= D) return;
  const float xv = __bfloat162float(x[(long long)b * D + d]);
  const float dtv = dt[(long long)b * D + d];
  float* hst = state + ((long long)b * D + d) * N;
  float acc = 0.f;
  for (int n = 0; n < N; ++n) {
    const float hn = __expf(dtv * A[(long long)d * N + n]) * hst[n] + dtv * bc[n] * xv;
    hst[n] = hn;
    acc = fmaf(hn, bc[N + n], acc);
  }
  y[(long long)b * D + d] = __float2bfloat16(acc + (Dskip ? Dskip[d] * xv : 0.f));
}

}  // namespace mmb

MMB_API int mmb_gated_delta_step(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state, void* out,
                                 int B, int H, int dk, int dv, float scale, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (dk <= 0 || dv <= 0 || dk > 4096) return (int)cudaErrorInvalidValue;
  return mmb::launch(mmb::gated_delta_step_kernel, dim3((unsigned)H, (unsigned)B), dim3(256), (size_t)2 * dk * 4, stream, 1, (const bf16*)q,
                     (const bf16*)k, (const bf16*)v, g, beta, state, (bf16*)out, H, dk, dv, scale);
}

MMB_API int mmb_selective_scan_step(const void* x, const float* dt, const float* A, const float* Bm, const float* Cm, const float* Dskip,
                                    float* state, void* y, int B, int D, int N, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (D <= 0 || N <= 0 || N > 4096) return (int)cudaErrorInvalidValue;
  return mmb::launch(mmb::selective_scan_step_kernel, dim3((unsigned)((D + 255) / 256), (unsigned)B), dim3(256), (size_t)2 * N * 4, stream, 1,
                     (const bf16*)x, dt, A, Bm, Cm, Dskip, state, (bf16*)y, D, N);
}
