// Whole-sequence scans of the recurrent layer families (prompt passes): RWKV v5 / v6 WKV, the Mamba selective scan and the
// gated delta rule.  One launch walks all T tokens of a sequence; the state never leaves the SM while it does:
//
//  * WKV and the gated delta rule keep a state S [dk, dv] per head.  Thread c owns value column c and holds S[:, c] in
//    registers (dk <= 128 floats); the per-token vectors that all columns share (r, k, w, or q, k) are staged in shared
//    memory once per token, two barriers per token.
//  * The selective scan keeps h [N] per channel in registers (N <= 128); B_t and C_t are staged per token.
//
// The recurrences are sequential in t by nature; parallelism comes from heads x batch x columns (tens of thousands of
// threads for real models).  fp32 state and accumulation throughout, bf16 or fp32 inputs converted on load.
#include "api_ext.h"
#include "common.cuh"
#include "launch.h"

namespace mmb {

// ------------------------------------------------------------------------------------------------ WKV (RWKV v5 / v6)
// r, k [B, T, H, dk], v [B, T, H, dv], w [B, T, H, dk] (v6) or [H, dk] (v5: w_tstride = 0), u [H, dk].
//   o_t = r_t (S + (u * k_t) v_t^T);  S <- diag(w_t) S + k_t v_t^T.     grid (H, B), dv threads.
template <int DK>
__global__ void wkv_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ w,
                           const float* __restrict__ u, float* __restrict__ state, float* __restrict__ out, int T, int H, int dv,
                           long long w_bstride, long long w_tstride) {
  __shared__ float rs[DK], ks[DK], ws[DK], us[DK];
  const int h = blockIdx.x, b = blockIdx.y, c = threadIdx.x;
  float S[DK];
  float* Sg = state + ((long long)(b * H + h) * DK) * dv;
#pragma unroll
  for (int i = 0; i < DK; ++i) S[i] = (c < dv) ? Sg[(long long)i * dv + c] : 0.f;
  for (int i = threadIdx.x; i < DK; i += blockDim.x) us[i] = u[h * DK + i];
  for (int t = 0; t < T; ++t) {
    const long long base = ((long long)(b * T + t) * H + h);
    __syncthreads();
    for (int i = threadIdx.x; i < DK; i += blockDim.x) {
      rs[i] = r[base * DK + i];
      ks[i] = k[base * DK + i];
      ws[i] = w[b * w_bstride + t * w_tstride + (long long)h * DK + i];
    }
    __syncthreads();
    if (c < dv) {
      const float vc = v[base * dv + c];
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i) {
        const float kv = ks[i] * vc;
        o = fmaf(rs[i], fmaf(us[i], kv, S[i]), o);
        S[i] = fmaf(ws[i], S[i], kv);
      }
      out[base * dv + c] = o;
    }
  }
  if (c < dv) {
#pragma unroll
    for (int i = 0; i < DK; ++i) Sg[(long long)i * dv + c] = S[i];
  }
}

// ------------------------------------------------------------------------------------------------ gated delta rule
// q, k [B, T, H, dk], v [B, T, H, dv], g, beta [B, T, H].  S <- S exp(g_t); m = S^T k_t; d = (v_t - m) beta_t;
// S <- S + k_t d^T; o_t = S^T (q_t * scale).      grid (H, B), dv threads.
template <int DK>
__global__ void gated_delta_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                        const float* __restrict__ g, const float* __restrict__ beta, float* __restrict__ state,
                                        float* __restrict__ out, int T, int H, int dv, float scale) {
  __shared__ float qs[DK], ks[DK];
  const int h = blockIdx.x, b = blockIdx.y, c = threadIdx.x;
  float S[DK];
  float* Sg = state + ((long long)(b * H + h) * DK) * dv;
#pragma unroll
  for (int i = 0; i < DK; ++i) S[i] = (c < dv) ? Sg[(long long)i * dv + c] : 0.f;
  for (int t = 0; t < T; ++t) {
    const long long base = ((long long)(b * T + t) * H + h);
    __syncthreads();
    for (int i = threadIdx.x; i < DK; i += blockDim.x) {
      qs[i] = q[base * DK + i] * scale;
      ks[i] = k[base * DK + i];
    }
    __syncthreads();
    if (c < dv) {
      const float decay = __expf(g[base]), bt = beta[base];
      float m = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i) {
        S[i] *= decay;
        m = fmaf(S[i], ks[i], m);
      }
      const float d = (v[base * dv + c] - m) * bt;
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i) {
        S[i] = fmaf(ks[i], d, S[i]);
        o = fmaf(S[i], qs[i], o);
      }
      out[base * dv + c] = o;
    }
  }
  if (c < dv) {
#pragma unroll
    for (int i = 0; i < DK; ++i) Sg[(long long)i * dv + c] = S[i];
  }
}

// ------------------------------------------------------------------------------------------------ selective scan (Mamba)
// x, dt [B, T, D], A [D, N], Bm, Cm [B, T, N], Dskip [D] or null, state h fp32 [B, D, N].
//   h <- exp(dt A) h + dt B_t x;  y_t = <h, C_t> + Dskip x.       grid (ceil(D / 128), B), 128 threads.
template <int N>
__global__ void __launch_bounds__(128) selective_scan_kernel(const float* __restrict__ x, const float* __restrict__ dt, const float* __restrict__ A,
                                                             const float* __restrict__ Bm, const float* __restrict__ Cm,
                                                             const float* __restrict__ Dskip, float* __restrict__ state, float* __restrict__ y,
                                                             int T, int D) {
  __shared__ float bs[N], cs[N];
  const int b = blockIdx.y, d = blockIdx.x * 128 + threadIdx.x;
  const bool live = d < D;
  float h[N], a[N];
#pragma unroll
  for (int n = 0; n < N; ++n) {
    h[n] = live ? state[((long long)b * D + d) * N + n] : 0.f;
    a[n] = live ? A[(long long)d * N + n] : 0.f;
  }
  const float dsk = (live && Dskip != nullptr) ? Dskip[d] : 0.f;
  for (int t = 0; t < T; ++t) {
    const long long bt = (long long)b * T + t;
    __syncthreads();
    for (int n = threadIdx.x; n < N; n += 128) {
      bs[n] = Bm[bt * N + n];
      cs[n] = Cm[bt * N + n];
    }
    __syncthreads();
    if (live) {
      const float xv = x[bt * D + d], dtv = dt[bt * D + d];
      float acc = 0.f;
#pragma unroll
      for (int n = 0; n < N; ++n) {
        h[n] = fmaf(__expf(dtv * a[n]), h[n], dtv * bs[n] * xv);
        acc = fmaf(h[n], cs[n], acc);
      }
      y[bt * D + d] = acc + dsk * xv;
    }
  }
  if (live) {
#pragma unroll
    for (int n = 0; n < N; ++n) state[((long long)b * D + d) * N + n] = h[n];
  }
}

}  // namespace mmb

MMB_API int mmb_wkv(const float* r, const float* k, const float* v, const float* w, const float* u, float* state, float* out, int B, int T,
                    int H, int dk, int dv, long long w_bstride, long long w_tstride, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (dv <= 0 || dv > 1024) return (int)cudaErrorInvalidValue;
  const dim3 grid((unsigned)H, (unsigned)B), block((unsigned)((dv + 31) / 32 * 32));
  switch (dk) {
    case 16: mmb::wkv_kernel<16><<<grid, block, 0, stream>>>(r, k, v, w, u, state, out, T, H, dv, w_bstride, w_tstride); break;
    case 32: mmb::wkv_kernel<32><<<grid, block, 0, stream>>>(r, k, v, w, u, state, out, T, H, dv, w_bstride, w_tstride); break;
    case 64: mmb::wkv_kernel<64><<<grid, block, 0, stream>>>(r, k, v, w, u, state, out, T, H, dv, w_bstride, w_tstride); break;
    case 128: mmb::wkv_kernel<128><<<grid, block, 0, stream>>>(r, k, v, w, u, state, out, T, H, dv, w_bstride, w_tstride); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

MMB_API int mmb_gated_delta_scan(const float* q, const float* k, const float* v, const float* g, const float* beta, float* state, float* out,
                                 int B, int T, int H, int dk, int dv, float scale, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (dv <= 0 || dv > 1024) return (int)cudaErrorInvalidValue;
  const dim3 grid((unsigned)H, (unsigned)B), block((unsigned)((dv + 31) / 32 * 32));
  switch (dk) {
    case 16: mmb::gated_delta_scan_kernel<16><<<grid, block, 0, stream>>>(q, k, v, g, beta, state, out, T, H, dv, scale); break;
    case 32: mmb::gated_delta_scan_kernel<32><<<grid, block, 0, stream>>>(q, k, v, g, beta, state, out, T, H, dv, scale); break;
    case 64: mmb::gated_delta_scan_kernel<64><<<grid, block, 0, stream>>>(q, k, v, g, beta, state, out, T, H, dv, scale); break;
    case 128: mmb::gated_delta_scan_kernel<128><<<grid, block, 0, stream>>>(q, k, v, g, beta, state, out, T, H, dv, scale); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

MMB_API int mmb_selective_scan(const float* x, const float* dt, const float* A, const float* Bm, const float* Cm, const float* Dskip,
                               float* state, float* y, int B, int T, int D, int N, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  const dim3 grid((unsigned)((D + 127) / 128), (unsigned)B);
  switch (N) {
    case 8: mmb::selective_scan_kernel<8><<<grid, 128, 0, stream>>>(x, dt, A, Bm, Cm, Dskip, state, y, T, D); break;
    case 16: mmb::selective_scan_kernel<16><<<grid, 128, 0, stream>>>(x, dt, A, Bm, Cm, Dskip, state, y, T, D); break;
    case 32: mmb::selective_scan_kernel<32><<<grid, 128, 0, stream>>>(x, dt, A, Bm, Cm, Dskip, state, y, T, D); break;
    case 64: mmb::selective_scan_kernel<64><<<grid, 128, 0, stream>>>(x, dt, A, Bm, Cm, Dskip, state, y, T, D); break;
    case 128: mmb::selective_scan_kernel<128><<<grid, 128, 0, stream>>>(x, dt, A, Bm, Cm, Dskip, state, y, T, D); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}
