// Tensor-parallel prefill: the kernels that complete a row-parallel projection whose GEMM epilogue already
// scattered the partial sums to the owners of the token rows (gemm_sm100.cu, reduce-scatter epilogue).
//   rs_finish: owner side - wait for the tp partials, sum them in rank order, optionally add the residual and apply
//              the next RMSNorm to the owned rows, and store the result rows into every peer's gathered buffer(s)
//              (all-gather by NVLink peer stores), then raise the ag flags;
//   tp_wait:   consumer side - bounded wait until all ranks' slices of the gathered buffer have arrived.
// Peer memory is only touched with plain loads / stores of this repository's own kernels.
#include "api_gemm.h"
#include "common.cuh"
#include "launch.h"
#include "tp_comm.cuh"

namespace mmb {

__device__ __forceinline__ uint4 pack8_bf16(const float* v) {
  uint4 o;
  o.x = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(v[0])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(v[1])) << 16);
  o.y = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(v[2])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(v[3])) << 16);
  o.z = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(v[4])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(v[5])) << 16);
  o.w = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(v[6])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(v[7])) << 16);
  return o;
}

// One CTA per owned token row (grid-stride).  Dynamic shared memory: the row as fp32 (only used with the fused norm).
__global__ void __launch_bounds__(256) rs_finish_kernel(const MmbRsFinishParams p) {
  extern __shared__ __align__(16) float row_s[];
  __shared__ float red_s[8];
  pdl_launch_dependents();
  pdl_wait();
  TpIn tin;
  tin.buf = p.in_buf;
  tin.flags = p.in_flags;
  tin.step = p.step;
  tin.status = p.status;
  tin.tp = p.tp;
  tin.slot_stride = (long long)p.rows * p.N;
  tp_wait(tin);
  const bf16* resid = reinterpret_cast<const bf16*>(p.resid);
  const bf16* nw = reinterpret_cast<const bf16*>(p.norm_w);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const int grow = p.rank * p.rows + row;                  // global token row
    if (grow >= p.M) break;
    float ss = 0.f;
    for (int c = tid * 8; c < p.N; c += 256 * 8) {
      const long long e0 = (long long)row * p.N + c;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < p.tp; ++r) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(p.in_buf + r * tin.slot_stride + e0));
        const float4 b = __ldcg(reinterpret_cast<const float4*>(p.in_buf + r * tin.slot_stride + e0 + 4));
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      }
      const long long dst = (long long)grow * p.N + c;
      if (resid != nullptr) {
        // same roundings as the unfused sequence: the projection output to bf16, then the residual sum to bf16
        const uint4 hv = *reinterpret_cast<const uint4*>(resid + dst);
        const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[2 * e] = __bfloat162float(__float2bfloat16(acc[2 * e])) + __uint_as_float(hw[e] << 16);
          acc[2 * e + 1] = __bfloat162float(__float2bfloat16(acc[2 * e + 1])) + __uint_as_float(hw[e] & 0xffff0000u);
        }
      }
      const uint4 o = pack8_bf16(acc);
      for (int r = 0; r < p.tp; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.ag_peer_bufs[r]) + dst) = o;
      if (nw != nullptr) {
        const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = __uint_as_float(ow[e] << 16), hi = __uint_as_float(ow[e] & 0xffff0000u);
          row_s[c + 2 * e] = lo;
          row_s[c + 2 * e + 1] = hi;
          ss = fmaf(lo, lo, fmaf(hi, hi, ss));
        }
      }
    }
    if (nw != nullptr) {
      ss = warp_sum(ss);
      if (lane == 0) red_s[warp] = ss;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) tot += red_s[w];
      const float rstd = rsqrtf(tot / (float)p.N + p.eps);
      for (int c = tid * 8; c < p.N; c += 256 * 8) {        // every thread normalizes the columns it produced
        const uint4 wv = *reinterpret_cast<const uint4*>(nw + c);
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        float y[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          y[2 * e] = row_s[c + 2 * e] * rstd * __uint_as_float(ww[e] << 16);
          y[2 * e + 1] = row_s[c + 2 * e + 1] * rstd * __uint_as_float(ww[e] & 0xffff0000u);
        }
        const uint4 o = pack8_bf16(y);
        const long long dst = (long long)grow * p.N + c;
        for (int r = 0; r < p.tp; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.ag2_peer_bufs[r]) + dst) = o;
      }
      __syncthreads();     // red_s is reused by the next row
    }
  }
  TpOut tout;
  tout.peer_slots = nullptr;
  tout.peer_flags = p.ag_peer_flags;
  tout.counter = p.counter;
  tout.step = p.step;
  tout.tp = p.tp;
  tp_signal(tout, gridDim.x);
}

__global__ void __launch_bounds__(32) tp_wait_kernel(const unsigned* flags, const unsigned* step, int* status, int tp) {
  pdl_launch_dependents();
  pdl_wait();
  TpIn tin;
  tin.buf = nullptr;
  tin.flags = flags;
  tin.step = step;
  tin.status = status;
  tin.tp = tp;
  tin.slot_stride = 0;
  tp_wait(tin);
}

}  // namespace mmb

MMB_API int mmb_tp_rs_finish(const MmbRsFinishParams* pp, cudaStream_t stream) {
  const MmbRsFinishParams& p = *pp;
  if (p.rows <= 0) return 0;
  if (p.N % 8 != 0 || p.tp < 1 || p.tp > 32) return (int)cudaErrorInvalidValue;
  if (p.norm_w != nullptr && p.ag2_peer_bufs == nullptr) return (int)cudaErrorInvalidValue;
  const size_t smem = p.norm_w != nullptr ? (size_t)p.N * 4 : 0;
  if (smem > 160 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(mmb::rs_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  // a few rows per CTA at most: the kernel is a bandwidth-bound sweep and its CTAs all raise one counter at the end
  int blocks = p.rows < 148 * 4 ? p.rows : 148 * 4;
  return mmb::launch(mmb::rs_finish_kernel, dim3((unsigned)blocks), dim3(256), smem, stream, 1, p);
}

MMB_API int mmb_tp_wait(const unsigned* flags, const unsigned* step, int* status, int tp, cudaStream_t stream) {
  if (tp < 1 || tp > 32) return (int)cudaErrorInvalidValue;
  return mmb::launch(mmb::tp_wait_kernel, dim3(1), dim3(32), 0, stream, 1, flags, step, status, tp);
}
