// Tensor-parallel prefill: the kernels that complete a row-parallel projection whose GEMM epilogue already
// scattered the partial sums to the owners of the token rows (gemm_sm100.cu, reduce-scatter epilogue).
//   rs_finish: owner side - wait for the tp partials, sum them in rank order, add the residual, and store the reduced
//              rows into every peer's gathered buffer (all-gather by NVLink peer stores), then raise the ag flags;
//   tp_wait:   consumer side - bounded wait until all ranks' slices of the gathered buffer have arrived.
// Peer memory is only touched with plain loads / stores of this repository's own kernels.
#include "api_gemm.h"
#include "common.cuh"
#include "launch.h"
#include "tp_comm.cuh"

namespace mmb {

__global__ void __launch_bounds__(256) rs_finish_kernel(const MmbRsFinishParams p) {
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
  const long long n_vec = (long long)p.rows * p.N / 8;       // N is a multiple of 8
  for (long long v = (long long)blockIdx.x * 256 + threadIdx.x; v < n_vec; v += (long long)gridDim.x * 256) {
    const long long e0 = v * 8;
    const int row = (int)(e0 / p.N);
    const int grow = p.rank * p.rows + row;                  // global token row
    if (grow >= p.M) continue;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < p.tp; ++r) {
      const float4 a = __ldcg(reinterpret_cast<const float4*>(p.in_buf + r * tin.slot_stride + e0));
      const float4 b = __ldcg(reinterpret_cast<const float4*>(p.in_buf + r * tin.slot_stride + e0 + 4));
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    uint4 o;
    o.x = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[0])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[1])) << 16);
    o.y = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[2])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[3])) << 16);
    o.z = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[4])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[5])) << 16);
    o.w = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[6])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[7])) << 16);
    const long long dst = (long long)grow * p.N + (e0 - (long long)row * p.N);
    for (int r = 0; r < p.tp; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.ag_peer_bufs[r]) + dst) = o;
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
  const long long n_vec = (long long)p.rows * p.N / 8;
  long long blocks = (n_vec + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  return mmb::launch(mmb::rs_finish_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, 1, p);
}

MMB_API int mmb_tp_wait(const unsigned* flags, const unsigned* step, int* status, int tp, cudaStream_t stream) {
  if (tp < 1 || tp > 32) return (int)cudaErrorInvalidValue;
  return mmb::launch(mmb::tp_wait_kernel, dim3(1), dim3(32), 0, stream, 1, flags, step, status, tp);
}
