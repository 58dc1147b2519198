// All-reduce through the NVSwitch in ONE kernel: `multimem.ld_reduce` sums the tp copies of a slice inside the switch,
// `multimem.st` writes the sum back into every rank's copy.  Used where a tensor-parallel partial is too large for the
// slot exchange of the decode kernels (MoE outputs of prompt passes, 17-32-token batches) instead of a collective call.
//
// Every rank holds the same symmetric buffer (fp32 [n]) that is also mapped through a multicast object (`mc`), and two flag
// words per source rank.  One call = one step s (= *step + 1, the same on every rank because all ranks make the same calls):
//   1. arrive: CTA 0 publishes s in arrive[rank] on every peer (release at system scope: this rank's copy, written by the
//      previous kernel of the stream, is complete); every CTA waits - bounded - until all tp arrive flags show s;
//   2. rank r owns the r-th slice: v = multimem.ld_reduce.add over the slice (the switch reads all copies), multimem.st v;
//   3. done: the last CTA to finish publishes s in done[rank] on every peer, waits - bounded - for all done flags (every
//      slice of this rank's copy has landed) and advances *step.  The next kernel of the stream reads the reduced copy.
// On an expired wait the kernel records 150 + source rank in the status word and returns without touching the data.
#include "api_gemm.h"
#include "common.cuh"
#include "launch.h"
#include "tp_comm.cuh"

namespace mmb {

__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_f32x4(float* mc_addr, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

// Bounded wait of the first tp threads of a CTA for flags[0..tp) >= want.  Returns the CTA-wide verdict.
__device__ __forceinline__ bool mc_wait_all(const unsigned* flags, unsigned want, int tp, int* status) {
  bool ok = true;
  if ((int)threadIdx.x < tp) {
    const unsigned* f = flags + threadIdx.x;
    if (ld_acquire_sys(f) < want) {
      const unsigned long long t0 = tp_now_ns(), lim = wait_limit_ns(status);
      unsigned it = 0;
      while (ld_acquire_sys(f) < want) {
        if ((++it & 63u) == 0u && tp_now_ns() - t0 > lim) {
          if (status) atomicExch(status, 150 + (int)threadIdx.x);
          ok = false;
          break;
        }
      }
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

__global__ void __launch_bounds__(512) mc_all_reduce_kernel(const MmbMcAllReduceParams p) {
  const unsigned s = *reinterpret_cast<const volatile unsigned*>(p.step) + 1u;
  if (blockIdx.x == 0 && (int)threadIdx.x < p.tp) {
    __threadfence_system();
    st_release_sys(p.peer_flags[threadIdx.x] + p.rank, s);
  }
  const bool arrived = mc_wait_all(p.local_flags, s, p.tp, p.status);
  if (arrived) {
    const long long n4 = p.n >> 2;
    const long long per = (n4 + p.tp - 1) / p.tp;
    const long long lo = (long long)p.rank * per, hi = min(n4, lo + per);
    float* mc = p.mc;
    for (long long i = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += (long long)gridDim.x * blockDim.x) {
      const float4 v = multimem_ld_reduce_f32x4(mc + i * 4);
      multimem_st_f32x4(mc + i * 4, v);
    }
  }
  __syncthreads();
  __shared__ int last_s;
  if (threadIdx.x == 0) {
    __threadfence_system();
    last_s = (atomicAdd(p.counter, 1u) == gridDim.x - 1u) ? 1 : 0;
  }
  __syncthreads();
  if (!last_s) return;
  // last CTA: publish "my slice is everywhere", wait until every rank's slice is here, advance the step
  if (threadIdx.x == 0) {
    __threadfence();
    atomicExch(p.counter, 0u);
  }
  if (arrived && (int)threadIdx.x < p.tp) st_release_sys(p.peer_flags[threadIdx.x] + p.tp + p.rank, s);
  const bool done = arrived && mc_wait_all(p.local_flags + p.tp, s, p.tp, p.status);
  if (done && threadIdx.x == 0) {
    *p.step = s;
    __threadfence();
  }
}

}  // namespace mmb

MMB_API int mmb_mc_all_reduce(const MmbMcAllReduceParams* pp, cudaStream_t stream) {
  const MmbMcAllReduceParams& p = *pp;
  if (p.n <= 0) return 0;
  if (p.mc == nullptr || p.peer_flags == nullptr || p.local_flags == nullptr || p.step == nullptr || p.counter == nullptr || p.tp < 1 ||
      p.tp > 32 || p.rank < 0 || p.rank >= p.tp || (p.n & 3) != 0 || (reinterpret_cast<uintptr_t>(p.mc) & 15) != 0)
    return (int)cudaErrorInvalidValue;
  const long long per4 = ((p.n >> 2) + p.tp - 1) / p.tp;
  long long blocks = (per4 + 511) / 512;
  if (blocks > 148 * 2) blocks = 148 * 2;
  if (blocks < 1) blocks = 1;
  mmb::mc_all_reduce_kernel<<<(unsigned)blocks, 512, 0, stream>>>(p);
  return (int)cudaGetLastError();
}
