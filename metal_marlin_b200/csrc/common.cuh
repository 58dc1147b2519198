// Shared device helpers for the sm_100a kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MMB_API extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

namespace mmb {

constexpr int kWarp = 32;

// Split cluster barrier.  A CTA may only touch another CTA's shared memory once that CTA has started; arriving
// at kernel entry and waiting right before the first remote access gives that guarantee without exposing the
// barrier latency.  Both must be executed by every thread of every CTA of the cluster.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `red` is >= 32 floats of shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

// 16-byte streaming load that does not pollute L1 (weights are read once per step).
__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t hi16) { return __uint_as_float(hi16 << 16); }

// m16n8k16, fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// m16n8k16, bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Expand the eight E2M1 codes of a tile-layout word into the four fp16x2 registers of an m16n8k16 A fragment.  In each
// 16-bit half the word holds the signs of registers 0..3 in bits 15..12 and their 3-bit magnitudes in bits 11..9, 8..6,
// 5..3, 2..0, so every register is an independent (shift, mask) pair of the same word: no serial shift chain, and the
// shifts can run as multiplies beside the logic ops.  The fp16 values equal e2m1 * 2^-14 (the exponent field is used
// as-is, so code 1 lands on an fp16 subnormal); the caller folds 2^14 into the group scale.
__device__ __forceinline__ void e2m1x8_to_f16x2(uint32_t q, uint32_t& a0, uint32_t& a1, uint32_t& a2, uint32_t& a3) {
  const uint32_t q3 = q << 3;
  a0 = q & 0x8E008E00u;
  a1 = ((q << 1) & 0x80008000u) | (q3 & 0x0E000E00u);
  a2 = ((q << 2) & 0x80008000u) | ((q << 6) & 0x0E000E00u);
  a3 = (q3 & 0x80008000u) | ((q << 9) & 0x0E000E00u);
}
constexpr float kE2M1F16Rescale = 16384.0f;  // 2^14

// Same codes to bf16x2 holding e2m1 * 2^-126 (bf16 subnormal trick): magnitudes go to bits 8..6.
__device__ __forceinline__ void e2m1x8_to_bf16x2_raw(uint32_t q, uint32_t& a0, uint32_t& a1, uint32_t& a2,
                                                     uint32_t& a3) {
  const uint32_t q3 = q << 3;
  a0 = (q & 0x80008000u) | ((q >> 3) & 0x01C001C0u);
  a1 = ((q << 1) & 0x80008000u) | (q & 0x01C001C0u);
  a2 = ((q << 2) & 0x80008000u) | (q3 & 0x01C001C0u);
  a3 = (q3 & 0x80008000u) | ((q << 6) & 0x01C001C0u);
}

// Programmatic dependent launch: pdl_launch_dependents() lets the next kernel of the stream start its
// independent prologue; pdl_wait() blocks until the previous kernel has completed and its writes are visible.
// Both are no-ops for kernels launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ------------------------------------------------------------------------------------------ mbarrier / bulk copies
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // 2 s: every mbarrier wait gives up after this long

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false when the limit expired or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0u) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kWaitLimitNs) return false;
    }
  }
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// Bulk copy global -> shared (TMA engine, no tensor map): 16-byte aligned addresses, size a multiple of 16.
// Completion is signalled on the mbarrier as `bytes` of transaction count.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

}  // namespace mmb
