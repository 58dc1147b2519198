// Device-side tensor-parallel exchange used inside the compute kernels (no separate collective launch).
//
// Protocol for one "site" (a place in the layer graph where partial sums of a row-parallel projection
// must be combined across the tp ranks):
//   * every rank owns a receive buffer  fp32 [tp][rows][width]  and a flag word per source rank, both in
//     memory that all peers can address (NVLink peer mappings);
//   * the PRODUCER kernel (the row-parallel GEMV / GEMM) stores its partial result straight into slot
//     `my_rank` of every peer's buffer from its epilogue; the last CTA to finish publishes the step
//     number into flag[my_rank] on every peer with a system-scope release store;
//   * the CONSUMER kernel (whatever reads the combined activation next: a GEMV prologue, the MoE router,
//     the LM head) waits - bounded - until all tp flags reached the current step and adds the tp slots in
//     rank order while it stages its input, so every rank computes a bit-identical sum.
// A site is used once per step and steps are globally ordered by the data dependencies, so one buffer per
// site needs no double buffering.  Waits give up after kTpWaitNs and record a code in the status word.
#pragma once
#include "common.cuh"

namespace mmb {

constexpr unsigned long long kTpWaitNs = 1000000000ull;   // 1 s

// Limit of a bounded wait: word 1 of the status array, when positive, gives it in microseconds (a host-side setting for
// tests and for deployments that want to give up sooner); otherwise one second.
__device__ __forceinline__ unsigned long long wait_limit_ns(const int* status) {
  if (status != nullptr) {
    const int us = *reinterpret_cast<const volatile int*>(status + 1);
    if (us > 0) return (unsigned long long)us * 1000ull;
  }
  return kTpWaitNs;
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long tp_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct TpIn {
  const float* buf;          // local fp32 [tp][slot_stride]
  const unsigned* flags;     // local [tp]
  const unsigned* step;      // device scalar: current step number
  int* status;               // optional error word
  int tp;
  long long slot_stride;     // elements between consecutive source slots
};

struct TpOut {
  float* const* peer_slots;      // device array [tp]: my slot inside rank r's receive buffer
  unsigned* const* peer_flags;   // device array [tp]: flag[my_rank] on rank r
  unsigned* counter;             // local CTA completion counter (starts at 0, left at 0)
  const unsigned* step;
  int tp;
  float* mc_slot = nullptr;      // optional: my slot addressed through the NVSwitch multicast mapping of the buffers
};

// All threads of the CTA call this before reading the receive buffer.
__device__ __forceinline__ void tp_wait(const TpIn& t) {
  if ((int)threadIdx.x < t.tp) {
    const unsigned want = *t.step;
    const unsigned* f = t.flags + threadIdx.x;
    if (ld_acquire_sys(f) < want) {
      const unsigned long long t0 = tp_now_ns(), lim = wait_limit_ns(t.status);
      unsigned it = 0;
      while (ld_acquire_sys(f) < want) {
        if ((++it & 63u) == 0u && tp_now_ns() - t0 > lim) {
          if (t.status) atomicExch(t.status, 100 + (int)threadIdx.x);
          break;
        }
      }
    }
  }
  __syncthreads();
}

// Sum of the tp partial slots at element idx, in rank order, bypassing L1 (the lines are rewritten by peers
// every step).
__device__ __forceinline__ float tp_sum(const TpIn& t, long long idx) {
  float s = 0.f;
  for (int r = 0; r < t.tp; ++r) s += __ldcg(t.buf + r * t.slot_stride + idx);
  return s;
}
__device__ __forceinline__ float2 tp_sum2(const TpIn& t, long long idx) {
  float2 s = make_float2(0.f, 0.f);
  for (int r = 0; r < t.tp; ++r) {
    const float2 v = __ldcg(reinterpret_cast<const float2*>(t.buf + r * t.slot_stride + idx));
    s.x += v.x;
    s.y += v.y;
  }
  return s;
}

// Store one value of this rank's partial into every peer: one multimem store that the NVSwitch replicates into all
// ranks' buffers when the buffers are bound to a multicast object, else tp plain peer stores.
__device__ __forceinline__ void tp_push(const TpOut& t, long long idx, float v) {
  if (t.mc_slot != nullptr) {
    asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(t.mc_slot + idx), "f"(v) : "memory");
    return;
  }
  for (int r = 0; r < t.tp; ++r) t.peer_slots[r][idx] = v;
}

// Called by all threads of every CTA of the producer grid after their tp_push calls.  The CTA barrier orders every
// thread's peer stores before thread 0's system-scope fence (fences are cumulative over writes observed through the
// barrier), so one fence per CTA - not one per thread - publishes them; the CTA that finds the counter complete
// raises the flags.
__device__ __forceinline__ void tp_signal(const TpOut& t, unsigned total_ctas) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned old = atomicAdd(t.counter, 1u);
    if (old == total_ctas - 1u) {
      __threadfence();
      atomicExch(t.counter, 0u);
      const unsigned step = *t.step;
      for (int r = 0; r < t.tp; ++r) st_release_sys(t.peer_flags[r], step);
    }
  }
}

}  // namespace mmb
