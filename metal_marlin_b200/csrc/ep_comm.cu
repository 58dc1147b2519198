// Expert-parallel token exchange inside our own kernels, over NVLink peer memory (no collective library call, no host
// synchronisation on the routing result).
//
// One MoE layer with every rank holding different tokens and a slice of the experts:
//   1. ep_dispatch (sender): one warp per (token, slot) pair copies the token's row straight into region `rank` of the
//      expert owner's receive buffer, with (local expert id, pair index) beside it; positions come from local atomics
//      (the order of rows inside a region is irrelevant: every row is an independent GEMM row).  The last CTA publishes
//      the per-destination row counts and the step number in the owners' flag words (system-scope release).
//   2. ep_recv_group (expert owner, one CTA): bounded wait for every sender's flag, then the counting sort of the
//      received rows by expert, the tile list of the grouped tcgen05 GEMM, and for every sorted row the ADDRESS of its
//      slot in the sender's return buffer.
//   3. gather + gate/up GEMM + SwiGLU + down GEMM (existing kernels); the down projection's epilogue stores each output
//      row at that address, i.e. directly into the token owner's memory (GEMM -> combine without an intermediate).
//   4. ep_signal: publishes the step in the senders' return flags.
//   5. ep_combine (token owner): bounded wait for every expert owner's return flag, then the routing-weighted sum of a
//      token's slots in slot order (+ shared expert / residual), fp32 accumulation: deterministic.
// Every wait gives up after kTpWaitNs, records a code in the status word and carries on with what has arrived, so a
// missing rank costs a wrong result and an error code, never a hung context.
#include "api_ext.h"
#include "common.cuh"
#include "launch.h"
#include "tp_comm.cuh"

namespace mmb {

constexpr int kEpMaxRanks = 32;
constexpr int kEpMaxExperts = 1024;

__device__ __forceinline__ bool ep_wait_flag(const unsigned* f, unsigned want, const int* status) {
  if (ld_acquire_sys(f) >= want) return true;
  const unsigned long long t0 = tp_now_ns(), lim = wait_limit_ns(status);
  unsigned it = 0;
  while (ld_acquire_sys(f) < want) {
    if ((++it & 63u) == 0u && tp_now_ns() - t0 > lim) return false;
  }
  return true;
}

__global__ void __launch_bounds__(256) ep_dispatch_kernel(MmbEpDispatchParams p) {
  __shared__ int s_last;
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = p.T * p.topk, vec = p.H / 8;
  for (int pair = blockIdx.x * 8 + warp; pair < n; pair += gridDim.x * 8) {
    const int e = p.ids[pair];                       // the same for the whole warp
    if (e < 0) continue;
    const int d = min(e / p.experts_per_rank, p.ep - 1);
    int pos = 0;
    if (lane == 0) pos = atomicAdd(&p.send_cnt[d], 1);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (pos >= p.cap) {
      if (lane == 0 && p.status) atomicExch(p.status, 120);
      continue;
    }
    const long long row = (long long)p.rank * p.cap + pos;
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(p.x) + (long long)(pair / p.topk) * p.ldx);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.peer_recv_x[d]) + row * p.H);
    for (int c = lane; c < vec; c += 32) dst[c] = src[c];
    if (lane == 0) *reinterpret_cast<int2*>(p.peer_recv_meta[d] + row * 2) = make_int2(e - d * p.experts_per_rank, pair);
  }
  // publish: every CTA's peer stores are fenced before its arrival on the counter; the last CTA sends counts and flags
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(p.counter, 1u) == gridDim.x - 1u;
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    if ((int)threadIdx.x < p.ep) {
      const int d = threadIdx.x;
      const int c = min(atomicExch(&p.send_cnt[d], 0), p.cap);
      p.peer_recv_cnt[d][p.rank] = c;
      __threadfence_system();
      st_release_sys(p.peer_flags[d], *p.step);
    }
    if (threadIdx.x == 0) atomicExch(p.counter, 0u);
  }
}

__global__ void __launch_bounds__(1024) ep_recv_group_kernel(MmbEpRecvParams p) {
  __shared__ int cnt[kEpMaxExperts];
  __shared__ int off[kEpMaxExperts + 1];
  __shared__ int tbase[kEpMaxExperts + 1];
  __shared__ int scnt[kEpMaxRanks];
  __shared__ int s_fits;
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, E = p.E_local, n = (p.n_rows_max > 0) ? min(p.n_rows_max, p.ep * p.cap) : p.ep * p.cap;
  if (tid < p.ep) {
    int c = 0;
    if (ep_wait_flag(p.flags + tid, *p.step, p.status)) c = min(max(__ldcg(p.recv_cnt + tid), 0), p.cap);
    else if (p.status) atomicExch(p.status, 121 + tid);
    scnt[tid] = c;
  }
  for (int e = tid; e < E; e += 1024) cnt[e] = 0;
  __syncthreads();
  for (int s = 0; s < p.ep; ++s)
    for (int j = tid; j < scnt[s]; j += 1024) {
      const int e = __ldcg(p.recv_meta + ((long long)s * p.cap + j) * 2);
      if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
  __syncthreads();
  if (tid == 0) {
    int o = 0, t = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = o;
      tbase[e] = t;
      o += cnt[e];
      t += (cnt[e] + p.token_tile - 1) / p.token_tile;
    }
    off[E] = o;
    tbase[E] = t;
    // the caller sized the row arrays for a bound on this pass; more rows than that: run nothing and report
    s_fits = (o <= n) ? 1 : 0;
    if (!s_fits && p.status) atomicExch(p.status, 120);
    p.n_tiles[0] = s_fits ? min(t, p.max_tiles) : 0;
    p.n_tiles[1] = s_fits ? o : 0;        // rows received in all: later kernels sweep these, not the worst-case capacity
  }
  __syncthreads();
  if (!s_fits) {
    // clear the tile list and the row tables: no row is scheduled
    for (int ti = tid; ti < p.max_tiles; ti += 1024) {
      p.tile_expert[ti] = 0;
      p.tile_row0[ti] = 0;
      p.tile_rows[ti] = 0;
    }
    for (int i = tid; i < n; i += 1024) {
      p.order[i] = -1;
      p.row_dst[i] = 0;
    }
    return;
  }
  for (int e = tid; e < E; e += 1024) {
    const int nt = tbase[e + 1] - tbase[e];
    for (int j = 0; j < nt; ++j) {
      const int ti = tbase[e] + j;
      if (ti < p.max_tiles) {
        p.tile_expert[ti] = e;
        p.tile_row0[ti] = off[e] + j * p.token_tile;
        p.tile_rows[ti] = min(p.token_tile, cnt[e] - j * p.token_tile);
      }
    }
    cnt[e] = off[e];          // becomes the write cursor of the expert
  }
  for (int ti = tbase[E] + tid; ti < p.max_tiles; ti += 1024) {
    p.tile_expert[ti] = 0;
    p.tile_row0[ti] = 0;
    p.tile_rows[ti] = 0;
  }
  for (int i = off[E] + tid; i < n; i += 1024) {
    p.order[i] = -1;
    p.row_dst[i] = 0;
  }
  __syncthreads();
  for (int s = 0; s < p.ep; ++s) {
    const long long ret = p.ret_peer[s];
    for (int j = tid; j < scnt[s]; j += 1024) {
      const int2 m = __ldcg(reinterpret_cast<const int2*>(p.recv_meta + ((long long)s * p.cap + j) * 2));
      if (m.x >= 0 && m.x < E) {
        const int pos = atomicAdd(&cnt[m.x], 1);
        p.order[pos] = s * p.cap + j;
        p.row_dst[pos] = ret + (long long)m.y * p.H * 2;
      }
    }
  }
}

__global__ void __launch_bounds__(32) ep_signal_kernel(unsigned* const* peer_flags, const unsigned* step, int ep) {
  pdl_wait();                      // everything earlier in the stream is complete and flushed
  if ((int)threadIdx.x < ep) {
    __threadfence_system();
    st_release_sys(peer_flags[threadIdx.x], *step);
  }
}

__global__ void __launch_bounds__(256) ep_combine_kernel(MmbEpCombineParams p) {
  pdl_launch_dependents();
  pdl_wait();
  if ((int)threadIdx.x < p.ep) {
    if (!ep_wait_flag(p.flags + threadIdx.x, *p.step, p.status) && p.status) atomicExch(p.status, 140 + (int)threadIdx.x);
  }
  __syncthreads();
  const int vec = p.N / 8;
  const bf16* y = reinterpret_cast<const bf16*>(p.ret_y);
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < (long long)p.T * vec; i += (long long)gridDim.x * 256) {
    const int t = (int)(i / vec), c = (int)(i % vec);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto add_row = [&](const uint4 v, float w) {
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += w * __uint_as_float(u[j] << 16);
        acc[2 * j + 1] += w * __uint_as_float(u[j] & 0xffff0000u);
      }
    };
    for (int k = 0; k < p.topk; ++k) {
      const int pair = t * p.topk + k;
      if (p.ids[pair] < 0) continue;
      // rows written by peers during this launch's lifetime: read at L2
      add_row(__ldcg(reinterpret_cast<const uint4*>(y + (long long)pair * p.N) + c), p.weights[pair]);
    }
    if (p.add0) add_row(*(reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(p.add0) + (long long)t * p.N) + c), 1.f);
    if (p.add1) add_row(*(reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(p.add1) + (long long)t * p.N) + c), 1.f);
    uint4 o;
    o.x = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[0])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[1])) << 16);
    o.y = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[2])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[3])) << 16);
    o.z = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[4])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[5])) << 16);
    o.w = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[6])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[7])) << 16);
    *(reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.out) + (long long)t * p.N) + c) = o;
  }
}

}  // namespace mmb

MMB_API int mmb_ep_dispatch(const MmbEpDispatchParams* p, cudaStream_t stream) {
  if (p->ep < 1 || p->ep > mmb::kEpMaxRanks || p->H % 8 != 0 || p->ldx % 8 != 0 || p->topk < 1 || p->cap < 1 || p->experts_per_rank < 1 ||
      p->rank < 0 || p->rank >= p->ep || p->T < 0)
    return (int)cudaErrorInvalidValue;
  // T == 0 still launches: the (zero) counts and the flags must reach the peers
  long long blocks = ((long long)p->T * p->topk + 7) / 8;
  blocks = blocks < 1 ? 1 : (blocks > 148 * 8 ? 148 * 8 : blocks);
  return mmb::launch(mmb::ep_dispatch_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, 1, *p);
}

MMB_API int mmb_ep_recv_group(const MmbEpRecvParams* p, cudaStream_t stream) {
  if (p->ep < 1 || p->ep > mmb::kEpMaxRanks || p->E_local < 1 || p->E_local > mmb::kEpMaxExperts || p->token_tile < 1 || p->max_tiles < 1 ||
      p->cap < 1)
    return (int)cudaErrorInvalidValue;
  return mmb::launch(mmb::ep_recv_group_kernel, dim3(1), dim3(1024), 0, stream, 1, *p);
}

MMB_API int mmb_ep_signal(unsigned* const* peer_flags, const unsigned* step, int ep, cudaStream_t stream) {
  if (ep < 1 || ep > mmb::kEpMaxRanks) return (int)cudaErrorInvalidValue;
  return mmb::launch(mmb::ep_signal_kernel, dim3(1), dim3(32), 0, stream, 1, peer_flags, step, ep);
}

MMB_API int mmb_ep_combine(const MmbEpCombineParams* p, cudaStream_t stream) {
  if (p->ep < 1 || p->ep > mmb::kEpMaxRanks || p->N % 8 != 0 || p->topk < 1) return (int)cudaErrorInvalidValue;
  long long blocks = ((long long)p->T * (p->N / 8) + 255) / 256;
  blocks = blocks < 1 ? 1 : (blocks > 148 * 8 ? 148 * 8 : blocks);
  return mmb::launch(mmb::ep_combine_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, 1, *p);
}
