// On-device sampler: repetition penalty, temperature, top-k, top-p, min-p, categorical draw, one CTA
// per row, token ids written to device memory (the decode loop never syncs with the host).
//
//   greedy (temperature <= 0)                   : block arg-max, ties -> lowest index
//   temperature only                            : Gumbel-max over the full vocabulary (exact, one pass)
//   top-k / top-p / min-p                       : 4-pass radix select of the k-th largest logit,
//                                                 candidates (<= 1024) gathered to shared memory,
//                                                 bitonic sort, nucleus cut, inverse-CDF draw
// When top-k is off the candidate set is capped at the 1024 largest logits; a nucleus that would
// extend past the cap is truncated there.
// Randomness: Philox-4x32-10 keyed by (seed), counter (offset, row, index).
#include "api.h"
#include "common.cuh"
#include "tp_comm.cuh"

namespace mmb {

constexpr int kSampThreads = 1024;
constexpr int kMaxCand = 1024;

__device__ __forceinline__ uint4 philox4x32(uint4 ctr, uint2 key) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}
__device__ __forceinline__ float u01(uint32_t r) { return ((float)(r >> 8) + 0.5f) * (1.0f / 16777216.0f); }

__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax argmax_combine(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ ArgMax block_argmax(ArgMax a, ArgMax* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = argmax_combine(a, b);
  }
  __syncthreads();
  if (lane == 0) red[w] = a;
  __syncthreads();
  ArgMax r = red[0];
  for (int j = 1; j < (int)(blockDim.x >> 5); ++j) r = argmax_combine(r, red[j]);
  return r;
}

__global__ void __launch_bounds__(kSampThreads) sample_kernel(const MmbSampleParams p) {
  extern __shared__ uint32_t bitmap[];                 // ceil(V / 32) words when a history is given
  __shared__ ArgMax red_am[32];
  __shared__ float red_f[32];
  __shared__ int hist[256];
  __shared__ float cand_v[kMaxCand];
  __shared__ int cand_i[kMaxCand];
  __shared__ int n_cand;
  __shared__ uint32_t sel_prefix;
  __shared__ int sel_remaining;
  const int tid = threadIdx.x;
  const long long row = blockIdx.x;
  const float* lg = p.logits + row * p.V;
  const float temp = p.temperature ? p.temperature[row] : 0.f;
  const int top_k = p.top_k ? p.top_k[row] : 0;
  const float top_p = p.top_p ? p.top_p[row] : 1.f;
  const float min_p = p.min_p ? p.min_p[row] : 0.f;
  const float rp = p.rep_penalty ? p.rep_penalty[row] : 1.f;
  const unsigned long long rng_off = p.offset + (p.offset_dev ? (unsigned long long)(*p.offset_dev) : 0ull);
  const unsigned long long seed = p.seed_dev ? (unsigned long long)p.seed_dev[row] : p.seed;   // per-row seeds survive graph replays
  const bool use_hist = (p.history != nullptr) && (rp != 1.f) && (p.hist_len > 0);
  if (use_hist) {
    const int words = (p.V + 31) / 32;
    for (int i = tid; i < words; i += kSampThreads) bitmap[i] = 0u;
    __syncthreads();
    for (int i = tid; i < p.hist_len; i += kSampThreads) {
      const long long t = p.history[row * p.hist_len + i];
      if (t >= 0 && t < p.V) atomicOr(&bitmap[t >> 5], 1u << (t & 31));
    }
    __syncthreads();
  }
  const float inv_t = (temp > 0.f) ? 1.f / temp : 1.f;
  auto logit_at = [&](int i) -> float {
    float v = lg[i];
    if (use_hist && ((bitmap[i >> 5] >> (i & 31)) & 1u)) v = (v > 0.f) ? v / rp : v * rp;
    return v * inv_t;
  };

  // ---- max (also the greedy answer)
  ArgMax am;
  am.v = -INFINITY;
  am.i = 0x7fffffff;
  for (int i = tid; i < p.V; i += kSampThreads) {
    ArgMax c;
    c.v = logit_at(i);
    c.i = i;
    am = argmax_combine(am, c);
  }
  am = block_argmax(am, red_am);
  const float vmax = am.v;
  // log partition function of the tempered (penalised) distribution
  float z = 0.f;
  for (int i = tid; i < p.V; i += kSampThreads) z += __expf(logit_at(i) - vmax);
  z = block_sum(z, red_f);

  const bool filtered = (top_k > 0) || (top_p < 1.f) || (min_p > 0.f);
  if (temp <= 0.f) {
    if (tid == 0) {
      p.out_ids[row] = am.i;
      if (p.out_logprob) p.out_logprob[row] = -__logf(z);
    }
    return;
  }
  if (!filtered) {
    // Gumbel-max: argmax(l_i + G_i)
    ArgMax gm;
    gm.v = -INFINITY;
    gm.i = 0x7fffffff;
    for (int i0 = tid * 4; i0 < p.V; i0 += kSampThreads * 4) {
      const uint4 r = philox4x32(make_uint4((uint32_t)rng_off, (uint32_t)(rng_off >> 32), (uint32_t)row, (uint32_t)(i0 >> 2)),
                                 make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
      const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = i0 + j;
        if (i < p.V) {
          ArgMax c;
          c.v = logit_at(i) - __logf(-__logf(u01(rr[j])));
          c.i = i;
          gm = argmax_combine(gm, c);
        }
      }
    }
    gm = block_argmax(gm, red_am);
    if (tid == 0) {
      p.out_ids[row] = gm.i;
      if (p.out_logprob) p.out_logprob[row] = logit_at(gm.i) - vmax - __logf(z);
    }
    return;
  }

  // ---- radix select: key of the k-th largest value
  const int k_sel = min(p.V, (top_k > 0) ? min(top_k, kMaxCand) : kMaxCand);
  if (tid == 0) {
    sel_prefix = 0u;
    sel_remaining = k_sel;
  }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = sel_prefix;
    const uint32_t pmask = (pass == 0) ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < p.V; i += kSampThreads) {
      const uint32_t key = float_key(logit_at(i));
      if ((key & pmask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int rem = sel_remaining;
      int dgt = 255;
      for (; dgt > 0; --dgt) {
        if (hist[dgt] >= rem) break;
        rem -= hist[dgt];
      }
      sel_prefix = prefix | ((uint32_t)dgt << shift);
      sel_remaining = rem;
    }
    __syncthreads();
  }
  const uint32_t kth_key = sel_prefix;     // every key >= kth_key is in the top-k (ties included)
  if (tid == 0) n_cand = 0;
  __syncthreads();
  for (int i = tid; i < p.V; i += kSampThreads) {
    const float v = logit_at(i);
    if (float_key(v) >= kth_key) {
      const int slot = atomicAdd(&n_cand, 1);
      if (slot < kMaxCand) {
        cand_v[slot] = v;
        cand_i[slot] = i;
      }
    }
  }
  __syncthreads();
  const int nc = min(n_cand, kMaxCand);
  for (int i = tid; i < kMaxCand; i += kSampThreads)
    if (i >= nc) {
      cand_v[i] = -INFINITY;
      cand_i[i] = 0x7fffffff;
    }
  __syncthreads();
  // ---- bitonic sort, descending by value then ascending by index
  for (int size = 2; size <= kMaxCand; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int i = tid;
      const int j = i ^ stride;
      if (j > i && i < kMaxCand) {
        const bool desc = ((i & size) == 0);
        const float vi = cand_v[i], vj = cand_v[j];
        const int ii = cand_i[i], ij = cand_i[j];
        const bool i_before_j = (vi > vj) || (vi == vj && ii < ij);
        if (i_before_j != desc) {
          cand_v[i] = vj;
          cand_v[j] = vi;
          cand_i[i] = ij;
          cand_i[j] = ii;
        }
      }
      __syncthreads();
    }
  }
  // ---- nucleus over the kept set (thread 0; <= 1024 sequential steps)
  if (tid == 0) {
    const int keep_k = (top_k > 0) ? min(nc, top_k) : nc;
    // denominator: the kept set when top-k is on (filters compose like successive renormalised
    // warpers), the full vocabulary otherwise
    float zk = 0.f;
    for (int i = 0; i < keep_k; ++i) zk += __expf(cand_v[i] - vmax);
    const float denom = (top_k > 0) ? zk : z;
    int n_keep = keep_k;
    if (top_p < 1.f) {
      float cum = 0.f;
      n_keep = 0;
      for (int i = 0; i < keep_k; ++i) {
        ++n_keep;
        cum += __expf(cand_v[i] - vmax) / denom;
        if (cum >= top_p) break;
      }
    }
    if (min_p > 0.f) {
      const float thr = __logf(min_p);
      int n2 = 0;
      for (int i = 0; i < n_keep; ++i)
        if (cand_v[i] - cand_v[0] >= thr) ++n2; else break;
      n_keep = max(1, n2);
    }
    float zz = 0.f;
    for (int i = 0; i < n_keep; ++i) zz += __expf(cand_v[i] - vmax);
    const uint4 r = philox4x32(make_uint4((uint32_t)rng_off, (uint32_t)(rng_off >> 32), (uint32_t)row, 0xffffffffu),
                               make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    const float target = u01(r.x) * zz;
    float cum = 0.f;
    int pick = n_keep - 1;
    for (int i = 0; i < n_keep; ++i) {
      cum += __expf(cand_v[i] - vmax);
      if (cum >= target) {
        pick = i;
        break;
      }
    }
    p.out_ids[row] = cand_i[pick];
    if (p.out_logprob) p.out_logprob[row] = cand_v[pick] - vmax - __logf(z);
  }
}

__global__ void __launch_bounds__(kSampThreads) argmax_kernel(const float* __restrict__ logits, int64_t* __restrict__ out,
                                                              int V) {
  __shared__ ArgMax red_am[32];
  const long long row = blockIdx.x;
  const float* lg = logits + row * V;
  ArgMax am;
  am.v = -INFINITY;
  am.i = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += kSampThreads) {
    ArgMax c;
    c.v = lg[i];
    c.i = i;
    am = argmax_combine(am, c);
  }
  am = block_argmax(am, red_am);
  if (threadIdx.x == 0) out[row] = am.i;
}

// Vocab-parallel greedy head: each rank arg-maxes its vocabulary shard, pushes (value, global index) for
// every row to all peers, waits for the tp pairs and picks the winner (ties -> lowest index), so all ranks
// end the step with the same token without moving the logits.  One CTA; B rows are handled in turn.
__global__ void __launch_bounds__(kSampThreads) tp_argmax_kernel(const float* __restrict__ logits, int64_t* __restrict__ out,
                                                                 int B, int Vloc, int vocab_offset, const MmbTpExchange x) {
  __shared__ ArgMax red_am[32];
  const int tid = threadIdx.x;
  for (int b = 0; b < B; ++b) {
    const float* lg = logits + (long long)b * Vloc;
    ArgMax am;
    am.v = -INFINITY;
    am.i = 0x7fffffff;
    for (int i = tid; i < Vloc; i += kSampThreads) {
      ArgMax c;
      c.v = lg[i];
      c.i = i;
      am = argmax_combine(am, c);
    }
    am = block_argmax(am, red_am);
    if (tid < x.tp) {
      float* dst = x.out_peer_slots[tid] + 2 * b;
      dst[0] = am.v;
      dst[1] = __int_as_float(am.i + vocab_offset);
    }
    __syncthreads();
  }
  __threadfence_system();
  __syncthreads();
  if (tid < x.tp) st_release_sys(x.out_peer_flags[tid], *x.step);
  TpIn tin;
  tin.buf = x.in_buf;
  tin.flags = x.in_flags;
  tin.step = x.step;
  tin.status = x.status;
  tin.tp = x.tp;
  tin.slot_stride = x.in_slot_stride;
  tp_wait(tin);
  for (int b = tid; b < B; b += kSampThreads) {
    ArgMax best;
    best.v = -INFINITY;
    best.i = 0x7fffffff;
    for (int r = 0; r < x.tp; ++r) {
      ArgMax c;
      c.v = __ldcg(x.in_buf + r * x.in_slot_stride + 2 * b);
      c.i = __float_as_int(__ldcg(x.in_buf + r * x.in_slot_stride + 2 * b + 1));
      best = argmax_combine(best, c);
    }
    out[b] = best.i;
  }
}

}  // namespace mmb

MMB_API int mmb_tp_argmax(const float* logits, int64_t* out, int B, int Vloc, int vocab_offset, const MmbTpExchange* x,
                          cudaStream_t stream) {
  if (B <= 0) return 0;
  if (x->tp < 1 || x->tp > 32 || x->out_peer_slots == nullptr || x->in_buf == nullptr) return (int)cudaErrorInvalidValue;
  mmb::tp_argmax_kernel<<<1, mmb::kSampThreads, 0, stream>>>(logits, out, B, Vloc, vocab_offset, *x);
  return (int)cudaGetLastError();
}

MMB_API int mmb_sample(const MmbSampleParams* pp, cudaStream_t stream) {
  const MmbSampleParams& p = *pp;
  if (p.B <= 0) return 0;
  size_t smem = 0;
  if (p.history != nullptr && p.hist_len > 0) smem = (size_t)((p.V + 31) / 32) * 4;
  if (smem > 32 * 1024) return (int)cudaErrorInvalidValue;   // vocabularies above ~260k need a larger bitmap
  mmb::sample_kernel<<<p.B, mmb::kSampThreads, smem, stream>>>(p);
  return (int)cudaGetLastError();
}

MMB_API int mmb_argmax(const float* logits, int64_t* out, int B, int V, cudaStream_t stream) {
  if (B <= 0) return 0;
  mmb::argmax_kernel<<<B, mmb::kSampThreads, 0, stream>>>(logits, out, V);
  return (int)cudaGetLastError();
}
