// Decode chain kernel (see api_chain.h): the weight-streaming links between two attention calls of a small-batch decode
// step as phases of one persistent grid.
//
// Grid: one CTA per SM, 16 warps.  A phase stages its activation rows once per CTA in shared memory (fp16, in the order
// the MMA B fragments are read; residual add and RMSNorm fused, rounded like the unfused kernels), then the CTAs walk the
// phase's units - a 16-row tile of the matrix, or a gate / up tile pair - round-robin.  The warps of a CTA form groups of
// `wpt` (as large as still gives every unit a group in one round) that split a unit's K axis, keep four 512-byte weight
// blocks per warp in flight in registers, expand E2M1 to fp16 A fragments (three integer operations per register) for
// mma.sync m16n8k16 and apply each quantization group's scale to a per-group accumulator in fp32, so the W4A16 arithmetic
// is exact like in the stand-alone kernels (gemv.cu).  Partial tiles meet in shared memory; outputs go to global memory
// (L2) for the next phase, which reads them with ld.global.cg after a grid barrier.
//
// Grid barrier: arrival counter in global memory, one atomic per CTA, acquire spin by thread 0 with a wall-clock limit.
#include "api_chain.h"
#include "common.cuh"
#include "router_select.cuh"

namespace mmb {

constexpr int kCW = 16;                 // warps per CTA
constexpr int kCT = kCW * 32;
constexpr unsigned long long kChainWaitNs = 500000000ull;    // 0.5 s per barrier
constexpr int kMaxSlots = 16;           // topk + shared experts per token
constexpr int kPF = 4;                  // weight blocks a warp keeps in flight

struct ChainShared {
  float red[kCW][2][128];
  float ss_red[kCW][8];
  float rstd[8];
  float logit[kMaxExperts];
  float choice[kMaxExperts];
  float group[64];
  int slot_e[8][kMaxSlots];
  float slot_w[8][kMaxSlots];
  int sel_ids[8 * 32];
  float sel_w[8 * 32];
  int ok;
};

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ldcg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
// Activations another CTA wrote earlier in this launch are read through L2 (ld.global.cg), never through this SM's L1.
__device__ __forceinline__ float ld_bf16_cg(const bf16* p) {
  return __uint_as_float((uint32_t)__ldcg(reinterpret_cast<const unsigned short*>(p)) << 16);
}

// Position of element k of a staged row (fragment order inside every 32-element block).
__device__ __forceinline__ int xs_off(int k) { return (k & ~31) + ((k >> 4) & 1) * 4 + ((k >> 3) & 1) * 2 + ((k & 7) >> 1) * 8 + (k & 1); }

// All CTAs of the grid; returns false when the wait ran out or another CTA gave up.
__device__ bool grid_barrier(const MmbChainParams& p, ChainShared* sh, unsigned& epoch, int code) {
  __syncthreads();
  if (threadIdx.x == 0) {
    bool ok = true;
    ++epoch;
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.sync) : "memory");      // orders this CTA's earlier writes (after bar.sync: cumulative)
    const unsigned target = epoch * gridDim.x;
    if (ld_acquire_u32(p.sync) < target) {
      const unsigned long long t0 = globaltimer_ns();
      for (unsigned it = 1;; ++it) {
        if (ld_acquire_u32(p.sync) >= target) break;
        if ((it & 63u) == 0u) {
          if (ld_acquire_u32(p.sync + 2) != 0u) {
            ok = false;
            break;
          }
          if (globaltimer_ns() - t0 > kChainWaitNs) {
            if (p.status) atomicExch(p.status, code);
            atomicExch(p.sync + 2, 1u);
            ok = false;
            break;
          }
        }
      }
    }
    __threadfence();
    sh->ok = ok ? 1 : 0;
  }
  __syncthreads();
  return sh->ok != 0;
}

// Rows [B] of x (+ delta), rounded to bf16 like an unfused add, optionally normalised (rounded to bf16 like an unfused
// RMSNorm), staged as fp16 in fragment order; columns [Kx, K) are zero.  `resid` (written by one CTA) receives x + delta.
__device__ void stage_rows(const bf16* x, long long ldx, const bf16* delta, long long ldd, bf16* resid, long long ldr,
                           const bf16* nw, int B, int K, int Kx, float eps, __half* xs, int XS, ChainShared* sh) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int j = 0; j < B; ++j) {
    float ss = 0.f;
    __half* dst = xs + (long long)j * XS;
    for (int k = tid * 8; k < K; k += kCT * 8) {
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (k < Kx) {
        const uint4 xv = ldcg16(x + (long long)j * ldx + k);
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[2 * e] = __uint_as_float(xw[e] << 16);
          v[2 * e + 1] = __uint_as_float(xw[e] & 0xffff0000u);
        }
        if (delta != nullptr) {
          const uint4 dv = ldcg16(delta + (long long)j * ldd + k);
          const uint32_t dw[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            v[2 * e] = __bfloat162float(__float2bfloat16(v[2 * e] + __uint_as_float(dw[e] << 16)));
            v[2 * e + 1] = __bfloat162float(__float2bfloat16(v[2 * e + 1] + __uint_as_float(dw[e] & 0xffff0000u)));
          }
          if (resid != nullptr) {
            uint4 o;
            o.x = (__float_as_uint(v[0]) >> 16) | (__float_as_uint(v[1]) & 0xffff0000u);
            o.y = (__float_as_uint(v[2]) >> 16) | (__float_as_uint(v[3]) & 0xffff0000u);
            o.z = (__float_as_uint(v[4]) >> 16) | (__float_as_uint(v[5]) & 0xffff0000u);
            o.w = (__float_as_uint(v[6]) >> 16) | (__float_as_uint(v[7]) & 0xffff0000u);
            *reinterpret_cast<uint4*>(resid + (long long)j * ldr + k) = o;
          }
        } else if (resid != nullptr) {
          *reinterpret_cast<uint4*>(resid + (long long)j * ldr + k) = xv;
        }
      }
      __half* blk = dst + (k & ~31) + ((k >> 4) & 1) * 4 + ((k >> 3) & 1) * 2;
      if (nw != nullptr) {
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
#pragma unroll
        for (int tt = 0; tt < 4; ++tt)      // park the bf16 bits; pass B rewrites them
          *reinterpret_cast<uint32_t*>(blk + tt * 8) = (__float_as_uint(v[2 * tt]) >> 16) | (__float_as_uint(v[2 * tt + 1]) & 0xffff0000u);
      } else {
#pragma unroll
        for (int tt = 0; tt < 4; ++tt)
          *reinterpret_cast<__half2*>(blk + tt * 8) = __floats2half2_rn(fminf(fmaxf(v[2 * tt], -65504.f), 65504.f),
                                                                        fminf(fmaxf(v[2 * tt + 1], -65504.f), 65504.f));
      }
    }
    if (nw != nullptr) {
      ss = warp_sum(ss);
      if (lane == 0) sh->ss_red[warp][j] = ss;
    }
  }
  __syncthreads();
  if (nw != nullptr) {
    if (tid < B) {
      float tot = 0.f;
      for (int w = 0; w < kCW; ++w) tot += sh->ss_red[w][tid];
      sh->rstd[tid] = rsqrtf(tot / (float)Kx + eps);
    }
    __syncthreads();
    for (int j = 0; j < B; ++j) {
      const float rs = sh->rstd[j];
      __half* dst = xs + (long long)j * XS;
      for (int k = tid * 8; k < Kx; k += kCT * 8) {
        const uint4 nv = __ldg(reinterpret_cast<const uint4*>(nw + k));
        const uint32_t nww[4] = {nv.x, nv.y, nv.z, nv.w};
        __half* blk = dst + (k & ~31) + ((k >> 4) & 1) * 4 + ((k >> 3) & 1) * 2;
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
          const uint32_t bits = *reinterpret_cast<const uint32_t*>(blk + tt * 8);
          float a = __bfloat162float(__float2bfloat16(__uint_as_float(bits << 16) * rs * __uint_as_float(nww[tt] << 16)));
          float b = __bfloat162float(__float2bfloat16(__uint_as_float(bits & 0xffff0000u) * rs * __uint_as_float(nww[tt] & 0xffff0000u)));
          a = fminf(fmaxf(a, -65504.f), 65504.f);
          b = fminf(fmaxf(b, -65504.f), 65504.f);
          *reinterpret_cast<__half2*>(blk + tt * 8) = __floats2half2_rn(a, b);
        }
      }
    }
    __syncthreads();
  }
}

struct GemvJob {
  MmbChainMat W;
  int act;            // 1: a unit is the pair (gate tile rt, up tile rt + n_rt / 2)
  int per_token;      // 1: units enumerate (token, [slot,] tile); the token's own row is the only column
  int nslot;          // gate|up with per_token: slots to run per token, starting at slot_first
  int slot_first;
  int nseg;           // down with per_token: segments (slots) of the virtual K axis; otherwise 1
  int B;
  bf16* out;
  long long ld_tok;   // output elements per token
  int I;              // gate|up: output features per slot
  int S;              // gate|up: slots per token in `out`
};


__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Ask L2 for every weight block (and scale block) this warp will read in job `j`, so that the phase that runs the job
// finds its weights on chip: the HBM transfer then overlaps the phase before it and the grid barrier between them.
// `slots_known`: the expert tables of this CTA are valid (jobs over routed experts cannot be requested earlier).
__device__ void l2_prefetch_job(const GemvJob& j, const ChainShared* sh, bool slots_known) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (j.W.q == nullptr) return;
  if (j.per_token && !slots_known) return;
  const int n_rt = (j.W.N + 15) >> 4;
  const int tps = j.act ? (n_rt >> 1) : n_rt;
  int n_units = tps;
  if (j.per_token) n_units = j.B * (j.nseg > 1 ? 1 : j.nslot) * tps;
  int wpt = kCW;
  while (wpt > 1 && n_units > (int)gridDim.x * (kCW / wpt)) wpt >>= 1;
  const int G = kCW / wpt, grp = warp / wpt, wi = warp - grp * wpt, TG = gridDim.x * G;
  const int KC = j.W.K >> 6, NG = j.W.K >> j.W.gs_shift;
  const int cpg = max(1, (1 << j.W.gs_shift) >> 6);
  const int total = (j.nseg * KC) / cpg;
  const int c0 = (int)(((long long)wi * total) / wpt) * cpg, c1 = (int)(((long long)(wi + 1) * total) / wpt) * cpg;
  const uint4* qb = reinterpret_cast<const uint4*>(j.W.q);
  const uint32_t* sb = reinterpret_cast<const uint32_t*>(j.W.s);
  for (int u = blockIdx.x * G + grp; u < n_units; u += TG) {
    int tok = 0, rt0 = u, e = 0;
    if (j.per_token) {
      const int per_tok = (j.nseg > 1 ? 1 : j.nslot) * tps;
      tok = u / per_tok;
      const int r = u - tok * per_tok;
      if (j.nseg > 1) {
        rt0 = r;
      } else {
        e = sh->slot_e[tok][j.slot_first + r / tps];
        rt0 = r - (r / tps) * tps;
      }
    }
    for (int tsel = 0; tsel < (j.act ? 2 : 1); ++tsel) {
      const int rt = rt0 + tsel * (n_rt >> 1);
      if (j.nseg > 1) {
        for (int c = c0 + (lane >> 2); c < c1; c += 8) {        // four 128-byte lines per 512-byte block
          const int seg = c / KC, cc = c - seg * KC;
          const int es = sh->slot_e[tok][seg];
          if (es >= 0) prefetch_l2(reinterpret_cast<const unsigned char*>(qb + (long long)es * j.W.stride_q + ((long long)rt * KC + cc) * 32) + (lane & 3) * 128);
        }
        if (wi == 0 && lane < j.nseg) {
          const int es = sh->slot_e[tok][lane];
          if (es >= 0) prefetch_l2(sb + (long long)es * j.W.stride_s + (long long)rt * NG * 8);
        }
      } else if (e >= 0) {
        const unsigned char* base = reinterpret_cast<const unsigned char*>(qb + (long long)e * j.W.stride_q + ((long long)rt * KC + c0) * 32);
        for (int i = lane; i < (c1 - c0) * 4; i += 32) prefetch_l2(base + (long long)i * 128);
        if (wi == 0) {
          const unsigned char* sbase = reinterpret_cast<const unsigned char*>(sb + (long long)e * j.W.stride_s + (long long)rt * NG * 8);
          for (int i = lane; i * 128 < NG * 32; i += 32) prefetch_l2(sbase + (long long)i * 128);
        }
      }
    }
  }
}

// One warp's share of one 16-row tile: chunks [c0, c1) of the (virtual) K axis.
__device__ __forceinline__ void gemv_tile(const GemvJob& j, const ChainShared* sh, const __half* xrow, int tok, int rt, int c0, int c1,
                                          int fixed_e, float (&acc)[4]) {
  const int lane = threadIdx.x & 31, g = lane >> 2;
  const int KC = j.W.K >> 6, NG = j.W.K >> j.W.gs_shift, gs = 1 << j.W.gs_shift, gmask = gs - 1;
  const uint4* qb = reinterpret_cast<const uint4*>(j.W.q);
  const uint32_t* sb = reinterpret_cast<const uint32_t*>(j.W.s);
  float gacc[4] = {0.f, 0.f, 0.f, 0.f};
  acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
  const int n = c1 - c0;
  uint4 wbuf[kPF];
  uint32_t sbuf[kPF];
  auto fetch = [&](int c, uint4& w, uint32_t& s) {
    int seg = 0, cc = c, e = fixed_e;
    if (j.nseg > 1) {
      seg = c / KC;
      cc = c - seg * KC;
      e = sh->slot_e[tok][seg];
    }
    if (e < 0) {
      w = make_uint4(0, 0, 0, 0);
      s = 0u;
      return;
    }
    w = ldg_stream(qb + (long long)e * j.W.stride_q + ((long long)rt * KC + cc) * 32 + lane);
    s = __ldg(sb + (long long)e * j.W.stride_s + (long long)rt * NG * 8 + ((cc * 64) >> j.W.gs_shift) * 8 + g);
  };
#pragma unroll
  for (int i = 0; i < kPF; ++i)
    if (i < n) fetch(c0 + i, wbuf[i], sbuf[i]);
  for (int base = 0; base < n; base += kPF) {
    uint4 wc[kPF];
    uint32_t sc[kPF];
#pragma unroll
    for (int i = 0; i < kPF; ++i) {
      wc[i] = wbuf[i];
      sc[i] = sbuf[i];
    }
#pragma unroll
    for (int i = 0; i < kPF; ++i)
      if (base + kPF + i < n) fetch(c0 + base + kPF + i, wbuf[i], sbuf[i]);
#pragma unroll
    for (int i = 0; i < kPF; ++i) {
      if (base + i >= n) break;
      const int c = c0 + base + i;
      int seg = 0, cc = c;
      float mult = kE2M1F16Rescale;
      if (j.nseg > 1) {
        seg = c / KC;
        cc = c - seg * KC;
        mult *= sh->slot_w[tok][seg];
      }
      const __half* xp = xrow + (long long)seg * j.W.K + cc * 64;
      const uint4 xv0 = *reinterpret_cast<const uint4*>(xp);
      const uint4 xv1 = *reinterpret_cast<const uint4*>(xp + 32);
      const uint32_t bb[8] = {xv0.x, xv0.y, xv0.z, xv0.w, xv1.x, xv1.y, xv1.z, xv1.w};
      const uint32_t qq[4] = {wc[i].x, wc[i].y, wc[i].z, wc[i].w};
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t a0, a1, a2, a3;
        e2m1x8_to_f16x2(qq[ks], a0, a1, a2, a3);
        mma_f16_16816(gacc, a0, a1, a2, a3, bb[2 * ks], bb[2 * ks + 1]);
      }
      if ((((cc + 1) * 64) & gmask) == 0) {       // quantization group complete: its scale, in fp32
        const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&sc[i]));
        const float slo = sf.x * mult, shi = sf.y * mult;
        acc[0] = fmaf(gacc[0], slo, acc[0]);
        acc[1] = fmaf(gacc[1], slo, acc[1]);
        acc[2] = fmaf(gacc[2], shi, acc[2]);
        acc[3] = fmaf(gacc[3], shi, acc[3]);
        gacc[0] = gacc[1] = gacc[2] = gacc[3] = 0.f;
      }
    }
  }
}

__device__ void run_gemv(const GemvJob& j, const __half* xs, int XS, ChainShared* sh) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int n_rt = (j.W.N + 15) >> 4;
  const int tps = j.act ? (n_rt >> 1) : n_rt;                         // units per matrix
  int n_units = tps;
  if (j.per_token) n_units = j.B * (j.nseg > 1 ? 1 : j.nslot) * tps;
  int wpt = kCW;
  while (wpt > 1 && n_units > (int)gridDim.x * (kCW / wpt)) wpt >>= 1;
  const int G = kCW / wpt, grp = warp / wpt, wi = warp - grp * wpt, TG = gridDim.x * G;
  const int KC = j.W.K >> 6;
  const int cpg = max(1, (1 << j.W.gs_shift) >> 6);                    // chunks per quantization group
  const int total = (j.nseg * KC) / cpg;
  const int c0 = (int)(((long long)wi * total) / wpt) * cpg, c1 = (int)(((long long)(wi + 1) * total) / wpt) * cpg;
  const int n_valid = j.act ? (j.W.N >> 1) : j.W.N;
  for (int u = blockIdx.x * G + grp; u < n_units; u += TG) {
    int tok = 0, sl = 0, rt0 = u, e = 0;
    if (j.per_token) {
      const int per_tok = (j.nseg > 1 ? 1 : j.nslot) * tps;
      tok = u / per_tok;
      const int r = u - tok * per_tok;
      if (j.nseg > 1) {
        rt0 = r;
      } else {
        sl = j.slot_first + r / tps;
        rt0 = r - (r / tps) * tps;
        e = sh->slot_e[tok][sl];
      }
    }
    const __half* xrow = xs + (long long)(j.per_token ? tok : min(g, j.B - 1)) * XS + t * 8;
    float accg[4], accu[4] = {0.f, 0.f, 0.f, 0.f};
    gemv_tile(j, sh, xrow, tok, rt0, c0, c1, e, accg);
    if (j.act) gemv_tile(j, sh, xrow, tok, rt0 + (n_rt >> 1), c0, c1, e, accu);
    float* r0 = &sh->red[warp][0][0];
    r0[g * 8 + 2 * t] = accg[0];
    r0[g * 8 + 2 * t + 1] = accg[1];
    r0[(g + 8) * 8 + 2 * t] = accg[2];
    r0[(g + 8) * 8 + 2 * t + 1] = accg[3];
    if (j.act) {
      float* r1 = &sh->red[warp][1][0];
      r1[g * 8 + 2 * t] = accu[0];
      r1[g * 8 + 2 * t + 1] = accu[1];
      r1[(g + 8) * 8 + 2 * t] = accu[2];
      r1[(g + 8) * 8 + 2 * t + 1] = accu[3];
    }
    if (wpt > 1) asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(wpt * 32) : "memory");
    else __syncwarp();
    const int w0 = grp * wpt;
    for (int o = wi * 32 + lane; o < 128; o += wpt * 32) {
      const int row = o >> 3, col = o & 7;
      if (j.per_token ? (col != 0) : (col >= j.B)) continue;
      const int nf = rt0 * 16 + row;
      if (nf >= n_valid) continue;
      float v = 0.f;
      for (int w2 = 0; w2 < wpt; ++w2) v += sh->red[w0 + w2][0][o];
      if (j.act) {
        float uu = 0.f;
        for (int w2 = 0; w2 < wpt; ++w2) uu += sh->red[w0 + w2][1][o];
        v = silu(v) * uu;
      }
      long long idx;
      if (j.per_token && j.nseg == 1) idx = ((long long)tok * j.S + sl) * j.I + nf;
      else idx = (long long)(j.per_token ? tok : col) * j.ld_tok + nf;
      j.out[idx] = __float2bfloat16(v);
    }
    if (wpt > 1) asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(wpt * 32) : "memory");
    else __syncwarp();
  }
}

__global__ void __launch_bounds__(kCT, 1) decode_chain_kernel(const MmbChainParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ ChainShared sh_s;
  ChainShared* sh = &sh_s;
  __half* xs = reinterpret_cast<__half*>(smem_raw);
  const int XS = p.stage_k + 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int B = p.B, H = p.H;
  const int S = p.moe ? (p.topk + p.n_shared) : 1;
  const int I = p.gate_up.N >> 1;
  unsigned epoch = 0;
  bool alive = true;
  const bool first_cta = blockIdx.x == 0;

  // ---- the jobs of the launch, built up front so that every phase can ask L2 for the weights of the next one
  GemvJob jA{}, jBs{}, jBd{}, jC{}, jD{}, jE{}, jF{};
  jA.W = p.o; jA.nseg = 1; jA.B = B; jA.out = reinterpret_cast<bf16*>(p.delta_attn); jA.ld_tok = H;
  jBs.W = p.gate_up; jBs.act = 1; jBs.per_token = 1; jBs.nslot = p.n_shared; jBs.slot_first = p.topk; jBs.nseg = 1; jBs.B = B;
  jBs.out = reinterpret_cast<bf16*>(p.hmid); jBs.I = I; jBs.S = S;
  jBd.W = p.gate_up; jBd.act = 1; jBd.nseg = 1; jBd.B = B; jBd.out = reinterpret_cast<bf16*>(p.hmid); jBd.ld_tok = I;
  jC = jBs; jC.nslot = p.topk; jC.slot_first = 0;
  jD.W = p.down; jD.per_token = p.moe ? 1 : 0; jD.nslot = 1; jD.nseg = p.moe ? S : 1; jD.B = B;
  jD.out = reinterpret_cast<bf16*>(p.delta_mlp); jD.ld_tok = H;
  jE.W = p.qa_kva; jE.nseg = 1; jE.B = B; jE.out = reinterpret_cast<bf16*>(p.a_out); jE.ld_tok = p.qa_kva.N;
  jF.W = p.q_b; jF.nseg = 1; jF.B = B; jF.out = reinterpret_cast<bf16*>(p.q_out); jF.ld_tok = p.q_b.N;
  const bool hasA = p.phases & MMB_CHAIN_A, hasB = p.phases & MMB_CHAIN_B, hasC = (p.phases & MMB_CHAIN_C) && p.moe,
             hasD = p.phases & MMB_CHAIN_D, hasE = p.phases & MMB_CHAIN_E, hasF = p.phases & MMB_CHAIN_F, hasG = p.phases & MMB_CHAIN_G;
  // shared-expert slots are known from the start (routed slots are filled in by phase C)
  if (tid < 8 * kMaxSlots) {
    const int b = tid / kMaxSlots, sl = tid % kMaxSlots;
    sh->slot_e[b][sl] = (p.moe && sl >= p.topk && sl < S) ? p.E + (sl - p.topk) : -1;
    sh->slot_w[b][sl] = 1.f;
  }
  __syncthreads();
  // weights of the first phase of the launch (nobody asked for them yet), requested before anything else
  if (hasA) l2_prefetch_job(jA, sh, true);
  else if (hasE) l2_prefetch_job(jE, sh, true);

  // ------------------------------------------------------------------ A: o_proj
  if (alive && hasA) {
    stage_rows(reinterpret_cast<const bf16*>(p.attn_o), p.o.K, nullptr, 0, nullptr, 0, nullptr, B, p.o.K, p.o.K, p.eps, xs, XS, sh);
    if (hasB) l2_prefetch_job(p.moe ? jBs : jBd, sh, true);
    run_gemv(jA, xs, XS, sh);
    alive = grid_barrier(p, sh, epoch, 300);
  }
  // ------------------------------------------------------------------ B: h_mid, post norm, router logits (+ shared experts) or dense gate|up
  if (alive && hasB) {
    stage_rows(reinterpret_cast<const bf16*>(p.h_in), H, reinterpret_cast<const bf16*>(p.delta_attn), H,
               first_cta ? reinterpret_cast<bf16*>(p.h_mid) : nullptr, H, reinterpret_cast<const bf16*>(p.post_norm), B, H, H, p.eps, xs, XS,
               sh);
    if (p.moe) {
      const bf16* Wr = reinterpret_cast<const bf16*>(p.router_w);
      for (int e = blockIdx.x; e < p.E; e += gridDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k = tid * 8; k < H; k += kCT * 8) {
          const uint4 w4 = ldg_stream(reinterpret_cast<const uint4*>(Wr + (long long)e * H + k));
          const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
          const int off = (k & ~31) + ((k >> 4) & 1) * 4 + ((k >> 3) & 1) * 2;
          for (int b = 0; b < B; ++b) {
            const __half* xb = xs + (long long)b * XS + off;
#pragma unroll
            for (int tt = 0; tt < 4; ++tt) {
              const float2 xv = __half22float2(*reinterpret_cast<const __half2*>(xb + tt * 8));
              acc[b] = fmaf(__uint_as_float(ww[tt] << 16), xv.x, acc[b]);
              acc[b] = fmaf(__uint_as_float(ww[tt] & 0xffff0000u), xv.y, acc[b]);
            }
          }
        }
        for (int b = 0; b < B; ++b) {
          const float v = warp_sum(acc[b]);
          if (lane == 0) sh->ss_red[warp][b] = v;
        }
        __syncthreads();
        if (tid < B) {
          float tot = 0.f;
          for (int w = 0; w < kCW; ++w) tot += sh->ss_red[w][tid];
          p.logits[(long long)tid * p.E + e] = tot;
        }
        __syncthreads();
      }
      if (p.n_shared > 0) run_gemv(jBs, xs, XS, sh);   // the shared experts do not depend on the routing
    } else {
      if (hasD) l2_prefetch_job(jD, sh, true);
      run_gemv(jBd, xs, XS, sh);
    }
    alive = grid_barrier(p, sh, epoch, 301);
  }
  // ------------------------------------------------------------------ C: selection (every CTA for itself) + routed gate|up
  if (alive && hasC) {
    if (warp == 0) {
      MmbRouterParams rp{};
      rp.E = p.E;
      rp.topk = p.topk;
      rp.scoring = p.scoring;
      rp.renorm = p.renorm;
      rp.routed_scale = p.routed_scale;
      rp.n_group = p.n_group;
      rp.topk_group = p.topk_group;
      rp.bias = p.router_bias;
      rp.ids = sh->sel_ids;
      rp.weights = sh->sel_w;
      rp.counts = nullptr;
      for (int b = 0; b < B; ++b) {
        for (int e = lane; e < p.E; e += 32) sh->logit[e] = __ldcg(p.logits + (long long)b * p.E + e);
        __syncwarp();
        router_select(rp, b, sh->logit, sh->choice, sh->group, lane);
        __syncwarp();
      }
    }
    __syncthreads();
    if (tid < 8 * kMaxSlots) {
      const int b = tid / kMaxSlots, sl = tid % kMaxSlots;
      if (b < B && sl < p.topk) {
        const int e = sh->sel_ids[b * p.topk + sl];
        const float w = sh->sel_w[b * p.topk + sl];
        sh->slot_e[b][sl] = e;
        sh->slot_w[b][sl] = w;
        if (first_cta) {
          p.ids[b * p.topk + sl] = e;
          p.weights[b * p.topk + sl] = w;
        }
      }
    }
    __syncthreads();
    if (!hasB)      // stand-alone use of this phase: the staged rows of phase B are not there
      stage_rows(reinterpret_cast<const bf16*>(p.h_mid), H, nullptr, 0, nullptr, 0, reinterpret_cast<const bf16*>(p.post_norm), B, H, H,
                 p.eps, xs, XS, sh);
    l2_prefetch_job(jC, sh, true);              // this phase's own weights: known only now
    if (hasD) l2_prefetch_job(jD, sh, true);    // and the down projections of the same experts
    run_gemv(jC, xs, XS, sh);
    alive = grid_barrier(p, sh, epoch, 302);
  }
  // ------------------------------------------------------------------ D: down
  if (alive && hasD) {
    if (p.moe && !hasC) {
      // stand-alone: the routed slots come from the ids / weights a previous launch left in global memory
      if (tid < 8 * kMaxSlots) {
        const int b = tid / kMaxSlots, sl = tid % kMaxSlots;
        if (b < B && sl < p.topk) {
          sh->slot_e[b][sl] = __ldcg(p.ids + b * p.topk + sl);
          sh->slot_w[b][sl] = __ldcg(p.weights + b * p.topk + sl);
        }
      }
      __syncthreads();
    }
    stage_rows(reinterpret_cast<const bf16*>(p.hmid), (long long)S * I, nullptr, 0, nullptr, 0, nullptr, B, S * I, S * I, p.eps, xs, XS, sh);
    if (hasE) l2_prefetch_job(jE, sh, true);
    run_gemv(jD, xs, XS, sh);
    alive = grid_barrier(p, sh, epoch, 303);
  }
  // ------------------------------------------------------------------ E: h_out, input norm, q_a | kv_a
  if (alive && hasE) {
    const bool has_delta = hasD || p.delta_mlp != nullptr;
    stage_rows(reinterpret_cast<const bf16*>(p.h_mid), H, has_delta ? reinterpret_cast<const bf16*>(p.delta_mlp) : nullptr, H,
               first_cta ? reinterpret_cast<bf16*>(p.h_out) : nullptr, H, reinterpret_cast<const bf16*>(p.in_norm), B, H, H, p.eps, xs, XS, sh);
    if (hasF) l2_prefetch_job(jF, sh, true);
    run_gemv(jE, xs, XS, sh);
    alive = grid_barrier(p, sh, epoch, 304);
  }
  // ------------------------------------------------------------------ F: q_b; last CTA first writes the new latent row
  if (alive && hasF) {
    const bf16* a = reinterpret_cast<const bf16*>(p.a_out);
    const int lda = p.qa_kva.N, dl = p.R + p.dr;
    if (hasG) {
      // W_uk^T rows of phase G (bf16, one row per warp and trip)
      const bf16* W = reinterpret_cast<const bf16*>(p.w_ukT);
      const int rows = p.nh * p.R, gw = blockIdx.x * kCW + warp, nwarps = gridDim.x * kCW;
      for (int r = gw; r < rows; r += nwarps)
        if (lane * 64 < p.dn) prefetch_l2(W + (long long)r * p.dn + lane * 64);
    }
    if (blockIdx.x == gridDim.x - 1) {
      const bf16* nw = reinterpret_cast<const bf16*>(p.kv_norm);
      bf16* cache = reinterpret_cast<bf16*>(p.cache);
      float* sm = sh->logit;                         // R <= kMaxExperts floats
      for (int j = 0; j < B; ++j) {
        const long long slot = p.slots[j];
        const bf16* src = a + (long long)j * lda + p.q_lora;
        float ss = 0.f;
        for (int d = tid; d < p.R; d += kCT) {
          const float v = ld_bf16_cg(src + d);
          sm[d] = v;
          ss += v * v;
        }
        ss = warp_sum(ss);
        if (lane == 0) sh->ss_red[warp][0] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < kCW; ++w) tot += sh->ss_red[w][0];
        const float rs = rsqrtf(tot / (float)p.R + p.eps);
        if (slot >= 0) {
          bf16* dst = cache + slot * dl;
          for (int d = tid; d < p.R; d += kCT) dst[d] = __float2bfloat16(sm[d] * rs * __bfloat162float(nw[d]));
          const int half = p.dr / 2;
          for (int f = tid; f < half; f += kCT) {
            float sn, cs;
            sincosf((float)p.positions[j] * p.inv_freq[f], &sn, &cs);
            const int ia = p.interleaved ? 2 * f : f, ib = p.interleaved ? 2 * f + 1 : f + half;
            const float va = ld_bf16_cg(src + p.R + ia), vb = ld_bf16_cg(src + p.R + ib);
            dst[p.R + ia] = __float2bfloat16((va * cs - vb * sn) * p.mscale);
            dst[p.R + ib] = __float2bfloat16((vb * cs + va * sn) * p.mscale);
          }
        }
        __syncthreads();
      }
    }
    stage_rows(a, lda, nullptr, 0, nullptr, 0, reinterpret_cast<const bf16*>(p.q_a_norm), B, p.q_b.K, p.q_lora, p.eps, xs, XS, sh);
    run_gemv(jF, xs, XS, sh);
    alive = grid_barrier(p, sh, epoch, 305);
  }
  // ------------------------------------------------------------------ G: absorb W_uk^T, RoPE(q_rope)
  if (alive && hasG) {
    const bf16* q = reinterpret_cast<const bf16*>(p.q_out);
    bf16* qf = reinterpret_cast<bf16*>(p.q_full);
    const bf16* W = reinterpret_cast<const bf16*>(p.w_ukT);
    const int dq = p.dn + p.dr, dl = p.R + p.dr, ldq = p.q_b.N;
    const int rows = p.nh * p.R;
    const int gw = blockIdx.x * kCW + warp, nwarps = gridDim.x * kCW;
    for (int r = gw; r < rows; r += nwarps) {
      const int h = r / p.R, rr = r - h * p.R;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (lane * 8 < p.dn) {
        const uint4 wv = ldg_stream(reinterpret_cast<const uint4*>(W + ((long long)h * p.R + rr) * p.dn + lane * 8));
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        for (int b = 0; b < B; ++b) {
          const uint4 xv = ldcg16(q + (long long)b * ldq + h * dq + lane * 8);
          const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[b] = fmaf(__uint_as_float(ww[e] << 16), __uint_as_float(xw[e] << 16), acc[b]);
            acc[b] = fmaf(__uint_as_float(ww[e] & 0xffff0000u), __uint_as_float(xw[e] & 0xffff0000u), acc[b]);
          }
        }
      }
      for (int b = 0; b < B; ++b) {
        const float v = warp_sum(acc[b]);
        if (lane == 0) qf[((long long)b * p.nh + h) * dl + rr] = __float2bfloat16(v);
      }
    }
    const int half = p.dr / 2;
    for (int i = blockIdx.x * kCT + tid; i < B * p.nh * half; i += gridDim.x * kCT) {
      const int b = i / (p.nh * half), rem = i - b * (p.nh * half), h = rem / half, f = rem - h * half;
      const bf16* src = q + (long long)b * ldq + h * dq + p.dn;
      float sn, cs;
      sincosf((float)p.positions[b] * p.inv_freq[f], &sn, &cs);
      const int ia = p.interleaved ? 2 * f : f, ib = p.interleaved ? 2 * f + 1 : f + half;
      const float va = ld_bf16_cg(src + ia), vb = ld_bf16_cg(src + ib);
      bf16* dst = qf + ((long long)b * p.nh + h) * dl + p.R;
      dst[ia] = __float2bfloat16((va * cs - vb * sn) * p.mscale);
      dst[ib] = __float2bfloat16((vb * cs + va * sn) * p.mscale);
    }
  }
  // weights the next kernels start with: ask L2 for them now, they arrive while this launch drains and the next one starts
  for (int r = 0; r < 2; ++r) {
    const unsigned char* base = reinterpret_cast<const unsigned char*>(p.pf_ptr[r]);
    if (base == nullptr) continue;
    const long long lines = p.pf_bytes[r] >> 7;
    for (long long i = (long long)blockIdx.x * kCT + tid; i < lines; i += (long long)gridDim.x * kCT) prefetch_l2(base + i * 128);
  }
  // ------------------------------------------------------------------ exit: the last CTA clears the counters for the next launch
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned prev = atomicAdd(p.sync + 1, 1u);
    if (prev == gridDim.x - 1) {
      atomicExch(p.sync, 0u);
      atomicExch(p.sync + 1, 0u);
    }
  }
}

}  // namespace mmb

MMB_API int mmb_decode_chain(const MmbChainParams* pp, cudaStream_t stream) {
  using namespace mmb;
  const MmbChainParams& p = *pp;
  if (p.B < 1 || p.B > 8 || p.sync == nullptr || p.stage_k <= 0 || (p.stage_k & 63)) return (int)cudaErrorInvalidValue;
  if (p.moe && (p.topk + p.n_shared > kMaxSlots || p.E > kMaxExperts || p.topk > 32 || p.n_group > 64)) return (int)cudaErrorInvalidValue;
  if ((p.phases & MMB_CHAIN_F) && p.R > kMaxExperts) return (int)cudaErrorInvalidValue;
  if ((p.phases & MMB_CHAIN_G) && (p.dn > 256 || (p.dn & 7))) return (int)cudaErrorInvalidValue;
  static int n_sm = 0;
  static size_t smem_set = 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (n_sm == 0) {
    e = cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
  }
  const size_t smem = (size_t)p.B * (p.stage_k + 32) * 2;
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > smem_set) {
    e = cudaFuncSetAttribute(decode_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    smem_set = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)n_sm);
  cfg.blockDim = dim3(kCT);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;      // all CTAs resident together: the grid barriers need it
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, decode_chain_kernel, p);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}
