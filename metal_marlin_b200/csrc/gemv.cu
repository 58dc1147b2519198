// Weight-streaming small-M kernels (decode): FP4 tile-layout GEMV on mma.sync with fp32
// accumulation and exact per-group scaling, plus a bf16 GEMV for unquantized matrices.
//
// FP4 kernel design (sm_100a, HBM-bound):
//  * one CTA owns R row tiles (16 rows each); its 8 warps split the (virtual) K axis, every
//    warp streaming whole 512-byte tile blocks with one 16-byte load per lane;
//  * the eight nibbles of a word are turned into an fp16 A fragment with 3 integer ops per
//    register (no multiply): the fp16 value is e2m1 * 2^-14 and the factor is folded into the
//    group scale, which is applied in fp32 to a per-group accumulator -> exact W4A16 math;
//  * activations are staged once per CTA in shared memory as fp16 (optionally after a fused
//    residual add + RMSNorm), laid out so B-fragment loads are conflict free;
//  * MoE: the expert of a slot is read from device memory (no host sync); the down projection
//    treats the (slot, k) pairs of a token as one long virtual K axis, so the weighted sum over
//    experts needs no atomics and is deterministic.
#include "api.h"
#include "common.cuh"
#include "launch.h"
#include "tp_comm.cuh"

namespace mmb {

constexpr int kMaxSeg = 16;

struct SegPtr {
  const uint4* q;
  const uint32_t* s;
  float mult;
};

// Expert of a (token, slot): read from device memory, so routing never touches the host.
__device__ __forceinline__ SegPtr seg_lookup(const MmbFp4GemvParams& p, int token, int sl) {
  SegPtr r;
  int e = 0;
  r.mult = 1.f;
  if (p.mode != 0) {
    if (sl < p.topk) {
      e = __ldg(p.expert_ids + token * p.topk + sl);
      if (p.mode == 2) r.mult = __ldg(p.expert_w + token * p.topk + sl);
    } else {
      e = p.shared_base + (sl - p.topk);
    }
  }
  if (e < 0) {
    r.q = nullptr;
    r.s = nullptr;
    r.mult = 0.f;
  } else {
    r.q = reinterpret_cast<const uint4*>(p.qw) + (long long)e * p.expert_stride_q;
    r.s = reinterpret_cast<const uint32_t*>(p.sc) + (long long)e * p.expert_stride_s;
  }
  return r;
}

constexpr int kDepth = 4;   // 16-byte weight loads kept in flight per lane

// NWARPS warps per CTA (8 or 16), R row tiles per CTA.  Decode GEMVs are latency bound: the launcher picks
// NWARPS so that a warp owns only about two 64-wide chunks, which keeps the dependent instruction chain of
// every warp short.
template <int R, bool BIG_GROUPS, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32, 1) fp4_gemv_kernel(const MmbFp4GemvParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float red[NWARPS * 128];
  __shared__ float ss_red[NWARPS][8];
  __shared__ float rstd_s[8];
  constexpr int kGemvThreads = NWARPS * 32;
  constexpr int kGemvWarps = NWARPS;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  constexpr int WPT = kGemvWarps / R;

  const int S = (p.mode == 0) ? 1 : (p.topk + p.n_shared);
  int m0, mt, token = 0, slot = 0;
  if (p.mode == 0) {
    m0 = blockIdx.y * 8;
    mt = min(8, p.M - m0);
  } else if (p.mode == 1) {
    token = blockIdx.y / S;
    slot = blockIdx.y % S;
    m0 = token;
    mt = 1;
  } else {
    token = blockIdx.y;
    m0 = token;
    mt = 1;
  }
  const int nseg = (p.mode == 2) ? S : 1;
  const int Kv = nseg * p.K;   // virtual K
  const int XS = Kv + 32;      // smem row stride in halves: rows are 64 bytes apart mod 128 -> 16-byte loads of a
                               // quarter warp (2 rows x 4 lanes) touch distinct banks
  __half* xs = reinterpret_cast<__half*>(smem_raw);

  // ---- work assignment of this warp (depends on launch parameters only)
  const int n_rt = (p.N + 15) >> 4;
  const int ti = warp / WPT, wi = warp % WPT;
  int rt;
  if (p.act == 1) {
    rt = (ti == 0) ? (int)blockIdx.x : (int)blockIdx.x + (n_rt >> 1);   // R == 2 enforced by the launcher
  } else {
    rt = blockIdx.x * R + ti;
  }
  const int KC = p.K >> 6;                 // chunks per segment
  const int NG = p.K >> p.gs_shift;        // groups per segment
  const int gs = 1 << p.gs_shift;
  const int unit_chunks = (gs >= 64) ? (gs >> 6) : 1;
  const int total_units = (nseg * KC) / unit_chunks;
  int c_begin = (int)(((long long)wi * total_units) / WPT) * unit_chunks;
  int c_end = (int)(((long long)(wi + 1) * total_units) / WPT) * unit_chunks;
  if (rt >= n_rt) c_end = c_begin;

  // ---- issue the first weight loads before anything else: their DRAM latency overlaps the x staging
  uint4 w[kDepth];
  uint32_t sw[kDepth];      // group scale word travelling with each chunk (BIG_GROUPS)
  int ld_seg = -1;
  SegPtr lseg;
  lseg.q = nullptr;
  lseg.s = nullptr;
  lseg.mult = 0.f;
  const int cpg_shift_ld = p.gs_shift - 6;      // log2(chunks per group) when the group spans whole chunks
  auto load_chunk = [&](int ci, uint32_t& scale_word) -> uint4 {
    int sidx = 0, cc = ci;
    if (nseg > 1) {
      sidx = ci / KC;
      cc = ci - sidx * KC;
    }
    if (sidx != ld_seg) {
      lseg = seg_lookup(p, token, (p.mode == 1) ? slot : sidx);
      ld_seg = sidx;
    }
    if (lseg.q == nullptr) {
      scale_word = 0u;
      return make_uint4(0, 0, 0, 0);
    }
    if (BIG_GROUPS) scale_word = __ldg(lseg.s + ((long long)rt * NG + (cc >> cpg_shift_ld)) * 8 + g);
    return ldg_stream(lseg.q + ((long long)rt * KC + cc) * 32 + lane);
  };
  // Dense weights never change, so their first fetches are issued before waiting for the previous kernel;
  // MoE fetches depend on the router's expert ids and must come after the wait.
#pragma unroll
  for (int i = 0; i < kDepth; ++i) {
    w[i] = make_uint4(0, 0, 0, 0);
    sw[i] = 0u;
  }
  if (p.mode == 0) {
#pragma unroll
    for (int i = 0; i < kDepth; ++i)
      if (c_begin + i < c_end) w[i] = load_chunk(c_begin + i, sw[i]);
  }
  // the RMSNorm weight is static as well: fetch this thread's first slices now (the rest, for K > 4096, is
  // read where it is used)
  const bf16* nw = reinterpret_cast<const bf16*>(p.norm_w);
  constexpr int kNormCh = 2;
  uint4 nwv[kNormCh];
  if (nw != nullptr) {
#pragma unroll
    for (int j = 0; j < kNormCh; ++j) {
      const int k = tid * 8 + j * kGemvThreads * 8;
      nwv[j] = (k < p.Kx) ? *reinterpret_cast<const uint4*>(nw + k) : make_uint4(0, 0, 0, 0);
    }
  }
  pdl_launch_dependents();
  pdl_wait();
  if (p.mode != 0) {
#pragma unroll
    for (int i = 0; i < kDepth; ++i)
      if (c_begin + i < c_end) w[i] = load_chunk(c_begin + i, sw[i]);
  }

  // ---- stage activations as fp16 (optional residual add + RMSNorm), 8 elements per thread per trip
  const bf16* xg = reinterpret_cast<const bf16*>(p.x);
  const bf16* dg = reinterpret_cast<const bf16*>(p.delta);
  bf16* ro = reinterpret_cast<bf16*>(p.resid_out);
  const int rows_to_stage = (p.mode == 2) ? nseg : mt;
  // tensor-parallel consumer: the residual delta is the sum of the tp partials peers pushed into the local buffer
  const bool has_tin = p.tpx.in_buf != nullptr;
  TpIn tin;
  tin.buf = p.tpx.in_buf;
  tin.flags = p.tpx.in_flags;
  tin.step = p.tpx.step;
  tin.status = p.tpx.status;
  tin.tp = p.tpx.tp;
  tin.slot_stride = p.tpx.in_slot_stride;
  if (has_tin) tp_wait(tin);

  // value of (x + delta) for 8 consecutive elements of row j, rounded to bf16 like an unfused add would
  auto load8 = [&](int j, long long row, int k, float (&v)[8]) {
    const uint4 xv = *reinterpret_cast<const uint4*>(xg + row + k);
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[2 * e] = __uint_as_float(xw[e] << 16);
      v[2 * e + 1] = __uint_as_float(xw[e] & 0xffff0000u);
    }
    if (has_tin) {
      const long long idx = (long long)(m0 + j) * p.Kx + k;
      float d[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < tin.tp; ++r) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(tin.buf + r * tin.slot_stride + idx));
        const float4 b = __ldcg(reinterpret_cast<const float4*>(tin.buf + r * tin.slot_stride + idx + 4));
        d[0] += a.x; d[1] += a.y; d[2] += a.z; d[3] += a.w;
        d[4] += b.x; d[5] += b.y; d[6] += b.z; d[7] += b.w;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = __bfloat162float(__float2bfloat16(v[e] + d[e]));
    } else if (dg != nullptr) {
      const uint4 dv = *reinterpret_cast<const uint4*>(dg + row + k);
      const uint32_t dw[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[2 * e] = __bfloat162float(__float2bfloat16(v[2 * e] + __uint_as_float(dw[e] << 16)));
        v[2 * e + 1] = __bfloat162float(__float2bfloat16(v[2 * e + 1] + __uint_as_float(dw[e] & 0xffff0000u)));
      }
    }
  };

  if (nw != nullptr) {
    // pass 1: sum of squares per token row; one combined block reduction for all rows
    float ss[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) ss[j] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < rows_to_stage) {
        const long long row = (long long)(m0 + j) * p.ldx;
        for (int k = tid * 8; k < p.Kx; k += kGemvThreads * 8) {
          float v[8];
          load8(j, row, k, v);
#pragma unroll
          for (int e = 0; e < 8; ++e) ss[j] = fmaf(v[e], v[e], ss[j]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < rows_to_stage) {
        const float sred = warp_sum(ss[j]);
        if (lane == 0) ss_red[warp][j] = sred;
      }
    }
    __syncthreads();
    if (tid < rows_to_stage) {
      float tot = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < kGemvWarps; ++w2) tot += ss_red[w2][tid];
      rstd_s[tid] = rsqrtf(tot / (float)p.Kx + p.eps);
    }
    __syncthreads();
  }
  for (int j = 0; j < rows_to_stage; ++j) {
    long long row;
    __half* dst;
    if (p.mode == 2) {
      row = (long long)(token * S + j) * p.ldx;
      dst = xs + (long long)j * p.K;
    } else {
      row = (long long)(m0 + j) * p.ldx;
      dst = xs + (long long)j * XS;
    }
    const float rs = (nw != nullptr) ? rstd_s[j] : 1.f;
    for (int jj = 0, k = tid * 8; k < p.K; ++jj, k += kGemvThreads * 8) {
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (k < p.Kx) {
        load8(j, row, k, v);
        if ((dg != nullptr || has_tin) && ro != nullptr && blockIdx.x == 0 && (p.mode != 1 || slot == 0)) {
          uint4 o;
          o.x = (__float_as_uint(v[0]) >> 16) | (__float_as_uint(v[1]) & 0xffff0000u);
          o.y = (__float_as_uint(v[2]) >> 16) | (__float_as_uint(v[3]) & 0xffff0000u);
          o.z = (__float_as_uint(v[4]) >> 16) | (__float_as_uint(v[5]) & 0xffff0000u);
          o.w = (__float_as_uint(v[6]) >> 16) | (__float_as_uint(v[7]) & 0xffff0000u);
          *reinterpret_cast<uint4*>(ro + (long long)(m0 + j) * p.Kx + k) = o;
        }
        if (nw != nullptr) {
          const uint4 nv = (jj == 0) ? nwv[0] : ((jj == 1) ? nwv[1] : *reinterpret_cast<const uint4*>(nw + k));
          const uint32_t nww[4] = {nv.x, nv.y, nv.z, nv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // round to bf16 like an unfused norm kernel would, so fused and unfused paths agree
            v[2 * e] = __bfloat162float(__float2bfloat16(v[2 * e] * rs * __uint_as_float(nww[e] << 16)));
            v[2 * e + 1] = __bfloat162float(__float2bfloat16(v[2 * e + 1] * rs * __uint_as_float(nww[e] & 0xffff0000u)));
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = fminf(fmaxf(v[e], -65504.f), 65504.f);
      }
      // fragment order inside each 32-wide block: lane t finds (b0, b1) of both k16 steps in 16 contiguous bytes
      __half* blk = dst + (k & ~31) + ((k >> 4) & 1) * 4 + ((k >> 3) & 1) * 2;
#pragma unroll
      for (int tt = 0; tt < 4; ++tt)
        *reinterpret_cast<__half2*>(blk + tt * 8) = __floats2half2_rn(v[2 * tt], v[2 * tt + 1]);
    }
  }
  __syncthreads();

  // ---- main loop: kDepth loads stay in flight per lane.  Per 64-wide chunk: two 16-byte shared loads give
  // the B fragments of its four k16 steps (the staging above stored x in fragment order), 4 x (12 integer
  // ops + 1 MMA), and once per quantization group the scale is applied to the group accumulator in fp32.
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  {
    const int gmask = gs - 1;
    const int cpg_shift = p.gs_shift - 6;                 // log2(chunks per group), valid when BIG_GROUPS
    const int cpg_mask = BIG_GROUPS ? ((1 << cpg_shift) - 1) : 0;
    const __half* xbase = xs + min(g, mt - 1) * ((p.mode == 2) ? 0 : XS) + t * 8;
    float gacc[4] = {0.f, 0.f, 0.f, 0.f};
    uint32_t s2 = 0;
    int pr_seg = -1;
    SegPtr pseg;
    pseg.q = nullptr;
    pseg.s = nullptr;
    pseg.mult = 0.f;
    const uint32_t* sbase = nullptr;
    float mult = 0.f;
    for (int c = c_begin; c < c_end; c += kDepth) {
#pragma unroll
      for (int i = 0; i < kDepth; ++i) {
        const int ci = c + i;
        if (ci >= c_end) break;
        int sidx = 0, cc = ci;
        if (nseg > 1) {
          sidx = ci / KC;
          cc = ci - sidx * KC;
        }
        if (sidx != pr_seg) {
          pseg = seg_lookup(p, token, (p.mode == 1) ? slot : sidx);
          pr_seg = sidx;
          sbase = (pseg.s != nullptr) ? pseg.s + (long long)rt * NG * 8 + g : nullptr;
          mult = pseg.mult * kE2M1F16Rescale;
        }
        const uint32_t qq[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
        const uint32_t s_cur = sw[i];
        if (ci + kDepth < c_end) w[i] = load_chunk(ci + kDepth, sw[i]);
        const __half* xp = xbase + (long long)sidx * p.K + cc * 64;
        const uint4 xv0 = *reinterpret_cast<const uint4*>(xp);
        const uint4 xv1 = *reinterpret_cast<const uint4*>(xp + 32);
        const uint32_t bb[8] = {xv0.x, xv0.y, xv0.z, xv0.w, xv1.x, xv1.y, xv1.z, xv1.w};
        if (BIG_GROUPS) s2 = s_cur;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          if (!BIG_GROUPS) {
            const int kabs = cc * 64 + ks * 16;
            if ((kabs & gmask) == 0) s2 = (sbase != nullptr) ? __ldg(sbase + (kabs >> p.gs_shift) * 8) : 0u;
          }
          uint32_t a0, a1, a2, a3;
          e2m1x8_to_f16x2(qq[ks], a0, a1, a2, a3);
          mma_f16_16816(gacc, a0, a1, a2, a3, bb[2 * ks], bb[2 * ks + 1]);
          if (!BIG_GROUPS) {
            const int kabs = cc * 64 + ks * 16;
            if (((kabs + 16) & gmask) == 0) {
              const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&s2));
              const float slo = sf.x * mult, shi = sf.y * mult;
              acc[0] = fmaf(gacc[0], slo, acc[0]);
              acc[1] = fmaf(gacc[1], slo, acc[1]);
              acc[2] = fmaf(gacc[2], shi, acc[2]);
              acc[3] = fmaf(gacc[3], shi, acc[3]);
              gacc[0] = gacc[1] = gacc[2] = gacc[3] = 0.f;
            }
          }
        }
        if (BIG_GROUPS) {
          if (((cc + 1) & cpg_mask) == 0) {
            const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&s2));
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
  }
  // ---- cross-warp reduction and epilogue
  {
    float* r = red + warp * 128;
    r[g * 8 + 2 * t] = acc[0];
    r[g * 8 + 2 * t + 1] = acc[1];
    r[(g + 8) * 8 + 2 * t] = acc[2];
    r[(g + 8) * 8 + 2 * t + 1] = acc[3];
  }
  __syncthreads();
  const int et = tid >> 7;            // epilogue tile (threads beyond R * 128 only take part in the barriers)
  const int row = (tid & 127) >> 3, col = tid & 7;
  const bool active = (et < R) && (col < mt);
  float v = 0.f;
  if (active) {
#pragma unroll
    for (int w2 = 0; w2 < WPT; ++w2) v += red[(et * WPT + w2) * 128 + row * 8 + col];
  }
  const long long orow = (p.mode == 1) ? (long long)blockIdx.y : (long long)(m0 + col);
  if (p.tpx.out_peer_slots != nullptr) {
    // tensor-parallel producer: this rank's partial goes straight into every peer's receive buffer
    TpOut tout;
    tout.peer_slots = p.tpx.out_peer_slots;
    tout.peer_flags = p.tpx.out_peer_flags;
    tout.counter = p.tpx.out_counter;
    tout.step = p.tpx.step;
    tout.tp = p.tpx.tp;
    const int n = (blockIdx.x * R + et) * 16 + row;
    if (active && n < p.N) tp_push(tout, orow * p.N + n, v);
    tp_signal(tout, gridDim.x * gridDim.y);
    return;
  }
  if (!active) return;
  bf16* out = reinterpret_cast<bf16*>(p.out);
  if (p.act == 1) {
    if (et != 0) return;
    float u = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < WPT; ++w2) u += red[(WPT + w2) * 128 + row * 8 + col];
    const int n = blockIdx.x * 16 + row;
    if (n < (p.N >> 1)) out[orow * p.ldo + n] = __float2bfloat16(silu(v) * u);
  } else {
    const int n = (blockIdx.x * R + et) * 16 + row;
    if (n < p.N) {
      if (p.bias) v += __bfloat162float(reinterpret_cast<const bf16*>(p.bias)[n]);
      if (p.out_add) v += __bfloat162float(reinterpret_cast<const bf16*>(p.out_add)[orow * p.ldo + n]);
      out[orow * p.ldo + n] = __float2bfloat16(v);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// bf16 GEMV: one warp per output row, 16-byte loads along K, x staged in shared memory as fp32.
template <int MT>
__global__ void __launch_bounds__(256) bf16_gemv_kernel(const MmbBf16GemvParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float red_small[32];
  __shared__ float rstd_s[8];
  float* xs = reinterpret_cast<float*>(smem_raw);   // [MT][K]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int m0 = blockIdx.y * MT;
  const int mt = min(MT, p.M - m0);
  const bf16* xg = reinterpret_cast<const bf16*>(p.x);
  const bf16* dg = reinterpret_cast<const bf16*>(p.delta);
  const bf16* nw = reinterpret_cast<const bf16*>(p.norm_w);
  const bool has_tin = p.tpx.in_buf != nullptr;
  TpIn tin;
  tin.buf = p.tpx.in_buf;
  tin.flags = p.tpx.in_flags;
  tin.step = p.tpx.step;
  tin.status = p.tpx.status;
  tin.tp = p.tpx.tp;
  tin.slot_stride = p.tpx.in_slot_stride;
  // first weight rows of this warp are requested before waiting for the producer of x
  const bf16* W = reinterpret_cast<const bf16*>(p.w);
  const int rows_per_cta = 8 * 4;   // 8 warps x 4 rows
  const int n0 = blockIdx.x * rows_per_cta + warp * 4;
  uint4 wpre[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int n = n0 + r;
    wpre[r] = (n < p.N && lane * 8 < p.K) ? ldg_stream(reinterpret_cast<const uint4*>(W + (long long)n * p.K + lane * 8))
                                         : make_uint4(0, 0, 0, 0);
  }
  pdl_launch_dependents();
  pdl_wait();
  if (has_tin) tp_wait(tin);
  for (int j = 0; j < mt; ++j) {
    const long long row = (long long)(m0 + j) * p.ldx;
    float ss = 0.f;
    for (int k = tid; k < p.K; k += 256) {
      float v = __bfloat162float(xg[row + k]);
      if (has_tin) v = __bfloat162float(__float2bfloat16(v + tp_sum(tin, (long long)(m0 + j) * p.K + k)));
      else if (dg) v = __bfloat162float(__float2bfloat16(v + __bfloat162float(dg[row + k])));
      xs[j * p.K + k] = v;
      ss += v * v;
    }
    if (nw != nullptr) {
      ss = block_sum(ss, red_small);
      if (tid == 0) rstd_s[j] = rsqrtf(ss / (float)p.K + p.eps);
    }
  }
  __syncthreads();
  if (nw != nullptr) {
    for (int j = 0; j < mt; ++j) {
      const float rs = rstd_s[j];
      for (int k = tid; k < p.K; k += 256)
        xs[j * p.K + k] = __bfloat162float(__float2bfloat16(xs[j * p.K + k] * rs * __bfloat162float(nw[k])));
    }
    __syncthreads();
  }
  float acc[4][MT];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int j = 0; j < MT; ++j) acc[r][j] = 0.f;
  for (int k = lane * 8; k < p.K; k += 256) {
    uint4 wv[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int n = n0 + r;
      if (k == lane * 8) wv[r] = wpre[r];
      else wv[r] = (n < p.N) ? ldg_stream(reinterpret_cast<const uint4*>(W + (long long)n * p.K + k)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const uint32_t ww[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float w0 = __uint_as_float(ww[2 * e] << 16), w1 = __uint_as_float(ww[2 * e] & 0xffff0000u);
        const float w2 = __uint_as_float(ww[2 * e + 1] << 16), w3 = __uint_as_float(ww[2 * e + 1] & 0xffff0000u);
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          if (j < mt) {
            const float4 xv = *reinterpret_cast<const float4*>(xs + j * p.K + k + 4 * e);
            acc[r][j] = fmaf(w0, xv.x, acc[r][j]);
            acc[r][j] = fmaf(w1, xv.y, acc[r][j]);
            acc[r][j] = fmaf(w2, xv.z, acc[r][j]);
            acc[r][j] = fmaf(w3, xv.w, acc[r][j]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int j = 0; j < MT; ++j) acc[r][j] = warp_sum(acc[r][j]);
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int n = n0 + r;
      if (n >= p.N) continue;
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        if (j < mt) {
          const long long o = (long long)(m0 + j) * p.ldo + n;
          if (p.out_f32) reinterpret_cast<float*>(p.out)[o] = acc[r][j];
          else reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16(acc[r][j]);
        }
      }
    }
  }
}

template <typename K>
static int set_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

}  // namespace mmb

MMB_API int mmb_fp4_gemv(const MmbFp4GemvParams* pp, cudaStream_t stream) {
  using namespace mmb;
  const MmbFp4GemvParams& p = *pp;
  if (p.K % 64 != 0 || p.Kx > p.K || (p.Kx & 7) || (p.ldx & 7) || p.M <= 0 || p.N <= 0) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(p.x) & 15) || (reinterpret_cast<uintptr_t>(p.delta) & 15) ||
      (reinterpret_cast<uintptr_t>(p.norm_w) & 15) || (reinterpret_cast<uintptr_t>(p.resid_out) & 15))
    return (int)cudaErrorInvalidValue;
  if ((1 << p.gs_shift) < 16) return (int)cudaErrorInvalidValue;
  const int S = (p.mode == 0) ? 1 : (p.topk + p.n_shared);
  if (S > kMaxSeg) return (int)cudaErrorInvalidValue;
  if (p.mode == 2 && (p.norm_w != nullptr || p.delta != nullptr)) return (int)cudaErrorInvalidValue;
  const int n_rt = (p.N + 15) / 16;
  size_t smem;
  dim3 grid;
  int R;
  if (p.mode == 0) {
    const int mt = p.M < 8 ? p.M : 8;
    smem = (size_t)mt * (p.K + 32) * 2;
    grid.y = (p.M + 7) / 8;
  } else if (p.mode == 1) {
    smem = (size_t)(p.K + 32) * 2;
    grid.y = p.M * S;
  } else {
    smem = (size_t)(S * p.K + 32) * 2;
    grid.y = p.M;
  }
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (p.tpx.out_peer_slots != nullptr && (p.act != 0 || p.mode == 1)) return (int)cudaErrorInvalidValue;
  if (p.act == 1) {
    if (n_rt % 2 != 0) return (int)cudaErrorInvalidValue;
    R = 2;
    grid.x = n_rt / 2;
  } else {
    R = 1;
    grid.x = (n_rt + R - 1) / R;
  }
  grid.z = 1;
  int e;
  const bool big = p.gs_shift >= 6;
  // warps per row tile so that a warp owns ~2 chunks; CTA = R tiles x that many warps, 8..32 warps in total
  const int chunks = ((p.mode == 2) ? S : 1) * (p.K / 64);
  int wpt = 1;
  while (wpt * 2 < chunks && wpt * R < 16) wpt *= 2;
  int nw = wpt * R;
  if (nw < 8) nw = 8;
  if (nw > 16) nw = 16;     // 32 warps would cap a thread at 64 registers and spill
#define MMB_LAUNCH_GEMV(RR, BG, NW)                                                         \
  do {                                                                                      \
    if ((e = set_smem(fp4_gemv_kernel<RR, BG, NW>, smem))) return e;                         \
    return launch(fp4_gemv_kernel<RR, BG, NW>, grid, dim3(NW * 32), smem, stream, 1, p);     \
  } while (0)
#define MMB_DISPATCH_NW(RR, BG)             \
  do {                                      \
    if (nw == 8) MMB_LAUNCH_GEMV(RR, BG, 8);  \
    MMB_LAUNCH_GEMV(RR, BG, 16);            \
  } while (0)
  if (R == 2 && big) MMB_DISPATCH_NW(2, true);
  if (R == 2) MMB_DISPATCH_NW(2, false);
  if (big) MMB_DISPATCH_NW(1, true);
  MMB_DISPATCH_NW(1, false);
#undef MMB_DISPATCH_NW
#undef MMB_LAUNCH_GEMV
}

MMB_API int mmb_bf16_gemv(const MmbBf16GemvParams* pp, cudaStream_t stream) {
  using namespace mmb;
  const MmbBf16GemvParams& p = *pp;
  if (p.K % 8 != 0 || p.M <= 0) return (int)cudaErrorInvalidValue;
  dim3 grid((p.N + 31) / 32, 1, 1);
  int e;
  if (p.M == 1) {
    const size_t smem = (size_t)p.K * 4;
    if ((e = set_smem(bf16_gemv_kernel<1>, smem))) return e;
    return launch(bf16_gemv_kernel<1>, grid, dim3(256), smem, stream, 1, p);
  } else {
    const size_t smem = (size_t)4 * p.K * 4;
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    grid.y = (p.M + 3) / 4;
    if ((e = set_smem(bf16_gemv_kernel<4>, smem))) return e;
    return launch(bf16_gemv_kernel<4>, grid, dim3(256), smem, stream, 1, p);
  }
}
