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

namespace mmb {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = 8;
constexpr int kMaxSeg = 16;

struct SegInfo {
  const uint4* q[kMaxSeg];
  const uint32_t* s[kMaxSeg];
  float mult[kMaxSeg];
};

template <int R>
__global__ void __launch_bounds__(kGemvThreads) fp4_gemv_kernel(const MmbFp4GemvParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float red[kGemvWarps * 128];
  __shared__ float red_small[32];
  __shared__ float rstd_s[8];
  __shared__ SegInfo seg;

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
  const int XS = Kv + 8;       // smem row stride in halves (word stride = 4 mod 32: conflict free)
  __half* xs = reinterpret_cast<__half*>(smem_raw);

  // ---- segment table
  if (tid < nseg) {
    int e;
    float mult = 1.f;
    if (p.mode == 0) {
      e = 0;
    } else {
      const int sl = (p.mode == 1) ? slot : tid;
      if (sl < p.topk) {
        e = p.expert_ids[token * p.topk + sl];
        if (p.mode == 2) mult = p.expert_w[token * p.topk + sl];
      } else {
        e = p.shared_base + (sl - p.topk);
      }
    }
    if (e < 0) {
      seg.q[tid] = nullptr;
      seg.s[tid] = nullptr;
      seg.mult[tid] = 0.f;
    } else {
      seg.q[tid] = reinterpret_cast<const uint4*>(p.qw) + (long long)e * p.expert_stride_q;
      seg.s[tid] = reinterpret_cast<const uint32_t*>(p.sc) + (long long)e * p.expert_stride_s;
      seg.mult[tid] = mult;
    }
  }

  // ---- stage activations as fp16 (optional residual add + RMSNorm)
  const bf16* xg = reinterpret_cast<const bf16*>(p.x);
  const bf16* dg = reinterpret_cast<const bf16*>(p.delta);
  const bf16* nw = reinterpret_cast<const bf16*>(p.norm_w);
  bf16* ro = reinterpret_cast<bf16*>(p.resid_out);
  const int rows_to_stage = (p.mode == 2) ? nseg : mt;
  if (nw != nullptr) {
    // pass 1: sum of squares of bf16(x + delta) per token row
    for (int j = 0; j < rows_to_stage; ++j) {
      const long long row = (long long)(m0 + j) * p.ldx;
      float ss = 0.f;
      for (int k = tid * 2; k < p.Kx; k += kGemvThreads * 2) {
        float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(xg + row + k));
        if (dg) {
          float2 d = __bfloat1622float2(*reinterpret_cast<const bf162*>(dg + row + k));
          v = __bfloat1622float2(__floats2bfloat162_rn(v.x + d.x, v.y + d.y));
        }
        ss += v.x * v.x + v.y * v.y;
      }
      ss = block_sum(ss, red_small);
      if (tid == 0) rstd_s[j] = rsqrtf(ss / (float)p.Kx + p.eps);
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
    for (int k = tid * 2; k < p.K; k += kGemvThreads * 2) {
      float2 v = make_float2(0.f, 0.f);
      if (k < p.Kx) {
        v = __bfloat1622float2(*reinterpret_cast<const bf162*>(xg + row + k));
        if (dg) {
          float2 d = __bfloat1622float2(*reinterpret_cast<const bf162*>(dg + row + k));
          bf162 s2 = __floats2bfloat162_rn(v.x + d.x, v.y + d.y);
          v = __bfloat1622float2(s2);
          if (ro != nullptr && blockIdx.x == 0 && (p.mode != 1 || slot == 0))
            *reinterpret_cast<bf162*>(ro + (long long)(m0 + j) * p.Kx + k) = s2;
        }
        if (nw != nullptr) {
          float2 w2 = __bfloat1622float2(*reinterpret_cast<const bf162*>(nw + k));
          // round to bf16 like an unfused norm kernel would, so fused and unfused paths agree
          v = __bfloat1622float2(__floats2bfloat162_rn(v.x * rs * w2.x, v.y * rs * w2.y));
        }
        v.x = fminf(fmaxf(v.x, -65504.f), 65504.f);
        v.y = fminf(fmaxf(v.y, -65504.f), 65504.f);
      }
      *reinterpret_cast<__half2*>(dst + k) = __floats2half2_rn(v.x, v.y);
    }
  }
  __syncthreads();

  // ---- which row tile does this warp serve
  const int n_rt = (p.N + 15) >> 4;
  const int ti = warp / WPT, wi = warp % WPT;
  int rt;
  if (p.act == 1) {
    rt = (ti == 0) ? (int)blockIdx.x : (int)blockIdx.x + (n_rt >> 1);   // R == 2 enforced by the launcher
  } else {
    rt = blockIdx.x * R + ti;
  }
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (rt < n_rt) {
    const int KC = p.K >> 6;                 // chunks per segment
    const int NG = p.K >> p.gs_shift;        // groups per segment
    const int gs = 1 << p.gs_shift;
    const int unit_chunks = (gs >= 64) ? (gs >> 6) : 1;
    const int total_units = (nseg * KC) / unit_chunks;
    const int u0 = (int)(((long long)wi * total_units) / WPT), u1 = (int)(((long long)(wi + 1) * total_units) / WPT);
    const int c_begin = u0 * unit_chunks, c_end = u1 * unit_chunks;
    const int gmask = gs - 1;
    const int xrow = min(g, mt - 1) * ((p.mode == 2) ? 0 : XS);
    float gacc[4] = {0.f, 0.f, 0.f, 0.f};
    uint32_t s2 = 0;

    for (int c = c_begin; c < c_end; c += 4) {
      uint4 w[4];
      int sidx[4], cc[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int ci = c + i;
        if (nseg == 1) {
          sidx[i] = 0;
          cc[i] = ci;
        } else {
          sidx[i] = ci / KC;
          cc[i] = ci - sidx[i] * KC;
        }
        w[i] = make_uint4(0, 0, 0, 0);
        if (ci < c_end) {
          const uint4* base = seg.q[sidx[i]];
          if (base != nullptr) w[i] = ldg_stream(base + ((long long)rt * KC + cc[i]) * 32 + lane);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (c + i < c_end) {
          const uint32_t qq[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
          const uint32_t* sbase = seg.s[sidx[i]];
          const float mult = seg.mult[sidx[i]] * kE2M1F16Rescale;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const int kabs = cc[i] * 64 + ks * 16;          // k inside the segment
            if ((kabs & gmask) == 0)
              s2 = (sbase != nullptr) ? __ldg(sbase + ((long long)rt * NG + (kabs >> p.gs_shift)) * 8 + g) : 0u;
            uint32_t a0, a1, a2, a3;
            e2m1x8_to_f16x2(qq[ks], a0, a1, a2, a3);
            const __half* xb = xs + xrow + (long long)sidx[i] * p.K + kabs + 2 * t;
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(xb);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(xb + 8);
            mma_f16_16816(gacc, a0, a1, a2, a3, b0, b1);
            if (((kabs + 16) & gmask) == 0) {
              const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&s2));
              const float slo = sf.x * mult, shi = sf.y * mult;
              acc[0] += gacc[0] * slo;
              acc[1] += gacc[1] * slo;
              acc[2] += gacc[2] * shi;
              acc[3] += gacc[3] * shi;
              gacc[0] = gacc[1] = gacc[2] = gacc[3] = 0.f;
            }
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
  const int et = tid >> 7;            // epilogue tile
  const int row = (tid & 127) >> 3, col = tid & 7;
  if (et >= R || col >= mt) return;
  float v = 0.f;
#pragma unroll
  for (int w2 = 0; w2 < WPT; ++w2) v += red[(et * WPT + w2) * 128 + row * 8 + col];
  bf16* out = reinterpret_cast<bf16*>(p.out);
  const long long orow = (p.mode == 1) ? (long long)blockIdx.y : (long long)(m0 + col);
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
  for (int j = 0; j < mt; ++j) {
    const long long row = (long long)(m0 + j) * p.ldx;
    float ss = 0.f;
    for (int k = tid; k < p.K; k += 256) {
      float v = __bfloat162float(xg[row + k]);
      if (dg) v = __bfloat162float(__float2bfloat16(v + __bfloat162float(dg[row + k])));
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
  const bf16* W = reinterpret_cast<const bf16*>(p.w);
  const int rows_per_cta = 8 * 4;   // 8 warps x 4 rows
  const int n0 = blockIdx.x * rows_per_cta + warp * 4;
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
      wv[r] = (n < p.N) ? ldg_stream(reinterpret_cast<const uint4*>(W + (long long)n * p.K + k)) : make_uint4(0, 0, 0, 0);
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
  if (p.K % 64 != 0 || p.Kx > p.K || (p.Kx & 1) || p.M <= 0 || p.N <= 0) return (int)cudaErrorInvalidValue;
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
    smem = (size_t)mt * (p.K + 8) * 2;
    grid.y = (p.M + 7) / 8;
  } else if (p.mode == 1) {
    smem = (size_t)(p.K + 8) * 2;
    grid.y = p.M * S;
  } else {
    smem = (size_t)(S * p.K + 8) * 2;
    grid.y = p.M;
  }
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (p.act == 1) {
    if (n_rt % 2 != 0) return (int)cudaErrorInvalidValue;
    R = 2;
    grid.x = n_rt / 2;
  } else {
    // two row tiles per CTA when there are plenty of rows; one when rows are scarce so more SMs stream
    R = (n_rt >= 592) ? 2 : 1;
    grid.x = (n_rt + R - 1) / R;
  }
  grid.z = 1;
  int e;
  if (R == 2) {
    if ((e = set_smem(fp4_gemv_kernel<2>, smem))) return e;
    fp4_gemv_kernel<2><<<grid, kGemvThreads, smem, stream>>>(p);
  } else {
    if ((e = set_smem(fp4_gemv_kernel<1>, smem))) return e;
    fp4_gemv_kernel<1><<<grid, kGemvThreads, smem, stream>>>(p);
  }
  return (int)cudaGetLastError();
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
    bf16_gemv_kernel<1><<<grid, 256, smem, stream>>>(p);
  } else {
    const size_t smem = (size_t)4 * p.K * 4;
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    grid.y = (p.M + 3) / 4;
    if ((e = set_smem(bf16_gemv_kernel<4>, smem))) return e;
    bf16_gemv_kernel<4><<<grid, 256, smem, stream>>>(p);
  }
  return (int)cudaGetLastError();
}
