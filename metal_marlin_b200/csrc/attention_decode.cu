// Decode-time attention over a paged KV pool, plus the MLA prologue/epilogue kernels.
//
//  * mla_prep:     q_nope absorbed through W_uk^T (per head), RoPE on q_rope, and the new token's
//                  latent (RMSNorm(c_kv) | RoPE(k_rope)) scattered into the paged latent cache.
//  * paged_decode: split-KV flash-decoding.  All query heads that share a KV head form the M
//                  dimension of the MMA (MLA: every head shares the single 576-d latent, and V is
//                  its first 512 columns, so one KV tile in shared memory feeds both QK^T and PV).
//                  KV tiles (64 tokens) arrive through a 2-stage cp.async pipeline.
//  * decode_merge: log-sum-exp merge of the split partials, optionally followed by the per-head
//                  MLA value up-projection W_uv.
#include "api.h"
#include "common.cuh"

namespace mmb {

// ------------------------------------------------------------------------------------------------
// mla_prep: grid (H * 4 + 1, ceil(T / 8)), 256 threads.
constexpr int kPrepTok = 8;
__global__ void __launch_bounds__(256) mla_prep_kernel(const MmbMlaPrepParams p) {
  __shared__ float red[32];
  extern __shared__ float sm[];   // [kPrepTok][max(dn, R + dr)]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = blockIdx.y * kPrepTok;
  const int nt = min(kPrepTok, p.T - t0);
  const bf16* q = reinterpret_cast<const bf16*>(p.q);
  bf16* qf = reinterpret_cast<bf16*>(p.q_full);
  const int dq = p.dn + p.dr, dl = p.R + p.dr;
  if ((int)blockIdx.x < p.H * 4) {
    const int h = blockIdx.x >> 2, chunk = blockIdx.x & 3;
    // stage q_nope of the tile's tokens
    for (int j = 0; j < nt; ++j)
      for (int d = tid; d < p.dn; d += 256)
        sm[j * p.dn + d] = __bfloat162float(q[(long long)(t0 + j) * p.ld_q + h * dq + d]);
    __syncthreads();
    const bf16* W = reinterpret_cast<const bf16*>(p.w_ukT) + (long long)h * p.R * p.dn;
    const int rows_per_chunk = (p.R + 3) / 4;
    const int c_lo = chunk * rows_per_chunk, c_hi = min(p.R, c_lo + rows_per_chunk);
    for (int c = c_lo + warp; c < c_hi; c += 8) {
      float acc[kPrepTok];
#pragma unroll
      for (int j = 0; j < kPrepTok; ++j) acc[j] = 0.f;
      const bf16* wr = W + (long long)c * p.dn;
      for (int d = lane * 2; d < p.dn; d += 64) {
        const float2 wv = __bfloat1622float2(*reinterpret_cast<const bf162*>(wr + d));
#pragma unroll
        for (int j = 0; j < kPrepTok; ++j)
          if (j < nt) acc[j] = fmaf(wv.x, sm[j * p.dn + d], fmaf(wv.y, sm[j * p.dn + d + 1], acc[j]));
      }
#pragma unroll
      for (int j = 0; j < kPrepTok; ++j) {
        if (j < nt) {
          const float v = warp_sum(acc[j]);
          if (lane == 0) qf[((long long)(t0 + j) * p.H + h) * dl + c] = __float2bfloat16(v);
        }
      }
    }
    if (chunk == 0) {
      // RoPE on the rope part of q
      const int half = p.dr / 2;
      for (int i = tid; i < nt * half; i += 256) {
        const int j = i / half, f = i % half;
        const long long tk = t0 + j;
        const bf16* src = q + tk * p.ld_q + h * dq + p.dn;
        float sn, cs;
        sincosf((float)p.positions[tk] * p.inv_freq[f], &sn, &cs);
        const int ia = p.interleaved ? 2 * f : f, ib = p.interleaved ? 2 * f + 1 : f + half;
        const float a = __bfloat162float(src[ia]), b = __bfloat162float(src[ib]);
        bf16* dst = qf + (tk * p.H + h) * dl + p.R;
        dst[ia] = __float2bfloat16((a * cs - b * sn) * p.mscale);
        dst[ib] = __float2bfloat16((b * cs + a * sn) * p.mscale);
      }
    }
  } else {
    // latent cache write: RMSNorm(c_kv) | RoPE(k_rope)
    const bf16* kva = reinterpret_cast<const bf16*>(p.kva);
    const bf16* nw = reinterpret_cast<const bf16*>(p.kv_norm_w);
    bf16* cache = reinterpret_cast<bf16*>(p.cache);
    for (int j = 0; j < nt; ++j) {
      const long long tk = t0 + j;
      const long long slot = p.slots[tk];
      const bf16* src = kva + tk * p.ld_kva;
      float ss = 0.f;
      for (int d = tid; d < p.R; d += 256) {
        const float v = __bfloat162float(src[d]);
        sm[d] = v;
        ss += v * v;
      }
      ss = block_sum(ss, red);
      const float rs = rsqrtf(ss / (float)p.R + p.eps);
      if (slot >= 0) {
        bf16* dst = cache + slot * dl;
        for (int d = tid; d < p.R; d += 256) dst[d] = __float2bfloat16(sm[d] * rs * __bfloat162float(nw[d]));
        const int half = p.dr / 2;
        for (int f = tid; f < half; f += 256) {
          float sn, cs;
          sincosf((float)p.positions[tk] * p.inv_freq[f], &sn, &cs);
          const int ia = p.interleaved ? 2 * f : f, ib = p.interleaved ? 2 * f + 1 : f + half;
          const float a = __bfloat162float(src[p.R + ia]), b = __bfloat162float(src[p.R + ib]);
          dst[p.R + ia] = __float2bfloat16((a * cs - b * sn) * p.mscale);
          dst[p.R + ib] = __float2bfloat16((b * cs + a * sn) * p.mscale);
        }
      }
      __syncthreads();
    }
  }
}

// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = smem_u32(smem);
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  const uint32_t a = smem_u32(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  const uint32_t a = smem_u32(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(a));
}

constexpr int kTileTok = 64;

template <int DQK, int DV, int MT, bool SHARED_V>
struct DecodeSmem {
  static constexpr int KS = DQK + 8;                     // row strides in elements (16-byte skew)
  static constexpr int VS = DV + 8;
  static constexpr int PS = kTileTok + 8;
  static constexpr size_t q_bytes = (size_t)MT * 16 * KS * 2;
  static constexpr size_t k_bytes = (size_t)kTileTok * KS * 2;
  static constexpr size_t v_bytes = SHARED_V ? 0 : (size_t)kTileTok * VS * 2;
  static constexpr size_t s_bytes = (size_t)MT * 16 * kTileTok * 4;
  static constexpr size_t p_bytes = (size_t)MT * 16 * PS * 2;
  static constexpr size_t total = q_bytes + 2 * (k_bytes + v_bytes) + s_bytes + p_bytes + 3 * MT * 16 * 4;
};

// grid (splits, Hkv, B), 128 threads.
template <int DQK, int DV, int MT, bool SHARED_V>
__global__ void __launch_bounds__(128) paged_decode_kernel(const MmbPagedDecodeParams p) {
  using L = DecodeSmem<DQK, DV, MT, SHARED_V>;
  extern __shared__ __align__(128) unsigned char smem[];
  bf16* q_s = reinterpret_cast<bf16*>(smem);
  bf16* k_s[2];
  bf16* v_s[2];
  k_s[0] = reinterpret_cast<bf16*>(smem + L::q_bytes);
  k_s[1] = reinterpret_cast<bf16*>(smem + L::q_bytes + L::k_bytes + L::v_bytes);
  v_s[0] = SHARED_V ? k_s[0] : reinterpret_cast<bf16*>(smem + L::q_bytes + L::k_bytes);
  v_s[1] = SHARED_V ? k_s[1] : reinterpret_cast<bf16*>(smem + L::q_bytes + 2 * L::k_bytes + L::v_bytes);
  float* s_s = reinterpret_cast<float*>(smem + L::q_bytes + 2 * (L::k_bytes + L::v_bytes));
  bf16* p_s = reinterpret_cast<bf16*>(reinterpret_cast<unsigned char*>(s_s) + L::s_bytes);
  float* row_m = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(p_s) + L::p_bytes);
  float* row_l = row_m + MT * 16;
  float* row_c = row_l + MT * 16;
  constexpr int VSTR = SHARED_V ? L::KS : L::VS;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int Gh = p.Hq / p.Hkv;                  // query heads per KV head (<= MT * 16)
  const int ctx = p.ctx_lens[b];
  const int lo = (p.window > 0) ? max(0, ctx - p.window) : 0;
  const int lo_al = lo & ~(kTileTok - 1);
  const int n_tiles_total = (ctx - lo_al + kTileTok - 1) / kTileTok;
  const int tiles_per_split = (n_tiles_total + p.splits - 1) / p.splits;
  const int tile_begin = split * tiles_per_split;
  const int tile_end = min(n_tiles_total, tile_begin + tiles_per_split);

  const bf16* q = reinterpret_cast<const bf16*>(p.q) + ((long long)b * p.Hq + (long long)hkv * Gh) * DQK;
  const bf16* kp = reinterpret_cast<const bf16*>(p.k_pool);
  const bf16* vp = reinterpret_cast<const bf16*>(p.v_pool);
  const int* bt = p.block_tables + (long long)b * p.max_blocks;

  float* po = p.part_o + (((long long)b * p.Hq + (long long)hkv * Gh) * p.splits + split) * DV;
  float* pml = p.part_ml + (((long long)b * p.Hq + (long long)hkv * Gh) * p.splits + split) * 2;

  if (tile_begin >= tile_end) {   // empty split: neutral partial
    for (int r = 0; r < Gh; ++r) {
      for (int d = tid; d < DV; d += 128) po[(long long)r * p.splits * DV + d] = 0.f;
      if (tid == 0) {
        pml[(long long)r * p.splits * 2] = -INFINITY;
        pml[(long long)r * p.splits * 2 + 1] = 0.f;
      }
    }
    return;
  }

  // ---- stage Q (zero padded to MT*16 rows)
  for (int i = tid; i < MT * 16 * (DQK / 8); i += 128) {
    const int r = i / (DQK / 8), c = i % (DQK / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < Gh) v = *reinterpret_cast<const uint4*>(q + (long long)r * DQK + c * 8);
    *reinterpret_cast<uint4*>(q_s + r * L::KS + c * 8) = v;
  }
  if (tid < MT * 16) {
    row_m[tid] = -INFINITY;
    row_l[tid] = 0.f;
  }

  auto load_tile = [&](int tile, int buf) {
    const int tok0 = lo_al + tile * kTileTok;
    constexpr int KCH = DQK / 8;
    for (int i = tid; i < kTileTok * KCH; i += 128) {
      const int r = i / KCH, c = i % KCH;
      const int tok = tok0 + r;
      const bool valid = tok < ctx;
      long long slot = 0;
      if (valid) slot = (long long)bt[tok / p.block_size] * p.block_size + (tok % p.block_size);
      cp_async16(k_s[buf] + r * L::KS + c * 8, kp + (slot * p.Hkv + hkv) * DQK + c * 8, valid);
    }
    if (!SHARED_V) {
      constexpr int VCH = DV / 8;
      for (int i = tid; i < kTileTok * VCH; i += 128) {
        const int r = i / VCH, c = i % VCH;
        const int tok = tok0 + r;
        const bool valid = tok < ctx;
        long long slot = 0;
        if (valid) slot = (long long)bt[tok / p.block_size] * p.block_size + (tok % p.block_size);
        cp_async16(v_s[buf] + r * L::VS + c * 8, vp + (slot * p.Hkv + hkv) * DV + c * 8, valid);
      }
    }
    cp_async_commit();
  };

  constexpr int NVT = DV / 4 / 8;   // n8 tiles of V columns per warp
  float o[MT][NVT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int n = 0; n < NVT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[m][n][e] = 0.f;

  load_tile(tile_begin, 0);
  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int buf = (tile - tile_begin) & 1;
    if (tile + 1 < tile_end) {
      load_tile(tile + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();   // tile `buf` (and, first time, Q) visible to all warps

    // ---- S = Q K^T for this warp's 16 token columns
    {
      float s[MT][2][4];
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[m][n][e] = 0.f;
      const bf16* kb = k_s[buf] + (warp * 16 + g) * L::KS + 2 * t;
#pragma unroll 4
      for (int k0 = 0; k0 < DQK; k0 += 16) {
        uint32_t bfr[2][2];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          bfr[n][0] = *reinterpret_cast<const uint32_t*>(kb + n * 8 * L::KS + k0);
          bfr[n][1] = *reinterpret_cast<const uint32_t*>(kb + n * 8 * L::KS + k0 + 8);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          uint32_t a0, a1, a2, a3;
          ldmatrix_x4(a0, a1, a2, a3, q_s + (m * 16 + (lane & 15)) * L::KS + k0 + (lane >> 4) * 8);
#pragma unroll
          for (int n = 0; n < 2; ++n) mma_bf16_16816(s[m][n], a0, a1, a2, a3, bfr[n][0], bfr[n][1]);
        }
      }
      const int tok0 = lo_al + tile * kTileTok;
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = m * 16 + g + ((e >> 1) << 3);
            const int c = warp * 16 + n * 8 + 2 * t + (e & 1);
            const int tok = tok0 + c;
            const bool ok = (tok < ctx) && (tok >= lo);
            s_s[r * kTileTok + c] = ok ? s[m][n][e] * p.scale : -INFINITY;
          }
    }
    __syncthreads();

    // ---- online softmax: 4 threads per row, 16 columns each
    if (tid < MT * 16 * 4) {
      const int r = tid >> 2, part = tid & 3;
      const float* sr = s_s + r * kTileTok + part * 16;
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 16; ++c) mx = fmaxf(mx, sr[c]);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_old = row_m[r];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      bf16* pr = p_s + r * L::PS + part * 16;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float e = (m_new == -INFINITY) ? 0.f : __expf(sr[c] - m_new);
        const bf16 eb = __float2bfloat16(e);
        pr[c] = eb;
        sum += __bfloat162float(eb);
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if (part == 0) {
        const float corr = (m_new == -INFINITY) ? 1.f : __expf(m_old - m_new);
        row_c[r] = corr;
        row_l[r] = row_l[r] * corr + sum;
        row_m[r] = m_new;
      }
    }
    __syncthreads();

    // ---- O = O * corr + P V for this warp's DV/4 value columns
    {
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float c0 = row_c[m * 16 + g], c1 = row_c[m * 16 + g + 8];
#pragma unroll
        for (int n = 0; n < NVT; ++n) {
          o[m][n][0] *= c0;
          o[m][n][1] *= c0;
          o[m][n][2] *= c1;
          o[m][n][3] *= c1;
        }
      }
      const bf16* vb = v_s[buf] + warp * (DV / 4);
#pragma unroll
      for (int k0 = 0; k0 < kTileTok; k0 += 16) {
        uint32_t a[MT][4];
#pragma unroll
        for (int m = 0; m < MT; ++m)
          ldmatrix_x4(a[m][0], a[m][1], a[m][2], a[m][3], p_s + (m * 16 + (lane & 15)) * L::PS + k0 + (lane >> 4) * 8);
#pragma unroll
        for (int n = 0; n < NVT; n += 2) {
          uint32_t b0, b1, b2, b3;
          // matrices: (tok k0..+7, col n), (tok k0+8..+15, col n), (tok k0..+7, col n+1), (tok k0+8.., col n+1)
          const int rr = k0 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int cc = (n + (lane >> 4)) * 8;
          ldmatrix_x4_trans(b0, b1, b2, b3, vb + rr * VSTR + cc);
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            mma_bf16_16816(o[m][n], a[m][0], a[m][1], a[m][2], a[m][3], b0, b1);
            mma_bf16_16816(o[m][n + 1], a[m][0], a[m][1], a[m][2], a[m][3], b2, b3);
          }
        }
      }
    }
    __syncthreads();   // everyone done with buf / s_s / p_s before they are overwritten
  }

  // ---- write the partial (unnormalised O, running max, running sum)
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int n = 0; n < NVT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = m * 16 + g + ((e >> 1) << 3);
        const int c = warp * (DV / 4) + n * 8 + 2 * t + (e & 1);
        if (r < Gh) po[(long long)r * p.splits * DV + c] = o[m][n][e];
      }
  if (tid < Gh) {
    pml[(long long)tid * p.splits * 2] = row_m[tid];
    pml[(long long)tid * p.splits * 2 + 1] = row_l[tid];
  }
}

// ------------------------------------------------------------------------------------------------
// decode_merge: grid (Hq, ceil(B / 8)), 256 threads.
constexpr int kMergeTok = 8;
__global__ void __launch_bounds__(256) decode_merge_kernel(const float* __restrict__ part_o,
                                                           const float* __restrict__ part_ml,
                                                           const bf16* __restrict__ w_uv, bf16* __restrict__ out, int B,
                                                           int Hq, int dv, int dvo, int splits) {
  extern __shared__ float o_s[];   // [kMergeTok][dv]
  const int h = blockIdx.x, b0 = blockIdx.y * kMergeTok;
  const int nb = min(kMergeTok, B - b0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int j = 0; j < nb; ++j) {
    const long long base = ((long long)(b0 + j) * Hq + h) * splits;
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
    float Lsum = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = part_ml[(base + s) * 2], ls = part_ml[(base + s) * 2 + 1];
      if (ls > 0.f) Lsum += ls * __expf(ms - M);
    }
    const float inv = (Lsum > 0.f) ? 1.f / Lsum : 0.f;
    for (int d = tid; d < dv; d += 256) {
      float acc = 0.f;
      for (int s = 0; s < splits; ++s) {
        const float ms = part_ml[(base + s) * 2], ls = part_ml[(base + s) * 2 + 1];
        if (ls > 0.f) acc += part_o[(base + s) * dv + d] * __expf(ms - M);
      }
      o_s[j * dv + d] = acc * inv;
    }
  }
  __syncthreads();
  if (w_uv == nullptr) {
    for (int j = 0; j < nb; ++j)
      for (int d = tid; d < dv; d += 256) out[((long long)(b0 + j) * Hq + h) * dv + d] = __float2bfloat16(o_s[j * dv + d]);
    return;
  }
  // round the merged latent to bf16 first (matches an unfused pipeline that stores it)
  for (int i = tid; i < nb * dv; i += 256) o_s[i] = __bfloat162float(__float2bfloat16(o_s[i]));
  __syncthreads();
  const bf16* W = w_uv + (long long)h * dvo * dv;
  for (int r = warp; r < dvo; r += 8) {
    float acc[kMergeTok];
#pragma unroll
    for (int j = 0; j < kMergeTok; ++j) acc[j] = 0.f;
    const bf16* wr = W + (long long)r * dv;
    for (int d = lane * 8; d < dv; d += 256) {
      const uint4 wv = *reinterpret_cast<const uint4*>(wr + d);
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float w0 = __uint_as_float(ww[e] << 16), w1 = __uint_as_float(ww[e] & 0xffff0000u);
#pragma unroll
        for (int j = 0; j < kMergeTok; ++j)
          if (j < nb) acc[j] = fmaf(w0, o_s[j * dv + d + 2 * e], fmaf(w1, o_s[j * dv + d + 2 * e + 1], acc[j]));
      }
    }
#pragma unroll
    for (int j = 0; j < kMergeTok; ++j) {
      if (j < nb) {
        const float v = warp_sum(acc[j]);
        if (lane == 0) out[((long long)(b0 + j) * Hq + h) * dvo + r] = __float2bfloat16(v);
      }
    }
  }
}

template <int DQK, int DV, int MT, bool SHARED_V>
static int launch_decode(const MmbPagedDecodeParams& p, cudaStream_t stream) {
  using L = DecodeSmem<DQK, DV, MT, SHARED_V>;
  auto kern = paged_decode_kernel<DQK, DV, MT, SHARED_V>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::total);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(p.splits, p.Hkv, p.B);
  kern<<<grid, 128, L::total, stream>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace mmb

MMB_API int mmb_mla_prep(const MmbMlaPrepParams* pp, cudaStream_t stream) {
  const MmbMlaPrepParams& p = *pp;
  if (p.T <= 0) return 0;
  if ((p.dn & 1) || (p.dr & 1)) return (int)cudaErrorInvalidValue;
  const int width = (p.dn > p.R + p.dr) ? p.dn : (p.R + p.dr);
  const size_t smem = (size_t)mmb::kPrepTok * width * 4;
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  dim3 grid(p.H * 4 + 1, (p.T + mmb::kPrepTok - 1) / mmb::kPrepTok);
  mmb::mla_prep_kernel<<<grid, 256, smem, stream>>>(p);
  return (int)cudaGetLastError();
}

MMB_API int mmb_paged_decode(const MmbPagedDecodeParams* pp, cudaStream_t stream) {
  using namespace mmb;
  const MmbPagedDecodeParams& p = *pp;
  if (p.B <= 0) return 0;
  if (p.Hq % p.Hkv != 0 || p.splits < 1) return (int)cudaErrorInvalidValue;
  const int Gh = p.Hq / p.Hkv;
  const bool shared = (p.v_pool == nullptr);
  if (shared && p.dqk == 576 && p.dv == 512 && Gh <= 32) return launch_decode<576, 512, 2, true>(p, stream);
  if (shared && p.dqk == 96 && p.dv == 64 && Gh <= 16) return launch_decode<96, 64, 1, true>(p, stream);   // tiny MLA (tests)
  if (!shared && p.dqk == 128 && p.dv == 128 && Gh <= 16) return launch_decode<128, 128, 1, false>(p, stream);
  if (!shared && p.dqk == 64 && p.dv == 64 && Gh <= 16) return launch_decode<64, 64, 1, false>(p, stream);
  if (!shared && p.dqk == 256 && p.dv == 256 && Gh <= 16) return launch_decode<256, 256, 1, false>(p, stream);
  return (int)cudaErrorNotSupported;
}

MMB_API int mmb_decode_merge(const float* part_o, const float* part_ml, const void* w_uv, void* out, int B, int Hq, int dv,
                             int dvo, int splits, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (dv % 8 != 0) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)mmb::kMergeTok * dv * 4;
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  dim3 grid(Hq, (B + mmb::kMergeTok - 1) / mmb::kMergeTok);
  mmb::decode_merge_kernel<<<grid, 256, smem, stream>>>(part_o, part_ml, (const bf16*)w_uv, (bf16*)out, B, Hq, dv, dvo,
                                                        splits);
  return (int)cudaGetLastError();
}
