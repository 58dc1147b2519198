// Decode-time attention over a paged KV pool, plus the MLA prologue/epilogue kernels.
//
//  * mla_prep:     q_nope absorbed through W_uk^T (per head), RoPE on q_rope, and the new token's
//                  latent (RMSNorm(c_kv) | RoPE(k_rope)) scattered into the paged latent cache.
//  * paged_decode: split-KV flash-decoding.  All query heads that share a KV head form the M
//                  dimension of the MMA (MLA: every head shares the single 576-d latent, and V is
//                  its first 512 columns, so one KV tile in shared memory feeds both QK^T and PV).
//                  KV tiles (64 tokens) arrive through a 2-stage cp.async pipeline; tiles that cannot
//                  contain this step's token are requested before the kernel waits for its producer.
//  * decode_merge: log-sum-exp merge of the split partials, optionally followed by the per-head
//                  MLA value up-projection W_uv.  One thread-block cluster per head: each CTA merges a
//                  slice of the latent and the slices are exchanged through distributed shared memory.
#include <cooperative_groups.h>

#include "api.h"
#include "common.cuh"
#include "kv_quant.cuh"
#include "launch.h"

namespace cg = cooperative_groups;

namespace mmb {

// ------------------------------------------------------------------------------------------------
// mla_prep: grid (H * ceil(R / 32) + 1, ceil(T / 8)), 256 threads.  Each CTA of the first group owns 32
// rows of one head's W_uk^T (4 per warp); the weight rows are requested before the query is staged so the
// DRAM round trip overlaps it.  The last CTA writes the new latent into the paged cache.
// Sums of 8 per-lane values over the 32 lanes of a warp in 9 shuffles: halve the value count while halving the lane
// span (xor 16, 8, 4), then finish the 4-lane groups.  Lane 4 * j returns the sum of value j (other lanes: partial
// garbage of no use).
__device__ __forceinline__ float warp_sum8(const float (&acc)[8], int lane) {
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
  float v4[4], v2[2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float send = b4 ? acc[i] : acc[i + 4];
    const float keep = b4 ? acc[i + 4] : acc[i];
    v4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float send = b3 ? v4[i] : v4[i + 2];
    const float keep = b3 ? v4[i + 2] : v4[i];
    v2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
  float v1 = (b2 ? v2[1] : v2[0]) + __shfl_xor_sync(0xffffffffu, b2 ? v2[0] : v2[1], 4);
  v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
  v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
  return v1;
}

constexpr int kPrepTok = 8;
constexpr int kPrepRows = 32;
__global__ void __launch_bounds__(256) mla_prep_kernel(const MmbMlaPrepParams p) {
  __shared__ float red[32];
  extern __shared__ __align__(16) float sm[];   // [kPrepTok][max(256, R + dr)]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = blockIdx.y * kPrepTok;
  const int nt = min(kPrepTok, p.T - t0);
  const bf16* q = reinterpret_cast<const bf16*>(p.q);
  bf16* qf = reinterpret_cast<bf16*>(p.q_full);
  const int dq = p.dn + p.dr, dl = p.R + p.dr;
  const int n_chunks = p.skip_absorb ? 1 : (p.R + kPrepRows - 1) / kPrepRows;
  if ((int)blockIdx.x < p.H * n_chunks) {
    const int h = blockIdx.x / n_chunks, chunk = blockIdx.x % n_chunks;
    const bf16* W = reinterpret_cast<const bf16*>(p.w_ukT) + (long long)h * p.R * p.dn;
    // this warp's four rows; one 16-byte load per lane per row (dn <= 256)
    uint4 wv[4];
    int crow[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      crow[r] = chunk * kPrepRows + warp * 4 + r;
      wv[r] = make_uint4(0, 0, 0, 0);
      if (!p.skip_absorb && crow[r] < p.R && lane * 8 < p.dn) wv[r] = ldg_stream(reinterpret_cast<const uint4*>(W + (long long)crow[r] * p.dn + lane * 8));
    }
    pdl_launch_dependents();
    pdl_wait();
    // query rows in shared memory, 256 floats per token, element d at [(d / 4) % 2][d / 8][d % 4]: the eight values a
    // lane multiplies with its weight word are two lane-contiguous float4 (no bank conflicts)
    if (!p.skip_absorb) {
      for (int i = tid; i < kPrepTok * 256; i += 256) {
        const int j = i >> 8, pos = i & 255;
        const int d = ((pos >> 2) & 31) * 8 + (pos >> 7) * 4 + (pos & 3);
        sm[i] = (j < nt && d < p.dn) ? __bfloat162float(q[(long long)(t0 + j) * p.ld_q + h * dq + d]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if (p.skip_absorb || crow[r] >= p.R) continue;
      const float wf[8] = {__uint_as_float(wv[r].x << 16), __uint_as_float(wv[r].x & 0xffff0000u),
                           __uint_as_float(wv[r].y << 16), __uint_as_float(wv[r].y & 0xffff0000u),
                           __uint_as_float(wv[r].z << 16), __uint_as_float(wv[r].z & 0xffff0000u),
                           __uint_as_float(wv[r].w << 16), __uint_as_float(wv[r].w & 0xffff0000u)};
      float acc[kPrepTok];
#pragma unroll
      for (int j = 0; j < kPrepTok; ++j) {
        const float4 x0 = *reinterpret_cast<const float4*>(sm + j * 256 + lane * 4);
        const float4 x1 = *reinterpret_cast<const float4*>(sm + j * 256 + 128 + lane * 4);
        acc[j] = fmaf(wf[0], x0.x, fmaf(wf[1], x0.y, fmaf(wf[2], x0.z, wf[3] * x0.w)));
        acc[j] = fmaf(wf[4], x1.x, fmaf(wf[5], x1.y, fmaf(wf[6], x1.z, fmaf(wf[7], x1.w, acc[j]))));
      }
      const float v1 = warp_sum8(acc, lane);
      const int j = lane >> 2;
      if ((lane & 3) == 0 && j < nt) qf[((long long)(t0 + j) * p.H + h) * dl + crow[r]] = __float2bfloat16(v1);
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
    pdl_launch_dependents();
    pdl_wait();
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
      if (p.cache_scale != nullptr) {
        // FP8 cache: the finished row (bf16-rounded like the bf16 cache would hold it) goes back to shared memory, its
        // amax gives the scale, then E4M3 bytes.  All threads take this branch together (slot is per token).
        float amax = 0.f;
        for (int d = tid; d < p.R; d += 256) {
          const float v = __bfloat162float(__float2bfloat16(sm[d] * rs * __bfloat162float(nw[d])));
          sm[d] = v;
          amax = fmaxf(amax, fabsf(v));
        }
        const int half = p.dr / 2;
        for (int f = tid; f < half; f += 256) {
          float sn, cs;
          sincosf((float)p.positions[tk] * p.inv_freq[f], &sn, &cs);
          const int ia = p.interleaved ? 2 * f : f, ib = p.interleaved ? 2 * f + 1 : f + half;
          const float a = __bfloat162float(src[p.R + ia]), b = __bfloat162float(src[p.R + ib]);
          const float ra = __bfloat162float(__float2bfloat16((a * cs - b * sn) * p.mscale));
          const float rb = __bfloat162float(__float2bfloat16((b * cs + a * sn) * p.mscale));
          sm[p.R + ia] = ra;
          sm[p.R + ib] = rb;
          amax = fmaxf(amax, fmaxf(fabsf(ra), fabsf(rb)));
        }
        amax = block_max(amax, red);
        if (slot >= 0) {
          const int fmt = p.cache_fmt;
          const float sc = amax > 0.f ? amax / kvq_range(fmt) : 1.f, inv = 1.f / sc;
          if (kvq_is4(fmt)) {
            unsigned char* dst8 = reinterpret_cast<unsigned char*>(p.cache) + slot * (dl / 2);
            for (int d = tid; d < dl / 2; d += 256)
              dst8[d] = (unsigned char)(kvq_encode(sm[2 * d] * inv, fmt) | (kvq_encode(sm[2 * d + 1] * inv, fmt) << 4));
          } else {
            unsigned char* dst8 = reinterpret_cast<unsigned char*>(p.cache) + slot * dl;
            for (int d = tid; d < dl; d += 256) dst8[d] = (unsigned char)kvq_encode(sm[d] * inv, fmt);
          }
          if (tid == 0) p.cache_scale[slot] = sc;
        }
      } else if (slot >= 0) {
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

__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gmem));
}

// In-place expansion of a tile of quantized rows to bf16 x row scale.  BPV = 1: D code bytes sit in the upper half of a bf16
// row of stride RS elements; BPV = 2 (4-bit codes, two per byte): D / 2 bytes sit in its last quarter.  Called by all NT
// threads of the CTA: every thread first reads its 16-byte pieces, the CTA synchronizes, then the 32- / 64-byte results are
// written (a piece's result overlaps other pieces' source bytes).
template <int D, int RS, int NT, int TT, int BPV>
__device__ __forceinline__ void expand_fp8_rows(bf16* rows, const float* row_scale, int nvalid, int tid, int fmt) {
  constexpr int UPR = D / (16 * BPV);                        // pieces per row
  constexpr int PER = (TT * UPR + NT - 1) / NT;              // pieces per thread
  constexpr int SRC0 = 2 * D - D / BPV;                      // byte offset of the codes inside the row
  uint4 raw[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int u = tid + i * NT, r = u / UPR, c = u - r * UPR;
    raw[i] = make_uint4(0, 0, 0, 0);
    if (r < nvalid) raw[i] = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(rows + r * RS) + SRC0 + c * 16);
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int u = tid + i * NT, r = u / UPR, c = u - r * UPR;
    if (r >= nvalid) continue;
    const float sc = row_scale[r];
    const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
    if (BPV == 1) {
      uint32_t o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float2 f = kvq_decode8x2(w[e >> 1] >> ((e & 1) * 16), fmt);
        const bf162 b2 = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        o[e] = *reinterpret_cast<const uint32_t*>(&b2);
      }
      uint4* dst = reinterpret_cast<uint4*>(rows + r * RS + c * 16);
      dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
      dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    } else {
      uint4* dst = reinterpret_cast<uint4*>(rows + r * RS + c * 32);
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {                       // one 32-bit word = 8 values = one 16-byte result
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const bf162 b2 = __floats2bfloat162_rn(kvq_decode4((w[q4] >> (8 * e)) & 0xfu, fmt) * sc, kvq_decode4((w[q4] >> (8 * e + 4)) & 0xfu, fmt) * sc);
          o[e] = *reinterpret_cast<const uint32_t*>(&b2);
        }
        dst[q4] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  __syncthreads();
}

// NW warps: in QK^T each warp owns 64 / NW token columns, in PV it owns DV / NW value columns.
// TT tokens per tile.  TT = 64: one CTA per SM (the two K/V buffers fill the shared memory).  TT = 32 (MLA shape only): half
// the tile, query rows stored compactly (the rows beyond the head group share one zero row) -> two CTAs per SM, so one
// CTA's barrier-separated phases (QK^T, soft-max, PV) overlap the other's; used when the grid has more CTAs than SMs.
template <int DQK, int DV, int MT, bool SHARED_V, int NW, int TT>
struct DecodeSmem {
  static constexpr int KS = DQK + 8;                     // row strides in elements (16-byte skew)
  static constexpr int VS = DV + 8;
  static constexpr int PS = TT + 8;
  static constexpr int SS = TT + 4;                      // fp32 score row stride
  static constexpr int QR = (TT == 32) ? 24 : MT * 16;   // query rows held (compact form: up to 23 heads + the zero row)
  static constexpr size_t q_bytes = (size_t)QR * KS * 2;
  static constexpr size_t k_bytes = (size_t)TT * KS * 2;
  static constexpr size_t v_bytes = SHARED_V ? 0 : (size_t)TT * VS * 2;
  static constexpr size_t s_bytes = (size_t)MT * 16 * SS * 4;
  static constexpr size_t p_bytes = (size_t)MT * 16 * PS * 2;
  static constexpr size_t total = q_bytes + 2 * (k_bytes + v_bytes) + s_bytes + p_bytes + 3 * MT * 16 * 4;
  static_assert(TT == 32 || ((64 / NW) % 8 == 0), "each warp needs whole n8 tiles of token columns");
  static_assert(TT == 64 || (MT * (TT / 8) == NW), "compact form: one 16 x 8 score tile per warp");
  static_assert((DV / NW) % 16 == 0, "each warp needs pairs of n8 tiles of value columns");
};

// grid (splits, Hkv, B), NW * 32 threads.  FP8: the pools hold E4M3 bytes and a scale per (slot, head); a row's bytes land
// in the upper half of its bf16 row in shared memory and are expanded in place (all reads, a barrier, all writes).
template <int DQK, int DV, int MT, bool SHARED_V, int NW, int FP8, int TT>
__global__ void __launch_bounds__(NW * 32, (TT == 32) ? 2 : 1) paged_decode_kernel(const MmbPagedDecodeParams p) {
  using L = DecodeSmem<DQK, DV, MT, SHARED_V, NW, TT>;
  constexpr int NT = NW * 32;
  constexpr int kTileTok = TT;          // shadows the file-level default inside this kernel
  constexpr int NQ = (TT == 64) ? 64 / NW / 8 : 1;       // n8 tiles of token columns per warp in QK^T
  constexpr int NVT = DV / NW / 8;      // n8 tiles of value columns per warp in PV
  extern __shared__ __align__(128) unsigned char smem[];
  bf16* q_s = reinterpret_cast<bf16*>(smem);
  bf16* const k_s0 = reinterpret_cast<bf16*>(smem + L::q_bytes);
  bf16* const k_s1 = reinterpret_cast<bf16*>(smem + L::q_bytes + L::k_bytes + L::v_bytes);
  bf16* const v_s0 = SHARED_V ? k_s0 : reinterpret_cast<bf16*>(smem + L::q_bytes + L::k_bytes);
  bf16* const v_s1 = SHARED_V ? k_s1 : reinterpret_cast<bf16*>(smem + L::q_bytes + 2 * L::k_bytes + L::v_bytes);
  float* s_s = reinterpret_cast<float*>(smem + L::q_bytes + 2 * (L::k_bytes + L::v_bytes));
  bf16* p_s = reinterpret_cast<bf16*>(reinterpret_cast<unsigned char*>(s_s) + L::s_bytes);
  float* row_m = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(p_s) + L::p_bytes);
  float* row_l = row_m + MT * 16;
  float* row_c = row_l + MT * 16;
  constexpr int VSTR = SHARED_V ? L::KS : L::VS;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int Gh = p.Hq / p.Hkv;                  // query heads per KV head (<= MT * 16)
  // ctx_lens / block_tables were written long before the producer of q started, so they may be read now
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
    pdl_launch_dependents();
    pdl_wait();
    for (int r = 0; r < Gh; ++r) {
      for (int d = tid; d < DV; d += NT) po[(long long)r * p.splits * DV + d] = 0.f;
      if (tid == 0) {
        pml[(long long)r * p.splits * 2] = -INFINITY;
        pml[(long long)r * p.splits * 2 + 1] = 0.f;
      }
    }
    return;
  }

  // K / V rows of a tile and the query rows arrive by bulk copies (one per row, issued by one lane each) that
  // signal an mbarrier per buffer; rows past the end of the sequence are zero-filled with plain stores.
  __shared__ __align__(8) uint64_t bar_kv[2];
  __shared__ __align__(8) uint64_t bar_q;
  __shared__ int abort_s;
  __shared__ float scale_s[2][2][kTileTok];     // [buffer][K | V][row]
  if (tid == 0) {
    mbar_init(&bar_kv[0], 1);
    mbar_init(&bar_kv[1], 1);
    mbar_init(&bar_q, 1);
    abort_s = 0;
    fence_barrier_init();
  }
  __syncthreads();
  const bool pow2_blocks = (p.block_size & (p.block_size - 1)) == 0;
  const int bs_shift = pow2_blocks ? (31 - __clz(p.block_size)) : 0;
  auto load_tile = [&](int tile, int buf) {
    const int tok0 = lo_al + tile * kTileTok;
    const int nvalid = min(kTileTok, ctx - tok0);
    bf16* kd = buf ? k_s1 : k_s0;
    bf16* vd = buf ? v_s1 : v_s0;
    // FP8 = 0: bf16 rows; 1: one code byte per value; 2: two 4-bit codes per byte
    if (tid == 0) mbar_expect_tx(&bar_kv[buf], (uint32_t)nvalid * (uint32_t)((DQK + (SHARED_V ? 0 : DV)) * 2 / (FP8 == 0 ? 1 : 2 * FP8)));
    if (tid < nvalid) {
      const int tok = tok0 + tid;
      const long long slot = pow2_blocks ? (((long long)__ldg(bt + (tok >> bs_shift)) << bs_shift) + (tok & (p.block_size - 1)))
                                         : ((long long)__ldg(bt + tok / p.block_size) * p.block_size + (tok % p.block_size));
      if (FP8) {
        const long long row = slot * p.Hkv + hkv;
        constexpr int KB8 = DQK / (FP8 ? FP8 : 1), VB8 = DV / (FP8 ? FP8 : 1);      // code bytes per row
        bulk_g2s(reinterpret_cast<unsigned char*>(kd + tid * L::KS) + 2 * DQK - KB8, reinterpret_cast<const unsigned char*>(p.k_pool) + row * KB8, KB8,
                 &bar_kv[buf]);
        cp_async_4(&scale_s[buf][0][tid], p.k_scale + row);
        if (!SHARED_V) {
          bulk_g2s(reinterpret_cast<unsigned char*>(vd + tid * L::VS) + 2 * DV - VB8, reinterpret_cast<const unsigned char*>(p.v_pool) + row * VB8, VB8,
                   &bar_kv[buf]);
          cp_async_4(&scale_s[buf][1][tid], p.v_scale + row);
        }
      } else {
        bulk_g2s(kd + tid * L::KS, kp + (slot * p.Hkv + hkv) * DQK, DQK * 2, &bar_kv[buf]);
        if (!SHARED_V) bulk_g2s(vd + tid * L::VS, vp + (slot * p.Hkv + hkv) * DV, DV * 2, &bar_kv[buf]);
      }
    }
    if (FP8) cp_async_commit();      // one group per tile from every thread, so the waits below can count groups
    if (nvalid < kTileTok) {
      constexpr int KCH = DQK / 8, VCH = DV / 8;
      for (int i = tid; i < (kTileTok - nvalid) * KCH; i += NT)
        *reinterpret_cast<uint4*>(kd + (nvalid + i / KCH) * L::KS + (i % KCH) * 8) = make_uint4(0, 0, 0, 0);
      if (!SHARED_V)
        for (int i = tid; i < (kTileTok - nvalid) * VCH; i += NT)
          *reinterpret_cast<uint4*>(vd + (nvalid + i / VCH) * L::VS + (i % VCH) * 8) = make_uint4(0, 0, 0, 0);
    }
  };

  // The cache row of this step's token (position ctx - 1) is written by the previous kernel; every other
  // row is older.  A first tile that does not contain it can be requested before waiting.
  const bool first_is_old = (lo_al + (tile_begin + 1) * kTileTok) <= ctx - 1;
  if (first_is_old) load_tile(tile_begin, 0);
  // query rows beyond the group are zero and never change
  for (int i = tid; i < (L::QR - Gh) * (DQK / 8); i += NT)
    *reinterpret_cast<uint4*>(q_s + (Gh + i / (DQK / 8)) * L::KS + (i % (DQK / 8)) * 8) = make_uint4(0, 0, 0, 0);
  pdl_launch_dependents();
  pdl_wait();
  if (tid == 0) mbar_expect_tx(&bar_q, (uint32_t)Gh * (uint32_t)(DQK * 2));
  if (tid >= 64 && tid < 64 + Gh) bulk_g2s(q_s + (tid - 64) * L::KS, q + (long long)(tid - 64) * DQK, DQK * 2, &bar_q);
  if (!first_is_old) load_tile(tile_begin, 0);

  if (tid < MT * 16) {
    row_m[tid] = -INFINITY;
    row_l[tid] = 0.f;
  }

  float o[MT][NVT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int n = 0; n < NVT; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[m][n][e] = 0.f;

  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int buf = (tile - tile_begin) & 1;
    if (tile + 1 < tile_end) load_tile(tile + 1, buf ^ 1);
    if (FP8) {      // this tile's scales (the group before the one just committed, if any)
      if (tile + 1 < tile_end) cp_async_wait<1>();
      else cp_async_wait<0>();
    }
    bool landed = mbar_wait(&bar_kv[buf], (uint32_t)((tile - tile_begin) >> 1) & 1u, &abort_s);
    if (tile == tile_begin) landed = mbar_wait(&bar_q, 0u, &abort_s) && landed;
    if (!landed) abort_s = 1;
    // tile `buf` (and, first time, Q and the zero rows) visible to all warps; a wait that expired ends the loop
    // for the whole CTA at once
    if (!__syncthreads_and(landed ? 1 : 0)) {
      if (tid == 0 && p.status != nullptr) atomicExch(p.status, 200);
      break;
    }
    const bf16* kt = buf ? k_s1 : k_s0;
    const bf16* vt = buf ? v_s1 : v_s0;
    if (FP8) {
      const int nvalid = min(kTileTok, ctx - (lo_al + tile * kTileTok));
      expand_fp8_rows<DQK, L::KS, NT, TT, FP8 ? FP8 : 1>(buf ? k_s1 : k_s0, scale_s[buf][0], nvalid, tid, p.kv_fmt);
      if (!SHARED_V) expand_fp8_rows<DV, L::VS, NT, TT, FP8 ? FP8 : 1>(buf ? v_s1 : v_s0, scale_s[buf][1], nvalid, tid, p.kv_fmt);
    }

    // ---- S = Q K^T for this warp's token columns
    {
      // two accumulator sets (even / odd k16 steps) halve the dependent MMA chain of this latency-bound loop
      // this warp's part of S: all MT row tiles x its NQ column tiles (64-token tiles), or one 16 x 8 tile (32-token tiles)
      constexpr int MQ = (TT == 64) ? MT : 1;
      const int m_first = (TT == 64) ? 0 : warp / (TT / 8);
      const int col_base = (TT == 64) ? warp * (64 / NW) : (warp % (TT / 8)) * 8;
      float s[MQ][NQ][4], s_odd[MQ][NQ][4];
#pragma unroll
      for (int m = 0; m < MQ; ++m)
#pragma unroll
        for (int n = 0; n < NQ; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[m][n][e] = s_odd[m][n][e] = 0.f;
      const bf16* kb = kt + (col_base + g) * L::KS + 2 * t;
      static_assert(DQK % 32 == 0, "the QK^T loop consumes two k16 steps per trip");
#pragma unroll 2
      for (int k0 = 0; k0 < DQK; k0 += 32) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int kk = k0 + half * 16;
          uint32_t bfr[NQ][2];
#pragma unroll
          for (int n = 0; n < NQ; ++n) {
            bfr[n][0] = *reinterpret_cast<const uint32_t*>(kb + n * 8 * L::KS + kk);
            bfr[n][1] = *reinterpret_cast<const uint32_t*>(kb + n * 8 * L::KS + kk + 8);
          }
#pragma unroll
          for (int m = 0; m < MQ; ++m) {
            uint32_t a0, a1, a2, a3;
            // compact query rows: rows beyond the head group read the zero row kept at the end
            const int qrow = min((m_first + m) * 16 + (lane & 15), L::QR - 1);
            ldmatrix_x4(a0, a1, a2, a3, q_s + qrow * L::KS + kk + (lane >> 4) * 8);
#pragma unroll
            for (int n = 0; n < NQ; ++n) {
              if (half == 0) mma_bf16_16816(s[m][n], a0, a1, a2, a3, bfr[n][0], bfr[n][1]);
              else mma_bf16_16816(s_odd[m][n], a0, a1, a2, a3, bfr[n][0], bfr[n][1]);
            }
          }
        }
      }
#pragma unroll
      for (int m = 0; m < MQ; ++m)
#pragma unroll
        for (int n = 0; n < NQ; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[m][n][e] += s_odd[m][n][e];
      const int tok0 = lo_al + tile * kTileTok;
#pragma unroll
      for (int m = 0; m < MQ; ++m)
#pragma unroll
        for (int n = 0; n < NQ; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = (m_first + m) * 16 + g + ((e >> 1) << 3);
            const int c = col_base + n * 8 + 2 * t + (e & 1);
            const int tok = tok0 + c;
            const bool ok = (tok < ctx) && (tok >= lo);
            s_s[r * L::SS + c] = ok ? s[m][n][e] * p.scale : -INFINITY;
          }
    }
    __syncthreads();

    // ---- online softmax: 4 threads per row, a quarter of the tile's columns each
    if (tid < MT * 16 * 4) {
      constexpr int CPT = TT / 4;
      const int r = tid >> 2, part = tid & 3;
      const float* sr = s_s + r * L::SS + part * CPT;
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < CPT; ++c) mx = fmaxf(mx, sr[c]);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_old = row_m[r];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      bf16* pr = p_s + r * L::PS + part * CPT;
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
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

    // ---- O = O * corr + P V for this warp's value columns
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
      const bf16* vb = vt + warp * (DV / NW);
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
      for (int e = 0; e < 4; e += 2) {
        const int r = m * 16 + g + ((e >> 1) << 3);
        const int c = warp * (DV / NW) + n * 8 + 2 * t;
        if (r < Gh) *reinterpret_cast<float2*>(po + (long long)r * p.splits * DV + c) = make_float2(o[m][n][e], o[m][n][e + 1]);
      }
  if (tid < Gh) {
    pml[(long long)tid * p.splits * 2] = row_m[tid];
    pml[(long long)tid * p.splits * 2 + 1] = row_l[tid];
  }
}

// ------------------------------------------------------------------------------------------------
// decode_merge: grid (Hq * CL, ceil(B / 8)) in clusters of CL CTAs (one cluster per head), 256 threads.
// CTA c of a cluster merges latent columns [c * dv / CL, (c + 1) * dv / CL) of every token of the tile and
// writes them into the shared memory of all CTAs of the cluster (DSMEM); after the cluster barrier each CTA
// applies its 32-row slab of W_uv (requested before anything else) to the full merged latent.
constexpr int kMergeTok = 8;
constexpr int kMergeRows = 32;
// position of latent element d inside a token's row of the merged-latent tile: [d / 256][(d / 4) % 2][(d / 8) % 32][d % 4]
__device__ __forceinline__ int merge_perm(int d) { return (((d >> 8) * 2 + ((d >> 2) & 1)) << 7) + (((d >> 3) & 31) << 2) + (d & 3); }
__global__ void __launch_bounds__(256) decode_merge_kernel(const float* __restrict__ part_o,
                                                           const float* __restrict__ part_ml,
                                                           const bf16* __restrict__ w_uv, bf16* __restrict__ out, int B,
                                                           int Hq, int dv, int dvo, int splits, int CL) {
  extern __shared__ __align__(16) float o_s[];   // [kMergeTok][DS] merged latent (permuted), then weights and partial sums
  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (CL > 1) ? (int)cluster.block_rank() : 0;
  if (CL > 1) cluster_arrive();   // matched by cluster_wait() before the first remote shared-memory store
  const int h = blockIdx.x / CL, b0 = blockIdx.y * kMergeTok;
  const int nb = min(kMergeTok, B - b0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // weight rows of this warp: slabs of 32 rows, slab index = crank, crank + CL, ...; the first slab's rows are
  // requested now (up to two 16-byte loads per lane per row, dv <= 512)
  uint4 wv[4][2];
  const bf16* W = (w_uv != nullptr) ? w_uv + (long long)h * dvo * dv : nullptr;
  if (W != nullptr) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = crank * kMergeRows + warp * 4 + r;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int d = u * 256 + lane * 8;
        wv[r][u] = (row < dvo && d < dv) ? ldg_stream(reinterpret_cast<const uint4*>(W + (long long)row * dv + d))
                                         : make_uint4(0, 0, 0, 0);
      }
    }
  }
  pdl_launch_dependents();
  pdl_wait();
  // ---- merge this CTA's column slice.  The partial outputs of the first token are requested first, then the
  // split weights are computed (one warp per token: lanes cover the splits) while those loads are in flight.
  // Merged latent layout in shared memory: element d of a token sits at merge_perm(d), which puts the eight
  // values a lane multiplies with one 16-byte weight word into two lane-contiguous float4 (no bank conflicts).
  const int DS = (dv <= 256) ? 256 : 512;          // row stride of o_s
  float* wgt = o_s + kMergeTok * DS;               // [kMergeTok][splits]: exp(m_s - M) / L, 0 for empty splits
  float* red = wgt + kMergeTok * splits;           // [tokens in flight][groups][per] partial sums
  const int per = (dv + CL - 1) / CL;
  const int d_lo = crank * per, d_hi = min(dv, d_lo + per);
  const int quads = (d_hi - d_lo + 3) >> 2;        // float4 columns of the slice (dv and per are multiples of 4)
  // thread rows of `quads` threads: tok_par tokens are merged at once, each by `groups` rows that split the splits
  const int pq = per >> 2;                         // thread-row width (the last CTA's slice may be shorter: quads <= pq)
  const int TG = max(1, 256 / pq);
  const int tok_par = min(nb, TG);
  const int groups = max(1, min(splits, TG / tok_par));
  const int cq = tid % pq, trow = tid / pq;
  const int tj = trow % tok_par, sg = trow / tok_par;
  const bool worker = trow < tok_par * groups && cq < quads;
  float4 pre[4];
  if (worker) {
    const long long base = ((long long)(b0 + tj) * Hq + h) * splits;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int s = sg + i * groups;
      pre[i] = (s < splits) ? __ldcg(reinterpret_cast<const float4*>(part_o + (base + s) * dv + d_lo + cq * 4))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  if (warp < nb) {
    const long long base = ((long long)(b0 + warp) * Hq + h) * splits;
    float2 mlr[2];
    float M = -INFINITY;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int s = lane + 32 * i;
      mlr[i] = (s < splits) ? __ldcg(reinterpret_cast<const float2*>(part_ml + (base + s) * 2)) : make_float2(-INFINITY, 0.f);
      if (mlr[i].y > 0.f) M = fmaxf(M, mlr[i].x);
    }
    for (int s = lane + 64; s < splits; s += 32) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + (base + s) * 2));
      if (ml.y > 0.f) M = fmaxf(M, ml.x);
    }
    M = warp_max(M);
    float Lsum = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int s = lane + 32 * i;
      const float w = (mlr[i].y > 0.f) ? __expf(mlr[i].x - M) : 0.f;
      if (s < splits) wgt[warp * splits + s] = w;
      Lsum += mlr[i].y * w;
    }
    for (int s = lane + 64; s < splits; s += 32) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + (base + s) * 2));
      const float w = (ml.y > 0.f) ? __expf(ml.x - M) : 0.f;
      wgt[warp * splits + s] = w;
      Lsum += ml.y * w;
    }
    Lsum = warp_sum(Lsum);
    const float inv = (Lsum > 0.f) ? 1.f / Lsum : 0.f;
    __syncwarp();
    for (int s = lane; s < splits; s += 32) wgt[warp * splits + s] *= inv;
  }
  __syncthreads();
  if (CL > 1) cluster_wait();
  for (int j0 = 0; j0 < nb; j0 += tok_par) {
    const int j = j0 + tj;
    if (worker && j < nb) {
      const long long base = ((long long)(b0 + j) * Hq + h) * splits;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s0 = sg, round = 0; s0 < splits; s0 += 4 * groups, ++round) {
        float4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int s = s0 + i * groups;
          if (j0 == 0 && round == 0) v[i] = pre[i];
          else v[i] = (s < splits) ? __ldcg(reinterpret_cast<const float4*>(part_o + (base + s) * dv + d_lo + cq * 4))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int s = s0 + i * groups;
          const float w = (s < splits) ? wgt[j * splits + s] : 0.f;
          if (w != 0.f) {
            acc.x = fmaf(v[i].x, w, acc.x);
            acc.y = fmaf(v[i].y, w, acc.y);
            acc.z = fmaf(v[i].z, w, acc.z);
            acc.w = fmaf(v[i].w, w, acc.w);
          }
        }
      }
      *reinterpret_cast<float4*>(red + (tj * groups + sg) * per + cq * 4) = acc;
    }
    __syncthreads();
    // four consecutive latent elements per thread: one 16-byte store per CTA of the cluster
    for (int idx = tid; idx < tok_par * pq; idx += 256) {
      const int t2 = idx / pq, qd = idx - t2 * pq;
      if (j0 + t2 >= nb || qd >= quads) continue;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int gI = 0; gI < groups; ++gI) {
        const float4 r4 = *reinterpret_cast<const float4*>(red + (t2 * groups + gI) * per + qd * 4);
        a.x += r4.x; a.y += r4.y; a.z += r4.z; a.w += r4.w;
      }
      // round the merged latent to bf16 (an unfused pipeline would store it in bf16)
      a.x = __bfloat162float(__float2bfloat16(a.x));
      a.y = __bfloat162float(__float2bfloat16(a.y));
      a.z = __bfloat162float(__float2bfloat16(a.z));
      a.w = __bfloat162float(__float2bfloat16(a.w));
      const int pd = (j0 + t2) * DS + merge_perm(d_lo + qd * 4);      // d_lo and the quad start are multiples of 4: contiguous
      if (CL > 1) {
        for (int c = 0; c < CL; ++c) *reinterpret_cast<float4*>(cluster.map_shared_rank(o_s, c) + pd) = a;
      } else {
        *reinterpret_cast<float4*>(o_s + pd) = a;
      }
    }
    __syncthreads();
  }
  if (CL > 1) cluster.sync();
  else __syncthreads();
  if (W == nullptr) {
    for (int j = 0; j < nb; ++j)
      for (int d = d_lo + tid; d < d_hi; d += 256)
        out[((long long)(b0 + j) * Hq + h) * dv + d] = __float2bfloat16(o_s[j * DS + merge_perm(d)]);
    return;
  }
  // Up-projection: the warp's four rows against the eight tokens; every 16-byte pair of the merged latent is read once
  // per token and used for all four rows.
  for (int slab = crank; slab * kMergeRows < dvo; slab += CL) {
    const int row0 = slab * kMergeRows + warp * 4;
    float acc[4][kMergeTok];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int j = 0; j < kMergeTok; ++j) acc[r][j] = 0.f;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int d = u * 256 + lane * 8;
      if (d >= dv) continue;
      float wf[4][8];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        uint4 w4 = make_uint4(0, 0, 0, 0);
        if (slab == crank) w4 = wv[r][u];
        else if (row0 + r < dvo) w4 = ldg_stream(reinterpret_cast<const uint4*>(W + (long long)(row0 + r) * dv + d));
        wf[r][0] = __uint_as_float(w4.x << 16); wf[r][1] = __uint_as_float(w4.x & 0xffff0000u);
        wf[r][2] = __uint_as_float(w4.y << 16); wf[r][3] = __uint_as_float(w4.y & 0xffff0000u);
        wf[r][4] = __uint_as_float(w4.z << 16); wf[r][5] = __uint_as_float(w4.z & 0xffff0000u);
        wf[r][6] = __uint_as_float(w4.w << 16); wf[r][7] = __uint_as_float(w4.w & 0xffff0000u);
      }
#pragma unroll
      for (int j = 0; j < kMergeTok; ++j) {
        if (j < nb) {
          const float4 x0 = *reinterpret_cast<const float4*>(o_s + j * DS + (u * 2) * 128 + lane * 4);
          const float4 x1 = *reinterpret_cast<const float4*>(o_s + j * DS + (u * 2 + 1) * 128 + lane * 4);
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            acc[r][j] = fmaf(wf[r][0], x0.x, fmaf(wf[r][1], x0.y, fmaf(wf[r][2], x0.z, fmaf(wf[r][3], x0.w, acc[r][j]))));
            acc[r][j] = fmaf(wf[r][4], x1.x, fmaf(wf[r][5], x1.y, fmaf(wf[r][6], x1.z, fmaf(wf[r][7], x1.w, acc[r][j]))));
          }
        }
      }
    }
    static_assert(kMergeTok == 8, "warp_sum8 reduces eight tokens at once");
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float v = warp_sum8(acc[r], lane);
      if (row0 + r < dvo && (lane & 3) == 0 && (lane >> 2) < nb)
        out[((long long)(b0 + (lane >> 2)) * Hq + h) * dvo + row0 + r] = __float2bfloat16(v);
    }
  }
}

template <int DQK, int DV, int MT, bool SHARED_V, int NW, int FP8, int TT = 64>
static int launch_decode_impl(const MmbPagedDecodeParams& p, cudaStream_t stream) {
  using L = DecodeSmem<DQK, DV, MT, SHARED_V, NW, TT>;
  auto kern = paged_decode_kernel<DQK, DV, MT, SHARED_V, NW, FP8, TT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::total);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(p.splits, p.Hkv, p.B);
  return launch(kern, grid, dim3(NW * 32), L::total, stream, 1, p);
}
template <int DQK, int DV, int MT, bool SHARED_V, int NW>
static int launch_decode(const MmbPagedDecodeParams& p, cudaStream_t stream) {
  if (p.k_scale != nullptr) {
    if ((!SHARED_V && p.v_scale == nullptr) || p.kv_fmt < 0 || p.kv_fmt > 3) return (int)cudaErrorInvalidValue;
    if (kvq_is4(p.kv_fmt)) {
      if constexpr (DQK % 32 == 0 && DV % 32 == 0) return launch_decode_impl<DQK, DV, MT, SHARED_V, NW, 2>(p, stream);
      return (int)cudaErrorNotSupported;
    }
    return launch_decode_impl<DQK, DV, MT, SHARED_V, NW, 1>(p, stream);
  }
  return launch_decode_impl<DQK, DV, MT, SHARED_V, NW, 0>(p, stream);
}

}  // namespace mmb

MMB_API int mmb_mla_prep(const MmbMlaPrepParams* pp, cudaStream_t stream) {
  const MmbMlaPrepParams& p = *pp;
  if (p.T <= 0) return 0;
  if ((p.dn & 7) || (p.dr & 1) || p.dn > 256) return (int)cudaErrorInvalidValue;
  const int width = (256 > p.R + p.dr) ? 256 : (p.R + p.dr);      // absorb CTAs: 256 floats per token; latent CTA: one row
  const size_t smem = (size_t)mmb::kPrepTok * width * 4;
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  dim3 grid(p.H * (p.skip_absorb ? 1 : (p.R + mmb::kPrepRows - 1) / mmb::kPrepRows) + 1, (p.T + mmb::kPrepTok - 1) / mmb::kPrepTok);
  return mmb::launch(mmb::mla_prep_kernel, grid, dim3(256), smem, stream, 1, p);
}

MMB_API int mmb_paged_decode(const MmbPagedDecodeParams* pp, cudaStream_t stream) {
  using namespace mmb;
  const MmbPagedDecodeParams& p = *pp;
  if (p.B <= 0) return 0;
  if (p.Hq % p.Hkv != 0 || p.splits < 1) return (int)cudaErrorInvalidValue;
  const int Gh = p.Hq / p.Hkv;
  const bool shared = (p.v_pool == nullptr);
  if (shared && p.dqk == 576 && p.dv == 512 && Gh <= 23 && (long long)p.B * p.Hkv * p.splits > 148 && p.k_scale == nullptr)
    return launch_decode_impl<576, 512, 2, true, 8, 0, 32>(p, stream);      // more CTAs than SMs: two smaller CTAs per SM
  if (shared && p.dqk == 576 && p.dv == 512 && Gh <= 32) return launch_decode<576, 512, 2, true, 8>(p, stream);
  if (shared && p.dqk == 96 && p.dv == 64 && Gh <= 16) return launch_decode<96, 64, 1, true, 4>(p, stream);   // tiny MLA (tests)
  if (!shared && p.dqk == 128 && p.dv == 128 && Gh <= 16) return launch_decode<128, 128, 1, false, 8>(p, stream);
  if (!shared && p.dqk == 64 && p.dv == 64 && Gh <= 16) return launch_decode<64, 64, 1, false, 4>(p, stream);
  if (!shared && p.dqk == 256 && p.dv == 256 && Gh <= 16) return launch_decode<256, 256, 1, false, 8>(p, stream);
  return (int)cudaErrorNotSupported;
}

MMB_API int mmb_decode_merge(const float* part_o, const float* part_ml, const void* w_uv, void* out, int B, int Hq, int dv,
                             int dvo, int splits, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (dv % 8 != 0 || dv > 512) return (int)cudaErrorInvalidValue;
  // cluster size: one CTA per 32-row slab of the up-projection, at most 8 (portable cluster size)
  int cl = 1;
  if (w_uv != nullptr) {
    const int slabs = (dvo + mmb::kMergeRows - 1) / mmb::kMergeRows;
    while (cl < 8 && cl < slabs) cl *= 2;
  }
  // shared memory: merged latent [8][dv], split weights [8][splits], per-group partial sums [groups][dv / cl]
  const int per = (dv + cl - 1) / cl;
  if (per % 4 != 0 || splits < 1) return (int)cudaErrorInvalidValue;
  int trows = 256 / (per / 4);          // thread rows of the merge; the partial-sum area holds one slice per row
  if (trows < 1) trows = 1;
  const int ds = (dv <= 256) ? 256 : 512;
  const size_t smem = ((size_t)mmb::kMergeTok * ds + (size_t)mmb::kMergeTok * splits + (size_t)trows * per) * 4;
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  dim3 grid(Hq * cl, (B + mmb::kMergeTok - 1) / mmb::kMergeTok);
  return mmb::launch(mmb::decode_merge_kernel, grid, dim3(256), smem, stream, cl, part_o, part_ml, (const bf16*)w_uv,
                     (bf16*)out, B, Hq, dv, dvo, splits, cl);
}
