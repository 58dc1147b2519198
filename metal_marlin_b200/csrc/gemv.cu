// Weight-streaming small-M kernels (decode): FP4 tile-layout GEMV on mma.sync with fp32
// accumulation and exact per-group scaling, plus a bf16 GEMV for unquantized matrices.
//
// FP4 kernel design (sm_100a; decode GEMVs are bound by latency and instruction fetch before bandwidth):
//  * warp groups own 16-row tiles (or gate/up tile pairs) and split the (virtual) K axis; each warp streams
//    whole 512-byte tile blocks through a private cp.async ring in shared memory, 16 bytes per lane per block;
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
  if (p.mode == 3) {
    e = __ldg(p.tile_expert + sl);
  } else if (p.mode != 0) {
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

constexpr int kRing = 8;    // weight chunks (512 B per warp) kept in flight per warp through cp.async

// Barrier over one warp group of the CTA (ids 1..15; id 0 is __syncthreads).
__device__ __forceinline__ void group_bar(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Where ring position (it, v) of a warp lives: v counts the chunks of one unit in the order the warp walks
// them (tile 0 of the unit, then tile 1 when the SwiGLU epilogue is fused).  A "run" is the stretch of
// consecutive positions that stay inside one row tile and one expert segment: inside a run the weight address
// just advances by one 512-byte block per chunk, so this lookup is only needed at run starts.
struct GemvLoc {
  const uint4* q;        // this lane's 16 bytes of the first chunk (null: expert id < 0 -> zeros)
  const uint32_t* s;     // scale words of the row tile for this lane's row pair (null like q)
  float mult;            // routing weight of the segment (mode 2) or 1
  int slot, rt0;         // unit: MoE slot (mode 1) and first row tile
  int tsel;              // tile of the unit (0 / 1)
  int sidx, cc;          // segment and chunk inside the segment
  int run;               // chunks in the run, starting with this one
};

// Division by a value fixed for the launch as one multiply-high: exact while dividend * divisor < 2^32 (unit and chunk
// counts here are far below that).
struct FastDiv {
  uint32_t magic;      // ceil(2^32 / d); unused for d == 1
  int d;
  __host__ __device__ void set(int div) {
    d = div;
    magic = (div > 1) ? 0xFFFFFFFFu / (unsigned)div + 1u : 0u;
  }
  __device__ __forceinline__ int div(int u) const { return (d > 1) ? (int)__umulhi((uint32_t)u, magic) : u; }
};
// The divisors of a launch (row tiles per slot, chunks per segment, slots per token), prepared on the host.
struct GemvDivs {
  FastDiv tps, kc, od;
};

struct GemvGeom {
  int gi, TG, tiles_per_slot, n_rt, cpw, c_begin, KC, NG, nseg, token, lane, g;
  int upi, upi_shift, UB, grp, G, item0, item_stride;   // grouped mode: the CTA walks items of UB units, upi (a power of two) per group
  FastDiv tps_div, kc_div;
};

__device__ __forceinline__ GemvLoc gemv_locate(const MmbFp4GemvParams& p, const GemvGeom& ge, int it, int v) {
  GemvLoc L;
  int u = ge.gi + it * ge.TG;
  if (p.mode == 3) {
    const int n = it >> ge.upi_shift;
    u = (ge.item0 + n * ge.item_stride) * ge.UB + ge.grp + (it - (n << ge.upi_shift)) * ge.G;
  }
  if (p.mode == 1 || p.mode == 3) {       // slot = MoE slot (mode 1) or tile-list entry (mode 3)
    L.slot = ge.tps_div.div(u);
    L.rt0 = u - L.slot * ge.tiles_per_slot;
  } else {
    L.slot = 0;
    L.rt0 = u;
  }
  L.tsel = (v >= ge.cpw) ? 1 : 0;
  const int off = v - L.tsel * ge.cpw;
  const int ci = ge.c_begin + off;
  const int rt = L.rt0 + L.tsel * (ge.n_rt >> 1);
  L.sidx = 0;
  L.cc = ci;
  if (ge.nseg > 1) {
    L.sidx = ge.kc_div.div(ci);
    L.cc = ci - L.sidx * ge.KC;
  }
  const SegPtr sp = seg_lookup(p, ge.token, (p.mode == 1 || p.mode == 3) ? L.slot : L.sidx);
  L.mult = sp.mult;
  L.q = (sp.q != nullptr) ? sp.q + ((long long)rt * ge.KC + L.cc) * 32 + ge.lane : nullptr;
  L.s = (sp.s != nullptr) ? sp.s + (long long)rt * ge.NG * 8 + ge.g : nullptr;
  L.run = min(ge.cpw - off, ge.KC - L.cc);
  return L;
}

// NWARPS warps per CTA (8: two CTAs per SM, so the next kernel's CTAs become resident and prefetch while this
// one drains; 16: one CTA per SM).  The warps form groups of `wpt`; a group owns one unit of work at a time - a
// 16-row tile, or a gate/up tile pair when the SwiGLU epilogue is fused - and splits its K axis; the groups of
// the whole grid walk the units round-robin, so the activation is staged once per CTA however many tiles it
// ends up processing.  Every warp streams its weights through a private ring of kRing 512-byte blocks in
// shared memory filled by cp.async, which runs on across tile and unit boundaries; the code of the loop exists
// once (no unrolled register ring), which matters because these kernels are short enough to be bound by
// instruction fetch.
//
// GROUPED (mode 3) serves a batch routed through a mixture of experts: rows are sorted by expert and cut into
// tiles of at most 8 rows by a device-built list.  A CTA walks work items - (tile, block of UB units) - stages
// the tile's rows once per item, and its groups take `upi` units each; the weight rings run on across items.
//
// GM selects the loop shape by quantization group size: 0 - groups below 64 (scale word fetched per k16 step), 1 - groups
// of 64 (one 64-wide chunk per trip), 2 - groups of 128 and more (two chunks and one scale word per trip: the per-trip
// bookkeeping of loader and consumer is paid once per 1 KB of weights, which matters because the fully loaded kernel
// is bound by instruction issue, not by DRAM).
//
// MB row blocks (dense mode only): a CTA holds 8 * MB token rows and every expanded weight fragment feeds MB MMAs, one per
// block of 8 rows, so the expansion - the bulk of the instructions - is paid once for 16 tokens (MB = 2; four blocks
// measured slower: staging 32 rows per CTA costs more than the expansion saved).  The extra accumulators need more
// registers than two resident 8-warp CTAs leave, so that variant runs one CTA per SM.
template <int GM, int NWARPS, bool GROUPED, int MB>
__global__ void __launch_bounds__(NWARPS * 32, (NWARPS == 8 && MB == 1) ? 2 : 1) fp4_gemv_kernel(const MmbFp4GemvParams p, const int wpt, const int mrows, const GemvDivs divs) {
  static_assert(MB == 1 || (!GROUPED && NWARPS == 8), "row blocks exist for the dense 8-warp kernel");
  constexpr bool BIG_GROUPS = GM > 0;
  constexpr int CPI = (GM == 2) ? 2 : 1;       // chunks per trip
  constexpr int kRingIt = kRing / CPI;         // ring slots (one trip's weights each)
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float red[2][NWARPS][2][128];
  __shared__ float ss_red[NWARPS][8 * MB];
  __shared__ float rstd_s[8 * MB];
  constexpr int kGemvThreads = NWARPS * 32;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;

  constexpr bool grouped = GROUPED;
  const int S = (p.mode == 0 || grouped) ? 1 : (p.topk + p.n_shared);
  int m0, mt, token = 0;
  if (grouped) {
    m0 = 0;
    mt = 8;                             // per unit: the tile's row count
  } else if (p.mode == 0) {
    m0 = blockIdx.y * mrows;            // mrows <= 8 * MB token rows per CTA (fewer when K is so large that they do not fit)
    mt = min(mrows, p.M - m0);
  } else {
    token = blockIdx.y;
    m0 = token;
    mt = 1;
  }
  const int nseg = (p.mode == 2) ? S : 1;
  const int Kv = nseg * p.K;   // virtual K
  const int XS = Kv + 32;      // smem row stride in halves: rows are 64 bytes apart mod 128 -> 16-byte loads of a
                               // quarter warp (2 rows x 4 lanes) touch distinct banks
  // rows of the staging area: mode 2 stages its S segments as one row of S * K; grouped mode restages up to 8 rows per item
  const int rows_to_stage = (p.mode == 2) ? 1 : mt;
  __half* xs = reinterpret_cast<__half*>(smem_raw);
  const uint32_t ring_q = smem_u32(smem_raw) + (uint32_t)((((size_t)rows_to_stage * XS * 2) + 127) & ~(size_t)127) +
                          (uint32_t)warp * (kRing * 512) + (uint32_t)lane * 16;
  const uint32_t ring_s = smem_u32(smem_raw) + (uint32_t)((((size_t)rows_to_stage * XS * 2) + 127) & ~(size_t)127) +
                          (uint32_t)NWARPS * (kRing * 512) + (uint32_t)warp * (kRing * 128) + (uint32_t)lane * 4;

  // ---- work assignment of this warp (depends on launch parameters only)
  GemvGeom ge;
  ge.n_rt = (p.N + 15) >> 4;
  const int NT = (p.act == 1) ? 2 : 1;                                   // tiles per unit
  ge.tiles_per_slot = (p.act == 1) ? (ge.n_rt >> 1) : ge.n_rt;
  const int n_units = ((p.mode == 1) ? S : 1) * ge.tiles_per_slot;
  const int G = NWARPS / wpt;                                            // groups per CTA
  ge.TG = gridDim.x * G;                                                 // groups in the grid (per blockIdx.y)
  const int grp = warp / wpt, wi = warp - grp * wpt;
  ge.gi = blockIdx.x * G + grp;
  // units of this group (grouped mode: known after the wait, the tile count lives on the device)
  int n_iter = (!grouped && ge.gi < n_units) ? (n_units - ge.gi + ge.TG - 1) / ge.TG : 0;
  ge.KC = p.K >> 6;                        // chunks per segment
  ge.kc_div = divs.kc;
  ge.NG = p.K >> p.gs_shift;               // groups per segment
  ge.nseg = nseg;
  ge.token = token;
  ge.lane = lane;
  ge.g = g;
  ge.G = G;
  ge.grp = grp;
  ge.upi = grouped ? mrows : 1;            // grouped launches pass the units per item and group in this argument
  ge.upi_shift = 31 - __clz(ge.upi);
  ge.tps_div = divs.tps;
  ge.UB = G * ge.upi;
  ge.item0 = blockIdx.x;
  ge.item_stride = gridDim.x;
  const int gs = 1 << p.gs_shift;
  {
    const int unit_chunks = (gs >= 64) ? (gs >> 6) : 1;
    const int total_units = (nseg * ge.KC) / unit_chunks;
    ge.c_begin = (int)(((long long)wi * total_units) / wpt) * unit_chunks;
    ge.cpw = (int)(((long long)(wi + 1) * total_units) / wpt) * unit_chunks - ge.c_begin;   // chunks per tile
  }
  const int cv = NT * ge.cpw;                                            // chunks of this warp per unit
  const int cpg_shift = BIG_GROUPS ? (p.gs_shift - 6) : 0;               // log2(chunks per quantization group)

  // ---- loader: one cp.async (16 bytes per lane) per chunk, plus the 4-byte scale word of the lane's row pair
  int l_it = 0, l_v = 0, l_cnt = 0, l_run = 0, l_cc = 0, l_qb = 0, l_sb = 0;     // l_qb / l_sb: bytes to copy (0 = zero fill: no expert)
  const uint4* l_q = reinterpret_cast<const uint4*>(p.qw);
  const uint32_t* l_s = reinterpret_cast<const uint32_t*>(p.sc);
  auto issue = [&]() {
    if (cv > 0 && l_it < n_iter) {
      if (l_run == 0) {
        const GemvLoc L = gemv_locate(p, ge, l_it, l_v);
        l_qb = (L.q != nullptr) ? 16 : 0;
        l_sb = (L.s != nullptr) ? 4 : 0;
        l_q = (L.q != nullptr) ? L.q : reinterpret_cast<const uint4*>(p.qw);
        l_s = (L.s != nullptr) ? L.s : reinterpret_cast<const uint32_t*>(p.sc);
        l_cc = L.cc;
        l_run = L.run;
      }
      const uint32_t slot = (uint32_t)l_cnt & (kRingIt - 1);
#pragma unroll
      for (int c = 0; c < CPI; ++c)
        cp_async_16(ring_q + slot * (CPI * 512) + c * 512, l_q + c * 32, l_qb);
      if (BIG_GROUPS)       // the chunks of a trip share their quantization group
        cp_async_4(ring_s + slot * 128, l_sb ? (const void*)(l_s + (l_cc >> cpg_shift) * 8) : (const void*)l_s, l_sb);
      if (l_qb) l_q += 32 * CPI;
      l_cc += CPI;
      l_run -= CPI;
      l_v += CPI;
      if (l_v == cv) {
        l_v = 0;
        ++l_it;
      }
    }
    cp_async_commit_group();
    ++l_cnt;
  };

  // the RMSNorm weight is static: fetch this thread's first slices before waiting (the rest, for K beyond two
  // trips of the CTA, is read where it is used)
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
  // Dense weights never change, so the ring is filled before waiting for the previous kernel; MoE fetches depend
  // on the router's expert ids and must come after the wait.
#pragma unroll 1
  for (int phase = 0; phase < 2; ++phase) {
    if (phase == 1) {
      pdl_launch_dependents();
      pdl_wait();
      if (grouped) {
        const int n_items = min(*p.n_tiles, p.max_tiles) * (ge.tiles_per_slot / ge.UB);
        n_iter = ((int)blockIdx.x < n_items) ? ((n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x) * ge.upi : 0;
      }
    }
    if ((p.mode == 0) == (phase == 0)) {
#pragma unroll 1
      for (int i = 0; i < kRingIt; ++i) issue();
    }
  }

  // ---- stage activations as fp16 (optional residual add + RMSNorm), 8 elements per thread per trip
  const bf16* xg = reinterpret_cast<const bf16*>(p.x);
  const bf16* dg = reinterpret_cast<const bf16*>(p.delta);
  bf16* ro = reinterpret_cast<bf16*>(p.resid_out);
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

  // Pass A reads global memory once: x (+ delta or the tp partial sums), rounded to bf16 like an unfused add;
  // writes the new residual; without a norm it stores the final fp16 value, with a norm it parks the bf16 bits
  // in the same shared-memory slots (fragment order) and accumulates the sum of squares.  Pass B (norm only)
  // has every thread rewrite its own slots with bf16(v * rstd * w) as fp16.
  const int stage_k = (p.mode == 2) ? Kv : p.K;          // staged width of a row (columns beyond Kx are zero)
  if (MB > 1) {
    // Many rows (dense mode, no exchange): one warp per row, so a row's loads are all in flight together, its sum of
    // squares needs one warp reduction, and pass B touches only slots the same lane wrote - no CTA barrier per row.
#pragma unroll 1
    for (int j = warp; j < rows_to_stage; j += NWARPS) {
      __half* dst = xs + (long long)j * XS;
      float ss = 0.f;
#pragma unroll 4
      for (int k = lane * 8; k < stage_k; k += 256) {
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (k < p.Kx) {
          const long long src = (long long)(m0 + j) * p.ldx + k;
          const uint4 xv = *reinterpret_cast<const uint4*>(xg + src);
          const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            v[2 * e] = __uint_as_float(xw[e] << 16);
            v[2 * e + 1] = __uint_as_float(xw[e] & 0xffff0000u);
          }
          if (dg != nullptr) {
            const uint4 dv = *reinterpret_cast<const uint4*>(dg + src);
            const uint32_t dw[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              v[2 * e] = __bfloat162float(__float2bfloat16(v[2 * e] + __uint_as_float(dw[e] << 16)));
              v[2 * e + 1] = __bfloat162float(__float2bfloat16(v[2 * e + 1] + __uint_as_float(dw[e] & 0xffff0000u)));
            }
            if (ro != nullptr && blockIdx.x == 0) {
              uint4 o;
              o.x = (__float_as_uint(v[0]) >> 16) | (__float_as_uint(v[1]) & 0xffff0000u);
              o.y = (__float_as_uint(v[2]) >> 16) | (__float_as_uint(v[3]) & 0xffff0000u);
              o.z = (__float_as_uint(v[4]) >> 16) | (__float_as_uint(v[5]) & 0xffff0000u);
              o.w = (__float_as_uint(v[6]) >> 16) | (__float_as_uint(v[7]) & 0xffff0000u);
              *reinterpret_cast<uint4*>(ro + (long long)(m0 + j) * p.Kx + k) = o;
            }
          }
        }
        __half* blk = dst + (k & ~31) + ((k >> 4) & 1) * 4 + ((k >> 3) & 1) * 2;
        if (nw != nullptr) {
#pragma unroll
          for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
#pragma unroll
          for (int tt = 0; tt < 4; ++tt)
            *reinterpret_cast<uint32_t*>(blk + tt * 8) = (__float_as_uint(v[2 * tt]) >> 16) | (__float_as_uint(v[2 * tt + 1]) & 0xffff0000u);
        } else {
#pragma unroll
          for (int tt = 0; tt < 4; ++tt)
            *reinterpret_cast<__half2*>(blk + tt * 8) = __floats2half2_rn(fminf(fmaxf(v[2 * tt], -65504.f), 65504.f),
                                                                          fminf(fmaxf(v[2 * tt + 1], -65504.f), 65504.f));
        }
      }
      if (nw != nullptr) {
        const float rs = rsqrtf(warp_sum(ss) / (float)p.Kx + p.eps);
#pragma unroll 4
        for (int k = lane * 8; k < p.Kx; k += 256) {
          const uint4 nv = *reinterpret_cast<const uint4*>(nw + k);
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
    }
  }
#pragma unroll 1
  for (int j = 0; j < ((grouped || MB > 1) ? 0 : rows_to_stage); ++j) {
    float ss = 0.f;
    __half* dst = xs + (long long)j * XS;
#pragma unroll 1
    for (int k = tid * 8; k < stage_k; k += kGemvThreads * 8) {
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      bool valid = k < p.Kx;
      long long src = (long long)(m0 + j) * p.ldx + k;
      if (p.mode == 2) {
        const int sg = k / p.K, off = k - sg * p.K;       // segment rows of h are ldx apart
        valid = off < p.Kx;
        src = (long long)(token * S + sg) * p.ldx + off;
      }
      if (valid) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xg + src);
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
          const uint4 dv = *reinterpret_cast<const uint4*>(dg + src);
          const uint32_t dw[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            v[2 * e] = __bfloat162float(__float2bfloat16(v[2 * e] + __uint_as_float(dw[e] << 16)));
            v[2 * e + 1] = __bfloat162float(__float2bfloat16(v[2 * e + 1] + __uint_as_float(dw[e] & 0xffff0000u)));
          }
        }
        if ((dg != nullptr || has_tin) && ro != nullptr && blockIdx.x == 0) {
          uint4 o;
          o.x = (__float_as_uint(v[0]) >> 16) | (__float_as_uint(v[1]) & 0xffff0000u);
          o.y = (__float_as_uint(v[2]) >> 16) | (__float_as_uint(v[3]) & 0xffff0000u);
          o.z = (__float_as_uint(v[4]) >> 16) | (__float_as_uint(v[5]) & 0xffff0000u);
          o.w = (__float_as_uint(v[6]) >> 16) | (__float_as_uint(v[7]) & 0xffff0000u);
          *reinterpret_cast<uint4*>(ro + (long long)(m0 + j) * p.Kx + k) = o;
        }
      }
      // fragment order inside each 32-wide block: lane t finds (b0, b1) of both k16 steps in 16 contiguous bytes
      __half* blk = dst + (k & ~31) + ((k >> 4) & 1) * 4 + ((k >> 3) & 1) * 2;
      if (nw != nullptr) {
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
#pragma unroll
        for (int tt = 0; tt < 4; ++tt)    // bf16 bits parked in the fp16 slots until pass B
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
      if (lane == 0) ss_red[warp][j] = ss;
    }
  }
  if (!grouped && MB == 1 && nw != nullptr) {
    __syncthreads();
    if (tid < rows_to_stage) {
      float tot = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < NWARPS; ++w2) tot += ss_red[w2][tid];
      rstd_s[tid] = rsqrtf(tot / (float)p.Kx + p.eps);
    }
    __syncthreads();
#pragma unroll 1
    for (int j = 0; j < rows_to_stage; ++j) {
      const float rs = rstd_s[j];
      __half* dst = xs + (long long)j * XS;
#pragma unroll 1
      for (int jj = 0, k = tid * 8; k < p.Kx; ++jj, k += kGemvThreads * 8) {
        const uint4 nv = (jj == 0) ? nwv[0] : ((jj == 1) ? nwv[1] : *reinterpret_cast<const uint4*>(nw + k));
        const uint32_t nww[4] = {nv.x, nv.y, nv.z, nv.w};
        __half* blk = dst + (k & ~31) + ((k >> 4) & 1) * 4 + ((k >> 3) & 1) * 2;
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
          const uint32_t bits = *reinterpret_cast<const uint32_t*>(blk + tt * 8);
          // round to bf16 like an unfused norm kernel would, so fused and unfused paths agree
          float a = __bfloat162float(__float2bfloat16(__uint_as_float(bits << 16) * rs * __uint_as_float(nww[tt] << 16)));
          float b = __bfloat162float(__float2bfloat16(__uint_as_float(bits & 0xffff0000u) * rs * __uint_as_float(nww[tt] & 0xffff0000u)));
          a = fminf(fmaxf(a, -65504.f), 65504.f);
          b = fminf(fmaxf(b, -65504.f), 65504.f);
          *reinterpret_cast<__half2*>(blk + tt * 8) = __floats2half2_rn(a, b);
        }
      }
    }
  }
  __syncthreads();

  // ---- main loop.  Per 64-wide chunk: one 16-byte shared load of the lane's weight words, two 16-byte shared
  // loads with the B fragments of its four k16 steps (the staging above stored x in fragment order),
  // 4 x (12 integer ops + 1 MMA), and once per quantization group the scale applied to the group accumulator
  // in fp32.
  const bool tp_out = p.tpx.out_peer_slots != nullptr;
  TpOut tout;
  tout.peer_slots = p.tpx.out_peer_slots;
  tout.peer_flags = p.tpx.out_peer_flags;
  tout.counter = p.tpx.out_counter;
  tout.step = p.tpx.step;
  tout.tp = p.tpx.tp;
  tout.mc_slot = p.tpx.out_mc_slot;
  bf16* const out = reinterpret_cast<bf16*>(p.out);
  {
    const int gmask = gs - 1;
    const int cpg_mask = (1 << cpg_shift) - 1;
    const __half* xbase = xs + min(g, mt - 1) * ((p.mode == 2) ? 0 : XS) + t * 8;
    // row blocks beyond the first: element offset of this lane's row (clamped to the last staged row) from xbase
    int xoff[MB];
#pragma unroll
    for (int b = 0; b < MB; ++b) xoff[b] = (min(b * 8 + g, mt - 1) - min(g, mt - 1)) * XS;
    const FastDiv od_div = divs.od;
    const unsigned char* ring_q_gen = smem_raw + (ring_q - smem_u32(smem_raw));
    const unsigned char* ring_s_gen = smem_raw + (ring_s - smem_u32(smem_raw));
    int c_cnt = 0, c_run = 0, c_cc = 0, c_tsel = 0, c_slot = 0, c_rt0 = 0, ebuf = 0;
    float mult = 0.f;
    const __half* xp = xbase;
    const uint32_t* c_s = nullptr;
#pragma unroll 1
    for (int it = 0; it < n_iter; ++it) {
      if (grouped && (it & (ge.upi - 1)) == 0) {
        // new item: every group is done with the previous rows; stage the rows of this item's tile (already
        // normalized bf16, clamped into fp16, fragment order as above)
        const int item = ge.item0 + (it >> ge.upi_shift) * ge.item_stride;
        const int tj = ge.tps_div.div(item * ge.UB);
        __syncthreads();
        m0 = __ldg(p.tile_row0 + tj);
        mt = min(__ldg(p.tile_rows + tj), 8);
        // source rows first (eight independent loads), then one 16-byte load per row and trip, all in flight together
        int srows[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          srows[r] = -1;
          if (r < mt) {
            srows[r] = m0 + r;
            if (p.order_div > 0) {
              const int pair = __ldg(p.row_order + m0 + r);
              srows[r] = (pair >= 0) ? od_div.div(pair) : -1;
            }
          }
        }
#pragma unroll 1
        for (int k = tid * 8; k < p.K; k += kGemvThreads * 8) {
          uint4 xv[8];
#pragma unroll
          for (int r = 0; r < 8; ++r)
            xv[r] = (srows[r] >= 0) ? *reinterpret_cast<const uint4*>(xg + (long long)srows[r] * p.ldx + k) : make_uint4(0, 0, 0, 0);
          __half* blk0 = xs + (k & ~31) + ((k >> 4) & 1) * 4 + ((k >> 3) & 1) * 2;
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            if (r >= mt) break;
            const uint32_t xw[4] = {xv[r].x, xv[r].y, xv[r].z, xv[r].w};
            __half* blk = blk0 + (long long)r * XS;
#pragma unroll
            for (int tt = 0; tt < 4; ++tt)
              *reinterpret_cast<__half2*>(blk + tt * 8) =
                  __floats2half2_rn(fminf(fmaxf(__uint_as_float(xw[tt] << 16), -65504.f), 65504.f),
                                    fminf(fmaxf(__uint_as_float(xw[tt] & 0xffff0000u), -65504.f), 65504.f));
          }
        }
        __syncthreads();
        xbase = xs + min(g, mt - 1) * XS + t * 8;
      }
      float accg[MB][4];    // tile 0 of the unit
      float accu[MB][4];    // tile 1 (the up half when the SwiGLU epilogue is fused)
      float gacc[MB][4];
#pragma unroll
      for (int b = 0; b < MB; ++b)
#pragma unroll
        for (int e = 0; e < 4; ++e) accg[b][e] = accu[b][e] = gacc[b][e] = 0.f;
      uint32_t s2 = 0;
#pragma unroll 1
      for (int v = 0; v < cv; v += CPI) {
        if (c_run == 0) {
          const GemvLoc L = gemv_locate(p, ge, it, v);
          c_run = L.run;
          c_cc = L.cc;
          c_tsel = L.tsel;
          c_slot = L.slot;
          c_rt0 = L.rt0;
          c_s = L.s;
          mult = L.mult * kE2M1F16Rescale;
          xp = xbase + (long long)L.sidx * p.K + L.cc * 64;
        }
        cp_async_wait_group<kRingIt - 1>();
        const uint32_t slot = (uint32_t)c_cnt & (kRingIt - 1);
        uint4 wq[CPI];
#pragma unroll
        for (int c = 0; c < CPI; ++c) wq[c] = *reinterpret_cast<const uint4*>(ring_q_gen + slot * (CPI * 512) + c * 512);
        const uint32_t s_cur = BIG_GROUPS ? *reinterpret_cast<const uint32_t*>(ring_s_gen + slot * 128) : 0u;
        issue();   // refill the slot just read
        if (BIG_GROUPS) s2 = s_cur;
#pragma unroll
        for (int c = 0; c < CPI; ++c) {
          const uint32_t qq[4] = {wq[c].x, wq[c].y, wq[c].z, wq[c].w};
          uint32_t bb[MB][8];
#pragma unroll
          for (int b = 0; b < MB; ++b) {
            const uint4 xv0 = *reinterpret_cast<const uint4*>(xp + xoff[b] + c * 64);
            const uint4 xv1 = *reinterpret_cast<const uint4*>(xp + xoff[b] + c * 64 + 32);
            bb[b][0] = xv0.x; bb[b][1] = xv0.y; bb[b][2] = xv0.z; bb[b][3] = xv0.w;
            bb[b][4] = xv1.x; bb[b][5] = xv1.y; bb[b][6] = xv1.z; bb[b][7] = xv1.w;
          }
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            if (!BIG_GROUPS) {
              const int kabs = c_cc * 64 + ks * 16;
              if ((kabs & gmask) == 0) s2 = (c_s != nullptr) ? __ldg(c_s + (kabs >> p.gs_shift) * 8) : 0u;
            }
            uint32_t a0, a1, a2, a3;
            e2m1x8_to_f16x2(qq[ks], a0, a1, a2, a3);
#pragma unroll
            for (int b = 0; b < MB; ++b) mma_f16_16816(gacc[b], a0, a1, a2, a3, bb[b][2 * ks], bb[b][2 * ks + 1]);
            // group complete: apply its scale to the group accumulator in fp32 (big groups: once per trip at most)
            const bool flush = BIG_GROUPS ? (c == CPI - 1 && ks == 3 && (((c_cc + CPI) & cpg_mask) == 0))
                                          : (((c_cc * 64 + ks * 16 + 16) & gmask) == 0);
            if (flush) {
              const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&s2));
              const float slo = sf.x * mult, shi = sf.y * mult;
#pragma unroll
              for (int b = 0; b < MB; ++b) {
                if (c_tsel == 0) {
                  accg[b][0] = fmaf(gacc[b][0], slo, accg[b][0]);
                  accg[b][1] = fmaf(gacc[b][1], slo, accg[b][1]);
                  accg[b][2] = fmaf(gacc[b][2], shi, accg[b][2]);
                  accg[b][3] = fmaf(gacc[b][3], shi, accg[b][3]);
                } else {
                  accu[b][0] = fmaf(gacc[b][0], slo, accu[b][0]);
                  accu[b][1] = fmaf(gacc[b][1], slo, accu[b][1]);
                  accu[b][2] = fmaf(gacc[b][2], shi, accu[b][2]);
                  accu[b][3] = fmaf(gacc[b][3], shi, accu[b][3]);
                }
                gacc[b][0] = gacc[b][1] = gacc[b][2] = gacc[b][3] = 0.f;
              }
            }
          }
        }
        xp += 64 * CPI;
        c_cc += CPI;
        c_run -= CPI;
        ++c_cnt;
      }
      // ---- reduction over the warps of the group and epilogue of this unit.  `red` is double buffered by unit
      // parity, so one group barrier per unit is enough: a warp can only overwrite a buffer after passing the
      // barrier of the unit in between, which the readers of that buffer reach after they are done with it.
      if (cv == 0) {   // a warp without chunks of its own still needs the unit of its group for the epilogue
        const GemvLoc L = gemv_locate(p, ge, it, 0);
        c_slot = L.slot;
        c_rt0 = L.rt0;
      }
      const int w0 = grp * wpt;
#pragma unroll
      for (int b = 0; b < MB; ++b) {
        if (b * 8 >= mt) break;
        const int buf = ebuf;         // alternates per executed block epilogue (see the note on `red` above)
        ebuf ^= 1;
        {
          float* r = &red[buf][warp][0][0];
          r[g * 8 + 2 * t] = accg[b][0];
          r[g * 8 + 2 * t + 1] = accg[b][1];
          r[(g + 8) * 8 + 2 * t] = accg[b][2];
          r[(g + 8) * 8 + 2 * t + 1] = accg[b][3];
          if (NT == 2) {
            r += 128;
            r[g * 8 + 2 * t] = accu[b][0];
            r[g * 8 + 2 * t + 1] = accu[b][1];
            r[(g + 8) * 8 + 2 * t] = accu[b][2];
            r[(g + 8) * 8 + 2 * t + 1] = accu[b][3];
          }
        }
        if (wpt > 1) group_bar(1 + grp, wpt * 32);
        else __syncwarp();
        for (int o = wi * 32 + lane; o < 16 * 8; o += wpt * 32) {
          const int row = o >> 3, col = b * 8 + (o & 7);
          if (col >= mt) continue;
          float v = 0.f;
#pragma unroll 4
          for (int w2 = 0; w2 < wpt; ++w2) v += red[buf][w0 + w2][0][o];
          const long long orow = (p.mode == 1) ? (long long)token * S + c_slot : (long long)(m0 + col);
          if (grouped && p.expert_w != nullptr) {
            const int pair = __ldg(p.row_order + orow);
            v *= (pair >= 0) ? __ldg(p.expert_w + pair) : 0.f;
          }
          const int n = c_rt0 * 16 + row;
          if (p.act == 1) {
            float u = 0.f;
#pragma unroll 4
            for (int w2 = 0; w2 < wpt; ++w2) u += red[buf][w0 + w2][1][o];
            if (n < (p.N >> 1)) out[orow * p.ldo + n] = __float2bfloat16(silu(v) * u);
          } else if (n < p.N) {
            if (tp_out) {
              // tensor-parallel producer: this rank's partial goes straight into every peer's receive buffer
              tp_push(tout, orow * p.N + n, v);
            } else {
              if (p.bias) v += __bfloat162float(reinterpret_cast<const bf16*>(p.bias)[n]);
              if (p.out_add) v += __bfloat162float(reinterpret_cast<const bf16*>(p.out_add)[orow * p.ldo + n]);
              out[orow * p.ldo + n] = __float2bfloat16(v);
            }
          }
        }
      }
    }
  }
  cp_async_wait_group<0>();
  if (tp_out) tp_signal(tout, gridDim.x * gridDim.y);
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

// `static_bytes`: the kernel's statically declared shared memory, which counts against the same 48 KB default.
template <typename K>
static int set_smem(K kernel, size_t bytes, size_t static_bytes = 0) {
  if (bytes + static_bytes > 48 * 1024) {
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
  const int S = (p.mode == 0 || p.mode == 3) ? 1 : (p.topk + p.n_shared);
  if (S > kMaxSeg) return (int)cudaErrorInvalidValue;
  if (p.mode == 3 && (p.norm_w != nullptr || p.delta != nullptr || p.tpx.in_buf != nullptr || p.tpx.out_peer_slots != nullptr ||
                      p.tile_expert == nullptr || p.tile_row0 == nullptr || p.tile_rows == nullptr || p.n_tiles == nullptr ||
                      p.max_tiles <= 0 || p.Kx != p.K || ((p.order_div > 0 || p.expert_w != nullptr) && p.row_order == nullptr)))
    return (int)cudaErrorInvalidValue;
  if (p.mode == 2 && (p.norm_w != nullptr || p.delta != nullptr)) return (int)cudaErrorInvalidValue;
  const int n_rt = (p.N + 15) / 16;
  size_t smem;
  dim3 grid;
  int mrows = 8, mb = 1;
  if (p.mode == 0) {
    // token rows staged per CTA: up to 8 per row block; 2 row blocks (one CTA per SM) when more than 8 tokens come and
    // their rows fit beside the weight rings; fewer than 8 rows when K is so large that 8 do not fit
    const size_t row_bytes = (size_t)(p.K + 32) * 2;
    const size_t ring_bytes = (size_t)8 * kRing * (512 + 128);
    if (p.M > 8 && 16 * row_bytes + ring_bytes <= 204 * 1024) mb = 2;
    if (p.tpx.in_buf != nullptr || p.tpx.out_peer_slots != nullptr) mb = 1;       // the exchange paths are decode-size
    mrows = 8 * mb;
    const size_t budget = 170 * 1024 - (size_t)16 * kRing * (512 + 128);
    while (mb == 1 && mrows > 1 && (size_t)mrows * row_bytes > budget) mrows >>= 1;
    const int mt = p.M < mrows ? p.M : mrows;
    smem = (size_t)mt * row_bytes;
    grid.y = (p.M + mrows - 1) / mrows;
  } else if (p.mode == 3) {
    smem = (size_t)8 * (p.K + 32) * 2;
    grid.y = 1;
  } else if (p.mode == 1) {
    smem = (size_t)(p.K + 32) * 2;
    grid.y = p.M;
  } else {
    smem = (size_t)(S * p.K + 32) * 2;
    grid.y = p.M;
  }
  if (p.tpx.out_peer_slots != nullptr && (p.act != 0 || p.mode == 1)) return (int)cudaErrorInvalidValue;
  if (p.act == 1 && n_rt % 2 != 0) return (int)cudaErrorInvalidValue;
  grid.z = 1;
  const int gm = p.gs_shift >= 7 ? 2 : (p.gs_shift == 6 ? 1 : 0);
  // Work units per token tile: row tiles (tile pairs with the fused SwiGLU), times the MoE slots in mode 1.
  const int n_units = ((p.mode == 1) ? S : 1) * ((p.act == 1) ? n_rt / 2 : n_rt);
  const int chunks = ((p.mode == 2) ? S : 1) * (p.K / 64);
  const int gs = 1 << p.gs_shift;
  const int k_units = chunks / ((gs >= 64) ? (gs >> 6) : 1);      // indivisible pieces of the K axis
  // Warps per unit: as many as keep every warp of the machine busy (148 SMs x 16 warps) while a warp still owns
  // at least two 64-wide chunks of a tile.
  const int warp_slots = 148 * ((mb > 1) ? 8 : 16) / (int)grid.y;
  int wpt = (mb > 1) ? 8 : 16;
  while (wpt > 1 && ((long long)n_units * wpt > warp_slots || k_units < wpt || chunks < 2 * wpt)) wpt >>= 1;
  if (p.mode == 3) {
    // many units per CTA: a warp should own at least a ring's worth of chunks per unit; 8-warp CTAs, two per SM
    const int tps = (p.act == 1) ? n_rt / 2 : n_rt;
    const int unit_chunks = ((p.act == 1) ? 2 : 1) * chunks;
    wpt = 8;
    while (wpt > 1 && (unit_chunks < 4 * kRing * wpt || k_units < wpt)) wpt >>= 1;
    while (wpt < 8 && tps % (8 / wpt) != 0) wpt <<= 1;      // the groups of a CTA share the units of an item evenly
    if (p.grouped_wpt > 0) wpt = p.grouped_wpt;
    if (wpt > 8 || (wpt & (wpt - 1)) || k_units < wpt) return (int)cudaErrorInvalidValue;
    const int Gg = 8 / wpt;
    if (tps % Gg != 0) return (int)cudaErrorInvalidValue;
    // units per item and group: items of about a quarter of a wave each, so the tail stays short, but as many units
    // per staging of the rows as that allows
    int upi = 8;
    while (upi > 1 && (tps % (Gg * upi) != 0 || (long long)p.max_tiles * tps / (Gg * upi) < 4 * 296)) upi >>= 1;
    if (p.grouped_upi > 0) upi = p.grouped_upi;
    if (tps % (Gg * upi) != 0 || (upi & (upi - 1))) return (int)cudaErrorInvalidValue;
    mrows = upi;
  }
  const int nw = (wpt == 16) ? 16 : 8;
  const int G = nw / wpt;
  const int cta_units = (n_units + G - 1) / G;                   // CTAs needed for one unit per group
  int cap = ((nw == 8 && mb == 1) ? 296 : 148) / (int)grid.y;    // CTAs of one wave
  if (cap < 1) cap = 1;
  const int passes = (cta_units + cap - 1) / cap;
  grid.x = (cta_units + passes - 1) / passes;
  if (p.mode == 3) {
    const long long items = (long long)p.max_tiles * (((p.act == 1) ? n_rt / 2 : n_rt) / (G * mrows));
    grid.x = (unsigned)(items < 296 ? items : 296);
  }
  // dynamic shared memory: the staged activation rows, then every warp's weight ring (512 + 128 bytes per slot)
  smem = ((smem + 127) & ~(size_t)127) + (size_t)nw * kRing * (512 + 128);
  if (smem > (size_t)((mb > 1) ? 206 : 180) * 1024) return (int)cudaErrorInvalidValue;
  GemvDivs divs;
  divs.tps.set((p.act == 1) ? n_rt / 2 : n_rt);
  divs.kc.set(p.K / 64);
  divs.od.set(p.order_div > 0 ? p.order_div : 1);
  int e;
#define MMB_LAUNCH_GEMV(GM_, NW, GR, MB_)                                                                     \
  do {                                                                                                        \
    if ((e = set_smem(fp4_gemv_kernel<GM_, NW, GR, MB_>, smem, 34 * 1024))) return e;                                   \
    return launch(fp4_gemv_kernel<GM_, NW, GR, MB_>, grid, dim3(NW * 32), smem, stream, 1, p, wpt, mrows, divs);  \
  } while (0)
#define MMB_LAUNCH_GEMV_GM(NW, GR, MB_)                 \
  do {                                                  \
    if (gm == 2) MMB_LAUNCH_GEMV(2, NW, GR, MB_);       \
    if (gm == 1) MMB_LAUNCH_GEMV(1, NW, GR, MB_);       \
    MMB_LAUNCH_GEMV(0, NW, GR, MB_);                    \
  } while (0)
  if (p.mode == 3) MMB_LAUNCH_GEMV_GM(8, true, 1);
  if (mb == 2) MMB_LAUNCH_GEMV_GM(8, false, 2);
  if (nw == 8) MMB_LAUNCH_GEMV_GM(8, false, 1);
  MMB_LAUNCH_GEMV_GM(16, false, 1);
#undef MMB_LAUNCH_GEMV_GM
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
