// tcgen05 GEMM for sm_100a: out[M, N] = x[M, K] * W^T with fp32 accumulators in tensor memory.
//
// Orientation: the weight tile is the MMA "A" operand (128 output features = 128 TMEM lanes) and
// the token tile is the "B" operand (TN = 32..256 tokens = TMEM columns), so the same kernel serves
// batch-32 decode (TN = 32) and long prefill (TN = 256) without wasting the M = 128 instruction shape.
//
// CTA = 18 warps (the weight-expanding variants run two such CTAs per SM):
//   warp 0      TMA producer: x tile [TN x 64] bf16, 128-byte swizzle, one bulk tensor copy per stage
//               (bf16-weight variant: also the W tile)
//   warp 1      allocates TMEM, issues tcgen05.mma (one elected lane), commits stages back to the
//               producers through mbarriers
//   warps 2..17 FP4 variant: stream tile-layout weight blocks from global memory and expand E2M1 -> bf16 with
//               the group scale in registers into the 128-byte-swizzled K-major A tile.  The two warps of a
//               16-row block take alternate k blocks (a 16-byte load per lane and block, two blocks in
//               flight).  The kernel is bound by the latency of a warp's (barrier wait -> expand -> store ->
//               fence -> arrive) round trip, not by instruction count, L2 or the tensor pipe, so what counts
//               is warps in flight and few, fat trips: 8 warps measured 390 TFLOP/s on 4096 x 3072 x 2048,
//               16 warps splitting the k16 steps 547, 16 warps alternating k blocks 593.  Afterwards the
//               same warps run the epilogue: tcgen05.ld of their 32-lane TMEM quarter (warp % 4), the four
//               warps of a quarter taking the 32-column chunks round-robin.
// Every mbarrier wait is bounded (wall-clock limit); on expiry the kernel records a code in
// status[0], skips the remaining work, still frees its TMEM and returns.
#include <cuda.h>
#include <stdlib.h>

#include "api_gemm.h"
#include "common.cuh"
#include "tcgen05.cuh"
#include "tp_comm.cuh"

namespace mmb {

constexpr int kBK = 64;                 // K elements per stage (one 128-byte swizzle row of bf16)
constexpr int kTileRows = 128;          // output features per CTA
constexpr int kExpandWarps = 16;          // warps that expand FP4 weights: two per 16-row block and stage, two k16 steps each
constexpr int kExpandSplit = 2;           // stage classes: a k block is expanded by kExpandWarps / kExpandSplit warps
constexpr int kGemmThreads = (2 + kExpandWarps) * 32;

// kind::f16 instruction descriptor: D = f32, A = B = bf16, both K-major, M = 128, N = tn.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int tn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(tn >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);
}

// MINB = 2: two CTAs share an SM (half the pipeline depth each).  The FP4 / trellis main loops are bound by the latency of the
// expansion warps' round trips, not by the tensor pipe or shared memory, so a second resident CTA fills the idle issue slots
// and MMA time of the first; both accumulators fit the 512 TMEM columns (2 x 256).
template <int TN, int MINB>
struct GemmCfg {
  static constexpr int kStages = (MINB == 2) ? ((TN == 256) ? 2 : (TN == 128) ? 3 : 4) : ((TN <= 128) ? 6 : 4);
  static constexpr int a_bytes = kTileRows * kBK * 2;      // 16 KB
  static constexpr int b_bytes = TN * kBK * 2;
  static constexpr int stage_bytes = a_bytes + b_bytes;
  static constexpr int tmem_cols = (TN < 32) ? 32 : TN;
  static constexpr size_t smem_bytes = (size_t)kStages * stage_bytes + 1024 /*align slack*/ + 256 /*barriers*/;
};

struct PipeShared {
  uint64_t full_a[6];
  uint64_t full_b[6];
  uint64_t empty[6];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

// One lane's 32 codes of a codebook row (LSB-first, BITS each) -> four 16-byte chunks of the swizzled K-major A row.
template <int BITS>
__device__ __forceinline__ void cb_expand_row(const uint32_t (&words)[8], const float* lut_s, float zp, float sc, unsigned char* dst,
                                              int half, int r7) {
  constexpr unsigned cmask = (1u << BITS) - 1u;
#pragma unroll
  for (int cc = 0; cc < 4; ++cc) {
    uint32_t o4[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int b0 = (cc * 8 + e * 2) * BITS, b1 = b0 + BITS;
      const float w0 = (lut_s[(words[b0 >> 5] >> (b0 & 31)) & cmask] - zp) * sc;
      const float w1 = (lut_s[(words[b1 >> 5] >> (b1 & 31)) & cmask] - zp) * sc;
      const bf162 pr = __floats2bfloat162_rn(w0, w1);
      o4[e] = *reinterpret_cast<const uint32_t*>(&pr);
    }
    const int chunk = half * 4 + cc;
    *reinterpret_cast<uint4*>(dst + ((chunk ^ r7) * 16)) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
  }
}

// WFMT 0: FP4 tile-layout weights expanded by the warps 2..17.  WFMT 1: bf16 weights fetched by TMA.  WFMT 2: trellis weights
// (16 x 16 tiles of 2..8-bit codes, LSB-first bit stream) decoded by the same warps inside the main loop.  WFMT 3: codebook
// weights (row-major 2 / 4 / 8-bit codes, 256-entry value table, fp16 group scales and optional zero points).  WFMT 4: 2:4
// sparse FP4 weights (two kept E2M1 values + a 4-bit position word per group of four columns), scattered to a dense tile.
template <int TN, int WFMT, int MINB>
__global__ void __launch_bounds__(kGemmThreads, MINB)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
            const MmbFp4GemmParams p, const MmbBf16GemmParams pb) {
  using Cfg = GemmCfg<TN, MINB>;
  constexpr bool QW = WFMT != 1;       // weights are expanded by the warps of this CTA (parameters in `p`)
  extern __shared__ unsigned char smem_dyn[];
  __shared__ float lut_s[WFMT == 3 ? 256 : (WFMT == 4 ? 16 : 1)];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  PipeShared* ps = reinterpret_cast<PipeShared*>(tiles + (size_t)Cfg::kStages * Cfg::stage_bytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- problem decode
  const int M = QW ? p.M : pb.M, N = QW ? p.N : pb.N, K = QW ? p.K : pb.K;
  int* status = QW ? p.status : pb.status;
  const int n0 = blockIdx.x * kTileRows;
  const MmbAgWait& ag = QW ? p.ag : pb.ag;
  int tile_y = blockIdx.y;
  if (ag.flags != nullptr)      // all-gather fused into the load of x: start with the token tiles of this rank's own rows
    tile_y = (int)((blockIdx.y + (unsigned)((ag.rank * ag.rows) / TN)) % gridDim.y);
  int tok0 = tile_y * TN, tok_rows = TN, expert = 0;
  const int batch = blockIdx.z;
  if (QW && p.tile_expert != nullptr) {
    if ((int)blockIdx.y >= *p.n_tiles) return;
    expert = p.tile_expert[blockIdx.y];
    tok0 = p.tile_row0[blockIdx.y];
    tok_rows = p.tile_rows[blockIdx.y];
  }
  const int KB = K / kBK;

  if (tid == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&ps->full_a[s], QW ? kExpandWarps / kExpandSplit : 1);      // the warps of one stage class (see the expansion loop)
      mbar_init(&ps->full_b[s], 1);
      mbar_init(&ps->empty[s], 1);
    }
    mbar_init(&ps->acc_full, 1);
    ps->abort_flag = 0;
    fence_proxy_async_smem();
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&ps->tmem_base, Cfg::tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ps->tmem_base;
  volatile int* abort_flag = &ps->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool x_ready = true;
      if (ag.flags != nullptr) {
        // rows tok0 .. tok0 + TN - 1 arrive from their owners by peer stores; wait (bounded) for those ranks only
        const unsigned want = *ag.step;
        const int last_row = min(tok0 + TN, M) - 1;
        const int r_hi = min(last_row / ag.rows, ag.tp - 1);
        for (int r = tok0 / ag.rows; r <= r_hi && x_ready; ++r) {
          const unsigned* f = ag.flags + r;
          if (ld_acquire_sys(f) >= want) continue;
          const unsigned long long t0 = tp_now_ns();
          unsigned spins = 0;
          while (ld_acquire_sys(f) < want) {
            if ((++spins & 63u) == 0u && tp_now_ns() - t0 > wait_limit_ns(status)) {
              x_ready = false;
              break;
            }
          }
        }
        if (!x_ready) {
          if (atomicExch(&ps->abort_flag, 1) == 0 && status) atomicExch(status, 110);
        }
        asm volatile("fence.proxy.async;" ::: "memory");      // the rows are read through the async proxy (TMA)
      }
      for (int i = 0; i < KB && x_ready; ++i) {
        const int s = i % Cfg::kStages;
        const uint32_t ph = (uint32_t)(i / Cfg::kStages) & 1u;
        if (!mbar_wait(&ps->empty[s], ph ^ 1u, abort_flag)) {
          if (atomicExch(&ps->abort_flag, 1) == 0 && status) atomicExch(status, 1);
          break;
        }
        unsigned char* a_tile = tiles + (size_t)s * Cfg::stage_bytes;
        unsigned char* b_tile = a_tile + Cfg::a_bytes;
        if (QW) {
          mbar_expect_tx(&ps->full_b[s], Cfg::b_bytes);
          tma_load_2d(b_tile, &tmap_x, &ps->full_b[s], i * kBK, tok0);
        } else {
          mbar_expect_tx(&ps->full_b[s], Cfg::b_bytes);
          tma_load_3d(b_tile, &tmap_x, &ps->full_b[s], i * kBK, tok0, pb.x_batch_stride ? batch : 0);
          mbar_expect_tx(&ps->full_a[s], Cfg::a_bytes);
          tma_load_3d(a_tile, &tmap_w, &ps->full_a[s], i * kBK, n0, pb.w_batch_stride ? batch : 0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TN < 16 ? 16 : TN);
      bool ok = true;
      for (int i = 0; i < KB && ok; ++i) {
        const int s = i % Cfg::kStages;
        const uint32_t ph = (uint32_t)(i / Cfg::kStages) & 1u;
        ok = mbar_wait(&ps->full_a[s], ph, abort_flag) && mbar_wait(&ps->full_b[s], ph, abort_flag);
        if (!ok) {
          if (atomicExch(&ps->abort_flag, 1) == 0 && status) atomicExch(status, 2);
          break;
        }
        tc_fence_after();
        unsigned char* a_tile = tiles + (size_t)s * Cfg::stage_bytes;
        const uint64_t adesc = make_sw128_desc(a_tile);
        const uint64_t bdesc = make_sw128_desc(a_tile + Cfg::a_bytes);
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k)
          umma_bf16(tmem_base, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (uint32_t)((i | k) != 0));
        umma_commit(&ps->empty[s]);     // frees the stage once these MMAs have read it
      }
      if (ok) umma_commit(&ps->acc_full);
    }
  } else {
    // ------------------------------------------------------------------ weight expansion (FP4) + epilogue
    // Expansion work split: the k blocks (pipeline stages) are dealt round-robin to kSplit classes of warps; a warp
    // expands kRB 16-row blocks (all four k16 steps each) of every k block of its class.  Fewer, fatter trips per warp:
    // a trip is a serial (barrier wait -> expand -> store -> fence -> arrive) round trip whose latency, not the
    // instruction count, bounds the kernel, and the independent chains inside a trip overlap.
    constexpr int kSplit = kExpandSplit;      // 2; (4 classes x 2 row blocks measured slower: with 4 stages a class is then tied to one buffer)
    constexpr int kRB = kSplit * 8 / kExpandWarps;        // row blocks per warp (8 per 128-row tile)
    const int kh = (warp - 2) % kSplit;                   // stage class of this warp
    const int dw0 = ((warp - 2) / kSplit) * kRB;          // first 16-row block of this warp
    bool ok = true;
    if (WFMT == 0) {
      const int g = lane >> 2, t = lane & 3;
      const int KC = K >> 6;
      const int NG = K >> p.gs_shift;
      const int n_rt = (N + 15) >> 4;
      const uint4* qw = reinterpret_cast<const uint4*>(p.qw) + (long long)expert * p.expert_stride_q;
      const uint32_t* sc = reinterpret_cast<const uint32_t*>(p.sc) + (long long)expert * p.expert_stride_s;
      const bool big_groups = p.gs_shift >= 6;
      // per row block: weight words (one 16-byte word per lane and k block; the next two k blocks of the class are kept
      // in flight - the loads do not depend on the pipeline barriers), scale words of this lane's row pair, store row
      bool rt_ok[kRB];
      const uint4* wsrc[kRB];
      const uint32_t* sc_row[kRB];
      int st_row[kRB];
      uint4 w0[kRB], w1[kRB];
      uint32_t s0[kRB], s1[kRB];       // groups of 64 and more: the scale words of the next two k blocks of the class, fetched with the weights
#pragma unroll
      for (int j = 0; j < kRB; ++j) {
        // act == 1 (fused SwiGLU): the CTA's 128 lanes are 64 gate rows (blocks 0..3) and the 64 up rows of the same
        // output features (blocks 4..7), so both halves of a product meet in one accumulator tile
        const int blk = dw0 + j;
        const int rt = p.act ? (((blk & 4) ? (n_rt >> 1) : 0) + (int)blockIdx.x * 4 + (blk & 3)) : ((n0 >> 4) + blk);
        rt_ok[j] = p.act ? ((int)blockIdx.x * 4 + (blk & 3) < (n_rt >> 1)) : (rt < n_rt);
        wsrc[j] = qw + ((long long)rt * KC) * 32 + lane;
        sc_row[j] = sc + (long long)rt * NG * 8 + g;
        st_row[j] = ((dw0 + j) * 16 + g) * 128;
        w0[j] = (rt_ok[j] && kh < KB) ? ldg_stream(wsrc[j] + (long long)kh * 32) : make_uint4(0, 0, 0, 0);
        w1[j] = (rt_ok[j] && kh + kSplit < KB) ? ldg_stream(wsrc[j] + (long long)(kh + kSplit) * 32) : make_uint4(0, 0, 0, 0);
        s0[j] = (big_groups && rt_ok[j] && kh < KB) ? __ldg(sc_row[j] + (long long)((kh * kBK) >> p.gs_shift) * 8) : 0u;
        s1[j] = (big_groups && rt_ok[j] && kh + kSplit < KB) ? __ldg(sc_row[j] + (long long)(((kh + kSplit) * kBK) >> p.gs_shift) * 8) : 0u;
      }
      // store offsets inside a row of the A tile (128-byte swizzle: 16-byte chunk index XOR (row % 8); row % 8 == g)
      int st_col[4][2];
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        st_col[ks][0] = ((ks * 2) ^ g) * 16 + 4 * t;
        st_col[ks][1] = ((ks * 2 + 1) ^ g) * 16 + 4 * t;
      }
      for (int i = kh; i < KB; i += kSplit) {
        const int s = i % Cfg::kStages;
        const uint32_t ph = (uint32_t)(i / Cfg::kStages) & 1u;
        uint4 wcur[kRB];
        uint32_t scur[kRB];
#pragma unroll
        for (int j = 0; j < kRB; ++j) {
          wcur[j] = w0[j];
          w0[j] = w1[j];
          w1[j] = (rt_ok[j] && i + 2 * kSplit < KB) ? ldg_stream(wsrc[j] + (long long)(i + 2 * kSplit) * 32) : make_uint4(0, 0, 0, 0);
          scur[j] = s0[j];
          s0[j] = s1[j];
          s1[j] = (big_groups && rt_ok[j] && i + 2 * kSplit < KB) ? __ldg(sc_row[j] + (long long)(((i + 2 * kSplit) * kBK) >> p.gs_shift) * 8) : 0u;
        }
        if (!mbar_wait(&ps->empty[s], ph ^ 1u, abort_flag)) {
          if (atomicExch(&ps->abort_flag, 1) == 0 && status) atomicExch(status, 3);
          ok = false;
          break;
        }
        unsigned char* a_tile = tiles + (size_t)s * Cfg::stage_bytes;
#pragma unroll
        for (int j = 0; j < kRB; ++j) {
          const uint32_t qq[4] = {wcur[j].x, wcur[j].y, wcur[j].z, wcur[j].w};
          unsigned char* r0 = a_tile + st_row[j];         // rows g and g + 8 of the 16-row block
          unsigned char* r1 = r0 + 8 * 128;
          // groups of 64 and more: the four k16 steps of a k block share its group, so the scale word is fetched and
          // turned into the bf16 multipliers once per block
          bf162 m_lo, m_hi;
          bool fold = true;
          if (big_groups) {
            const uint32_t sw = scur[j];
            const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&sw));
            // fold the 2^126 subnormal rescale into the scale when it cannot overflow bf16
            fold = (fabsf(sf.x) < 2.f) && (fabsf(sf.y) < 2.f);
            m_lo = __float2bfloat162_rn(fold ? sf.x * 8.507059173023462e37f : sf.x);   // 2^126
            m_hi = __float2bfloat162_rn(fold ? sf.y * 8.507059173023462e37f : sf.y);
          }
#pragma unroll
          for (int kq = 0; kq < 4; ++kq) {
            if (!big_groups) {
              const int kabs = i * kBK + kq * 16;
              const uint32_t sw = rt_ok[j] ? __ldg(sc_row[j] + (long long)(kabs >> p.gs_shift) * 8) : 0u;
              const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&sw));
              fold = (fabsf(sf.x) < 2.f) && (fabsf(sf.y) < 2.f);
              m_lo = __float2bfloat162_rn(fold ? sf.x * 8.507059173023462e37f : sf.x);
              m_hi = __float2bfloat162_rn(fold ? sf.y * 8.507059173023462e37f : sf.y);
            }
            uint32_t a0, a1, a2, a3;
            e2m1x8_to_bf16x2_raw(qq[kq], a0, a1, a2, a3);
            if (!fold) {
              const bf162 big = __float2bfloat162_rn(8.507059173023462e37f);
              *reinterpret_cast<bf162*>(&a0) = __hmul2(*reinterpret_cast<bf162*>(&a0), big);
              *reinterpret_cast<bf162*>(&a1) = __hmul2(*reinterpret_cast<bf162*>(&a1), big);
              *reinterpret_cast<bf162*>(&a2) = __hmul2(*reinterpret_cast<bf162*>(&a2), big);
              *reinterpret_cast<bf162*>(&a3) = __hmul2(*reinterpret_cast<bf162*>(&a3), big);
            }
            // fragment registers: a0 = (row g, k 2t..), a1 = (row g+8, same k), a2 = (row g, k+8), a3 = (row g+8, k+8)
            *reinterpret_cast<bf162*>(&a0) = __hmul2(*reinterpret_cast<bf162*>(&a0), m_lo);
            *reinterpret_cast<bf162*>(&a1) = __hmul2(*reinterpret_cast<bf162*>(&a1), m_hi);
            *reinterpret_cast<bf162*>(&a2) = __hmul2(*reinterpret_cast<bf162*>(&a2), m_lo);
            *reinterpret_cast<bf162*>(&a3) = __hmul2(*reinterpret_cast<bf162*>(&a3), m_hi);
            *reinterpret_cast<uint32_t*>(r0 + st_col[kq][0]) = a0;
            *reinterpret_cast<uint32_t*>(r1 + st_col[kq][0]) = a1;
            *reinterpret_cast<uint32_t*>(r0 + st_col[kq][1]) = a2;
            *reinterpret_cast<uint32_t*>(r1 + st_col[kq][1]) = a3;
          }
        }
        fence_proxy_async_smem();       // generic-proxy stores -> visible to the tensor core (async proxy)
        __syncwarp();
        if (lane == 0) mbar_arrive(&ps->full_a[s]);
      }
    } else if (WFMT == 2) {
      // Trellis weights decoded in the main loop.  A 16 x 16 tile is 32 * bits bytes, LSB-first; lane l owns the 8 codes of
      // output row l / 2, input columns (l % 2) * 8 .. + 7, i.e. bytes [l * bits, (l + 1) * bits) of the tile - and those 8
      // values are exactly one 16-byte chunk of the swizzled K-major A row, so every lane makes one shared-memory store per
      // tile.  The four tiles of a k block are contiguous in memory; a lane fetches its bytes with aligned 32-bit loads
      // (neighbouring lanes read neighbouring words) and funnels them into place.  w = (code - (2^bits - 1) / 2) * sv[o] *
      // grid * scale[group, o] * su[i], rounded to bf16 once: the same value the stand-alone de-quantization kernel writes.
      constexpr float kGrid = 1.24371088f;
      const long long* desc0 = p.tr_desc + (long long)expert * p.tr_stride * 6;
      const uint8_t* codes[kRB];
      const float* scl[kRB];
      const float* su[kRB];
      float rowf[kRB], halfc[kRB];
      int bits[kRB], gsz[kRB], outf[kRB], tin[kRB], orow[kRB], st_off[kRB];
      bool rt_ok[kRB];
#pragma unroll
      for (int j = 0; j < kRB; ++j) {
        const int blk = dw0 + j;
        const int mat = p.tr_first + ((p.act && (blk & 4)) ? 1 : 0);
        const long long* d = desc0 + mat * 6;
        const int rt = p.act ? ((int)blockIdx.x * 4 + (blk & 3)) : ((n0 >> 4) + blk);
        codes[j] = reinterpret_cast<const uint8_t*>(d[0]);
        scl[j] = reinterpret_cast<const float*>(d[1]);
        su[j] = reinterpret_cast<const float*>(d[2]);
        const float* sv = reinterpret_cast<const float*>(d[3]);
        outf[j] = (int)(d[4] & 0xffffffffll);
        const int in_f = (int)(d[4] >> 32);
        bits[j] = (int)(d[5] & 0xffffffffll);
        gsz[j] = (int)(d[5] >> 32);
        tin[j] = (in_f + 15) >> 4;
        orow[j] = rt * 16 + (lane >> 1);
        rt_ok[j] = orow[j] < outf[j];
        rowf[j] = rt_ok[j] ? __ldg(sv + orow[j]) * kGrid : 0.f;
        halfc[j] = (float)((1 << bits[j]) - 1) * 0.5f;
        codes[j] += (long long)rt * tin[j] * (32 * bits[j]);          // first tile of this row block
        const int r = blk * 16 + (lane >> 1);                          // row inside the 128-row A tile
        st_off[j] = r * 128;
      }
      for (int i = kh; i < KB; i += kSplit) {
        const int s = i % Cfg::kStages;
        const uint32_t ph = (uint32_t)(i / Cfg::kStages) & 1u;
        // fetch this k block's bytes before waiting for the stage (the loads do not depend on the pipeline)
        unsigned long long cw[kRB][4];
        float sc[kRB][4];
#pragma unroll
        for (int j = 0; j < kRB; ++j) {
#pragma unroll
          for (int tt = 0; tt < 4; ++tt) {
            const int ti = i * 4 + tt;
            cw[j][tt] = 0ull;
            sc[j][tt] = 0.f;
            if (rt_ok[j] && ti < tin[j]) {
              const uint8_t* tile = codes[j] + (long long)ti * (32 * bits[j]);
              const int o = lane * bits[j], lo = o & 3;
              const uint32_t* w = reinterpret_cast<const uint32_t*>(tile + (o - lo));
              const int need = lo + bits[j];                            // bytes from the first aligned word on
              const uint32_t w0 = __ldg(w), w1 = need > 4 ? __ldg(w + 1) : 0u, w2 = need > 8 ? __ldg(w + 2) : 0u;
              unsigned long long v = ((unsigned long long)w1 << 32) | w0;
              v >>= 8 * lo;
              if (lo && need > 8) v |= (unsigned long long)w2 << (64 - 8 * lo);
              cw[j][tt] = v;
              sc[j][tt] = __ldg(scl[j] + (long long)((ti * 16) / gsz[j]) * outf[j] + orow[j]) * rowf[j];
            }
          }
        }
        if (!mbar_wait(&ps->empty[s], ph ^ 1u, abort_flag)) {
          if (atomicExch(&ps->abort_flag, 1) == 0 && status) atomicExch(status, 3);
          ok = false;
          break;
        }
        unsigned char* a_tile = tiles + (size_t)s * Cfg::stage_bytes;
#pragma unroll
        for (int j = 0; j < kRB; ++j) {
          const unsigned mask = (1u << bits[j]) - 1u;
          const int r7 = (lane >> 1) & 7;
#pragma unroll
          for (int tt = 0; tt < 4; ++tt) {
            const int col0 = (i * 4 + tt) * 16 + (lane & 1) * 8;
            uint32_t o4[4] = {0u, 0u, 0u, 0u};
            if (rt_ok[j] && (i * 4 + tt) < tin[j]) {
              const float4 s0 = __ldg(reinterpret_cast<const float4*>(su[j] + col0));
              const float4 s1 = __ldg(reinterpret_cast<const float4*>(su[j] + col0 + 4));
              const float sf[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
              const unsigned long long v = cw[j][tt];
              float wv[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) wv[e] = ((float)((unsigned)(v >> (e * bits[j])) & mask) - halfc[j]) * sc[j][tt] * sf[e];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const bf162 pr = __floats2bfloat162_rn(wv[2 * e], wv[2 * e + 1]);
                o4[e] = *reinterpret_cast<const uint32_t*>(&pr);
              }
            }
            const int chunk = tt * 2 + (lane & 1);
            *reinterpret_cast<uint4*>(a_tile + st_off[j] + ((chunk ^ r7) * 16)) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ps->full_a[s]);
      }
    } else if (WFMT == 3) {
      // Codebook weights decoded in the main loop.  Lane l owns output row l / 2 of a 16-row block and the 32 input columns
      // (l % 2) * 32 .. + 31 of the k block: 4 * bits contiguous bytes of the row-major code matrix (one or two vector loads,
      // requested before the stage wait) that become four 16-byte chunks of the swizzled K-major A row.
      for (int i2 = tid - 64; i2 < 256; i2 += kExpandWarps * 32) lut_s[i2] = __ldg(p.cb_lut + i2);
      asm volatile("bar.sync 6, %0;" ::"n"(kExpandWarps * 32) : "memory");
      const int bits = p.cb_bits;
      const int NG = K >> p.gs_shift;
      const long long row_bytes = (long long)K * bits / 8;
      const uint8_t* cbase = reinterpret_cast<const uint8_t*>(p.qw);
      const __half* sc_h = reinterpret_cast<const __half*>(p.sc);
      const __half* zp_h = reinterpret_cast<const __half*>(p.cb_zeros);
      const int half_k = (lane & 1) * 32;
      int orow[kRB], st_off[kRB];
      bool rt_ok[kRB];
#pragma unroll
      for (int j = 0; j < kRB; ++j) {
        const int blk = dw0 + j;
        orow[j] = n0 + blk * 16 + (lane >> 1);
        rt_ok[j] = orow[j] < N;
        st_off[j] = (blk * 16 + (lane >> 1)) * 128;
      }
      for (int i = kh; i < KB; i += kSplit) {
        const int s = i % Cfg::kStages;
        const uint32_t ph = (uint32_t)(i / Cfg::kStages) & 1u;
        uint4 cw[kRB][2];
        float scl[kRB], zpt[kRB];
#pragma unroll
        for (int j = 0; j < kRB; ++j) {
          cw[j][0] = cw[j][1] = make_uint4(0, 0, 0, 0);
          scl[j] = zpt[j] = 0.f;
          if (rt_ok[j]) {
            const int k0 = i * kBK + half_k;
            const uint8_t* src = cbase + (long long)orow[j] * row_bytes + (long long)k0 * bits / 8;
            if (bits == 8) {
              cw[j][0] = ldg_stream(reinterpret_cast<const uint4*>(src));
              cw[j][1] = ldg_stream(reinterpret_cast<const uint4*>(src) + 1);
            } else if (bits == 4) {
              cw[j][0] = ldg_stream(reinterpret_cast<const uint4*>(src));
            } else {
              const uint2 v2 = __ldg(reinterpret_cast<const uint2*>(src));
              cw[j][0] = make_uint4(v2.x, v2.y, 0, 0);
            }
            const long long gi = (long long)orow[j] * NG + (k0 >> p.gs_shift);
            scl[j] = __half2float(sc_h[gi]);
            zpt[j] = zp_h ? __half2float(zp_h[gi]) : 0.f;
          }
        }
        if (!mbar_wait(&ps->empty[s], ph ^ 1u, abort_flag)) {
          if (atomicExch(&ps->abort_flag, 1) == 0 && status) atomicExch(status, 3);
          ok = false;
          break;
        }
        unsigned char* a_tile = tiles + (size_t)s * Cfg::stage_bytes;
        const int r7 = (lane >> 1) & 7;
#pragma unroll
        for (int j = 0; j < kRB; ++j) {
          const uint32_t words[8] = {cw[j][0].x, cw[j][0].y, cw[j][0].z, cw[j][0].w, cw[j][1].x, cw[j][1].y, cw[j][1].z, cw[j][1].w};
          unsigned char* dst = a_tile + st_off[j];
          if (bits == 4) cb_expand_row<4>(words, lut_s, zpt[j], scl[j], dst, lane & 1, r7);
          else if (bits == 8) cb_expand_row<8>(words, lut_s, zpt[j], scl[j], dst, lane & 1, r7);
          else cb_expand_row<2>(words, lut_s, zpt[j], scl[j], dst, lane & 1, r7);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ps->full_a[s]);
      }
    } else if (WFMT == 4) {
      // 2:4 sparse FP4.  Lane l owns output row l / 2 of a 16-row block and the 32 dense columns (l % 2) * 32 .. + 31 of the
      // k block: 8 groups of four = 8 bytes of kept codes + 4 bytes of positions (both requested before the stage wait),
      // scattered into four 16-byte chunks of the swizzled K-major A row.
      if (tid - 64 < 16) {
        const int c = tid - 64, m = c & 7, e = m >> 1, f = m & 1;
        const float mag = e == 0 ? 0.5f * (float)f : (1.f + 0.5f * (float)f) * (float)(1 << (e - 1));
        lut_s[c] = (c & 8) ? -mag : mag;
      }
      asm volatile("bar.sync 6, %0;" ::"n"(kExpandWarps * 32) : "memory");
      const int NG = K >> p.gs_shift;
      const uint8_t* cbase = reinterpret_cast<const uint8_t*>(p.qw);
      const uint8_t* mbase = reinterpret_cast<const uint8_t*>(p.sp_meta);
      const __half* sc_h = reinterpret_cast<const __half*>(p.sc);
      const int half_k = (lane & 1) * 32;
      int orow[kRB], st_off[kRB];
      bool rt_ok[kRB];
#pragma unroll
      for (int j = 0; j < kRB; ++j) {
        const int blk = dw0 + j;
        orow[j] = n0 + blk * 16 + (lane >> 1);
        rt_ok[j] = orow[j] < N;
        st_off[j] = (blk * 16 + (lane >> 1)) * 128;
      }
      for (int i = kh; i < KB; i += kSplit) {
        const int s = i % Cfg::kStages;
        const uint32_t ph = (uint32_t)(i / Cfg::kStages) & 1u;
        uint2 cw[kRB];
        uint32_t mw[kRB];
        float scl[kRB];
#pragma unroll
        for (int j = 0; j < kRB; ++j) {
          cw[j] = make_uint2(0, 0);
          mw[j] = 0u;
          scl[j] = 0.f;
          if (rt_ok[j]) {
            const int k0 = i * kBK + half_k;
            cw[j] = __ldg(reinterpret_cast<const uint2*>(cbase + (long long)orow[j] * (K >> 2) + (k0 >> 2)));
            mw[j] = __ldg(reinterpret_cast<const uint32_t*>(mbase + (long long)orow[j] * (K >> 3) + (k0 >> 3)));
            scl[j] = __half2float(sc_h[(long long)orow[j] * NG + (k0 >> p.gs_shift)]);
          }
        }
        if (!mbar_wait(&ps->empty[s], ph ^ 1u, abort_flag)) {
          if (atomicExch(&ps->abort_flag, 1) == 0 && status) atomicExch(status, 3);
          ok = false;
          break;
        }
        unsigned char* a_tile = tiles + (size_t)s * Cfg::stage_bytes;
        const int r7 = (lane >> 1) & 7;
#pragma unroll
        for (int j = 0; j < kRB; ++j) {
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {                     // chunk cc = groups 2 cc and 2 cc + 1
            uint32_t o4[4];
#pragma unroll
            for (int g2 = 0; g2 < 2; ++g2) {
              const int g = cc * 2 + g2;
              const uint32_t word = g < 4 ? cw[j].x : cw[j].y;
              const uint32_t pair = (word >> ((g & 3) * 8)) & 0xffu;
              const uint32_t m4 = (mw[j] >> (g * 4)) & 0xfu;
              const int i0 = (int)(m4 & 3u), i1 = (int)(m4 >> 2);
              const float a = lut_s[pair & 0xfu] * scl[j], b = lut_s[pair >> 4] * scl[j];
              float v[4];
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) v[q4] = (q4 == i0 ? a : 0.f) + (q4 == i1 ? b : 0.f);
              const bf162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
              o4[g2 * 2] = *reinterpret_cast<const uint32_t*>(&p0);
              o4[g2 * 2 + 1] = *reinterpret_cast<const uint32_t*>(&p1);
            }
            const int chunk = (lane & 1) * 4 + cc;
            *reinterpret_cast<uint4*>(a_tile + st_off[j] + ((chunk ^ r7) * 16)) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ps->full_a[s]);
      }
    }
    // ---- epilogue: TMEM -> registers -> global
    if (ok) ok = mbar_wait(&ps->acc_full, 0u, abort_flag);
    if (!ok) {
      if (atomicExch(&ps->abort_flag, 1) == 0 && status) atomicExch(status, 4);
    } else {
      tc_fence_after();
      const int q = warp & 3;                    // TMEM lane quarter this warp may access
      const int n = n0 + q * 32 + lane;
      const int ldo = QW ? p.ldo : pb.ldo;
      const int c_first = ((warp - 2) >> 2) * 32; // the warps of a quarter take the 32-column chunks round-robin
      if (QW && p.act) {
        // fused SwiGLU: lanes 0..63 hold gate rows, lanes 64..127 the matching up rows.  The four warps that share a
        // 32-column chunk (one per lane quarter) pair up through shared memory: the up quarters park their values in a
        // column-major slab of the (now idle) pipeline stages, the gate quarters read them back and store silu(g) * u.
        // Two slabs per chunk group alternate, so one named barrier per chunk orders both directions.
        const int grp = (warp - 2) >> 2;                                   // chunk group 0..3
        float* slab = reinterpret_cast<float*>(tiles) + grp * (2 * 64 * 32);
        const int half_n = N >> 1;
        const int no = (int)blockIdx.x * 64 + (q & 1) * 32 + lane;        // output feature of this lane (gate quarters)
        int it = 0;
#pragma unroll 1
        for (int c0 = c_first; c0 < TN; c0 += (kExpandWarps / 4) * 32, ++it) {
          uint32_t v[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
          tmem_ld_wait();
          float* sl = slab + (it & 1) * (64 * 32);
          if (q >= 2) {
#pragma unroll
            for (int j = 0; j < 32; ++j) sl[j * 64 + (q & 1) * 32 + lane] = __uint_as_float(v[j]);
          }
          asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
          if (q < 2 && no < half_n) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int r = c0 + j;
              if (r < tok_rows && tok0 + r < M) {
                const float gv = __uint_as_float(v[j]), uv = sl[j * 64 + (q & 1) * 32 + lane];
                float f = gv / (1.f + __expf(-gv)) * uv;
                if (p.row_scale) f *= p.row_scale[tok0 + r];
                reinterpret_cast<bf16*>(p.out)[(long long)(tok0 + r) * ldo + no] = __float2bfloat16(f);
              }
            }
          }
        }
      } else {
#pragma unroll 1
      for (int c0 = c_first; c0 < TN; c0 += (kExpandWarps / 4) * 32) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
        tmem_ld_wait();
        if (n < N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int r = c0 + j;
            if (r < tok_rows && tok0 + r < M) {
              float f = __uint_as_float(v[j]);
              if (QW && p.rs_peer_bufs != nullptr) {
                // reduce-scatter epilogue: the partial goes to the rank that owns this token row
                const int row = tok0 + r, owner = row / p.rs_rows;
                p.rs_peer_bufs[owner][((long long)p.rs_rank * p.rs_rows + (row - owner * p.rs_rows)) * N + n] = f;
              } else if (QW && p.out_rows != nullptr) {
                // scatter epilogue: the row's destination (possibly in a peer's memory) comes from a device table
                bf16* dst = reinterpret_cast<bf16*>(p.out_rows[tok0 + r]);
                if (dst != nullptr) dst[n] = __float2bfloat16(f);
              } else if (QW) {
                if (p.row_scale) f *= p.row_scale[tok0 + r];
                reinterpret_cast<bf16*>(p.out)[(long long)(tok0 + r) * ldo + n] = __float2bfloat16(f);
              } else {
                const long long o = (long long)batch * pb.out_batch_stride + (long long)(tok0 + r) * ldo + n;
                if (pb.out_f32) reinterpret_cast<float*>(pb.out)[o] = f;
                else reinterpret_cast<bf16*>(pb.out)[o] = __float2bfloat16(f);
              }
            }
          }
        }
      }
      }
      if (QW && p.out_rows != nullptr) __threadfence_system();     // peer stores ordered before the grid completes
    }
  }
  if (QW && p.rs_peer_bufs != nullptr) {
    // all threads: make the peer stores visible system wide, then the last CTA of the grid raises the flags
    TpOut tout;
    tout.peer_slots = nullptr;
    tout.peer_flags = p.rs_peer_flags;
    tout.counter = p.rs_counter;
    tout.step = p.rs_step;
    tout.tp = p.rs_tp;
    tp_signal(tout, gridDim.x * gridDim.y * gridDim.z);
  }
  // ---- teardown: if something timed out give in-flight bulk copies time to land, then free TMEM
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::tmem_cols);
  }
}

// ------------------------------------------------------------------------------------------ host
// bf16 [batch, rows, cols] with row stride ld (elements); box = {64, box_rows, 1}, 128-byte swizzle, zero fill.
static int make_tmap(CUtensorMap* map, const void* base, long long cols, long long rows, long long batch, long long ld,
                     long long batch_stride, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16 != 0) return (int)cudaErrorInvalidValue;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)(batch > 0 ? batch : 1)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(batch_stride > 0 ? batch_stride : rows * ld) * 2};
  if (strides[1] % 16 != 0) return (int)cudaErrorInvalidValue;
  cuuint32_t box[3] = {(cuuint32_t)kBK, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}
static int make_tmap_2d(CUtensorMap* map, const void* base, long long cols, long long rows, long long ld, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16 != 0) return (int)cudaErrorInvalidValue;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int TN, int WFMT, int MINB>
static int launch_gemm_b(const CUtensorMap& mx, const CUtensorMap& mw, const MmbFp4GemmParams& p, const MmbBf16GemmParams& pb,
                         dim3 grid, cudaStream_t stream) {
  auto kern = gemm_kernel<TN, WFMT, MINB>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GemmCfg<TN, MINB>::smem_bytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  kern<<<grid, kGemmThreads, GemmCfg<TN, MINB>::smem_bytes, stream>>>(mx, mw, p, pb);
  return (int)cudaGetLastError();
}

// CTAs per SM of the weight-expanding variants: 2 unless MMB200_GEMM_CTAS=1 (the bf16 x bf16 variant is fed by TMA alone
// and keeps the deep single-CTA pipeline).
static int gemm_ctas_per_sm() {
  static int v = 0;
  if (v == 0) {
    const char* e = getenv("MMB200_GEMM_CTAS");
    v = (e != nullptr && e[0] == '1') ? 1 : 2;
  }
  return v;
}

template <int TN, int WFMT>
static int launch_gemm(const CUtensorMap& mx, const CUtensorMap& mw, const MmbFp4GemmParams& p, const MmbBf16GemmParams& pb,
                       dim3 grid, cudaStream_t stream) {
  if constexpr (WFMT != 1) {
    if (gemm_ctas_per_sm() == 2) return launch_gemm_b<TN, WFMT, 2>(mx, mw, p, pb, grid, stream);
  }
  return launch_gemm_b<TN, WFMT, 1>(mx, mw, p, pb, grid, stream);
}

static int pick_tn(int M, int forced) {
  if (forced == 32 || forced == 64 || forced == 128 || forced == 256) return forced;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 1024) return 128;
  return 256;
}

}  // namespace mmb

MMB_API int mmb_fp4_gemm(const MmbFp4GemmParams* pp, cudaStream_t stream) {
  using namespace mmb;
  MmbFp4GemmParams p = *pp;
  if (p.M <= 0 || p.N <= 0) return 0;
  if (p.K % 64 != 0 || p.Kx % 8 != 0 || p.Kx > p.K || (p.act != 0 && p.act != 1)) return (int)cudaErrorInvalidValue;
  // fused SwiGLU: N counts gate + up rows; every CTA takes 64 output features (needs N / 2 to be a multiple of 64)
  if (p.act == 1 && ((p.N & 127) != 0 || p.rs_peer_bufs != nullptr || p.out_rows != nullptr)) return (int)cudaErrorInvalidValue;
  const bool grouped = p.tile_expert != nullptr;
  if (p.ag.flags != nullptr && (grouped || p.ag.step == nullptr || p.ag.rows <= 0 || p.ag.tp < 1)) return (int)cudaErrorInvalidValue;
  const int TN = pick_tn(grouped ? (p.token_tile ? p.token_tile : 128) : p.M, p.token_tile);
  CUtensorMap mx;
  int e = make_tmap_2d(&mx, p.x, p.Kx, p.M, p.Kx, TN);
  if (e) return e;
  MmbBf16GemmParams pb{};
  dim3 grid((p.N + kTileRows - 1) / kTileRows, grouped ? p.max_tiles : (p.M + TN - 1) / TN, 1);     // act == 1: N / 128 CTAs of 64 + 64 rows
  switch (TN) {
    case 32: return launch_gemm<32, 0>(mx, mx, p, pb, grid, stream);
    case 64: return launch_gemm<64, 0>(mx, mx, p, pb, grid, stream);
    case 128: return launch_gemm<128, 0>(mx, mx, p, pb, grid, stream);
    default: return launch_gemm<256, 0>(mx, mx, p, pb, grid, stream);
  }
}

// Trellis weights (WFMT 2): `tr_desc` is a device table of MmbTrellisMat rows (6 x int64 each: codes, scales, su, sv,
// out | in << 32, bits | group << 32); matrix index = expert * tr_stride + tr_first (+ 1 for the up half with act = 1).
MMB_API int mmb_trellis_gemm(const MmbFp4GemmParams* pp, cudaStream_t stream) {
  using namespace mmb;
  MmbFp4GemmParams p = *pp;
  if (p.M <= 0 || p.N <= 0) return 0;
  if (p.tr_desc == nullptr || p.K % 64 != 0 || p.Kx % 8 != 0 || p.Kx > p.K || (p.act != 0 && p.act != 1)) return (int)cudaErrorInvalidValue;
  if (p.act == 1 && ((p.N & 127) != 0 || p.out_rows != nullptr)) return (int)cudaErrorInvalidValue;
  if (p.rs_peer_bufs != nullptr || p.ag.flags != nullptr) return (int)cudaErrorInvalidValue;
  const bool grouped = p.tile_expert != nullptr;
  const int TN = pick_tn(grouped ? (p.token_tile ? p.token_tile : 128) : p.M, p.token_tile);
  CUtensorMap mx;
  int e = make_tmap_2d(&mx, p.x, p.Kx, p.M, p.Kx, TN);
  if (e) return e;
  MmbBf16GemmParams pb{};
  dim3 grid((p.N + kTileRows - 1) / kTileRows, grouped ? p.max_tiles : (p.M + TN - 1) / TN, 1);
  switch (TN) {
    case 32: return launch_gemm<32, 2>(mx, mx, p, pb, grid, stream);
    case 64: return launch_gemm<64, 2>(mx, mx, p, pb, grid, stream);
    case 128: return launch_gemm<128, 2>(mx, mx, p, pb, grid, stream);
    default: return launch_gemm<256, 2>(mx, mx, p, pb, grid, stream);
  }
}

// Codebook weights (WFMT 3): plain mode only (no grouping, activation or exchange epilogues).
MMB_API int mmb_codebook_gemm(const MmbFp4GemmParams* pp, cudaStream_t stream) {
  using namespace mmb;
  MmbFp4GemmParams p = *pp;
  if (p.M <= 0 || p.N <= 0) return 0;
  if (p.qw == nullptr || p.sc == nullptr || p.cb_lut == nullptr || (p.cb_bits != 2 && p.cb_bits != 4 && p.cb_bits != 8)) return (int)cudaErrorInvalidValue;
  if (p.K % 64 != 0 || p.Kx != p.K || p.gs_shift < 5 || (p.K & ((1 << p.gs_shift) - 1)) != 0) return (int)cudaErrorInvalidValue;
  if (p.act != 0 || p.tile_expert != nullptr || p.rs_peer_bufs != nullptr || p.ag.flags != nullptr || p.out_rows != nullptr) return (int)cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(p.qw) & 15) return (int)cudaErrorInvalidValue;
  const int TN = pick_tn(p.M, p.token_tile);
  CUtensorMap mx;
  int e = make_tmap_2d(&mx, p.x, p.Kx, p.M, p.Kx, TN);
  if (e) return e;
  MmbBf16GemmParams pb{};
  dim3 grid((p.N + kTileRows - 1) / kTileRows, (p.M + TN - 1) / TN, 1);
  switch (TN) {
    case 32: return launch_gemm<32, 3>(mx, mx, p, pb, grid, stream);
    case 64: return launch_gemm<64, 3>(mx, mx, p, pb, grid, stream);
    case 128: return launch_gemm<128, 3>(mx, mx, p, pb, grid, stream);
    default: return launch_gemm<256, 3>(mx, mx, p, pb, grid, stream);
  }
}

// 2:4 sparse FP4 weights (WFMT 4): plain mode only.
MMB_API int mmb_sparse24_gemm(const MmbFp4GemmParams* pp, cudaStream_t stream) {
  using namespace mmb;
  MmbFp4GemmParams p = *pp;
  if (p.M <= 0 || p.N <= 0) return 0;
  if (p.qw == nullptr || p.sc == nullptr || p.sp_meta == nullptr) return (int)cudaErrorInvalidValue;
  if (p.K % 64 != 0 || p.Kx != p.K || p.gs_shift < 5 || (p.K & ((1 << p.gs_shift) - 1)) != 0) return (int)cudaErrorInvalidValue;
  if (p.act != 0 || p.tile_expert != nullptr || p.rs_peer_bufs != nullptr || p.ag.flags != nullptr || p.out_rows != nullptr) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(p.qw) & 7) || (reinterpret_cast<uintptr_t>(p.sp_meta) & 3)) return (int)cudaErrorInvalidValue;
  const int TN = pick_tn(p.M, p.token_tile);
  CUtensorMap mx;
  int e = make_tmap_2d(&mx, p.x, p.Kx, p.M, p.Kx, TN);
  if (e) return e;
  MmbBf16GemmParams pb{};
  dim3 grid((p.N + kTileRows - 1) / kTileRows, (p.M + TN - 1) / TN, 1);
  switch (TN) {
    case 32: return launch_gemm<32, 4>(mx, mx, p, pb, grid, stream);
    case 64: return launch_gemm<64, 4>(mx, mx, p, pb, grid, stream);
    case 128: return launch_gemm<128, 4>(mx, mx, p, pb, grid, stream);
    default: return launch_gemm<256, 4>(mx, mx, p, pb, grid, stream);
  }
}

MMB_API int mmb_bf16_gemm(const MmbBf16GemmParams* pp, cudaStream_t stream) {
  using namespace mmb;
  MmbBf16GemmParams pb = *pp;
  if (pb.M <= 0 || pb.N <= 0) return 0;
  if (pb.K % 64 != 0 || pb.ldx % 8 != 0 || pb.ldw % 8 != 0) return (int)cudaErrorInvalidValue;
  const int nb = pb.batch > 0 ? pb.batch : 1;
  if (pb.ag.flags != nullptr && (nb != 1 || pb.ag.step == nullptr || pb.ag.rows <= 0 || pb.ag.tp < 1)) return (int)cudaErrorInvalidValue;
  const int TN = pick_tn(pb.M, 0);
  CUtensorMap mx, mw;
  int e = make_tmap(&mx, pb.x, pb.K, pb.M, pb.x_batch_stride ? nb : 1, pb.ldx, pb.x_batch_stride, TN);
  if (e) return e;
  e = make_tmap(&mw, pb.w, pb.K, pb.N, pb.w_batch_stride ? nb : 1, pb.ldw, pb.w_batch_stride, kTileRows);
  if (e) return e;
  MmbFp4GemmParams p{};
  dim3 grid((pb.N + kTileRows - 1) / kTileRows, (pb.M + TN - 1) / TN, nb);
  switch (TN) {
    case 32: return launch_gemm<32, 1>(mx, mw, p, pb, grid, stream);
    case 64: return launch_gemm<64, 1>(mx, mw, p, pb, grid, stream);
    case 128: return launch_gemm<128, 1>(mx, mw, p, pb, grid, stream);
    default: return launch_gemm<256, 1>(mx, mw, p, pb, grid, stream);
  }
}
