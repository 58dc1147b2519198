// Causal prefill attention (optionally with a sliding window) on the tcgen05 tensor cores.
//
// One CTA owns 128 query rows of one head and walks the keys in tiles of KT (64 at head size 256, 128 at head size 128):
//   warp 0      TMA producer: Q once, then per tile the K rows [KT keys x D] and the V^T block [D x KT keys] into a
//               two-stage ring (cp.async.bulk.tensor, 128-byte swizzle, completion on mbarriers);
//   warp 1      one elected thread issues the MMAs: S = Q K^T (M 128, N KT, K = D) into one of two S buffers in TMEM,
//               O += P V (M 128, N = D, K = KT) into the O accumulator in TMEM; tcgen05.commit signals the mbarriers.
//               S of tile j + 1 is issued before P V of tile j, so it runs under the soft-max of tile j;
//   warps 2-9   soft-max, two threads per query row (its TMEM lane; each takes half of the tile's keys and half of the O
//               columns, row maxima exchanged through shared memory): tcgen05.ld of the scores, scale, causal mask (diagonal
//               tiles only), running maximum with LAZY rescaling (the reference maximum only moves when a row's maximum
//               grew by more than 2^8, decided per warp; only then does the warp wait for the previous P V and rescale
//               its O rows in TMEM with tcgen05.ld / tcgen05.st), exp2, P rounded to bf16 and stored as the K-major
//               swizzled A operand of the P V MMA (two P buffers); finally O / l -> global.
// TMEM: O in columns [0, D), S buffers at D and D + 128.
// Shared memory: Q 64 KB + 2 x (K 32 KB + V^T 32 KB + P 16 KB) at D = 256; 32 + 2 x (32 + 32 + 32) KB at D = 128.
// Every mbarrier wait is bounded; on expiry a code goes to the status word, the roles stop, TMEM is freed.
#include "api_ext.h"
#include "common.cuh"
#include "tcgen05.cuh"

namespace mmb {

constexpr int kFmThreads = 320;         // warp 0 TMA, warp 1 MMA, warps 2-9 soft-max (two per TMEM lane quarter)
constexpr float kFmLazyLog2 = 8.f;      // rescale O only when a row maximum grew by more than this (log2 units)

struct FmhaShared {
  uint64_t q_full, k_full[2], v_full[2], s_full[2], p_full[2], pv_done[2];
  uint64_t pair_bar[4];       // the two soft-max warps of a lane quarter meet here (64 arrivals), bounded like every wait
  uint32_t tmem_base;
  int abort_flag;
  float xmax[2][2][128];      // [tile parity][column half][row]: row maxima exchanged between the two warps of a row (the row
                              // sums take the idle parity once at the end)
};

// D: head size; KT: keys per tile (64 at D = 256, 128 at D = 128, so that K, V^T and P all fit twice).
template <int D, int KT>
struct FmhaCfg {
  static constexpr int KB = D / 64;                 // 64-wide k blocks of the head dimension (S = Q K^T)
  static constexpr int NKB = KT / 64;               // 64-key k blocks of a tile (O += P V)
  static constexpr int q_bytes = KB * 16384;
  static constexpr int k_blk = KT * 128;            // one k block of the K tile: KT rows x 128 B
  static constexpr int k_bytes = KB * k_blk;
  static constexpr int v_blk = D * 128;             // one 64-key block of V^T: D rows x 128 B
  static constexpr int v_bytes = NKB * v_blk;
  static constexpr int p_bytes = NKB * 16384;
  static constexpr size_t smem_bytes = (size_t)q_bytes + 2 * (k_bytes + v_bytes + p_bytes) + sizeof(FmhaShared);
  static_assert(smem_bytes <= 232448, "shared memory of one CTA");
};

// kind::f16 instruction descriptor: D = f32, A = B = bf16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t fm_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ float fm_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t fm_pack(float a, float b) {
  const bf162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <int D, int KT>
__global__ void __launch_bounds__(kFmThreads, 1)
fmha_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const MmbFmhaPrefillParams p) {
  using Cfg = FmhaCfg<D, KT>;
  extern __shared__ __align__(1024) unsigned char smem_fm[];      // the swizzled tiles need 1024-byte alignment
  unsigned char* Qs = smem_fm;
  unsigned char* Ks = Qs + Cfg::q_bytes;            // [2][k_bytes]
  unsigned char* Vs = Ks + 2 * Cfg::k_bytes;        // [2][v_bytes]
  unsigned char* Ps = Vs + 2 * Cfg::v_bytes;        // [2][p_bytes]
  FmhaShared* sh = reinterpret_cast<FmhaShared*>(Ps + 2 * Cfg::p_bytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qt = (int)gridDim.y - 1 - (int)blockIdx.y;       // all heads' tiles with the most keys start first
  const int q0 = qt * 128, h = blockIdx.x, hk = h / (p.Hq / p.Hk);
  const int q_off = p.n - p.t;
  // sliding window: a query at position x sees the keys (x - window, x]; tiles wholly in front of the first row's window
  // are never loaded, and tile numbers below count from the first visited tile j0
  const int win = p.window;
  const int j0 = win > 0 ? max(0, q_off + q0 - win + 1) / KT : 0;
  const int nt = (q_off + min(q0 + 127, p.t - 1)) / KT + 1 - j0;    // key tiles this query tile can see
  int* status = p.status;
  if ((smem_u32(smem_fm) & 1023u) != 0u) {      // no room for alignment slack: refuse rather than mis-address the tiles
    if (tid == 0 && status) atomicExch(status, 42);
    return;
  }

  if (tid == 0) {
    mbar_init(&sh->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh->k_full[i], 1);
      mbar_init(&sh->v_full[i], 1);
      mbar_init(&sh->s_full[i], 1);
      mbar_init(&sh->p_full[i], 8);
      mbar_init(&sh->pv_done[i], 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&sh->pair_bar[i], 64);
    sh->abort_flag = 0;
    fence_proxy_async_smem();
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_flag = &sh->abort_flag;
  auto fail = [&](int code) {
    if (atomicExch(&sh->abort_flag, 1) == 0 && status) atomicExch(status, code);
  };
  // tile j uses stage / buffer j & 1; its barriers are in phase (j >> 1) & 1
  auto ph = [](int j) { return (uint32_t)(j >> 1) & 1u; };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(&sh->q_full, Cfg::q_bytes);
      for (int kb = 0; kb < Cfg::KB; ++kb) tma_load_3d(Qs + kb * 16384, &tm_q, &sh->q_full, kb * 64, h, q0);
      for (int j = 0; j < nt; ++j) {
        const int s = j & 1;
        if (j >= 2 && !mbar_wait(&sh->s_full[s], ph(j - 2), abort_flag)) {      // K stage read by S(j-2)
          fail(31);
          break;
        }
        mbar_expect_tx(&sh->k_full[s], Cfg::k_bytes);
        for (int kb = 0; kb < Cfg::KB; ++kb)
          tma_load_3d(Ks + s * Cfg::k_bytes + kb * Cfg::k_blk, &tm_k, &sh->k_full[s], kb * 64, hk, (j0 + j) * KT);
        if (j >= 2 && !mbar_wait(&sh->pv_done[s], ph(j - 2), abort_flag)) {     // V stage read by PV(j-2)
          fail(32);
          break;
        }
        mbar_expect_tx(&sh->v_full[s], Cfg::v_bytes);
        for (int kb = 0; kb < Cfg::NKB; ++kb)
          tma_load_3d(Vs + s * Cfg::v_bytes + kb * Cfg::v_blk, &tm_v, &sh->v_full[s], (j0 + j) * KT + kb * 64, 0, hk);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t id_s = fm_idesc(KT), id_o = fm_idesc(D);
      bool ok = mbar_wait(&sh->q_full, 0u, abort_flag);
      if (!ok) fail(33);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&sh->k_full[s], ph(j), abort_flag)) {
          fail(34);
          return false;
        }
        tc_fence_after();
        const uint32_t ts = tmem_base + (uint32_t)(D + s * 128);
#pragma unroll
        for (int kb = 0; kb < Cfg::KB; ++kb) {
          const uint64_t ad = make_sw128_desc(Qs + kb * 16384), bd = make_sw128_desc(Ks + s * Cfg::k_bytes + kb * Cfg::k_blk);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(ts, ad + (uint64_t)(k * 2), bd + (uint64_t)(k * 2), id_s, (uint32_t)((kb | k) != 0));
        }
        umma_commit(&sh->s_full[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < nt && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < nt) ok = issue_s(j + 1);       // runs under the soft-max of tile j
        if (!ok) break;
        if (!mbar_wait(&sh->p_full[s], ph(j), abort_flag) || !mbar_wait(&sh->v_full[s], ph(j), abort_flag)) {
          fail(35);
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < Cfg::NKB; ++kb) {
          const uint64_t ad = make_sw128_desc(Ps + s * Cfg::p_bytes + kb * 16384), bd = make_sw128_desc(Vs + s * Cfg::v_bytes + kb * Cfg::v_blk);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base, ad + (uint64_t)(k * 2), bd + (uint64_t)(k * 2), id_o, (uint32_t)((j | kb | k) != 0));
        }
        umma_commit(&sh->pv_done[s]);
      }
    }
  } else {
    // ------------------------------------------------------------------ soft-max: two threads (of two warps) per query row
    constexpr int HC = KT / 2;                        // score columns per thread
    constexpr int NC = HC / 32;                       // 32-column chunks per thread
    const int quarter = warp & 3;                     // TMEM lane quarter this warp may access
    const int half = (warp - 2) >> 2;                 // which half of the columns (and of the O columns) this warp owns
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float c = p.scale * 1.4426950408889634f;
    const int my_pos = q_off + q0 + row;
    uint32_t pair_phase = 0;
    auto pair_sync = [&]() -> bool {                  // rendezvous of the two warps that share these rows
      mbar_arrive(&sh->pair_bar[quarter]);
      const bool r = mbar_wait(&sh->pair_bar[quarter], pair_phase, abort_flag);
      pair_phase ^= 1u;
      return r;
    };
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nt; ++j) {
      const int s = j & 1;
      if (!mbar_wait(&sh->s_full[s], ph(j), abort_flag)) {
        fail(36);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t ts = tmem_base + lane_addr + (uint32_t)(D + s * 128 + half * HC);
      uint32_t v[NC][32];
#pragma unroll
      for (int cc = 0; cc < NC; ++cc) tmem_ld32(ts + (uint32_t)(cc * 32), v[cc]);
      tmem_ld_wait();
      const int key0 = (j0 + j) * KT;
      const bool need_mask = (key0 + KT - 1 > q_off + q0) || (key0 + KT > p.n) || (win > 0 && key0 <= q_off + q0 + 127 - win);
      float mt = -INFINITY;
#pragma unroll
      for (int cc = 0; cc < NC; ++cc)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = __uint_as_float(v[cc][i]) * c;
          if (need_mask) {
            const int key = key0 + half * HC + cc * 32 + i;
            if (key > my_pos || key >= p.n || (win > 0 && key <= my_pos - win)) x = -INFINITY;
          }
          v[cc][i] = __float_as_uint(x);
          mt = fmaxf(mt, x);
        }
      // the row maximum over both halves: both threads of a row reach the same decisions below
      sh->xmax[s][half][row] = mt;
      if (!pair_sync()) {
        fail(40);
        ok = false;
        break;
      }
      mt = fmaxf(mt, sh->xmax[s][half ^ 1][row]);
      float alpha = 1.f;
      bool resc = false;
      if (j == 0) {
        m_ref = mt;
      } else {
        resc = __any_sync(0xffffffffu, mt > m_ref + kFmLazyLog2) != 0;
        if (resc) {
          const float mn = fmaxf(m_ref, mt);
          alpha = (m_ref == -INFINITY) ? 0.f : fm_exp2(m_ref - mn);
          m_ref = mn;
        }
      }
      const float mr = (m_ref == -INFINITY) ? 0.f : m_ref;
      float sum = 0.f;
      // probabilities, rounded to bf16 and packed in place: v[cc][0..15] hold the 32 keys of chunk cc
#pragma unroll
      for (int cc = 0; cc < NC; ++cc)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = fm_exp2(__uint_as_float(v[cc][i]) - mr), p1 = fm_exp2(__uint_as_float(v[cc][i + 1]) - mr);
          sum += p0 + p1;
          v[cc][i >> 1] = fm_pack(p0, p1);
        }
      // P buffer s was the A operand of PV(j-2)
      if (j >= 2 && !mbar_wait(&sh->pv_done[s], ph(j - 2), abort_flag)) {
        fail(37);
        ok = false;
        break;
      }
      if (resc) {
        // the O accumulator may only be touched between PV(j-1) and PV(j); this warp rescales its half of the columns
        if (!mbar_wait(&sh->pv_done[(j - 1) & 1], ph(j - 1), abort_flag)) {
          fail(39);
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll 1
        for (int c8 = 0; c8 < D / 64; ++c8) {
          uint32_t o[32];
          const uint32_t ta = tmem_base + lane_addr + (uint32_t)(half * (D / 2) + c8 * 32);
          tmem_ld32(ta, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(ta, o);
        }
        tmem_st_wait();
      }
      l = l * alpha + sum;
      // P as the A operand of the next MMA: [128 rows x 64 keys] K-major tiles, 16-byte chunk index XOR (row % 8)
      unsigned char* pb = Ps + s * Cfg::p_bytes;
#pragma unroll
      for (int cch = 0; cch < HC / 8; ++cch) {
        const int ch = half * (HC / 8) + cch;
        unsigned char* dst = pb + (ch >> 3) * 16384 + row * 128 + (((ch & 7) ^ (row & 7)) * 16);
        *reinterpret_cast<uint4*>(dst) = make_uint4(v[cch >> 2][(cch & 3) * 4], v[cch >> 2][(cch & 3) * 4 + 1], v[cch >> 2][(cch & 3) * 4 + 2],
                                                    v[cch >> 2][(cch & 3) * 4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->p_full[s]);
    }
    // ---- epilogue: O / l -> global, each warp its half of the columns
    if (ok) ok = mbar_wait(&sh->pv_done[(nt - 1) & 1], ph(nt - 1), abort_flag);
    if (!ok) {
      fail(38);
    } else {
      tc_fence_after();
      float (*xl)[128] = sh->xmax[nt & 1];           // the parity the last tile did not use
      xl[half][row] = l;
      if (!pair_sync()) fail(41);
      l += xl[half ^ 1][row];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool store = q0 + row < p.t;
      bf16* dst = reinterpret_cast<bf16*>(p.out) + (long long)(q0 + row) * p.o_tok_stride + (long long)h * p.o_head_stride + half * (D / 2);
#pragma unroll 1
      for (int c8 = 0; c8 < D / 64; ++c8) {
        uint32_t o[32];
        tmem_ld32(tmem_base + lane_addr + (uint32_t)(half * (D / 2) + c8 * 32), o);
        tmem_ld_wait();
        if (store) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = fm_pack(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
            w.y = fm_pack(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            w.z = fm_pack(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
            w.w = fm_pack(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c8 * 32 + i) = w;
          }
        }
      }
    }
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
    tmem_dealloc(tmem_base, 512);
  }
}

// bf16 tensor map with 128-byte swizzle; dims / strides innermost first (strides in elements, for dims 1 and 2).
static int fm_tmap(CUtensorMap* map, const void* base, long long d0, long long d1, long long d2, long long s1, long long s2, int b0, int b1,
                   int b2) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (s1 * 2) % 16 != 0 || (s2 * 2) % 16 != 0) return (int)cudaErrorInvalidValue;
  cuuint64_t dims[3] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)d2};
  cuuint64_t strides[2] = {(cuuint64_t)s1 * 2, (cuuint64_t)s2 * 2};
  cuuint32_t box[3] = {(cuuint32_t)b0, (cuuint32_t)b1, (cuuint32_t)b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int D, int KT>
static int launch_fmha(const MmbFmhaPrefillParams& p, cudaStream_t stream) {
  CUtensorMap mq, mk, mv;
  // q / k as (d, head, token): the head stride is the smaller one in [token, head, d] tensors
  int e = fm_tmap(&mq, p.q, D, p.Hq, p.t, p.q_head_stride, p.q_tok_stride, 64, 1, 128);
  if (e) return e;
  e = fm_tmap(&mk, p.k, D, p.Hk, p.n, p.k_head_stride, p.k_tok_stride, 64, 1, KT);
  if (e) return e;
  e = fm_tmap(&mv, p.vt, p.n_pad, D, p.Hk, p.n_pad, (long long)D * p.n_pad, 64, D, 1);
  if (e) return e;
  auto kern = fmha_prefill_kernel<D, KT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FmhaCfg<D, KT>::smem_bytes);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  dim3 grid(p.Hq, (p.t + 127) / 128, 1);
  kern<<<grid, kFmThreads, FmhaCfg<D, KT>::smem_bytes, stream>>>(mq, mk, mv, p);
  return (int)cudaGetLastError();
}

}  // namespace mmb

MMB_API int mmb_fmha_prefill(const MmbFmhaPrefillParams* pp, cudaStream_t stream) {
  const MmbFmhaPrefillParams& p = *pp;
  if (p.t <= 0) return 0;
  if (p.window < 0 || p.n < p.t || p.n_pad < p.n || p.n_pad % 8 != 0 || p.Hk < 1 || p.Hq % p.Hk != 0 || (p.D != 128 && p.D != 256)) return (int)cudaErrorInvalidValue;
  if (p.q_tok_stride % 8 || p.q_head_stride % 8 || p.k_tok_stride % 8 || p.k_head_stride % 8 || p.o_tok_stride % 8 || p.o_head_stride % 8 ||
      (reinterpret_cast<uintptr_t>(p.out) & 15))
    return (int)cudaErrorInvalidValue;
  // the tensor maps need strides that grow with the dimension: head stride <= token stride
  if (p.q_head_stride > p.q_tok_stride || p.k_head_stride > p.k_tok_stride) return (int)cudaErrorInvalidValue;
  return p.D == 128 ? mmb::launch_fmha<128, 128>(p, stream) : mmb::launch_fmha<256, 64>(p, stream);
}
