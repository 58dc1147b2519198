// Prefill attention: one CTA (8 warps) owns 128 query rows of one head of one sequence, each warp 16 of them with its
// scores, soft-max statistics and output accumulator entirely in registers (no cross-warp traffic); 64-key K / V tiles
// stream through a double-buffered cp.async pipeline in shared memory.  The probability tile never leaves registers:
// the accumulator fragment of S = Q K^T is re-used as the A fragment of P V.  Keys come either from contiguous
// rows or straight from the paged pool through the block table (no gather copy).
#include "api_ext.h"
#include "common.cuh"
#include "launch.h"

namespace mmb {

constexpr int kPfM = 128;     // query rows per CTA (8 warps x 16)
constexpr int kPfThreads = 256;
constexpr int kPfN = 64;      // keys per tile

__device__ __forceinline__ void pf_cp16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = smem_u32(smem);
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void pf_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void pf_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void pf_ldsm4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void pf_ldsm4t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ uint32_t pf_pack(float a, float b) {
  const bf162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <int D>
__global__ void __launch_bounds__(kPfThreads) prefill_attention_kernel(const MmbPrefillAttnParams p) {
  constexpr int LD = D + 8;              // shared-memory row stride in elements (16-byte skew: conflict-free ldmatrix)
  constexpr int CH = D / 8;              // 16-byte chunks per row
  extern __shared__ __align__(128) unsigned char smem_pf[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_pf);
  bf16* Ks = Qs + kPfM * LD;             // [2][kPfN][LD]
  bf16* Vs = Ks + 2 * kPfN * LD;         // [2][kPfN][LD]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int b = blockIdx.z, h = blockIdx.y, hk = h / (p.Hq / p.Hk);
  pdl_launch_dependents();
  pdl_wait();
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int q0 = blockIdx.x * kPfM;
  if (q0 >= q_len) return;
  const bool paged = p.cu_k == nullptr;
  const int k_begin = paged ? 0 : p.cu_k[b];
  const int kv_len = paged ? p.ctx_lens[b] : p.cu_k[b + 1] - k_begin;
  const int q_off = kv_len - q_len;      // position of query row 0 among the keys
  const int* bt = paged ? p.block_tables + (long long)b * p.max_blocks : nullptr;
  const bf16* qg = reinterpret_cast<const bf16*>(p.q) + (long long)(q_begin + q0) * p.q_tok_stride + (long long)h * p.q_head_stride;
  const bf16* kg = reinterpret_cast<const bf16*>(p.k) + (long long)hk * p.k_head_stride;
  const bf16* vg = reinterpret_cast<const bf16*>(p.v) + (long long)hk * p.v_head_stride;

  // key range of this query tile
  const int qpos_hi = q_off + min(q0 + kPfM, q_len) - 1;
  const int k_hi = p.causal ? min(kv_len, qpos_hi + 1) : kv_len;
  const int k_lo_win = (p.window > 0) ? max(0, q_off + q0 - p.window + 1) : 0;
  const int sinks = (p.window > 0) ? p.sinks : 0;
  const int tile_lo = (sinks > 0) ? 0 : k_lo_win / kPfN, tile_hi = (k_hi + kPfN - 1) / kPfN;
  const unsigned char* bmask = p.block_mask
      ? p.block_mask + ((long long)(p.block_heads > 1 ? h : 0) * ((p.max_q + kPfM - 1) / kPfM) + blockIdx.x) * p.n_kblocks
      : nullptr;
  const unsigned char* tmask = p.tree_mask ? p.tree_mask + (long long)q_begin * p.tree_ld : nullptr;
  // key tiles nobody in this query tile can see are skipped: block-sparse zeros, and the gap between the global tokens
  // and the start of the window
  auto next_tile = [&](int tl) {
    while (tl < tile_hi) {
      const bool in_gap = sinks > 0 && tl * kPfN >= sinks && (tl + 1) * kPfN <= k_lo_win;
      const bool off = bmask != nullptr && (tl >= p.n_kblocks || bmask[tl] == 0);
      if (!in_gap && !off) break;
      ++tl;
    }
    return tl;
  };

  auto load_kv = [&](int tile, int buf) {
    bf16* kd = Ks + buf * kPfN * LD;
    bf16* vd = Vs + buf * kPfN * LD;
    for (int i = tid; i < kPfN * CH; i += kPfThreads) {
      const int r = i / CH, c = i % CH;
      const int key = tile * kPfN + r;
      const bool ok = key < kv_len;
      long long row = 0;
      if (ok) row = paged ? ((long long)bt[key / p.block_size] * p.block_size + key % p.block_size) : (long long)(k_begin + key);
      pf_cp16(kd + r * LD + c * 8, kg + row * p.k_tok_stride + c * 8, ok);
      pf_cp16(vd + r * LD + c * 8, vg + row * p.v_tok_stride + c * 8, ok);
    }
  };
  for (int i = tid; i < kPfM * CH; i += kPfThreads) {
    const int r = i / CH, c = i % CH;
    pf_cp16(Qs + r * LD + c * 8, qg + (long long)r * p.q_tok_stride + c * 8, q0 + r < q_len);
  }
  const int tile_first = next_tile(tile_lo);
  if (tile_first < tile_hi) load_kv(tile_first, 0);
  pf_commit();

  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sl2 = p.scale * 1.4426950408889634f;
  const int qrow0 = q0 + warp * 16 + g;        // this thread's rows: qrow0 and qrow0 + 8 (relative to the sequence's queries)

  int buf = 0;
  for (int tile = tile_first, tile_next; tile < tile_hi; tile = tile_next, buf ^= 1) {
    tile_next = next_tile(tile + 1);
    if (tile_next < tile_hi) load_kv(tile_next, buf ^ 1);
    pf_commit();
    pf_wait<1>();
    __syncthreads();
    const bf16* kt = Ks + buf * kPfN * LD;
    const bf16* vt = Vs + buf * kPfN * LD;
    // ---- S = Q K^T (16 x 64 per warp)
    float s[kPfN / 8][4];
#pragma unroll
    for (int n = 0; n < kPfN / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll 2
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a0, a1, a2, a3;
      pf_ldsm4(a0, a1, a2, a3, Qs + (warp * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int n = 0; n < kPfN / 8; n += 2) {
        uint32_t b0, b1, b2, b3;
        pf_ldsm4(b0, b1, b2, b3, kt + (n * 8 + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16_16816(s[n], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(s[n + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // ---- mask + online soft-max (rows g and g + 8)
    const int key0 = tile * kPfN;
    const bool need_mask = (key0 + kPfN > kv_len) || (p.causal && key0 + kPfN - 1 > q_off + q0 + warp * 16) ||
                           (p.window > 0 && key0 < q_off + q0 + warp * 16 + 16 - p.window + 1) ||
                           (tmask != nullptr && key0 + kPfN > q_off);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < kPfN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[n][e] * sl2;
        if (need_mask) {
          const int key = key0 + n * 8 + 2 * t + (e & 1);
          const int qpos = q_off + qrow0 + ((e >> 1) << 3);
          bool ok = key < kv_len && (!p.causal || key <= qpos) && (p.window <= 0 || key > qpos - p.window || key < sinks);
          if (ok && tmask != nullptr && key >= q_off) {
            const int qr = qpos - q_off;
            ok = qr < q_len && tmask[(long long)qr * p.tree_ld + (key - q_off)] != 0;
          }
          if (!ok) v = -INFINITY;
        }
        s[n][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      msafe[r] = (m_new == -INFINITY) ? 0.f : m_new;
      corr[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - msafe[r]);
      m_run[r] = m_new;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < kPfN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = exp2f(s[n][e] - msafe[e >> 1]);
        s[n][e] = pv;
        rs[e >> 1] += pv;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
      l_run[r] = l_run[r] * corr[r] + rs[r];
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      o[n][0] *= corr[0];
      o[n][1] *= corr[0];
      o[n][2] *= corr[1];
      o[n][3] *= corr[1];
    }
    // ---- O += P V: the S accumulator fragments of two 8-key tiles are the A fragment of one 16-key step
#pragma unroll
    for (int kk = 0; kk < kPfN / 16; ++kk) {
      const uint32_t a0 = pf_pack(s[2 * kk][0], s[2 * kk][1]), a1 = pf_pack(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pf_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pf_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int n = 0; n < D / 8; n += 2) {
        uint32_t b0, b1, b2, b3;
        pf_ldsm4t(b0, b1, b2, b3, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + (n + (lane >> 4)) * 8);
        mma_bf16_16816(o[n], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(o[n + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();      // every warp is done with this buffer before the load of tile + 2 overwrites it
  }
  pf_wait<0>();
  // ---- normalise and store
  bf16* og = reinterpret_cast<bf16*>(p.out) + (long long)(q_begin) * p.o_tok_stride + (long long)h * p.o_head_stride;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = qrow0 + r * 8;
    if (row >= q_len) continue;
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
      *reinterpret_cast<bf162*>(og + (long long)row * p.o_tok_stride + n * 8 + 2 * t) = __floats2bfloat162_rn(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
  }
}

template <int D>
static int launch_prefill(const MmbPrefillAttnParams& p, cudaStream_t stream) {
  const size_t smem = (size_t)(kPfM + 4 * kPfN) * (D + 8) * 2;
  auto kern = prefill_attention_kernel<D>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((p.max_q + kPfM - 1) / kPfM, p.Hq, p.B);
  return launch(kern, grid, dim3(kPfThreads), smem, stream, 1, p);
}

}  // namespace mmb

MMB_API int mmb_prefill_attention(const MmbPrefillAttnParams* pp, cudaStream_t stream) {
  const MmbPrefillAttnParams& p = *pp;
  if (p.B <= 0 || p.max_q <= 0) return 0;
  if (p.Hk <= 0 || p.Hq % p.Hk != 0) return (int)cudaErrorInvalidValue;
  if ((p.q_tok_stride | p.q_head_stride | p.k_tok_stride | p.k_head_stride | p.v_tok_stride | p.v_head_stride) & 7) return (int)cudaErrorInvalidValue;
  if ((p.o_tok_stride | p.o_head_stride) & 1) return (int)cudaErrorInvalidValue;
  if (p.cu_k == nullptr && (p.block_tables == nullptr || p.ctx_lens == nullptr || p.block_size <= 0)) return (int)cudaErrorInvalidValue;
  if (p.Hq > 65535 || p.B > 65535) return (int)cudaErrorInvalidValue;
  switch (p.D) {
    case 64: return mmb::launch_prefill<64>(p, stream);
    case 128: return mmb::launch_prefill<128>(p, stream);
    case 256: return mmb::launch_prefill<256>(p, stream);
    default: return (int)cudaErrorNotSupported;
  }
}
