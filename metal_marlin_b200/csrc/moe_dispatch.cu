// MoE token dispatch on the device: counting sort of (token, slot) pairs by expert with the grouped-GEMM tile list,
// gather of the activation rows in expert order, and the combine (un-sort + sum over a token's slots + optional
// adds).  Three launches replace the chain of ~20 small framework kernels (argsort, scatter_add, cumsum, searchsorted,
// index_select, index_copy, sum) that otherwise dominates the grouped path at decode batch sizes.
#include "api_ext.h"
#include "common.cuh"
#include "launch.h"

namespace mmb {

constexpr int kGroupMaxExperts = 1024;

// One CTA.  ids int32 [n] (negative = dropped pair).  Outputs: order [n] (sorted position -> pair, -1 padded), inv [n]
// (pair -> sorted position or -1), tile_expert / tile_row0 / tile_rows [max_tiles], n_tiles [1].
__global__ void __launch_bounds__(1024) moe_group_kernel(const int* __restrict__ ids, int n, int E, int token_tile, int max_tiles,
                                                         int* __restrict__ order, int* __restrict__ inv, int* __restrict__ tile_expert,
                                                         int* __restrict__ tile_row0, int* __restrict__ tile_rows, int* __restrict__ n_tiles) {
  __shared__ int cnt[kGroupMaxExperts];
  __shared__ int off[kGroupMaxExperts + 1];
  __shared__ int tbase[kGroupMaxExperts + 1];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += 1024) cnt[e] = 0;
  __syncthreads();
  for (int i = tid; i < n; i += 1024) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int o = 0, t = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = o;
      tbase[e] = t;
      o += cnt[e];
      t += (cnt[e] + token_tile - 1) / token_tile;
    }
    off[E] = o;
    tbase[E] = t;
    *n_tiles = min(t, max_tiles);
  }
  __syncthreads();
  for (int e = tid; e < E; e += 1024) {
    const int nt = tbase[e + 1] - tbase[e];
    for (int j = 0; j < nt; ++j) {
      const int ti = tbase[e] + j;
      if (ti < max_tiles) {
        tile_expert[ti] = e;
        tile_row0[ti] = off[e] + j * token_tile;
        tile_rows[ti] = min(token_tile, cnt[e] - j * token_tile);
      }
    }
    cnt[e] = off[e];          // becomes the write cursor of the expert
  }
  for (int ti = tbase[E] + tid; ti < max_tiles; ti += 1024) {
    tile_expert[ti] = 0;
    tile_row0[ti] = 0;
    tile_rows[ti] = 0;
  }
  for (int i = off[E] + tid; i < n; i += 1024) order[i] = -1;
  __syncthreads();
  for (int i = tid; i < n; i += 1024) {
    const int e = ids[i];
    if (e >= 0 && e < E) {
      const int pos = atomicAdd(&cnt[e], 1);
      order[pos] = i;
      inv[i] = pos;
    } else {
      inv[i] = -1;
    }
  }
}

// xs[pos, :] = x[order[pos] / topk, :] (zero rows for padding); 8 bf16 per thread.
__global__ void __launch_bounds__(256) moe_gather_kernel(const bf16* __restrict__ x, const int* __restrict__ order, bf16* __restrict__ xs,
                                                         int n, int topk, int K, int ldx, const int* __restrict__ n_dev) {
  pdl_launch_dependents();
  pdl_wait();
  if (n_dev != nullptr) n = min(n, max(*n_dev, 0));      // rows beyond the device-side count are never read by a tile
  const int vec = K / 8;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < (long long)n * vec; i += (long long)gridDim.x * 256) {
    const int pos = (int)(i / vec), c = (int)(i % vec);
    const int pair = order[pos];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (pair >= 0) v = *reinterpret_cast<const uint4*>(x + (long long)(pair / topk) * ldx + c * 8);
    *reinterpret_cast<uint4*>(xs + (long long)pos * K + c * 8) = v;
  }
}

// out[t, :] = sum_k y[inv[t * topk + k], :] (+ add0[t, :] + add1[t, :]), fp32 accumulation, bf16 result.
__global__ void __launch_bounds__(256) moe_combine_kernel(const bf16* __restrict__ y, const int* __restrict__ inv, const bf16* __restrict__ add0,
                                                          const bf16* __restrict__ add1, bf16* __restrict__ out, int T, int topk, int N) {
  pdl_launch_dependents();
  pdl_wait();
  const int vec = N / 8;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < (long long)T * vec; i += (long long)gridDim.x * 256) {
    const int t = (int)(i / vec), c = (int)(i % vec);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto add_row = [&](const bf16* row) {
      const uint4 v = *reinterpret_cast<const uint4*>(row + c * 8);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __uint_as_float(w[j] << 16);
        acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
      }
    };
    for (int k = 0; k < topk; ++k) {
      const int pos = inv[t * topk + k];
      if (pos >= 0) add_row(y + (long long)pos * N);
    }
    if (add0) add_row(add0 + (long long)t * N);
    if (add1) add_row(add1 + (long long)t * N);
    uint4 o;
    o.x = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[0])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[1])) << 16);
    o.y = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[2])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[3])) << 16);
    o.z = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[4])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[5])) << 16);
    o.w = (uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[6])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16(acc[7])) << 16);
    *reinterpret_cast<uint4*>(out + (long long)t * N + c * 8) = o;
  }
}

}  // namespace mmb

MMB_API int mmb_moe_group(const int* ids, int n, int E, int token_tile, int max_tiles, int* order, int* inv, int* tile_expert, int* tile_row0,
                          int* tile_rows, int* n_tiles, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (E < 1 || E > mmb::kGroupMaxExperts || token_tile < 1 || max_tiles < 1) return (int)cudaErrorInvalidValue;
  return mmb::launch(mmb::moe_group_kernel, dim3(1), dim3(1024), 0, stream, 1, ids, n, E, token_tile, max_tiles, order, inv, tile_expert,
                     tile_row0, tile_rows, n_tiles);
}

MMB_API int mmb_moe_gather(const void* x, const int* order, void* xs, int n, int topk, int K, int ldx, const int* n_dev, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (K % 8 != 0 || ldx % 8 != 0 || topk < 1) return (int)cudaErrorInvalidValue;
  long long blocks = ((long long)n * (K / 8) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return mmb::launch(mmb::moe_gather_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, 1, (const bf16*)x, order, (bf16*)xs, n, topk, K, ldx, n_dev);
}

MMB_API int mmb_moe_combine(const void* y, const int* inv, const void* add0, const void* add1, void* out, int T, int topk, int N,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (N % 8 != 0 || topk < 1) return (int)cudaErrorInvalidValue;
  long long blocks = ((long long)T * (N / 8) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return mmb::launch(mmb::moe_combine_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, 1, (const bf16*)y, inv, (const bf16*)add0,
                     (const bf16*)add1, (bf16*)out, T, topk, N);
}
