// Trellis (2-8 bit uniform codebook, 16x16 tiles, LSB-first bit stream) weights: de-quantization to bf16 for the
// tensor-core GEMM path and a decode GEMV that reads the bit stream directly.
//
// Tile geometry: a tile holds 256 codes, code index = local_out * 16 + local_in, `bits` bits each, so lane l of a
// warp owns codes [8l, 8l + 8) = output row l / 2, input columns (l % 2) * 8 .. + 7, and those are exactly bytes
// [l * bits, (l + 1) * bits) of the tile: every lane reads `bits` contiguous bytes, no bit straddles lanes.
#include "api_ext.h"
#include "common.cuh"
#include "launch.h"

namespace mmb {

constexpr float kTrellisGridScale = 1.24371088f;

// the 8 codes of lane `lane` of a tile
__device__ __forceinline__ void trellis_lane_codes(const uint8_t* tile, int lane, int bits, int (&c)[8]) {
  unsigned long long v = 0;
  const uint8_t* p = tile + lane * bits;
  for (int b = 0; b < bits; ++b) v |= (unsigned long long)p[b] << (8 * b);
  const unsigned mask = (1u << bits) - 1u;
#pragma unroll
  for (int j = 0; j < 8; ++j) c[j] = (int)((v >> (j * bits)) & mask);
}

// grid: one warp per tile (8 warps per CTA)
__global__ void __launch_bounds__(256) trellis_dequant_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ scales,
                                                              const float* __restrict__ su, const float* __restrict__ sv,
                                                              bf16* __restrict__ out, int out_f, int in_f, int bits, int gs) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int ti_n = (in_f + 15) >> 4, to_n = (out_f + 15) >> 4;
  const long long tile = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tile >= (long long)ti_n * to_n) return;
  const int to = (int)(tile / ti_n), ti = (int)(tile % ti_n);
  int c[8];
  trellis_lane_codes(codes + tile * (32 * bits), lane, bits, c);
  const int o = to * 16 + (lane >> 1), i0 = ti * 16 + (lane & 1) * 8;
  if (o >= out_f) return;
  const float half = (float)((1 << bits) - 1) * 0.5f;
  const float row = sv[o] * kTrellisGridScale;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int i = i0 + j;
    if (i < in_f) out[(long long)o * in_f + i] = __float2bfloat16(((float)c[j] - half) * row * scales[(long long)(i / gs) * out_f + o] * su[i]);
  }
}

// grid (tiles_out), 256 threads: the 8 warps split the tiles of one tile row; x * su staged in shared memory as fp32.
constexpr int kTrellisMaxM = 4;
__global__ void __launch_bounds__(256) trellis_gemv_kernel(const bf16* __restrict__ x, const uint8_t* __restrict__ codes,
                                                           const float* __restrict__ scales, const float* __restrict__ su,
                                                           const float* __restrict__ sv, bf16* __restrict__ y, int M, int out_f,
                                                           int in_f, int bits, int gs, int ldx, int ldy) {
  extern __shared__ float xs[];            // [M][in_f]
  __shared__ float red[8][16][kTrellisMaxM];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int m = 0; m < M; ++m)
    for (int i = tid; i < in_f; i += 256) xs[m * in_f + i] = __bfloat162float(x[(long long)m * ldx + i]) * su[i];
  __syncthreads();
  const int ti_n = (in_f + 15) >> 4;
  const int to = blockIdx.x;
  const int o = to * 16 + (lane >> 1);
  const float half = (float)((1 << bits) - 1) * 0.5f;
  float acc[kTrellisMaxM] = {0.f, 0.f, 0.f, 0.f};
  for (int ti = warp; ti < ti_n; ti += 8) {
    int c[8];
    trellis_lane_codes(codes + ((long long)to * ti_n + ti) * (32 * bits), lane, bits, c);
    const int i0 = ti * 16 + (lane & 1) * 8;
    // group sizes are multiples of 16 (checked by the launcher), so a tile lies inside one scale group
    const float sc = (o < out_f) ? scales[(long long)(i0 / gs) * out_f + o] : 0.f;
#pragma unroll
    for (int m = 0; m < kTrellisMaxM; ++m) {
      if (m < M) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (i0 + j < in_f) s = fmaf((float)c[j] - half, xs[m * in_f + i0 + j], s);
        acc[m] = fmaf(s, sc, acc[m]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < kTrellisMaxM; ++m) {
    acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], 1);      // the two lanes of an output row
    if ((lane & 1) == 0) red[warp][lane >> 1][m] = acc[m];
  }
  __syncthreads();
  if (tid < 16 * kTrellisMaxM) {
    const int r = tid / kTrellisMaxM, m = tid % kTrellisMaxM;
    const int oo = to * 16 + r;
    if (m < M && oo < out_f) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) v += red[w][r][m];
      y[(long long)m * ldy + oo] = __float2bfloat16(v * sv[oo] * kTrellisGridScale);
    }
  }
}

// ---- mixture-of-experts decode on trellis weights (mixed bits per expert and per matrix).
// Expert matrices are described by a device table of MmbTrellisMat; the expert of every (token, slot) is read from device
// memory, so routing never touches the host and the launches can be captured in a CUDA graph.

// this warp's share of one 16-row tile row of matrix `mt` against the staged input (already multiplied by su)
__device__ __forceinline__ float trellis_row_partial(const MmbTrellisMat& mt, const float* xs, int to, int warp, int lane) {
  const int ti_n = (mt.in_f + 15) >> 4;
  const int o = to * 16 + (lane >> 1);
  const float half = (float)((1 << mt.bits) - 1) * 0.5f;
  float acc = 0.f;
  for (int ti = warp; ti < ti_n; ti += 8) {
    int c[8];
    trellis_lane_codes(mt.codes + ((long long)to * ti_n + ti) * (32 * mt.bits), lane, mt.bits, c);
    const int i0 = ti * 16 + (lane & 1) * 8;
    const float sc = (o < mt.out_f) ? mt.scales[(long long)(i0 / mt.gs) * mt.out_f + o] : 0.f;
    float sacc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (i0 + j < mt.in_f) sacc = fmaf((float)c[j] - half, xs[i0 + j], sacc);
    acc = fmaf(sacc, sc, acc);
  }
  return acc + __shfl_xor_sync(0xffffffffu, acc, 1);      // the two lanes of an output row
}

// grid (ceil(I / 16), T * topk), 256 threads.  h[slot, :] = silu(gate_e(x_t)) * up_e(x_t).
__global__ void __launch_bounds__(256) trellis_moe_gate_up_kernel(const bf16* __restrict__ x, const MmbTrellisMat* __restrict__ mats,
                                                                  const int* __restrict__ ids, bf16* __restrict__ h, int topk, int ldx,
                                                                  int ldh) {
  extern __shared__ float xs[];            // [2][in_f]: x * su of the gate and of the up matrix
  __shared__ float red[2][8][16];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int slot = blockIdx.y, token = slot / topk, to = blockIdx.x;
  const int e = ids[slot];
  if (e < 0) {
    if (tid < 16) h[(long long)slot * ldh + to * 16 + tid] = __float2bfloat16(0.f);
    return;
  }
  const MmbTrellisMat g = mats[e * 3 + 0], u = mats[e * 3 + 1];
  if (to * 16 >= g.out_f) return;
  for (int i = tid; i < g.in_f; i += 256) {
    const float xv = __bfloat162float(x[(long long)token * ldx + i]);
    xs[i] = xv * g.su[i];
    xs[g.in_f + i] = xv * u.su[i];
  }
  __syncthreads();
  const float pg = trellis_row_partial(g, xs, to, warp, lane);
  const float pu = trellis_row_partial(u, xs + g.in_f, to, warp, lane);
  if ((lane & 1) == 0) {
    red[0][warp][lane >> 1] = pg;
    red[1][warp][lane >> 1] = pu;
  }
  __syncthreads();
  if (tid < 16) {
    const int o = to * 16 + tid;
    if (o < g.out_f) {
      float vg = 0.f, vu = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        vg += red[0][w][tid];
        vu += red[1][w][tid];
      }
      // both projections rounded to bf16 like separate linears would return them
      vg = __bfloat162float(__float2bfloat16(vg * g.sv[o] * kTrellisGridScale));
      vu = __bfloat162float(__float2bfloat16(vu * u.sv[o] * kTrellisGridScale));
      h[(long long)slot * ldh + o] = __float2bfloat16(silu(vg) * vu);
    }
  }
}

// grid (ceil(H / 16), T * topk), 256 threads.  y[slot, :] = w[slot] * down_e(h[slot, :]) (fp32; the caller sums the slots).
__global__ void __launch_bounds__(256) trellis_moe_down_kernel(const bf16* __restrict__ h, const MmbTrellisMat* __restrict__ mats,
                                                               const int* __restrict__ ids, const float* __restrict__ wts,
                                                               float* __restrict__ y, int ldh, int ldy) {
  extern __shared__ float xs[];            // [in_f]
  __shared__ float red[8][16];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int slot = blockIdx.y, to = blockIdx.x;
  const int e = ids[slot];
  if (e < 0) {
    if (tid < 16) y[(long long)slot * ldy + to * 16 + tid] = 0.f;
    return;
  }
  const MmbTrellisMat d = mats[e * 3 + 2];
  if (to * 16 >= d.out_f) return;
  for (int i = tid; i < d.in_f; i += 256) xs[i] = __bfloat162float(h[(long long)slot * ldh + i]) * d.su[i];
  __syncthreads();
  const float pd = trellis_row_partial(d, xs, to, warp, lane);
  if ((lane & 1) == 0) red[warp][lane >> 1] = pd;
  __syncthreads();
  if (tid < 16) {
    const int o = to * 16 + tid;
    if (o < d.out_f) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) v += red[w][tid];
      v = __bfloat162float(__float2bfloat16(v * d.sv[o] * kTrellisGridScale));
      y[(long long)slot * ldy + o] = v * wts[slot];
    }
  }
}

}  // namespace mmb

MMB_API int mmb_trellis_moe(const void* x, const MmbTrellisMat* mats, const int* ids, const float* wts, void* h, float* y, int T, int topk,
                            int hidden, int inter, int ldx, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (topk < 1 || hidden % 16 != 0 || inter % 16 != 0 || (size_t)hidden * 8 > 160 * 1024 || (size_t)inter * 4 > 160 * 1024)
    return (int)cudaErrorInvalidValue;
  const size_t smem_gu = (size_t)hidden * 8, smem_d = (size_t)inter * 4;
  if (smem_gu > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(mmb::trellis_moe_gate_up_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_gu);
    if (e != cudaSuccess) return (int)e;
  }
  if (smem_d > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(mmb::trellis_moe_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_d);
    if (e != cudaSuccess) return (int)e;
  }
  int e = mmb::launch(mmb::trellis_moe_gate_up_kernel, dim3(inter / 16, T * topk), dim3(256), smem_gu, stream, 1, (const bf16*)x, mats, ids,
                      (bf16*)h, topk, ldx, inter);
  if (e) return e;
  return mmb::launch(mmb::trellis_moe_down_kernel, dim3(hidden / 16, T * topk), dim3(256), smem_d, stream, 1, (const bf16*)h, mats, ids, wts,
                     y, inter, hidden);
}

MMB_API int mmb_trellis_dequant(const uint8_t* codes, const float* scales, const float* su, const float* sv, void* out_bf16,
                                int out_f, int in_f, int bits, int group_size, cudaStream_t stream) {
  if (bits < 2 || bits > 8 || out_f <= 0 || in_f <= 0 || group_size <= 0) return (int)cudaErrorInvalidValue;
  const long long tiles = (long long)((out_f + 15) / 16) * ((in_f + 15) / 16);
  return mmb::launch(mmb::trellis_dequant_kernel, dim3((unsigned)((tiles + 7) / 8)), dim3(256), 0, stream, 1, codes, scales, su, sv,
                     (bf16*)out_bf16, out_f, in_f, bits, group_size);
}

MMB_API int mmb_trellis_gemv(const void* x, const uint8_t* codes, const float* scales, const float* su, const float* sv, void* y,
                             int M, int out_f, int in_f, int bits, int group_size, int ldx, int ldy, cudaStream_t stream) {
  if (bits < 2 || bits > 8 || M < 1 || M > mmb::kTrellisMaxM || group_size % 16 != 0) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)M * in_f * 4;
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(mmb::trellis_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return mmb::launch(mmb::trellis_gemv_kernel, dim3((unsigned)((out_f + 15) / 16)), dim3(256), smem, stream, 1, (const bf16*)x, codes,
                     scales, su, sv, (bf16*)y, M, out_f, in_f, bits, group_size, ldx, ldy);
}
