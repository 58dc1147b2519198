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

}  // namespace mmb

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
