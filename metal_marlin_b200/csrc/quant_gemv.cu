// Decode GEMV for the group-quantized formats other than FP4: INT8 / INT4 / INT2 (with or without zero points),
// FP8 (E4M3 / E5M2), NF4 / NF3 / NF2 and 3-bit integers (held as 4-bit codes on the device).  One kernel covers
// them through a 256-entry value table: w = (lut[code] - zero) * scale.
//
// Layout: codes packed LSB-first along the input axis, `bits` in {2, 4, 8} per code, row-major [out, in * bits / 8];
// scales / zeros fp16 [out, in / gs].  One warp per output row; a lane consumes 16 bytes of codes per step
// (64 / 32 / 16 weights), which the launcher keeps inside one scale group.
#include "api_ext.h"
#include "common.cuh"
#include "launch.h"

namespace mmb {

constexpr int kCbMaxM = 8;

template <int BITS>
__global__ void __launch_bounds__(256) codebook_gemv_kernel(const bf16* __restrict__ x, const uint8_t* __restrict__ codes,
                                                            const __half* __restrict__ scales, const __half* __restrict__ zeros,
                                                            const float* __restrict__ lut, bf16* __restrict__ y, int M, int out_f,
                                                            int in_f, int gs, int ldx, int ldy) {
  extern __shared__ float xs[];      // [M][in_f]
  __shared__ float lut_s[256];
  constexpr int CPB = 8 / BITS;      // codes per byte
  constexpr int CPL = 16 * CPB;      // codes per lane per step
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int o = blockIdx.x * 8 + warp;
  // the first code words of this row are static: request them before waiting for the producer of x
  const long long row_bytes = (long long)in_f * BITS / 8;
  const uint8_t* crow = codes + (long long)min(o, out_f - 1) * row_bytes;
  uint4 first = make_uint4(0, 0, 0, 0);
  if (lane * 16 < row_bytes) first = ldg_stream(reinterpret_cast<const uint4*>(crow + lane * 16));
  lut_s[tid] = lut[tid];
  pdl_launch_dependents();
  pdl_wait();
  for (int m = 0; m < M; ++m)
    for (int i = tid; i < in_f; i += 256) xs[m * in_f + i] = __bfloat162float(x[(long long)m * ldx + i]);
  __syncthreads();
  if (o >= out_f) return;
  const int ng = in_f / gs;
  float acc[kCbMaxM];
#pragma unroll
  for (int m = 0; m < kCbMaxM; ++m) acc[m] = 0.f;
  for (long long b0 = lane * 16; b0 < row_bytes; b0 += 32 * 16) {
    const uint4 v = (b0 == lane * 16) ? first : ldg_stream(reinterpret_cast<const uint4*>(crow + b0));
    const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
    const int i0 = (int)(b0 * CPB);
    const int gi = i0 / gs;
    const float sc = __half2float(scales[(long long)o * ng + gi]);
    const float zp = zeros ? __half2float(zeros[(long long)o * ng + gi]) : 0.f;
    float s1[kCbMaxM], s2[kCbMaxM];
#pragma unroll
    for (int m = 0; m < kCbMaxM; ++m) s1[m] = s2[m] = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
      for (int j = 0; j < 4 * CPB; ++j) {
        const float wv = lut_s[(w4[q] >> (j * BITS)) & ((1u << BITS) - 1u)];
        const int i = i0 + q * 4 * CPB + j;
#pragma unroll
        for (int m = 0; m < kCbMaxM; ++m) {
          if (m < M) {
            const float xv = xs[m * in_f + i];
            s1[m] = fmaf(wv, xv, s1[m]);
            s2[m] += xv;
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < kCbMaxM; ++m) acc[m] = fmaf(sc, s1[m] - zp * s2[m], acc[m]);
  }
  (void)CPL;
#pragma unroll
  for (int m = 0; m < kCbMaxM; ++m) {
    if (m < M) {
      const float v = warp_sum(acc[m]);
      if (lane == 0) y[(long long)m * ldy + o] = __float2bfloat16(v);
    }
  }
}

}  // namespace mmb

MMB_API int mmb_codebook_gemv_bits(
    const void* x, const uint8_t* codes, const void* scales, const void* zeros, const float* lut, void* y, int M, int out_f,
    int in_f, int group_size, int bits, int ldx, int ldy, cudaStream_t stream) {
  using namespace mmb;
  if (M < 1 || M > kCbMaxM || (bits != 2 && bits != 4 && bits != 8)) return (int)cudaErrorInvalidValue;
  const int cpl = 16 * (8 / bits);
  if (in_f % cpl != 0 || group_size % cpl != 0 || in_f % group_size != 0) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)M * in_f * 4;
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  const dim3 grid((unsigned)((out_f + 7) / 8));
#define MMB_CB_LAUNCH(B)                                                                                                   \
  do {                                                                                                                     \
    if (smem > 48 * 1024) {                                                                                                \
      cudaError_t e = cudaFuncSetAttribute(codebook_gemv_kernel<B>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                                                 \
    }                                                                                                                      \
    return launch(codebook_gemv_kernel<B>, grid, dim3(256), smem, stream, 1, (const bf16*)x, codes, (const __half*)scales,   \
                  (const __half*)zeros, lut, (bf16*)y, M, out_f, in_f, group_size, ldx, ldy);                               \
  } while (0)
  if (bits == 8) MMB_CB_LAUNCH(8);
  if (bits == 4) MMB_CB_LAUNCH(4);
  MMB_CB_LAUNCH(2);
#undef MMB_CB_LAUNCH
}

MMB_API int mmb_codebook_gemv(const void* x, const uint8_t* codes, const void* scales, const void* zeros, const float* lut, void* y,
                              int M, int out_f, int in_f, int group_size, int ldx, int ldy, cudaStream_t stream) {
  return mmb_codebook_gemv_bits(x, codes, scales, zeros, lut, y, M, out_f, in_f, group_size, 8, ldx, ldy, stream);
}
