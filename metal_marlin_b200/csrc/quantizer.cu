// Quantizer kernels: the column-serial inner loop of GPTQ over one lazy block, and fused round-to-nearest E2M1
// quantization + packing.  Both restate PyTorch code of this package operation by operation (same fp32 roundings, no
// fused multiply-add), so their results are bit-identical to it and either path can produce a checkpoint.
//
// Parity: reference src/cholesky.metal (`gptq_update_weights`), metal_marlin/gptq_accelerated.py (block loop),
// metal_marlin/fp4_metal.py (FP4 quantization on the device).
#include "api_ext.h"
#include "common.cuh"

namespace {

constexpr int GPTQ_WARPS = 8;
constexpr int GPTQ_MAX_BLOCK = 128;
constexpr int GPTQ_MAX_GRID = 256;

// Index of the grid value nearest to x: the number of midpoints strictly below x (ties go to the lower value), which
// is torch.bucketize(x, mids) with right=False.
__device__ __forceinline__ int nearest_index(float x, const float* mids, int n_mid) {
  int lo = 0, hi = n_mid;
  while (lo < hi) {
    const int m = (lo + hi) >> 1;
    if (mids[m] < x) lo = m + 1; else hi = m;
  }
  return lo;
}

// One warp per weight row.  Lane l holds columns l, l + 32, l + 64, l + 96 of the block in registers; the columns are
// visited in order, the owner broadcasts its value, every lane computes the same quantized value and error and
// subtracts err * Hinv[i, c] from the columns c >= i that it owns.
__global__ void __launch_bounds__(GPTQ_WARPS * 32)
gptq_block_kernel(float* __restrict__ W, float* __restrict__ Q, float* __restrict__ E, const float* __restrict__ Hinv,
                  const float* __restrict__ col_scale, const float* __restrict__ grid, float* __restrict__ err_rows,
                  int n_grid, int out_f, long ldw, long ldh, int i1, int B) {
  __shared__ float grid_s[GPTQ_MAX_GRID];
  __shared__ float mids_s[GPTQ_MAX_GRID];
  for (int i = threadIdx.x; i < n_grid; i += blockDim.x) {
    grid_s[i] = grid[i];
    if (i + 1 < n_grid) mids_s[i] = __fdiv_rn(__fadd_rn(grid[i + 1], grid[i]), 2.0f);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * GPTQ_WARPS + (threadIdx.x >> 5);
  if (row >= out_f) return;
  float* wrow = W + (long)row * ldw + i1;
  float* qrow = Q + (long)row * ldw + i1;
  const float* srow = col_scale + (long)row * ldw + i1;
  float w[4], s[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int c = t * 32 + lane;
    w[t] = c < B ? wrow[c] : 0.0f;
    s[t] = c < B ? srow[c] : 1.0f;
  }
  float err_sq = 0.0f;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    for (int l = 0; l < 32; ++l) {
      const int i = t * 32 + l;
      if (i >= B) break;
      const float wc = __shfl_sync(0xffffffffu, w[t], l);
      const float sc = __shfl_sync(0xffffffffu, s[t], l);
      const float q = __fmul_rn(grid_s[nearest_index(__fdiv_rn(wc, sc), mids_s, n_grid - 1)], sc);
      const float* hrow = Hinv + (long)(i1 + i) * ldh + i1;
      const float d = __fsub_rn(wc, q);
      const float e = __fdiv_rn(d, hrow[i]);
      if (lane == l) {
        qrow[i] = q;
        E[(long)row * B + i] = e;
        err_sq = __fadd_rn(err_sq, __fmul_rn(d, d));
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = u * 32 + lane;
        if (c >= i && c < B) w[u] = __fsub_rn(w[u], __fmul_rn(e, hrow[c]));
      }
    }
  }
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int c = t * 32 + lane;
    if (c < B) wrow[c] = w[t];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) err_sq += __shfl_xor_sync(0xffffffffu, err_sq, o);
  if (lane == 0) err_rows[row] += err_sq;
}

__device__ __forceinline__ float load_f32(const float* p, long i) { return p[i]; }
__device__ __forceinline__ float load_f32(const __nv_bfloat16* p, long i) { return __bfloat162float(p[i]); }

// One thread per output word (8 consecutive input columns of one row); the gs / 8 threads of a group (1..16, a power of
// two, inside one warp) share the absolute maximum by shuffles.
template <typename T>
__global__ void __launch_bounds__(256)
fp4_quantize_pack_kernel(const T* __restrict__ w, uint32_t* __restrict__ packed, __half* __restrict__ scales,
                         long n_words, int words_per_row, int lanes_per_group) {
  const long word = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = word < n_words;
  float v[8];
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    v[j] = live ? load_f32(w, word * 8 + j) : 0.0f;
    amax = fmaxf(amax, fabsf(v[j]));
  }
  for (int o = lanes_per_group >> 1; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  __half sh = __float2half_rn(__fdiv_rn(amax, 6.0f));
  if (!(__half2float(sh) > 0.0f)) sh = __ushort_as_half((unsigned short)1);    // smallest subnormal, 2^-24
  const float sf = __half2float(sh);
  uint32_t out = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float x = fminf(fmaxf(__fdiv_rn(v[j], sf), -6.0f), 6.0f);
    const float a = fabsf(x);
    // midpoints of the E2M1 magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6; a value on a midpoint takes the smaller magnitude
    const uint32_t mag = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
    out |= (mag | ((x < 0.0f && mag > 0) ? 8u : 0u)) << (4 * j);
  }
  if (live) {
    packed[word] = out;
    const int in_row = (int)(word % words_per_row);
    if (in_row % lanes_per_group == 0)
      scales[(word / words_per_row) * (words_per_row / lanes_per_group) + in_row / lanes_per_group] = sh;
  }
}

}  // namespace

extern "C" int mmb_gptq_block(float* W, float* Q, float* E, const float* Hinv, const float* col_scale, const float* grid,
                              float* err_rows, int n_grid, int out_f, long ldw, long ldh, int i1, int B,
                              cudaStream_t stream) {
  if (B < 1 || B > GPTQ_MAX_BLOCK || n_grid < 2 || n_grid > GPTQ_MAX_GRID || out_f < 1) return (int)cudaErrorInvalidValue;
  const int blocks = (out_f + GPTQ_WARPS - 1) / GPTQ_WARPS;
  gptq_block_kernel<<<blocks, GPTQ_WARPS * 32, 0, stream>>>(W, Q, E, Hinv, col_scale, grid, err_rows, n_grid, out_f, ldw,
                                                            ldh, i1, B);
  return (int)cudaGetLastError();
}

extern "C" int mmb_fp4_quantize_pack(const void* w, int w_is_bf16, uint32_t* packed, void* scales, long out_f, int in_f,
                                     int group_size, cudaStream_t stream) {
  const int lanes = group_size / 8;
  if (group_size < 8 || group_size > 128 || (lanes & (lanes - 1)) != 0 || in_f % group_size != 0)
    return (int)cudaErrorInvalidValue;
  const long n_words = out_f * (long)(in_f / 8);
  if (n_words == 0) return 0;
  const unsigned blocks = (unsigned)((n_words + 255) / 256);
  if (w_is_bf16)
    fp4_quantize_pack_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)w, packed, (__half*)scales, n_words, in_f / 8,
                                                         lanes);
  else
    fp4_quantize_pack_kernel<<<blocks, 256, 0, stream>>>((const float*)w, packed, (__half*)scales, n_words, in_f / 8, lanes);
  return (int)cudaGetLastError();
}
