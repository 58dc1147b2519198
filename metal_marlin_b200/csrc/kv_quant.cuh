// Quantized KV-cache rows: one fp32 scale per cached (token, head) row and 8- or 4-bit codes.
//   format 0  FP8 E4M3     1 byte / value    scale = amax / 448
//   format 1  INT8         1 byte / value    scale = amax / 127   (round to nearest even, symmetric)
//   format 2  FP4 E2M1     2 values / byte   scale = amax / 6     (low nibble = even element)
//   format 3  INT4         2 values / byte   scale = amax / 7     (two's complement nibbles)
// The writers (attention prologue kernels) and the readers (paged decode, gather for prompt passes) share these helpers, so
// a row is decoded exactly as it was encoded.
#pragma once
#include <cuda_fp8.h>

#include "common.cuh"

namespace mmb {

enum { KVQ_E4M3 = 0, KVQ_INT8 = 1, KVQ_E2M1 = 2, KVQ_INT4 = 3 };

__device__ __forceinline__ float kvq_range(int fmt) { return fmt == KVQ_E4M3 ? 448.f : (fmt == KVQ_INT8 ? 127.f : (fmt == KVQ_E2M1 ? 6.f : 7.f)); }
__host__ __device__ __forceinline__ bool kvq_is4(int fmt) { return fmt >= KVQ_E2M1; }

// `v` is the value divided by the row scale.
__device__ __forceinline__ unsigned kvq_encode(float v, int fmt) {
  if (fmt == KVQ_E4M3) return (unsigned)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
  if (fmt == KVQ_INT8) return (unsigned)__float2int_rn(fminf(fmaxf(v, -127.f), 127.f)) & 0xffu;
  if (fmt == KVQ_INT4) return (unsigned)__float2int_rn(fminf(fmaxf(v, -7.f), 7.f)) & 0xfu;
  const float a = fabsf(v);       // nearest of {0, .5, 1, 1.5, 2, 3, 4, 6}; a value on a midpoint takes the larger magnitude
  const unsigned m = a < 0.25f ? 0u : a < 0.75f ? 1u : a < 1.25f ? 2u : a < 1.75f ? 3u : a < 2.5f ? 4u : a < 3.5f ? 5u : a < 5.f ? 6u : 7u;
  return m | (v < 0.f ? 8u : 0u);
}

__device__ __forceinline__ float kvq_decode4(unsigned n, int fmt) {
  if (fmt == KVQ_INT4) return (float)(((int)(n << 28)) >> 28);
  const unsigned m = n & 7u, e = m >> 1, f = m & 1u;
  const float mag = e == 0u ? 0.5f * (float)f : (1.f + 0.5f * (float)f) * (float)(1u << (e - 1u));
  return (n & 8u) ? -mag : mag;
}

// Two 8-bit codes (low 16 bits of `w`) -> two floats.
__device__ __forceinline__ float2 kvq_decode8x2(unsigned w, int fmt) {
  if (fmt == KVQ_INT8) return make_float2((float)(signed char)(w & 0xffu), (float)(signed char)((w >> 8) & 0xffu));
  const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xffffu), __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&hr));
}

}  // namespace mmb
