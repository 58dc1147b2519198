// Memory-bound elementwise / normalisation kernels: RMSNorm (+residual), SwiGLU, RoPE, the fused
// per-head q/k norm + RoPE + paged K/V scatter, embedding gather.  One CTA per row, 16-byte
// accesses where the row length allows, fp32 math, bf16 storage.
#include "api.h"
#include "common.cuh"
#include "kv_quant.cuh"

namespace mmb {

__global__ void __launch_bounds__(256) rmsnorm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ delta,
                                                      const bf16* __restrict__ w, bf16* __restrict__ out,
                                                      bf16* __restrict__ resid_out, int dim, int ldx, int ldo,
                                                      float eps) {
  __shared__ float red[32];
  extern __shared__ float row_s[];   // dim floats
  const long long r = blockIdx.x;
  const bf16* xr = x + r * ldx;
  const bf16* dr = delta ? delta + r * ldx : nullptr;
  float ss = 0.f;
  for (int k = threadIdx.x * 2; k < dim; k += blockDim.x * 2) {
    float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(xr + k));
    if (dr) {
      float2 d = __bfloat1622float2(*reinterpret_cast<const bf162*>(dr + k));
      bf162 s2 = __floats2bfloat162_rn(v.x + d.x, v.y + d.y);
      v = __bfloat1622float2(s2);
      if (resid_out) *reinterpret_cast<bf162*>(resid_out + r * dim + k) = s2;
    }
    row_s[k] = v.x;
    row_s[k + 1] = v.y;
    ss += v.x * v.x + v.y * v.y;
  }
  ss = block_sum(ss, red);
  const float rs = rsqrtf(ss / (float)dim + eps);
  for (int k = threadIdx.x * 2; k < dim; k += blockDim.x * 2) {
    float2 wv = w ? __bfloat1622float2(*reinterpret_cast<const bf162*>(w + k)) : make_float2(1.f, 1.f);
    *reinterpret_cast<bf162*>(out + r * ldo + k) = __floats2bfloat162_rn(row_s[k] * rs * wv.x, row_s[k + 1] * rs * wv.y);
  }
}

// LayerNorm, one CTA per row: the row is read once into registers (8 values per thread and trip), mean and variance come
// from one pass of sums (fp32), the normalised row is written with 16-byte stores.
__global__ void __launch_bounds__(256) layernorm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ delta, const bf16* __restrict__ w,
                                                        const bf16* __restrict__ b, bf16* __restrict__ out, bf16* __restrict__ resid_out,
                                                        int dim, int ldx, int ldo, float eps) {
  __shared__ float red[32];
  extern __shared__ float rowbuf[];          // [dim] fp32 copy of the row (rows wider than the register budget)
  pdl_launch_dependents();
  pdl_wait();
  const long long r = blockIdx.x;
  const bf16* xr = x + r * ldx;
  float s = 0.f, q = 0.f;
  for (int k = threadIdx.x * 2; k < dim; k += 512) {
    float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(xr + k));
    if (delta != nullptr) {
      const float2 d = __bfloat1622float2(*reinterpret_cast<const bf162*>(delta + r * ldx + k));
      const bf162 s2 = __floats2bfloat162_rn(v.x + d.x, v.y + d.y);
      v = __bfloat1622float2(s2);
      if (resid_out != nullptr) *reinterpret_cast<bf162*>(resid_out + r * dim + k) = s2;
    }
    rowbuf[k] = v.x;
    rowbuf[k + 1] = v.y;
    s += v.x + v.y;
    q = fmaf(v.x, v.x, fmaf(v.y, v.y, q));
  }
  const float mean = block_sum(s, red) / (float)dim;
  const float var = fmaxf(block_sum(q, red) / (float)dim - mean * mean, 0.f);
  const float rstd = rsqrtf(var + eps);
  for (int k = threadIdx.x * 2; k < dim; k += 512) {
    float a = (rowbuf[k] - mean) * rstd, c = (rowbuf[k + 1] - mean) * rstd;
    if (w != nullptr) {
      const float2 ww = __bfloat1622float2(*reinterpret_cast<const bf162*>(w + k));
      a *= ww.x;
      c *= ww.y;
    }
    if (b != nullptr) {
      const float2 bb = __bfloat1622float2(*reinterpret_cast<const bf162*>(b + k));
      a += bb.x;
      c += bb.y;
    }
    *reinterpret_cast<bf162*>(out + r * ldo + k) = __floats2bfloat162_rn(a, c);
  }
}

__global__ void silu_mul_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int inter) {
  const long long r = blockIdx.x;            // rows on the x axis: prefill row counts exceed the 65535 limit of y
  const int k = (blockIdx.y * blockDim.x + threadIdx.x) * 2;
  if (k >= inter) return;
  float2 g = __bfloat1622float2(*reinterpret_cast<const bf162*>(gu + r * 2 * inter + k));
  float2 u = __bfloat1622float2(*reinterpret_cast<const bf162*>(gu + r * 2 * inter + inter + k));
  *reinterpret_cast<bf162*>(out + r * inter + k) = __floats2bfloat162_rn(silu(g.x) * u.x, silu(g.y) * u.y);
}

__global__ void add_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ out, long long n) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (i + 1 < n) {
    float2 x = __bfloat1622float2(*reinterpret_cast<const bf162*>(a + i));
    float2 y = __bfloat1622float2(*reinterpret_cast<const bf162*>(b + i));
    *reinterpret_cast<bf162*>(out + i) = __floats2bfloat162_rn(x.x + y.x, x.y + y.y);
  } else if (i < n) {
    out[i] = __float2bfloat16(__bfloat162float(a[i]) + __bfloat162float(b[i]));
  }
}

__global__ void embedding_kernel(const bf16* __restrict__ table, const int64_t* __restrict__ ids, bf16* __restrict__ out,
                                 int dim) {
  const long long r = blockIdx.x;
  const long long id = ids[r];
  const uint4* src = reinterpret_cast<const uint4*>(table + id * dim);
  uint4* dst = reinterpret_cast<uint4*>(out + r * dim);
  for (int k = threadIdx.x; k < dim / 8; k += blockDim.x) dst[k] = src[k];
}

__device__ __forceinline__ void rope_pair(float& a, float& b, float c, float s) {
  const float x = a * c - b * s, y = b * c + a * s;
  a = x;
  b = y;
}

// One CTA per token; threads loop over (head, pair).
__global__ void rope_kernel(bf16* __restrict__ q, bf16* __restrict__ k, const int* __restrict__ positions,
                            const float* __restrict__ inv_freq, int Hq, int Hk, int D, int rot_dim, int ldq, int ldk,
                            int interleaved, float mscale) {
  const long long tkn = blockIdx.x;
  const float pos = (float)positions[tkn];
  const int half = rot_dim / 2;
  const int total = (Hq + Hk) * half;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int h = i / half, j = i % half;
    bf16* base = (h < Hq) ? (q + tkn * ldq + (long long)h * D) : (k + tkn * ldk + (long long)(h - Hq) * D);
    float sn, cs;
    sincosf(pos * inv_freq[j], &sn, &cs);
    sn *= mscale;
    cs *= mscale;
    const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
    float a = __bfloat162float(base[ia]), b = __bfloat162float(base[ib]);
    rope_pair(a, b, cs, sn);
    base[ia] = __float2bfloat16(a);
    base[ib] = __float2bfloat16(b);
  }
}

// Qwen3-style attention prologue: per-head RMSNorm of q and k (optional), RoPE, K/V scatter to a paged
// pool [num_slots, Hk, D].  grid = (T, Hq + Hk); one warp-sized CTA per (token, head); D <= 256.
// One quantized row: `vals` (shared memory, D floats) -> codes at `dst` (D bytes, or D / 2 for the 4-bit formats).
__device__ __forceinline__ void kvq_store_row(unsigned char* dst, const float* vals, float inv, int D, int fmt) {
  if (kvq_is4(fmt)) {
    for (int i = threadIdx.x; i < D / 2; i += blockDim.x)
      dst[i] = (unsigned char)(kvq_encode(vals[2 * i] * inv, fmt) | (kvq_encode(vals[2 * i + 1] * inv, fmt) << 4));
  } else {
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = (unsigned char)kvq_encode(vals[i] * inv, fmt);
  }
}

// FP8 cache variant of the kernel below: same prologue; the K row (after norm + RoPE) and the V row are quantized to
// E4M3 with one scale per row (amax / 448) written beside them.
__global__ void __launch_bounds__(128) qk_norm_rope_cache_fp8_kernel(bf16* __restrict__ q, const bf16* __restrict__ k,
                                                                     const bf16* __restrict__ v, const bf16* __restrict__ qn_w,
                                                                     const bf16* __restrict__ kn_w, const int* __restrict__ positions,
                                                                     const float* __restrict__ inv_freq, const int64_t* __restrict__ slots,
                                                                     unsigned char* __restrict__ k_pool, unsigned char* __restrict__ v_pool,
                                                                     float* __restrict__ k_scale, float* __restrict__ v_scale, int Hq,
                                                                     int Hk, int D, int ldqkv, float eps, int interleaved, int fmt) {
  __shared__ float red[32];
  __shared__ float vals[256];
  const long long tkn = blockIdx.x;
  const int h = blockIdx.y;
  const bool is_q = h < Hq;
  const bf16* src = is_q ? (q + tkn * ldqkv + (long long)h * D) : (k + tkn * ldqkv + (long long)(h - Hq) * D);
  const bf16* nw = is_q ? qn_w : kn_w;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float x = __bfloat162float(src[i]);
    vals[i] = x;
    ss += x * x;
  }
  ss = block_sum(ss, red);
  if (nw != nullptr) {
    const float rs = rsqrtf(ss / (float)D + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x)
      vals[i] = __bfloat162float(__float2bfloat16(vals[i] * rs * __bfloat162float(nw[i])));
  }
  __syncthreads();
  const float pos = (float)positions[tkn];
  const int half = D / 2;
  const long long slot = slots ? slots[tkn] : -1;
  float amax = 0.f;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float sn, cs;
    sincosf(pos * inv_freq[j], &sn, &cs);
    const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
    float a = vals[ia], b = vals[ib];
    rope_pair(a, b, cs, sn);
    a = __bfloat162float(__float2bfloat16(a));
    b = __bfloat162float(__float2bfloat16(b));
    if (is_q) {
      bf16* dst = q + tkn * ldqkv + (long long)h * D;
      dst[ia] = __float2bfloat16(a);
      dst[ib] = __float2bfloat16(b);
    } else {
      vals[ia] = a;      // every pair is owned by one thread: in place
      vals[ib] = b;
      amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
    }
  }
  if (is_q || slot < 0) return;
  const long long row = slot * Hk + (h - Hq);
  amax = block_max(amax, red);
  const int row_bytes = kvq_is4(fmt) ? D / 2 : D;
  __syncthreads();       // all rotated values are in `vals`
  {
    const float sc = amax > 0.f ? amax / kvq_range(fmt) : 1.f, inv = 1.f / sc;
    kvq_store_row(k_pool + row * (long long)row_bytes, vals, inv, D, fmt);
    if (threadIdx.x == 0) k_scale[row] = sc;
  }
  if (v != nullptr) {
    const bf16* vs = v + tkn * ldqkv + (long long)(h - Hq) * D;
    float vmax = 0.f;
    __syncthreads();     // the K codes have been read out of `vals`
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      const float x = __bfloat162float(vs[i]);
      vals[i] = x;
      vmax = fmaxf(vmax, fabsf(x));
    }
    vmax = block_max(vmax, red);
    const float sc = vmax > 0.f ? vmax / kvq_range(fmt) : 1.f, inv = 1.f / sc;
    kvq_store_row(v_pool + row * (long long)row_bytes, vals, inv, D, fmt);
    if (threadIdx.x == 0) v_scale[row] = sc;
  }
}

// Paged quantized rows to contiguous bf16: grid (max_ctx, Hkv, B), one row per CTA of 64 threads (4 bytes per thread and trip).
__global__ void __launch_bounds__(64) kv_fp8_gather_kernel(const unsigned char* __restrict__ pool, const float* __restrict__ scale,
                                                           const int* __restrict__ block_tables, const int* __restrict__ ctx_lens,
                                                           const int* __restrict__ cu_k, bf16* __restrict__ out, int Hkv, int D,
                                                           int block_size, int max_blocks, int fmt) {
  const int t = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  if (t >= ctx_lens[b]) return;
  const long long slot = (long long)block_tables[(long long)b * max_blocks + t / block_size] * block_size + t % block_size;
  const long long row = slot * Hkv + h;
  const float sc = scale[row];
  bf16* dst = out + ((long long)(cu_k[b] + t) * Hkv + h) * D;
  if (kvq_is4(fmt)) {
    const unsigned char* src = pool + row * (long long)(D / 2);
    for (int i = threadIdx.x * 4; i < D / 2; i += 64 * 4) {      // 4 bytes = 8 values
      const uint32_t w = *reinterpret_cast<const uint32_t*>(src + i);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        *reinterpret_cast<bf162*>(dst + 2 * i + 2 * e) =
            __floats2bfloat162_rn(kvq_decode4((w >> (8 * e)) & 0xfu, fmt) * sc, kvq_decode4((w >> (8 * e + 4)) & 0xfu, fmt) * sc);
    }
    return;
  }
  const unsigned char* src = pool + row * (long long)D;
  for (int i = threadIdx.x * 4; i < D; i += 64 * 4) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(src + i);
#pragma unroll
    for (int e = 0; e < 4; e += 2) {
      const float2 f = kvq_decode8x2(w >> (8 * e), fmt);
      *reinterpret_cast<bf162*>(dst + i + e) = __floats2bfloat162_rn(f.x * sc, f.y * sc);
    }
  }
}

__global__ void __launch_bounds__(128) qk_norm_rope_cache_kernel(bf16* __restrict__ q, const bf16* __restrict__ k,
                                                                 const bf16* __restrict__ v, const bf16* __restrict__ qn_w,
                                                                 const bf16* __restrict__ kn_w,
                                                                 const int* __restrict__ positions,
                                                                 const float* __restrict__ inv_freq,
                                                                 const int64_t* __restrict__ slots, bf16* __restrict__ k_pool,
                                                                 bf16* __restrict__ v_pool, int Hq, int Hk, int D, int ldqkv,
                                                                 float eps, int interleaved) {
  __shared__ float red[32];
  __shared__ float vals[256];
  const long long tkn = blockIdx.x;
  const int h = blockIdx.y;
  const bool is_q = h < Hq;
  const bf16* src = is_q ? (q + tkn * ldqkv + (long long)h * D) : (k + tkn * ldqkv + (long long)(h - Hq) * D);
  const bf16* nw = is_q ? qn_w : kn_w;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float x = __bfloat162float(src[i]);
    vals[i] = x;
    ss += x * x;
  }
  ss = block_sum(ss, red);
  if (nw != nullptr) {
    const float rs = rsqrtf(ss / (float)D + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x)
      vals[i] = __bfloat162float(__float2bfloat16(vals[i] * rs * __bfloat162float(nw[i])));
  }
  __syncthreads();
  const float pos = (float)positions[tkn];
  const int half = D / 2;
  const long long slot = slots ? slots[tkn] : -1;
  bf16* dst;
  if (is_q) dst = q + tkn * ldqkv + (long long)h * D;
  else dst = (slot >= 0) ? k_pool + (slot * Hk + (h - Hq)) * (long long)D : nullptr;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float sn, cs;
    sincosf(pos * inv_freq[j], &sn, &cs);
    const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;
    float a = vals[ia], b = vals[ib];
    rope_pair(a, b, cs, sn);
    if (dst) {
      dst[ia] = __float2bfloat16(a);
      dst[ib] = __float2bfloat16(b);
    }
  }
  if (!is_q && slot >= 0 && v != nullptr) {
    const bf16* vs = v + tkn * ldqkv + (long long)(h - Hq) * D;
    bf16* vd = v_pool + (slot * Hk + (h - Hq)) * (long long)D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) vd[i] = vs[i];
  }
}

}  // namespace mmb

MMB_API int mmb_rmsnorm(const void* x, const void* delta, const void* w, void* out, void* resid_out, int rows, int dim,
                        int ldx, int ldo, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dim % 2 != 0 || dim * 4 > 160 * 1024) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)dim * 4;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(mmb::rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  mmb::rmsnorm_kernel<<<rows, 256, smem, stream>>>((const bf16*)x, (const bf16*)delta, (const bf16*)w, (bf16*)out,
                                                   (bf16*)resid_out, dim, ldx, ldo, eps);
  return (int)cudaGetLastError();
}

MMB_API int mmb_layernorm(const void* x, const void* delta, const void* w, const void* b, void* out, void* resid_out, int rows, int dim, int ldx,
                          int ldo, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dim <= 0 || (dim & 1) || (ldx & 1) || (ldo & 1)) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)dim * 4;
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(mmb::layernorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  mmb::layernorm_kernel<<<rows, 256, smem, stream>>>((const bf16*)x, (const bf16*)delta, (const bf16*)w, (const bf16*)b, (bf16*)out,
                                                     (bf16*)resid_out, dim, ldx, ldo, eps);
  return (int)cudaGetLastError();
}

MMB_API int mmb_silu_mul(const void* gate_up, void* out, int rows, int inter, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (inter % 2 != 0) return (int)cudaErrorInvalidValue;
  dim3 grid(rows, (inter / 2 + 255) / 256);
  mmb::silu_mul_kernel<<<grid, 256, 0, stream>>>((const bf16*)gate_up, (bf16*)out, inter);
  return (int)cudaGetLastError();
}

MMB_API int mmb_add(const void* a, const void* b, void* out, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long long pairs = (n + 1) / 2;
  mmb::add_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, stream>>>((const bf16*)a, (const bf16*)b, (bf16*)out, n);
  return (int)cudaGetLastError();
}

MMB_API int mmb_embedding(const void* table, const int64_t* ids, void* out, int n, int dim, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dim % 8 != 0) return (int)cudaErrorInvalidValue;
  mmb::embedding_kernel<<<n, 128, 0, stream>>>((const bf16*)table, ids, (bf16*)out, dim);
  return (int)cudaGetLastError();
}

MMB_API int mmb_rope(void* q, void* k, const int* positions, const float* inv_freq, int T, int Hq, int Hk, int D,
                     int rot_dim, int ldq, int ldk, int interleaved, float mscale, cudaStream_t stream) {
  if (T <= 0) return 0;
  mmb::rope_kernel<<<T, 256, 0, stream>>>((bf16*)q, (bf16*)k, positions, inv_freq, Hq, k ? Hk : 0, D, rot_dim, ldq, ldk,
                                          interleaved, mscale);
  return (int)cudaGetLastError();
}

MMB_API int mmb_qk_norm_rope_cache(void* q, const void* k, const void* v, const void* qn_w, const void* kn_w,
                                   const int* positions, const float* inv_freq, const int64_t* slots, void* k_pool,
                                   void* v_pool, int T, int Hq, int Hk, int D, int ldqkv, float eps, int interleaved,
                                   cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D > 256 || D % 2) return (int)cudaErrorInvalidValue;
  dim3 grid(T, Hq + Hk);
  mmb::qk_norm_rope_cache_kernel<<<grid, 128, 0, stream>>>((bf16*)q, (const bf16*)k, (const bf16*)v, (const bf16*)qn_w,
                                                           (const bf16*)kn_w, positions, inv_freq, slots, (bf16*)k_pool,
                                                           (bf16*)v_pool, Hq, Hk, D, ldqkv, eps, interleaved);
  return (int)cudaGetLastError();
}

MMB_API int mmb_qk_norm_rope_cache_fp8(void* q, const void* k, const void* v, const void* qn_w, const void* kn_w, const int* positions,
                                       const float* inv_freq, const int64_t* slots, void* k_pool, void* v_pool, float* k_scale,
                                       float* v_scale, int T, int Hq, int Hk, int D, int ldqkv, float eps, int interleaved, int kv_fmt,
                                       cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D > 256 || D % 8 || k_scale == nullptr || (v != nullptr && v_scale == nullptr) || kv_fmt < 0 || kv_fmt > 3) return (int)cudaErrorInvalidValue;
  dim3 grid(T, Hq + Hk);
  mmb::qk_norm_rope_cache_fp8_kernel<<<grid, 128, 0, stream>>>((bf16*)q, (const bf16*)k, (const bf16*)v, (const bf16*)qn_w,
                                                               (const bf16*)kn_w, positions, inv_freq, slots, (unsigned char*)k_pool,
                                                               (unsigned char*)v_pool, k_scale, v_scale, Hq, Hk, D, ldqkv, eps,
                                                               interleaved, kv_fmt);
  return (int)cudaGetLastError();
}

MMB_API int mmb_kv_fp8_gather(const void* pool, const float* scale, const int* block_tables, const int* ctx_lens, const int* cu_k,
                              void* out, int B, int Hkv, int D, int block_size, int max_blocks, int max_ctx, int kv_fmt,
                              cudaStream_t stream) {
  if (B <= 0 || max_ctx <= 0) return 0;
  if (D % 8 != 0 || Hkv > 65535 || B > 65535 || kv_fmt < 0 || kv_fmt > 3) return (int)cudaErrorInvalidValue;
  dim3 grid(max_ctx, Hkv, B);
  mmb::kv_fp8_gather_kernel<<<grid, 64, 0, stream>>>((const unsigned char*)pool, scale, block_tables, ctx_lens, cu_k, (bf16*)out, Hkv, D,
                                                     block_size, max_blocks, kv_fmt);
  return (int)cudaGetLastError();
}
