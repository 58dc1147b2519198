// Image preprocessing for vision-language models: bilinear resize (half-pixel centres, edge clamp) of uint8 HWC
// images, per-channel normalisation and, optionally, patch extraction in the order ViT patch embeddings read
// (channel-major inside a patch) - one pass, one launch.
#include "api_ext.h"
#include "common.cuh"
#include "launch.h"

namespace mmb {

__global__ void __launch_bounds__(256) vision_preprocess_kernel(const uint8_t* __restrict__ img, bf16* __restrict__ out, int B, int H,
                                                                int W, int oh, int ow, int patch, float m0, float m1, float m2,
                                                                float s0, float s1, float s2) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;     // one thread per output pixel
  const long long total = (long long)B * oh * ow;
  if (idx >= total) return;
  const int b = (int)(idx / ((long long)oh * ow));
  const int r = (int)(idx % ((long long)oh * ow));
  const int oy = r / ow, ox = r % ow;
  const float fy = ((float)oy + 0.5f) * (float)H / (float)oh - 0.5f;
  const float fx = ((float)ox + 0.5f) * (float)W / (float)ow - 0.5f;
  const int y0 = max(0, min(H - 1, (int)floorf(fy))), x0 = max(0, min(W - 1, (int)floorf(fx)));
  const int y1 = min(H - 1, y0 + 1), x1 = min(W - 1, x0 + 1);
  const float wy = fminf(fmaxf(fy - (float)y0, 0.f), 1.f), wx = fminf(fmaxf(fx - (float)x0, 0.f), 1.f);
  const uint8_t* base = img + (long long)b * H * W * 3;
  const float mean[3] = {m0, m1, m2}, istd[3] = {1.f / s0, 1.f / s1, 1.f / s2};
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    const float p00 = base[((long long)y0 * W + x0) * 3 + c], p01 = base[((long long)y0 * W + x1) * 3 + c];
    const float p10 = base[((long long)y1 * W + x0) * 3 + c], p11 = base[((long long)y1 * W + x1) * 3 + c];
    const float v = (p00 * (1.f - wx) + p01 * wx) * (1.f - wy) + (p10 * (1.f - wx) + p11 * wx) * wy;
    const float nv = (v * (1.f / 255.f) - mean[c]) * istd[c];
    long long o;
    if (patch > 0) {
      const int py = oy / patch, px = ox / patch, ly = oy % patch, lx = ox % patch;
      const int pw = ow / patch;
      o = (((long long)b * (oh / patch) * pw + (long long)py * pw + px) * 3 + c) * patch * patch + ly * patch + lx;
    } else {
      o = (((long long)b * 3 + c) * oh + oy) * ow + ox;
    }
    out[o] = __float2bfloat16(nv);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// General form: crop rectangle (centre crop = a centred rectangle), bilinear / bicubic / nearest resampling of the
// rectangle to out_h x out_w (half-pixel centres, indices clamped to the rectangle; the bicubic kernel is the Keys cubic with
// a = -0.75), normalisation, then CHW pixels or ViT patches; `merge` > 1 orders the patches by merge x merge groups (the
// spatial-merge order of Qwen2-VL style encoders).
__device__ __forceinline__ float cubic_w(float x) {       // Keys, a = -0.75
  const float a = -0.75f;
  x = fabsf(x);
  if (x <= 1.f) return ((a + 2.f) * x - (a + 3.f)) * x * x + 1.f;
  if (x < 2.f) return ((a * x - 5.f * a) * x + 8.f * a) * x - 4.f * a;
  return 0.f;
}

__global__ void __launch_bounds__(256) vision_preprocess_ex_kernel(const uint8_t* __restrict__ img, bf16* __restrict__ out, int B, int H, int W,
                                                                   int cy, int cx, int ch, int cw, int oh, int ow, int patch, int merge,
                                                                   int mode, float m0, float m1, float m2, float s0, float s1, float s2) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long total = (long long)B * oh * ow;
  if (idx >= total) return;
  const int b = (int)(idx / ((long long)oh * ow));
  const int r = (int)(idx % ((long long)oh * ow));
  const int oy = r / ow, ox = r % ow;
  const float fy = ((float)oy + 0.5f) * (float)ch / (float)oh - 0.5f;
  const float fx = ((float)ox + 0.5f) * (float)cw / (float)ow - 0.5f;
  const uint8_t* base = img + (long long)b * H * W * 3;
  const float mean[3] = {m0, m1, m2}, istd[3] = {1.f / s0, 1.f / s1, 1.f / s2};
  auto px = [&](int y, int x, int c) -> float {
    y = cy + max(0, min(ch - 1, y));
    x = cx + max(0, min(cw - 1, x));
    return (float)base[((long long)y * W + x) * 3 + c];
  };
  float v[3];
  if (mode == 2) {
    const int y = (int)floorf(((float)oy + 0.5f) * (float)ch / (float)oh), x = (int)floorf(((float)ox + 0.5f) * (float)cw / (float)ow);
#pragma unroll
    for (int c = 0; c < 3; ++c) v[c] = px(y, x, c);
  } else if (mode == 1) {
    const int y0 = (int)floorf(fy), x0 = (int)floorf(fx);
    const float ty = fy - (float)y0, tx = fx - (float)x0;
    float wy[4], wx[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      wy[i] = cubic_w(ty - (float)(i - 1));
      wx[i] = cubic_w(tx - (float)(i - 1));
    }
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float row = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) row = fmaf(wx[j], px(y0 - 1 + i, x0 - 1 + j, c), row);
        acc = fmaf(wy[i], row, acc);
      }
      v[c] = acc;
    }
  } else {
    const int y0 = (int)floorf(fy), x0 = (int)floorf(fx);
    const float wy = fy - (float)y0, wx = fx - (float)x0;
#pragma unroll
    for (int c = 0; c < 3; ++c)
      v[c] = (px(y0, x0, c) * (1.f - wx) + px(y0, x0 + 1, c) * wx) * (1.f - wy) + (px(y0 + 1, x0, c) * (1.f - wx) + px(y0 + 1, x0 + 1, c) * wx) * wy;
  }
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    const float nv = (v[c] * (1.f / 255.f) - mean[c]) * istd[c];
    long long o;
    if (patch > 0) {
      const int py = oy / patch, pxx = ox / patch, ly = oy % patch, lx = ox % patch;
      const int pw = ow / patch, phh = oh / patch;
      long long pi = (long long)py * pw + pxx;
      if (merge > 1) pi = ((long long)(py / merge) * (pw / merge) + pxx / merge) * merge * merge + (py % merge) * merge + (pxx % merge);
      o = (((long long)b * phh * pw + pi) * 3 + c) * patch * patch + ly * patch + lx;
    } else {
      o = (((long long)b * 3 + c) * oh + oy) * ow + ox;
    }
    out[o] = __float2bfloat16(nv);
  }
}

// Per-image, per-channel mean and standard deviation of pixel / 255 (dataset statistics, auto-normalisation).
// grid (B), 256 threads; out fp32 [B, 3, 2].
__global__ void __launch_bounds__(256) channel_stats_kernel(const uint8_t* __restrict__ img, float* __restrict__ out, int HW) {
  __shared__ float red[32];
  const uint8_t* base = img + (long long)blockIdx.x * HW * 3;
  float s[3] = {0.f, 0.f, 0.f}, q[3] = {0.f, 0.f, 0.f};
  for (int i = threadIdx.x; i < HW; i += 256) {
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      const float v = (float)base[(long long)i * 3 + c] * (1.f / 255.f);
      s[c] += v;
      q[c] = fmaf(v, v, q[c]);
    }
  }
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    const float ts = block_sum(s[c], red);
    const float tq = block_sum(q[c], red);
    if (threadIdx.x == 0) {
      const float mean = ts / (float)HW;
      out[(blockIdx.x * 3 + c) * 2] = mean;
      out[(blockIdx.x * 3 + c) * 2 + 1] = sqrtf(fmaxf(tq / (float)HW - mean * mean, 0.f));
    }
  }
}

}  // namespace mmb

MMB_API int mmb_vision_preprocess_ex(const uint8_t* images, void* out, int B, int H, int W, int crop_y, int crop_x, int crop_h, int crop_w,
                                     int out_h, int out_w, int patch, int merge, int mode, const float* mean3, const float* std3,
                                     cudaStream_t stream) {
  if (B <= 0) return 0;
  if (H <= 0 || W <= 0 || out_h <= 0 || out_w <= 0 || crop_h <= 0 || crop_w <= 0 || crop_y < 0 || crop_x < 0 || crop_y + crop_h > H ||
      crop_x + crop_w > W || mode < 0 || mode > 2)
    return (int)cudaErrorInvalidValue;
  if (patch > 0 && (out_h % patch || out_w % patch)) return (int)cudaErrorInvalidValue;
  if (patch > 0 && merge > 1 && ((out_h / patch) % merge || (out_w / patch) % merge)) return (int)cudaErrorInvalidValue;
  for (int c = 0; c < 3; ++c)
    if (std3[c] == 0.f) return (int)cudaErrorInvalidValue;
  const long long total = (long long)B * out_h * out_w;
  return mmb::launch(mmb::vision_preprocess_ex_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, 1, images, (bf16*)out, B,
                     H, W, crop_y, crop_x, crop_h, crop_w, out_h, out_w, patch, merge, mode, mean3[0], mean3[1], mean3[2], std3[0], std3[1],
                     std3[2]);
}

MMB_API int mmb_channel_stats(const uint8_t* images, float* out, int B, int H, int W, cudaStream_t stream) {
  if (B <= 0) return 0;
  mmb::channel_stats_kernel<<<B, 256, 0, stream>>>(images, out, H * W);
  return (int)cudaGetLastError();
}

MMB_API int mmb_vision_preprocess(const uint8_t* images, void* out, int B, int H, int W, int out_h, int out_w, int patch,
                                  const float* mean3, const float* std3, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (H <= 0 || W <= 0 || out_h <= 0 || out_w <= 0) return (int)cudaErrorInvalidValue;
  if (patch > 0 && (out_h % patch || out_w % patch)) return (int)cudaErrorInvalidValue;
  for (int c = 0; c < 3; ++c)
    if (std3[c] == 0.f) return (int)cudaErrorInvalidValue;
  const long long total = (long long)B * out_h * out_w;
  return mmb::launch(mmb::vision_preprocess_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, 1, images, (bf16*)out, B,
                     H, W, out_h, out_w, patch, mean3[0], mean3[1], mean3[2], std3[0], std3[1], std3[2]);
}
