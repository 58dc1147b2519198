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

}  // namespace mmb

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
