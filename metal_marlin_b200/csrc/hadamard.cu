// Block Walsh-Hadamard transform (orthonormal) on bf16 rows: the rotation MR-GPTQ-quantized layers apply to
// their input.  One CTA holds max(block, 512) consecutive elements of a row in shared memory as fp32 and runs
// the log2(block) butterfly stages on them.
#include "api_ext.h"
#include "common.cuh"
#include "launch.h"

namespace mmb {

__global__ void __launch_bounds__(256) hadamard_kernel(const bf16* __restrict__ x, bf16* __restrict__ out, long long total,
                                                       int block, int span) {
  extern __shared__ float hs[];
  pdl_launch_dependents();
  pdl_wait();
  const long long base = (long long)blockIdx.x * span;
  const int n = (int)min((long long)span, total - base);
  for (int i = threadIdx.x; i < n; i += 256) hs[i] = __bfloat162float(x[base + i]);
  __syncthreads();
  for (int h = 1; h < block; h <<= 1) {
    for (int i = threadIdx.x; i < n / 2; i += 256) {
      const int j = (i / h) * 2 * h + (i % h);
      const float a = hs[j], b = hs[j + h];
      hs[j] = a + b;
      hs[j + h] = a - b;
    }
    __syncthreads();
  }
  const float norm = rsqrtf((float)block);
  for (int i = threadIdx.x; i < n; i += 256) out[base + i] = __float2bfloat16(hs[i] * norm);
}

}  // namespace mmb

MMB_API int mmb_hadamard(const void* x, void* out, int rows, int dim, int block, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (block < 2 || block > 1024 || (block & (block - 1)) || dim % block) return (int)cudaErrorInvalidValue;
  const long long total = (long long)rows * dim;
  const int span = block > 512 ? block : 512 / block * block;      // whole blocks per CTA
  const unsigned grid = (unsigned)((total + span - 1) / span);
  return mmb::launch(mmb::hadamard_kernel, dim3(grid), dim3(256), (size_t)span * 4, stream, 1, (const bf16*)x, (bf16*)out, total,
                     block, span);
}
