// Paged decode attention with built-in scratch memory: split-KV attention followed by the merge of the split
// partials, where the partials live in a fixed device array of this module instead of caller-provided buffers.
// Nothing on this path allocates: no device or host allocation, no allocating library routine.  The launches
// are the same kernels the regular entry points use (mmb_paged_decode, mmb_decode_merge).
//
// Who needs this: hosts that own every byte of device memory themselves (an arena carved at start-up, a
// real-time serving loop where the allocator is off limits) and still want split-KV decode attention, which
// needs somewhere to keep per-split partial outputs between its two launches.
#include "attention_noalloc.h"

#include <stdio.h>

#include <mutex>

#include "api.h"
#include "common.cuh"

namespace {

// Capacity of the scratch.  8 MiB of partial outputs covers e.g. 32 sequences x 20 heads x 6 splits of a
// 512-wide MLA latent, or one sequence x 20 heads x 64 splits x 512; the pair array allows narrow heads
// (dv = 64) to use all of the partial-output space.
constexpr long long kMaxPartialFloats = 2ll << 20;
constexpr long long kMaxRows = 16ll << 10;
constexpr int kMaxDevices = 64;

// [ partial outputs : kMaxPartialFloats ][ (running max, running sum) pairs : 2 * kMaxRows ]
static __device__ __align__(256) __attribute__((used)) float g_noalloc_scratch[kMaxPartialFloats + 2 * kMaxRows];

std::mutex g_mu;
float* g_scratch_ptr[kMaxDevices] = {};   // address of g_noalloc_scratch on each device, filled on first use

thread_local char g_err[256] = "";

int fail(int code, const char* fmt, long long a = 0, long long b = 0, long long c = 0) {
  snprintf(g_err, sizeof(g_err), fmt, a, b, c);
  return code;
}

// Address of the scratch on the current device.  The first call per device asks the runtime for the symbol's
// address (this also makes sure the module is loaded on that device); later calls read the cached pointer.
int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(MMB_NOALLOC_SETUP_FAILED, "no usable current device (cudaGetDevice -> %lld, device %lld)", (long long)e, dev);
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(MMB_NOALLOC_SETUP_FAILED, "cudaGetSymbolAddress failed on device %lld with error %lld", dev, (long long)e);
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return MMB_NOALLOC_OK;
}

}  // namespace

MMB_API void mmb_paged_attention_noalloc_limits(long long* max_partial_floats, long long* max_rows) {
  if (max_partial_floats) *max_partial_floats = kMaxPartialFloats;
  if (max_rows) *max_rows = kMaxRows;
}

MMB_API const char* mmb_paged_attention_noalloc_error(void) { return g_err; }

MMB_API int mmb_paged_attention_noalloc(const void* q, const void* k_pool, const void* v_pool, const int* block_tables,
                                        const int* ctx_lens, const void* w_uv, void* out, int B, int Hq, int Hkv,
                                        int dqk, int dv, int dvo, int block_size, int max_blocks, int splits,
                                        float scale, int window, cudaStream_t stream) {
  g_err[0] = 0;
  if (!q || !k_pool || !block_tables || !ctx_lens || !out)
    return fail(MMB_NOALLOC_BAD_ARGUMENT, "q, k_pool, block_tables, ctx_lens and out must be non-null");
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || dqk <= 0 || dv <= 0 || block_size <= 0 || max_blocks <= 0 || splits <= 0)
    return fail(MMB_NOALLOC_BAD_ARGUMENT, "sizes must be positive (B %lld, Hq %lld, splits %lld)", B, Hq, splits);
  if (w_uv == nullptr && dvo != dv)
    return fail(MMB_NOALLOC_BAD_ARGUMENT, "dvo (%lld) must equal dv (%lld) without an up projection", dvo, dv);
  const long long rows = (long long)B * Hq * splits;
  if (rows > kMaxRows)
    return fail(MMB_NOALLOC_TOO_LARGE, "B * Hq * splits = %lld exceeds the scratch limit of %lld rows", rows, kMaxRows);
  if (rows * dv > kMaxPartialFloats)
    return fail(MMB_NOALLOC_TOO_LARGE, "B * Hq * splits * dv = %lld floats exceeds the scratch limit of %lld floats",
                rows * dv, kMaxPartialFloats);
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != MMB_NOALLOC_OK) return rc;
  float* part_o = scratch;
  float* part_ml = scratch + kMaxPartialFloats;
  // A (max, sum) pair with sum == 0 marks a split without keys, which the merge skips: start every pair of this
  // call from zero so that a pair no CTA writes can never carry a stale sum from an earlier call.
  cudaError_t e = cudaMemsetAsync(part_ml, 0, (size_t)rows * 2 * sizeof(float), stream);
  if (e != cudaSuccess) return fail((int)e, "cudaMemsetAsync of the pair array failed with error %lld", (long long)e);

  MmbPagedDecodeParams p{};
  p.q = q;
  p.k_pool = k_pool;
  p.v_pool = v_pool;
  p.block_tables = block_tables;
  p.ctx_lens = ctx_lens;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.B = B;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.dqk = dqk;
  p.dv = dv;
  p.block_size = block_size;
  p.max_blocks = max_blocks;
  p.splits = splits;
  p.scale = scale;
  p.window = window;
  rc = mmb_paged_decode(&p, stream);
  if (rc == (int)cudaErrorNotSupported || rc == (int)cudaErrorInvalidValue)
    return fail(MMB_NOALLOC_BAD_ARGUMENT, "unsupported head shape (dqk %lld, dv %lld, heads per KV head %lld)", dqk, dv,
                Hkv ? Hq / Hkv : 0);
  if (rc != 0) return fail(rc, "split-KV attention launch failed with error %lld", rc);
  rc = mmb_decode_merge(part_o, part_ml, w_uv, out, B, Hq, dv, dvo, splits, stream);
  if (rc == (int)cudaErrorInvalidValue) return fail(MMB_NOALLOC_BAD_ARGUMENT, "merge does not support dv = %lld", dv);
  if (rc != 0) return fail(rc, "merge launch failed with error %lld", rc);
  return MMB_NOALLOC_OK;
}
