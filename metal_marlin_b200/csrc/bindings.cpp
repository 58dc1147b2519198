// torch.ops.mmb200.* : thin argument-checking shims over the extern "C" kernel launchers.
// Every op writes into caller-provided output tensors (no allocation here), runs on the current
// CUDA stream and is therefore capturable in a CUDA graph.
#include <cstring>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include "api.h"
#include "api_gemm.h"
#include "api_ext.h"
#include "api_chain.h"
#include "api_vmm.h"

namespace {

using torch::Tensor;
using OptT = c10::optional<Tensor>;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline const void* cptr(const OptT& t) { return (t.has_value() && t->defined()) ? t->data_ptr() : nullptr; }
inline void* mptr(const OptT& t) { return (t.has_value() && t->defined()) ? t->data_ptr() : nullptr; }

inline void check(int err, const char* what) {
  TORCH_CHECK(err == 0, what, " failed: ", cudaGetErrorString((cudaError_t)err), " (", err, ")");
}
inline void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16, name, " must be a CUDA bf16 tensor");
}
inline int log2i(int64_t v) {
  int s = 0;
  while ((1LL << s) < v) ++s;
  TORCH_CHECK((1LL << s) == v, "group size must be a power of two, got ", v);
  return s;
}

// Tensor-parallel exchange descriptor: a CPU int64[9] tensor
// [in_buf, in_flags, in_slot_stride, out_peer_slots, out_peer_flags, out_counter, step, status, tp] (raw addresses).
inline void fill_tpx(const OptT& t, MmbTpExchange& x) {
  if (!t.has_value() || !t->defined()) return;
  TORCH_CHECK(!t->is_cuda() && t->scalar_type() == at::kLong && (t->numel() == 9 || t->numel() == 10), "tpx must be a CPU int64[9 | 10] tensor");
  const int64_t* v = t->data_ptr<int64_t>();
  x.in_buf = reinterpret_cast<const float*>(v[0]);
  x.in_flags = reinterpret_cast<const unsigned*>(v[1]);
  x.in_slot_stride = v[2];
  x.out_peer_slots = reinterpret_cast<float* const*>(v[3]);
  x.out_peer_flags = reinterpret_cast<unsigned* const*>(v[4]);
  x.out_counter = reinterpret_cast<unsigned*>(v[5]);
  x.step = reinterpret_cast<const unsigned*>(v[6]);
  x.status = reinterpret_cast<int*>(v[7]);
  x.tp = (int)v[8];
  if (t->numel() == 10) x.out_mc_slot = reinterpret_cast<float*>(v[9]);
}

void fp4_gemv(const Tensor& x, const Tensor& qw, const Tensor& sc, Tensor out, int64_t N, int64_t Kx, int64_t gs,
              const OptT& delta, const OptT& norm_w, const OptT& resid_out, double eps, int64_t act, const OptT& bias,
              const OptT& out_add, const OptT& tpx) {
  check_bf16(x, "x");
  check_bf16(out, "out");
  TORCH_CHECK(x.dim() == 2 && out.dim() == 2 && x.stride(1) == 1 && out.stride(1) == 1);
  TORCH_CHECK(qw.dim() == 4 && qw.is_contiguous() && sc.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  MmbFp4GemvParams p{};
  p.qw = qw.data_ptr();
  p.sc = sc.data_ptr();
  p.x = x.data_ptr();
  p.delta = cptr(delta);
  p.norm_w = cptr(norm_w);
  p.resid_out = mptr(resid_out);
  p.out = out.data_ptr();
  p.bias = cptr(bias);
  p.out_add = cptr(out_add);
  p.M = (int)x.size(0);
  p.N = (int)N;
  p.K = (int)qw.size(1) * 64;
  p.Kx = (int)Kx;
  p.ldx = (int)x.stride(0);
  p.ldo = (int)out.stride(0);
  p.gs_shift = log2i(gs);
  p.eps = (float)eps;
  p.act = (int)act;
  p.mode = 0;
  fill_tpx(tpx, p.tpx);
  TORCH_CHECK(qw.size(0) * 16 >= N && x.size(1) >= Kx);
  if (delta.has_value() && delta->defined()) TORCH_CHECK(delta->stride(0) == x.stride(0));
  check(mmb_fp4_gemv(&p, cur_stream()), "fp4_gemv");
}

// mode 1: gate-up for every (token, slot); x [T, Kx]; out [T * S, N or N/2].
// mode 2: down; x [T * S, Kx]; out [T, N].
void fp4_moe_gemv(const Tensor& x, const Tensor& qw, const Tensor& sc, Tensor out, int64_t N, int64_t Kx, int64_t gs,
                  int64_t mode, const Tensor& ids, const OptT& weights, int64_t n_shared, int64_t shared_base,
                  const OptT& norm_w, double eps, int64_t act, const OptT& out_add, const OptT& tpx) {
  check_bf16(x, "x");
  check_bf16(out, "out");
  TORCH_CHECK(qw.dim() == 5 && qw.is_contiguous() && sc.is_contiguous(), "expert bank must be [E, N/16, K/64, 32, 4]");
  TORCH_CHECK(ids.scalar_type() == at::kInt && ids.dim() == 2 && ids.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  MmbFp4GemvParams p{};
  p.qw = qw.data_ptr();
  p.sc = sc.data_ptr();
  p.x = x.data_ptr();
  p.norm_w = cptr(norm_w);
  p.out = out.data_ptr();
  p.out_add = cptr(out_add);
  p.M = (int)ids.size(0);
  p.N = (int)N;
  p.K = (int)qw.size(2) * 64;
  p.Kx = (int)Kx;
  p.ldx = (int)x.stride(0);
  p.ldo = (int)out.stride(0);
  p.gs_shift = log2i(gs);
  p.eps = (float)eps;
  p.act = (int)act;
  p.mode = (int)mode;
  p.expert_ids = ids.data_ptr<int>();
  if (weights.has_value() && weights->defined()) {
    TORCH_CHECK(weights->scalar_type() == at::kFloat && weights->is_contiguous());
    p.expert_w = weights->data_ptr<float>();
  }
  p.topk = (int)ids.size(1);
  p.n_shared = (int)n_shared;
  p.shared_base = (int)shared_base;
  fill_tpx(tpx, p.tpx);
  p.expert_stride_q = qw.stride(0) / 4;     // int32 elements -> 16-byte units
  p.expert_stride_s = sc.stride(0) / 2;     // fp16 elements -> 4-byte units
  TORCH_CHECK(mode == 1 || mode == 2);
  TORCH_CHECK(mode != 2 || p.expert_w != nullptr, "down projection needs routing weights");
  const int S = p.topk + p.n_shared;
  if (mode == 1) {
    TORCH_CHECK(x.size(0) == p.M && out.size(0) == (int64_t)p.M * S);
  } else {
    TORCH_CHECK(x.size(0) == (int64_t)p.M * S && out.size(0) == p.M);
  }
  check(mmb_fp4_gemv(&p, cur_stream()), "fp4_moe_gemv");
}

// Grouped MoE weight-streaming kernel over a device-built tile list (tiles of at most 8 sorted rows).
void fp4_grouped_gemv(const Tensor& x, const Tensor& qw, const Tensor& sc, Tensor out, int64_t N, int64_t gs, int64_t act,
                      const Tensor& tile_expert, const Tensor& tile_row0, const Tensor& tile_rows, const Tensor& n_tiles,
                      const OptT& row_order, int64_t order_div, const OptT& weights, int64_t wpt, int64_t upi) {
  check_bf16(x, "x");
  check_bf16(out, "out");
  TORCH_CHECK(qw.dim() == 5 && qw.is_contiguous() && sc.is_contiguous(), "expert bank must be [E, N/16, K/64, 32, 4]");
  TORCH_CHECK(x.stride(1) == 1 && out.stride(1) == 1);
  for (const Tensor* t : {&tile_expert, &tile_row0, &tile_rows, &n_tiles})
    TORCH_CHECK(t->scalar_type() == at::kInt && t->is_contiguous() && t->is_cuda());
  TORCH_CHECK(tile_row0.numel() == tile_expert.numel() && tile_rows.numel() == tile_expert.numel() && n_tiles.numel() == 1);
  c10::cuda::CUDAGuard guard(x.device());
  MmbFp4GemvParams p{};
  p.qw = qw.data_ptr();
  p.sc = sc.data_ptr();
  p.x = x.data_ptr();
  p.out = out.data_ptr();
  p.M = (int)out.size(0);
  p.N = (int)N;
  p.K = (int)qw.size(2) * 64;
  p.Kx = p.K;
  TORCH_CHECK(x.size(1) >= p.K, "grouped kernel needs rows of the padded width");
  p.ldx = (int)x.stride(0);
  p.ldo = (int)out.stride(0);
  p.gs_shift = log2i(gs);
  p.act = (int)act;
  p.mode = 3;
  p.expert_stride_q = qw.stride(0) / 4;
  p.expert_stride_s = sc.stride(0) / 2;
  p.tile_expert = tile_expert.data_ptr<int>();
  p.tile_row0 = tile_row0.data_ptr<int>();
  p.tile_rows = tile_rows.data_ptr<int>();
  p.n_tiles = n_tiles.data_ptr<int>();
  p.max_tiles = (int)tile_expert.numel();
  if (row_order.has_value() && row_order->defined()) {
    TORCH_CHECK(row_order->scalar_type() == at::kInt && row_order->is_contiguous() && row_order->numel() >= out.size(0));
    p.row_order = row_order->data_ptr<int>();
  }
  p.order_div = (int)order_div;
  if (weights.has_value() && weights->defined()) {
    TORCH_CHECK(weights->scalar_type() == at::kFloat && weights->is_contiguous());
    p.expert_w = weights->data_ptr<float>();
  }
  p.grouped_wpt = (int)wpt;
  p.grouped_upi = (int)upi;
  check(mmb_fp4_gemv(&p, cur_stream()), "fp4_grouped_gemv");
}

void bf16_gemv(const Tensor& x, const Tensor& w, Tensor out, const OptT& delta, const OptT& norm_w, double eps,
               const OptT& tpx) {
  check_bf16(x, "x");
  check_bf16(w, "w");
  TORCH_CHECK(w.is_contiguous() && x.stride(1) == 1 && out.stride(1) == 1);
  c10::cuda::CUDAGuard guard(x.device());
  MmbBf16GemvParams p{};
  p.w = w.data_ptr();
  p.x = x.data_ptr();
  p.delta = cptr(delta);
  p.norm_w = cptr(norm_w);
  p.out = out.data_ptr();
  p.M = (int)x.size(0);
  p.N = (int)w.size(0);
  p.K = (int)w.size(1);
  p.ldx = (int)x.stride(0);
  p.ldo = (int)out.stride(0);
  p.eps = (float)eps;
  p.out_f32 = out.scalar_type() == at::kFloat;
  fill_tpx(tpx, p.tpx);
  TORCH_CHECK(p.out_f32 || out.scalar_type() == at::kBFloat16);
  check(mmb_bf16_gemv(&p, cur_stream()), "bf16_gemv");
}

void rmsnorm(const Tensor& x, const OptT& delta, const OptT& w, Tensor out, const OptT& resid_out, double eps) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && out.stride(1) == 1);
  c10::cuda::CUDAGuard guard(x.device());
  check(mmb_rmsnorm(x.data_ptr(), cptr(delta), cptr(w), out.data_ptr(), mptr(resid_out), (int)x.size(0), (int)x.size(1),
                    (int)x.stride(0), (int)out.stride(0), (float)eps, cur_stream()),
        "rmsnorm");
}

void silu_mul(const Tensor& gate_up, Tensor out) {
  check_bf16(gate_up, "gate_up");
  TORCH_CHECK(gate_up.is_contiguous() && out.is_contiguous());
  c10::cuda::CUDAGuard guard(gate_up.device());
  check(mmb_silu_mul(gate_up.data_ptr(), out.data_ptr(), (int)gate_up.size(0), (int)gate_up.size(1) / 2, cur_stream()),
        "silu_mul");
}

void add(const Tensor& a, const Tensor& b, Tensor out) {
  check_bf16(a, "a");
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && out.is_contiguous());
  c10::cuda::CUDAGuard guard(a.device());
  check(mmb_add(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), cur_stream()), "add");
}

void embedding(const Tensor& table, const Tensor& ids, Tensor out) {
  check_bf16(table, "table");
  TORCH_CHECK(ids.scalar_type() == at::kLong && ids.is_contiguous() && table.is_contiguous() && out.is_contiguous());
  c10::cuda::CUDAGuard guard(table.device());
  check(mmb_embedding(table.data_ptr(), ids.data_ptr<int64_t>(), out.data_ptr(), (int)ids.numel(), (int)table.size(1),
                      cur_stream()),
        "embedding");
}

void rope(Tensor q, const OptT& k, const Tensor& positions, const Tensor& inv_freq, int64_t Hq, int64_t Hk, int64_t D,
          int64_t rot_dim, bool interleaved, double mscale) {
  check_bf16(q, "q");
  TORCH_CHECK(positions.scalar_type() == at::kInt && inv_freq.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(q.device());
  const int T = (int)positions.numel();
  check(mmb_rope(q.data_ptr(), mptr(k), positions.data_ptr<int>(), inv_freq.data_ptr<float>(), T, (int)Hq, (int)Hk, (int)D,
                 (int)rot_dim, (int)q.stride(0), k.has_value() && k->defined() ? (int)k->stride(0) : 0, interleaved ? 1 : 0,
                 (float)mscale, cur_stream()),
        "rope");
}

void qk_norm_rope_cache(Tensor q, const Tensor& k, const Tensor& v, const OptT& qn_w, const OptT& kn_w,
                        const Tensor& positions, const Tensor& inv_freq, const Tensor& slots, Tensor k_pool, Tensor v_pool,
                        int64_t Hq, int64_t Hk, int64_t D, double eps, bool interleaved) {
  check_bf16(q, "q");
  TORCH_CHECK(q.stride(0) == k.stride(0) && q.stride(0) == v.stride(0));
  TORCH_CHECK(positions.scalar_type() == at::kInt && slots.scalar_type() == at::kLong);
  c10::cuda::CUDAGuard guard(q.device());
  check(mmb_qk_norm_rope_cache(q.data_ptr(), k.data_ptr(), v.data_ptr(), cptr(qn_w), cptr(kn_w), positions.data_ptr<int>(),
                               inv_freq.data_ptr<float>(), slots.data_ptr<int64_t>(), k_pool.data_ptr(), v_pool.data_ptr(),
                               (int)positions.numel(), (int)Hq, (int)Hk, (int)D, (int)q.stride(0), (float)eps,
                               interleaved ? 1 : 0, cur_stream()),
        "qk_norm_rope_cache");
}

void qk_norm_rope_cache_fp8(Tensor q, const Tensor& k, const Tensor& v, const OptT& qn_w, const OptT& kn_w, const Tensor& positions,
                            const Tensor& inv_freq, const Tensor& slots, Tensor k_pool, Tensor v_pool, Tensor k_scale, Tensor v_scale,
                            int64_t Hq, int64_t Hk, int64_t D, double eps, bool interleaved, int64_t kv_fmt) {
  check_bf16(q, "q");
  TORCH_CHECK(q.stride(0) == k.stride(0) && q.stride(0) == v.stride(0));
  TORCH_CHECK(positions.scalar_type() == at::kInt && slots.scalar_type() == at::kLong);
  TORCH_CHECK(k_pool.size(-1) == (kv_fmt >= 2 ? D / 2 : D) && v_pool.size(-1) == k_pool.size(-1), "quantized KV pool row width does not match the format");
  TORCH_CHECK(k_pool.scalar_type() == at::kByte && v_pool.scalar_type() == at::kByte && k_scale.scalar_type() == at::kFloat &&
              v_scale.scalar_type() == at::kFloat && k_pool.is_contiguous() && v_pool.is_contiguous());
  c10::cuda::CUDAGuard guard(q.device());
  check(mmb_qk_norm_rope_cache_fp8(q.data_ptr(), k.data_ptr(), v.data_ptr(), cptr(qn_w), cptr(kn_w), positions.data_ptr<int>(),
                                   inv_freq.data_ptr<float>(), slots.data_ptr<int64_t>(), k_pool.data_ptr(), v_pool.data_ptr(),
                                   k_scale.data_ptr<float>(), v_scale.data_ptr<float>(), (int)positions.numel(), (int)Hq, (int)Hk, (int)D,
                                   (int)q.stride(0), (float)eps, interleaved ? 1 : 0, (int)kv_fmt, cur_stream()),
        "qk_norm_rope_cache_fp8");
}

// pool uint8 [num_slots, Hkv, D] + scale fp32 [num_slots, Hkv] -> out bf16 [sum ctx, Hkv, D] (rows cu_k[b] .. of sequence b)
void kv_fp8_gather(const Tensor& pool, const Tensor& scale, const Tensor& block_tables, const Tensor& ctx_lens, const Tensor& cu_k, Tensor out,
                   int64_t Hkv, int64_t D, int64_t block_size, int64_t max_ctx, int64_t kv_fmt) {
  check_bf16(out, "out");
  TORCH_CHECK(pool.size(-1) == (kv_fmt >= 2 ? D / 2 : D), "quantized KV pool row width does not match the format");
  TORCH_CHECK(pool.scalar_type() == at::kByte && pool.is_contiguous() && scale.scalar_type() == at::kFloat && out.is_contiguous());
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && block_tables.dim() == 2 && block_tables.is_contiguous() &&
              ctx_lens.scalar_type() == at::kInt && cu_k.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard guard(pool.device());
  check(mmb_kv_fp8_gather(pool.data_ptr(), scale.data_ptr<float>(), block_tables.data_ptr<int>(), ctx_lens.data_ptr<int>(),
                          cu_k.data_ptr<int>(), out.data_ptr(), (int)ctx_lens.numel(), (int)Hkv, (int)D, (int)block_size,
                          (int)block_tables.size(1), (int)max_ctx, (int)kv_fmt, cur_stream()),
        "kv_fp8_gather");
}

void mla_prep_impl(const Tensor& q, const Tensor& kva, const Tensor& w_ukT, const Tensor& kv_norm_w, const Tensor& positions,
                   const Tensor& inv_freq, const Tensor& slots, Tensor q_full, Tensor cache, int64_t H, int64_t dn, int64_t dr,
                   int64_t R, double eps, double mscale, bool interleaved, bool skip_absorb, Tensor* cache_scale, int64_t cache_fmt = 0);
void mla_prep(const Tensor& q, const Tensor& kva, const Tensor& w_ukT, const Tensor& kv_norm_w, const Tensor& positions,
              const Tensor& inv_freq, const Tensor& slots, Tensor q_full, Tensor cache, int64_t H, int64_t dn, int64_t dr,
              int64_t R, double eps, double mscale, bool interleaved, bool skip_absorb) {
  TORCH_CHECK(cache.scalar_type() == at::kBFloat16);
  mla_prep_impl(q, kva, w_ukT, kv_norm_w, positions, inv_freq, slots, q_full, cache, H, dn, dr, R, eps, mscale, interleaved, skip_absorb,
                nullptr);
}
// Quantized latent cache: `cache` uint8 [num_slots, R + dr] (8-bit formats) or [num_slots, (R + dr) / 2] (4-bit), `cache_scale`
// fp32 [num_slots]; `cache_fmt` as in kv_quant.cuh.
void mla_prep_fp8(const Tensor& q, const Tensor& kva, const Tensor& w_ukT, const Tensor& kv_norm_w, const Tensor& positions,
                  const Tensor& inv_freq, const Tensor& slots, Tensor q_full, Tensor cache, Tensor cache_scale, int64_t H, int64_t dn,
                  int64_t dr, int64_t R, double eps, double mscale, bool interleaved, bool skip_absorb, int64_t cache_fmt) {
  TORCH_CHECK(cache.scalar_type() == at::kByte && cache_scale.scalar_type() == at::kFloat && cache_scale.is_contiguous() &&
              cache_scale.numel() == cache.size(0) && cache_fmt >= 0 && cache_fmt <= 3);
  TORCH_CHECK(cache.size(-1) == (cache_fmt >= 2 ? (R + dr) / 2 : R + dr), "quantized latent cache row width does not match the format");
  mla_prep_impl(q, kva, w_ukT, kv_norm_w, positions, inv_freq, slots, q_full, cache, H, dn, dr, R, eps, mscale, interleaved, skip_absorb,
                &cache_scale, cache_fmt);
}
void mla_prep_impl(const Tensor& q, const Tensor& kva, const Tensor& w_ukT, const Tensor& kv_norm_w, const Tensor& positions,
                   const Tensor& inv_freq, const Tensor& slots, Tensor q_full, Tensor cache, int64_t H, int64_t dn, int64_t dr,
                   int64_t R, double eps, double mscale, bool interleaved, bool skip_absorb, Tensor* cache_scale, int64_t cache_fmt) {
  check_bf16(q, "q");
  check_bf16(kva, "kva");
  check_bf16(w_ukT, "w_ukT");
  TORCH_CHECK(w_ukT.is_contiguous() && q_full.is_contiguous() && cache.is_contiguous());
  TORCH_CHECK(positions.scalar_type() == at::kInt && slots.scalar_type() == at::kLong);
  c10::cuda::CUDAGuard guard(q.device());
  MmbMlaPrepParams p{};
  p.q = q.data_ptr();
  p.kva = kva.data_ptr();
  p.w_ukT = w_ukT.data_ptr();
  p.kv_norm_w = kv_norm_w.data_ptr();
  p.positions = positions.data_ptr<int>();
  p.inv_freq = inv_freq.data_ptr<float>();
  p.slots = slots.data_ptr<int64_t>();
  p.q_full = q_full.data_ptr();
  p.cache = cache.data_ptr();
  p.T = (int)positions.numel();
  p.H = (int)H;
  p.dn = (int)dn;
  p.dr = (int)dr;
  p.R = (int)R;
  p.ld_q = (int)q.stride(0);
  p.ld_kva = (int)kva.stride(0);
  p.eps = (float)eps;
  p.mscale = (float)mscale;
  p.interleaved = interleaved ? 1 : 0;
  p.skip_absorb = skip_absorb ? 1 : 0;
  p.cache_scale = cache_scale ? cache_scale->data_ptr<float>() : nullptr;
  p.cache_fmt = (int)cache_fmt;
  check(mmb_mla_prep(&p, cur_stream()), "mla_prep");
}

// Per-device status word for kernels whose op signature carries none (registered once per device from Python).
int* g_status_word[64] = {nullptr};
void set_status_word(Tensor status) {
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1);
  const int d = status.device().index();
  TORCH_CHECK(d >= 0 && d < 64);
  g_status_word[d] = status.data_ptr<int>();
}
inline int* status_word_of(const Tensor& t) {
  const int d = t.device().index();
  return (d >= 0 && d < 64) ? g_status_word[d] : nullptr;
}

void paged_decode_impl(const Tensor& q, const Tensor& k_pool, const OptT& v_pool, const Tensor& block_tables, const Tensor& ctx_lens,
                       Tensor part_o, Tensor part_ml, int64_t Hq, int64_t Hkv, int64_t dqk, int64_t dv, int64_t block_size, int64_t splits,
                       double scale, int64_t window, const Tensor* k_scale, const OptT* v_scale, int64_t kv_fmt = 0);
void paged_decode(const Tensor& q, const Tensor& k_pool, const OptT& v_pool, const Tensor& block_tables,
                  const Tensor& ctx_lens, Tensor part_o, Tensor part_ml, int64_t Hq, int64_t Hkv, int64_t dqk, int64_t dv,
                  int64_t block_size, int64_t splits, double scale, int64_t window) {
  check_bf16(k_pool, "k_pool");
  paged_decode_impl(q, k_pool, v_pool, block_tables, ctx_lens, part_o, part_ml, Hq, Hkv, dqk, dv, block_size, splits, scale, window, nullptr,
                    nullptr);
}
// FP8 pools: uint8 (E4M3) K / V pools with fp32 scales [num_slots, Hkv].
void paged_decode_fp8(const Tensor& q, const Tensor& k_pool, const OptT& v_pool, const Tensor& k_scale, const OptT& v_scale,
                      const Tensor& block_tables, const Tensor& ctx_lens, Tensor part_o, Tensor part_ml, int64_t Hq, int64_t Hkv, int64_t dqk,
                      int64_t dv, int64_t block_size, int64_t splits, double scale, int64_t window, int64_t kv_fmt) {
  TORCH_CHECK(k_pool.scalar_type() == at::kByte && k_scale.scalar_type() == at::kFloat && k_scale.is_contiguous());
  TORCH_CHECK(kv_fmt >= 0 && kv_fmt <= 3 && dqk % (kv_fmt >= 2 ? 32 : 16) == 0 && dv % (kv_fmt >= 2 ? 32 : 16) == 0,
              "quantized rows are copied in 16-byte pieces");
  TORCH_CHECK(k_pool.size(-1) == (kv_fmt >= 2 ? dqk / 2 : dqk), "quantized KV pool row width does not match the format");
  if (v_pool.has_value() && v_pool->defined())
    TORCH_CHECK(v_pool->scalar_type() == at::kByte && v_scale.has_value() && v_scale->defined() && v_scale->scalar_type() == at::kFloat);
  paged_decode_impl(q, k_pool, v_pool, block_tables, ctx_lens, part_o, part_ml, Hq, Hkv, dqk, dv, block_size, splits, scale, window, &k_scale,
                    &v_scale, kv_fmt);
}
void paged_decode_impl(const Tensor& q, const Tensor& k_pool, const OptT& v_pool, const Tensor& block_tables, const Tensor& ctx_lens,
                       Tensor part_o, Tensor part_ml, int64_t Hq, int64_t Hkv, int64_t dqk, int64_t dv, int64_t block_size, int64_t splits,
                       double scale, int64_t window, const Tensor* k_scale, const OptT* v_scale, int64_t kv_fmt) {
  check_bf16(q, "q");
  TORCH_CHECK(q.is_contiguous() && k_pool.is_contiguous() && block_tables.is_contiguous() && block_tables.dim() == 2);
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && ctx_lens.scalar_type() == at::kInt);
  TORCH_CHECK(part_o.scalar_type() == at::kFloat && part_ml.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(q.device());
  MmbPagedDecodeParams p{};
  p.q = q.data_ptr();
  p.k_pool = k_pool.data_ptr();
  p.v_pool = cptr(v_pool);
  p.block_tables = block_tables.data_ptr<int>();
  p.ctx_lens = ctx_lens.data_ptr<int>();
  p.part_o = part_o.data_ptr<float>();
  p.part_ml = part_ml.data_ptr<float>();
  p.B = (int)ctx_lens.numel();
  p.Hq = (int)Hq;
  p.Hkv = (int)Hkv;
  p.dqk = (int)dqk;
  p.dv = (int)dv;
  p.block_size = (int)block_size;
  p.max_blocks = (int)block_tables.size(1);
  p.splits = (int)splits;
  p.scale = (float)scale;
  p.window = (int)window;
  if (k_scale != nullptr) {
    p.k_scale = k_scale->data_ptr<float>();
    p.kv_fmt = (int)kv_fmt;
    if (v_scale != nullptr && v_scale->has_value() && (*v_scale)->defined()) p.v_scale = (*v_scale)->data_ptr<float>();
  }
  TORCH_CHECK(part_o.numel() >= (int64_t)p.B * Hq * splits * dv && part_ml.numel() >= (int64_t)p.B * Hq * splits * 2);
  p.status = status_word_of(q);
  check(mmb_paged_decode(&p, cur_stream()), "paged_decode");
}

// Decode chain (decode_chain.cu).  `desc` is a CPU byte tensor holding an MmbChainParams exactly as the C ABI lays it out
// (the Python side builds it with a ctypes mirror of the struct); all pointers in it are device addresses of tensors the
// caller keeps alive.
void decode_chain(const Tensor& desc, const Tensor& anchor) {
  TORCH_CHECK(!desc.is_cuda() && desc.scalar_type() == at::kByte && desc.is_contiguous() &&
                  desc.numel() == (int64_t)sizeof(MmbChainParams),
              "decode_chain: descriptor has ", desc.numel(), " bytes, the library expects ", sizeof(MmbChainParams));
  TORCH_CHECK(anchor.is_cuda());
  c10::cuda::CUDAGuard guard(anchor.device());
  MmbChainParams p;
  std::memcpy(&p, desc.data_ptr(), sizeof(p));
  check(mmb_decode_chain(&p, cur_stream()), "decode_chain");
}
int64_t decode_chain_param_bytes() { return (int64_t)sizeof(MmbChainParams); }

void decode_merge(const Tensor& part_o, const Tensor& part_ml, const OptT& w_uv, Tensor out, int64_t B, int64_t Hq,
                  int64_t dv, int64_t dvo, int64_t splits) {
  c10::cuda::CUDAGuard guard(part_o.device());
  check(mmb_decode_merge(part_o.data_ptr<float>(), part_ml.data_ptr<float>(), cptr(w_uv), out.data_ptr(), (int)B, (int)Hq,
                         (int)dv, (int)dvo, (int)splits, cur_stream()),
        "decode_merge");
}

void moe_router(const Tensor& x, const Tensor& w, const OptT& delta, const OptT& norm_w, const OptT& resid_out,
                const OptT& bias, Tensor ids, Tensor weights, const OptT& logits_out, const OptT& counts, int64_t topk,
                double eps, int64_t scoring, bool renorm, double routed_scale, int64_t n_group, int64_t topk_group,
                const OptT& tpx) {
  check_bf16(x, "x");
  check_bf16(w, "w");
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous() && ids.is_contiguous() && weights.is_contiguous());
  TORCH_CHECK(ids.scalar_type() == at::kInt && weights.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(x.device());
  MmbRouterParams p{};
  p.w = w.data_ptr();
  p.x = x.data_ptr();
  p.delta = cptr(delta);
  p.norm_w = cptr(norm_w);
  p.resid_out = mptr(resid_out);
  p.bias = (bias.has_value() && bias->defined()) ? bias->data_ptr<float>() : nullptr;
  p.ids = ids.data_ptr<int>();
  p.weights = weights.data_ptr<float>();
  p.logits_out = (logits_out.has_value() && logits_out->defined()) ? logits_out->data_ptr<float>() : nullptr;
  p.counts = (counts.has_value() && counts->defined()) ? counts->data_ptr<int>() : nullptr;
  p.T = (int)x.size(0);
  p.E = (int)w.size(0);
  p.K = (int)w.size(1);
  p.topk = (int)topk;
  p.eps = (float)eps;
  p.scoring = (int)scoring;
  p.renorm = renorm ? 1 : 0;
  p.routed_scale = (float)routed_scale;
  p.n_group = (int)n_group;
  p.topk_group = (int)topk_group;
  fill_tpx(tpx, p.tpx);
  check(mmb_moe_router(&p, cur_stream()), "moe_router");
}

void moe_select(const Tensor& logits, const OptT& bias, Tensor ids, Tensor weights, const OptT& counts, int64_t topk, int64_t scoring,
                bool renorm, double routed_scale, int64_t n_group, int64_t topk_group) {
  TORCH_CHECK(logits.scalar_type() == at::kFloat && logits.is_contiguous() && logits.dim() == 2);
  TORCH_CHECK(ids.scalar_type() == at::kInt && weights.scalar_type() == at::kFloat && ids.is_contiguous() && weights.is_contiguous());
  c10::cuda::CUDAGuard guard(logits.device());
  MmbRouterParams p{};
  p.bias = (bias.has_value() && bias->defined()) ? bias->data_ptr<float>() : nullptr;
  p.ids = ids.data_ptr<int>();
  p.weights = weights.data_ptr<float>();
  p.counts = (counts.has_value() && counts->defined()) ? counts->data_ptr<int>() : nullptr;
  p.T = (int)logits.size(0);
  p.E = (int)logits.size(1);
  p.topk = (int)topk;
  p.scoring = (int)scoring;
  p.renorm = renorm ? 1 : 0;
  p.routed_scale = (float)routed_scale;
  p.n_group = (int)n_group;
  p.topk_group = (int)topk_group;
  check(mmb_moe_select(&p, logits.data_ptr<float>(), cur_stream()), "moe_select");
}

void sample(const Tensor& logits, Tensor out_ids, const OptT& out_logprob, const OptT& temperature, const OptT& top_k,
            const OptT& top_p, const OptT& min_p, const OptT& history, const OptT& rep_penalty, int64_t seed,
            int64_t offset, const OptT& offset_dev, const OptT& seed_dev) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.is_contiguous() && logits.dim() == 2);
  TORCH_CHECK(out_ids.scalar_type() == at::kLong);
  c10::cuda::CUDAGuard guard(logits.device());
  MmbSampleParams p{};
  p.logits = logits.data_ptr<float>();
  p.out_ids = out_ids.data_ptr<int64_t>();
  auto fp = [](const OptT& t) -> const float* { return (t.has_value() && t->defined()) ? t->data_ptr<float>() : nullptr; };
  p.out_logprob = (out_logprob.has_value() && out_logprob->defined()) ? out_logprob->data_ptr<float>() : nullptr;
  p.temperature = fp(temperature);
  p.top_k = (top_k.has_value() && top_k->defined()) ? top_k->data_ptr<int>() : nullptr;
  p.top_p = fp(top_p);
  p.min_p = fp(min_p);
  p.rep_penalty = fp(rep_penalty);
  if (history.has_value() && history->defined()) {
    TORCH_CHECK(history->scalar_type() == at::kLong && history->is_contiguous() && history->dim() == 2);
    p.history = history->data_ptr<int64_t>();
    p.hist_len = (int)history->size(1);
  }
  p.B = (int)logits.size(0);
  p.V = (int)logits.size(1);
  p.seed = (unsigned long long)seed;
  p.offset = (unsigned long long)offset;
  if (offset_dev.has_value() && offset_dev->defined()) {
    TORCH_CHECK(offset_dev->scalar_type() == at::kLong);
    p.offset_dev = offset_dev->data_ptr<int64_t>();
  }
  if (seed_dev.has_value() && seed_dev->defined()) {
    TORCH_CHECK(seed_dev->scalar_type() == at::kLong && seed_dev->numel() >= logits.size(0));
    p.seed_dev = seed_dev->data_ptr<int64_t>();
  }
  check(mmb_sample(&p, cur_stream()), "sample");
}

void argmax(const Tensor& logits, Tensor out) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.is_contiguous() && logits.dim() == 2);
  c10::cuda::CUDAGuard guard(logits.device());
  check(mmb_argmax(logits.data_ptr<float>(), out.data_ptr<int64_t>(), (int)logits.size(0), (int)logits.size(1), cur_stream()),
        "argmax");
}

void tp_argmax(const Tensor& logits, Tensor out, int64_t vocab_offset, const Tensor& tpx) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.is_contiguous() && logits.dim() == 2);
  c10::cuda::CUDAGuard guard(logits.device());
  MmbTpExchange x{};
  fill_tpx(tpx, x);
  check(mmb_tp_argmax(logits.data_ptr<float>(), out.data_ptr<int64_t>(), (int)logits.size(0), (int)logits.size(1),
                      (int)vocab_offset, &x, cur_stream()),
        "tp_argmax");
}

// ---- tcgen05 GEMM (prefill / large M)
// ag: CPU int64[5] = flags, step, tp, rank, rows per rank (all-gather fused into the load of x)
MmbAgWait ag_from(const Tensor& ag) {
  TORCH_CHECK(!ag.is_cuda() && ag.scalar_type() == at::kLong && ag.numel() == 5, "ag must be a CPU int64[5] tensor");
  const int64_t* v = ag.data_ptr<int64_t>();
  MmbAgWait a{};
  a.flags = reinterpret_cast<const unsigned*>(v[0]);
  a.step = reinterpret_cast<const unsigned*>(v[1]);
  a.tp = (int)v[2];
  a.rank = (int)v[3];
  a.rows = (int)v[4];
  TORCH_CHECK(a.tp >= 1 && a.rows > 0 && a.rank >= 0 && a.rank < a.tp);
  return a;
}

void fp4_gemm_impl(const Tensor& x, const Tensor& qw, const Tensor& sc, Tensor out, int64_t N, int64_t gs, Tensor status, const Tensor* ag,
                   int act = 0);
void fp4_gemm(const Tensor& x, const Tensor& qw, const Tensor& sc, Tensor out, int64_t N, int64_t gs, Tensor status) {
  fp4_gemm_impl(x, qw, sc, out, N, gs, status, nullptr);
}
void fp4_gemm_ag(const Tensor& x, const Tensor& qw, const Tensor& sc, Tensor out, int64_t N, int64_t gs, Tensor status, const Tensor& ag) {
  fp4_gemm_impl(x, qw, sc, out, N, gs, status, &ag);
}
// SwiGLU fused into the epilogue: W holds gate rows [0, N/2) and up rows [N/2, N); out is [M, N/2].
void fp4_gemm_swiglu(const Tensor& x, const Tensor& qw, const Tensor& sc, Tensor out, int64_t N, int64_t gs, Tensor status) {
  TORCH_CHECK(N % 128 == 0 && out.size(1) == N / 2, "fused SwiGLU needs N / 2 to be a multiple of 64 and out [M, N / 2]");
  fp4_gemm_impl(x, qw, sc, out, N, gs, status, nullptr, 1);
}
void fp4_gemm_impl(const Tensor& x, const Tensor& qw, const Tensor& sc, Tensor out, int64_t N, int64_t gs, Tensor status, const Tensor* ag,
                   int act) {
  check_bf16(x, "x");
  check_bf16(out, "out");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && out.is_contiguous() && qw.is_contiguous() && sc.is_contiguous());
  TORCH_CHECK(status.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard guard(x.device());
  MmbFp4GemmParams p{};
  p.x = x.data_ptr();
  p.qw = qw.data_ptr();
  p.sc = sc.data_ptr();
  p.out = out.data_ptr();
  p.M = (int)x.size(0);
  p.N = (int)N;
  p.K = (int)qw.size(1) * 64;
  p.Kx = (int)x.size(1);
  p.ldo = (int)out.stride(0);
  p.gs_shift = log2i(gs);
  p.status = status.data_ptr<int>();
  if (ag != nullptr) p.ag = ag_from(*ag);
  p.act = act;
  check(mmb_fp4_gemm(&p, cur_stream()), "fp4_gemm");
}

// Row-parallel projection with the reduce-scatter epilogue: `rs` is a CPU int64[7] descriptor
// (peer buffer table, peer flag table, counter, step, tp, rank, rows per rank); nothing is written locally.
void fp4_gemm_rs(const Tensor& x, const Tensor& qw, const Tensor& sc, int64_t N, int64_t gs, Tensor status, const Tensor& rs) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && qw.is_contiguous() && sc.is_contiguous());
  TORCH_CHECK(!rs.is_cuda() && rs.scalar_type() == at::kLong && rs.numel() == 7, "rs must be a CPU int64[7] tensor");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t* v = rs.data_ptr<int64_t>();
  MmbFp4GemmParams p{};
  p.x = x.data_ptr();
  p.qw = qw.data_ptr();
  p.sc = sc.data_ptr();
  p.out = nullptr;
  p.M = (int)x.size(0);
  p.N = (int)N;
  p.K = (int)qw.size(1) * 64;
  p.Kx = (int)x.size(1);
  p.ldo = (int)N;
  p.gs_shift = log2i(gs);
  p.status = status.data_ptr<int>();
  p.rs_peer_bufs = reinterpret_cast<float* const*>(v[0]);
  p.rs_peer_flags = reinterpret_cast<unsigned* const*>(v[1]);
  p.rs_counter = reinterpret_cast<unsigned*>(v[2]);
  p.rs_step = reinterpret_cast<const unsigned*>(v[3]);
  p.rs_tp = (int)v[4];
  p.rs_rank = (int)v[5];
  p.rs_rows = (int)v[6];
  TORCH_CHECK(p.rs_rows > 0 && (int64_t)p.rs_rows * p.rs_tp >= p.M);
  check(mmb_fp4_gemm(&p, cur_stream()), "fp4_gemm_rs");
}

// desc: CPU int64[12] = in_buf, in_flags, ag_peer_bufs, ag_peer_flags, counter, step, status, tp, rank, rows, N, M;
// with resid / norm_w the owned rows get the residual add and the RMSNorm, and the normalized rows go to the
// second gathered buffer (ag2: device address of the peer table).
void tp_rs_finish_impl(const Tensor& desc, const OptT& resid, const OptT& norm_w, int64_t ag2, double eps);
void tp_rs_finish(const Tensor& desc) { tp_rs_finish_impl(desc, c10::nullopt, c10::nullopt, 0, 0.0); }
void tp_rs_finish_norm(const Tensor& desc, const OptT& resid, const Tensor& norm_w, int64_t ag2, double eps) {
  tp_rs_finish_impl(desc, resid, norm_w, ag2, eps);
}
void tp_rs_finish_impl(const Tensor& desc, const OptT& resid, const OptT& norm_w, int64_t ag2, double eps) {
  TORCH_CHECK(!desc.is_cuda() && desc.scalar_type() == at::kLong && desc.numel() == 12);
  const int64_t* v = desc.data_ptr<int64_t>();
  MmbRsFinishParams p{};
  p.in_buf = reinterpret_cast<const float*>(v[0]);
  p.in_flags = reinterpret_cast<const unsigned*>(v[1]);
  p.ag_peer_bufs = reinterpret_cast<void* const*>(v[2]);
  p.ag_peer_flags = reinterpret_cast<unsigned* const*>(v[3]);
  p.counter = reinterpret_cast<unsigned*>(v[4]);
  p.step = reinterpret_cast<const unsigned*>(v[5]);
  p.status = reinterpret_cast<int*>(v[6]);
  p.tp = (int)v[7];
  p.rank = (int)v[8];
  p.rows = (int)v[9];
  p.N = (int)v[10];
  p.M = (int)v[11];
  if (resid.has_value() && resid->defined()) {
    check_bf16(*resid, "resid");
    TORCH_CHECK(resid->is_contiguous() && resid->dim() == 2 && resid->size(0) >= p.M && resid->size(1) == p.N);
    p.resid = resid->data_ptr();
  }
  if (norm_w.has_value() && norm_w->defined()) {
    check_bf16(*norm_w, "norm_w");
    TORCH_CHECK(norm_w->is_contiguous() && norm_w->numel() == p.N && ag2 != 0);
    p.norm_w = norm_w->data_ptr();
    p.ag2_peer_bufs = reinterpret_cast<void* const*>(ag2);
    p.eps = (float)eps;
  }
  check(mmb_tp_rs_finish(&p, cur_stream()), "tp_rs_finish");
}

// desc: CPU int64[4] = flags, step, status, tp
void tp_wait(const Tensor& desc) {
  TORCH_CHECK(!desc.is_cuda() && desc.scalar_type() == at::kLong && desc.numel() == 4);
  const int64_t* v = desc.data_ptr<int64_t>();
  check(mmb_tp_wait(reinterpret_cast<const unsigned*>(v[0]), reinterpret_cast<const unsigned*>(v[1]), reinterpret_cast<int*>(v[2]), (int)v[3],
                    cur_stream()),
        "tp_wait");
}

// Grouped (MoE) GEMM: x rows are sorted by expert; the tile list lives on the device.
static void fp4_gemm_grouped_impl(const Tensor& x, const Tensor& qw, const Tensor& sc, Tensor out, int64_t N, int64_t gs,
                                  const Tensor& tile_expert, const Tensor& tile_row0, const Tensor& tile_rows, const Tensor& n_tiles,
                                  int64_t token_tile, const OptT& row_scale, Tensor status, const Tensor* out_rows, int act = 0);
// Grouped GEMM with SwiGLU in the epilogue (gate | up row halves of every expert): out [rows, N / 2].
void fp4_gemm_grouped_swiglu(const Tensor& x, const Tensor& qw, const Tensor& sc, Tensor out, int64_t N, int64_t gs,
                             const Tensor& tile_expert, const Tensor& tile_row0, const Tensor& tile_rows, const Tensor& n_tiles,
                             int64_t token_tile, Tensor status) {
  TORCH_CHECK(N % 128 == 0 && out.size(1) == N / 2, "fused SwiGLU needs N / 2 to be a multiple of 64 and out [rows, N / 2]");
  fp4_gemm_grouped_impl(x, qw, sc, out, N, gs, tile_expert, tile_row0, tile_rows, n_tiles, token_tile, c10::nullopt, status, nullptr, 1);
}
void fp4_gemm_grouped(const Tensor& x, const Tensor& qw, const Tensor& sc, Tensor out, int64_t N, int64_t gs,
                      const Tensor& tile_expert, const Tensor& tile_row0, const Tensor& tile_rows, const Tensor& n_tiles,
                      int64_t token_tile, const OptT& row_scale, Tensor status) {
  fp4_gemm_grouped_impl(x, qw, sc, out, N, gs, tile_expert, tile_row0, tile_rows, n_tiles, token_tile, row_scale, status, nullptr);
}
// Same GEMM with the scatter epilogue: row r of the result goes to the address out_rows[r] (int64 [M] on the device, 0 = skip;
// the addresses may be peer memory).  `out` only supplies the row width.
void fp4_gemm_grouped_scatter(const Tensor& x, const Tensor& qw, const Tensor& sc, Tensor out, int64_t N, int64_t gs,
                              const Tensor& tile_expert, const Tensor& tile_row0, const Tensor& tile_rows, const Tensor& n_tiles,
                              int64_t token_tile, Tensor status, const Tensor& out_rows) {
  TORCH_CHECK(out_rows.is_cuda() && out_rows.scalar_type() == at::kLong && out_rows.is_contiguous() && out_rows.numel() >= x.size(0));
  fp4_gemm_grouped_impl(x, qw, sc, out, N, gs, tile_expert, tile_row0, tile_rows, n_tiles, token_tile, c10::nullopt, status, &out_rows);
}
static void fp4_gemm_grouped_impl(const Tensor& x, const Tensor& qw, const Tensor& sc, Tensor out, int64_t N, int64_t gs,
                                  const Tensor& tile_expert, const Tensor& tile_row0, const Tensor& tile_rows, const Tensor& n_tiles,
                                  int64_t token_tile, const OptT& row_scale, Tensor status, const Tensor* out_rows, int act) {
  check_bf16(x, "x");
  check_bf16(out, "out");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && out.is_contiguous() && qw.dim() == 5 && qw.is_contiguous() &&
              sc.is_contiguous());
  TORCH_CHECK(tile_expert.scalar_type() == at::kInt && tile_row0.scalar_type() == at::kInt &&
              tile_rows.scalar_type() == at::kInt && n_tiles.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard guard(x.device());
  MmbFp4GemmParams p{};
  p.x = x.data_ptr();
  p.qw = qw.data_ptr();
  p.sc = sc.data_ptr();
  p.out = out.data_ptr();
  p.M = (int)x.size(0);
  p.N = (int)N;
  p.K = (int)qw.size(2) * 64;
  p.Kx = (int)x.size(1);
  p.ldo = (int)out.stride(0);
  p.gs_shift = log2i(gs);
  p.status = status.data_ptr<int>();
  p.tile_expert = tile_expert.data_ptr<int>();
  p.tile_row0 = tile_row0.data_ptr<int>();
  p.tile_rows = tile_rows.data_ptr<int>();
  p.n_tiles = n_tiles.data_ptr<int>();
  p.max_tiles = (int)tile_expert.numel();
  p.expert_stride_q = qw.stride(0) / 4;
  p.expert_stride_s = sc.stride(0) / 2;
  p.token_tile = (int)token_tile;
  if (row_scale.has_value() && row_scale->defined()) {
    TORCH_CHECK(row_scale->scalar_type() == at::kFloat && row_scale->is_contiguous());
    p.row_scale = row_scale->data_ptr<float>();
  }
  if (out_rows != nullptr) p.out_rows = reinterpret_cast<const long long*>(out_rows->data_ptr<int64_t>());
  p.act = act;
  check(mmb_fp4_gemm(&p, cur_stream()), "fp4_gemm_grouped");
}

// Trellis weights on the tensor cores (codes decoded inside the GEMM's main loop).  `desc` int64 [n_mats, 6] on the device:
// codes, scales, su, sv, out | in << 32, bits | group << 32 per matrix.  Dense: n_mats = 1 (or 2 with act = 1: gate, up).
// Grouped: matrices [expert * stride + first (+ 1 for the up half)], rows of x sorted by expert, tile list on the device.
void trellis_gemm(const Tensor& x, const Tensor& desc, Tensor out, int64_t N, int64_t K, int64_t act, int64_t first, int64_t stride,
                  const OptT& tile_expert, const OptT& tile_row0, const OptT& tile_rows, const OptT& n_tiles, int64_t token_tile,
                  const OptT& row_scale, const OptT& out_rows, Tensor status) {
  check_bf16(x, "x");
  check_bf16(out, "out");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && out.is_contiguous() && desc.is_cuda() && desc.scalar_type() == at::kLong &&
              desc.is_contiguous() && desc.dim() == 2 && desc.size(1) == 6);
  TORCH_CHECK(K % 64 == 0 && x.size(1) == K, "trellis_gemm: the input width must equal K and be a multiple of 64");
  TORCH_CHECK(act == 0 ? out.size(1) == N : (N % 128 == 0 && out.size(1) == N / 2));
  c10::cuda::CUDAGuard guard(x.device());
  MmbFp4GemmParams p{};
  if (out_rows.has_value() && out_rows->defined()) {
    // scatter epilogue: row r of the result goes to the address out_rows[r] (possibly peer memory); `out` gives the width
    TORCH_CHECK(out_rows->is_cuda() && out_rows->scalar_type() == at::kLong && out_rows->is_contiguous() && out_rows->numel() >= x.size(0) &&
                act == 0);
    p.out_rows = reinterpret_cast<const long long*>(out_rows->data_ptr<int64_t>());
  }
  p.x = x.data_ptr();
  p.out = out.data_ptr();
  p.M = (int)x.size(0);
  p.N = (int)N;
  p.K = (int)K;
  p.Kx = (int)K;
  p.ldo = (int)out.stride(0);
  p.status = status.data_ptr<int>();
  p.act = (int)act;
  p.tr_desc = reinterpret_cast<const long long*>(desc.data_ptr<int64_t>());
  p.tr_first = (int)first;
  p.tr_stride = (int)stride;
  if (tile_expert.has_value() && tile_expert->defined()) {
    TORCH_CHECK(tile_row0.has_value() && tile_rows.has_value() && n_tiles.has_value());
    TORCH_CHECK(tile_expert->scalar_type() == at::kInt && tile_row0->scalar_type() == at::kInt && tile_rows->scalar_type() == at::kInt &&
                n_tiles->scalar_type() == at::kInt);
    p.tile_expert = tile_expert->data_ptr<int>();
    p.tile_row0 = tile_row0->data_ptr<int>();
    p.tile_rows = tile_rows->data_ptr<int>();
    p.n_tiles = n_tiles->data_ptr<int>();
    p.max_tiles = (int)tile_expert->numel();
    p.token_tile = (int)token_tile;
  } else {
    TORCH_CHECK(desc.size(0) >= first + (act ? 2 : 1));
  }
  if (row_scale.has_value() && row_scale->defined()) {
    TORCH_CHECK(row_scale->scalar_type() == at::kFloat && row_scale->is_contiguous());
    p.row_scale = row_scale->data_ptr<float>();
  }
  check(mmb_trellis_gemm(&p, cur_stream()), "trellis_gemm");
}

// ---- expert-parallel exchange (ep_comm.cu).  Descriptors are CPU int64 tensors of device addresses.
// desc [8] = tables (device arrays of ep pointers) peer_recv_x, peer_recv_meta, peer_recv_cnt, peer_flags; then the local
// send_cnt, counter, step, status
void ep_dispatch(const Tensor& x, const Tensor& ids, const Tensor& desc, int64_t experts_per_rank, int64_t ep, int64_t rank, int64_t cap) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && ids.scalar_type() == at::kInt && ids.is_contiguous() && ids.dim() == 2 &&
              ids.size(0) == x.size(0));
  TORCH_CHECK(!desc.is_cuda() && desc.scalar_type() == at::kLong && desc.numel() == 8);
  const int64_t* v = desc.data_ptr<int64_t>();
  c10::cuda::CUDAGuard guard(x.device());
  MmbEpDispatchParams p{};
  p.x = x.data_ptr();
  p.ldx = (int)x.stride(0);
  p.ids = ids.data_ptr<int>();
  p.T = (int)x.size(0);
  p.topk = (int)ids.size(1);
  p.H = (int)x.size(1);
  p.experts_per_rank = (int)experts_per_rank;
  p.ep = (int)ep;
  p.rank = (int)rank;
  p.cap = (int)cap;
  p.peer_recv_x = reinterpret_cast<void* const*>(v[0]);
  p.peer_recv_meta = reinterpret_cast<int* const*>(v[1]);
  p.peer_recv_cnt = reinterpret_cast<int* const*>(v[2]);
  p.peer_flags = reinterpret_cast<unsigned* const*>(v[3]);
  p.send_cnt = reinterpret_cast<int*>(v[4]);
  p.counter = reinterpret_cast<unsigned*>(v[5]);
  p.step = reinterpret_cast<const unsigned*>(v[6]);
  p.status = reinterpret_cast<int*>(v[7]);
  check(mmb_ep_dispatch(&p, cur_stream()), "ep_dispatch");
}

// desc [6] = recv_meta, recv_cnt, flags, step, status, ret_peer table (device int64 [ep])
void ep_recv_group(const Tensor& desc, int64_t ep, int64_t cap, int64_t H, int64_t E_local, int64_t token_tile, Tensor order, Tensor row_dst,
                   Tensor tile_expert, Tensor tile_row0, Tensor tile_rows, Tensor n_tiles) {
  TORCH_CHECK(!desc.is_cuda() && desc.scalar_type() == at::kLong && desc.numel() == 6);
  TORCH_CHECK(order.is_cuda() && order.scalar_type() == at::kInt && order.numel() <= ep * cap && row_dst.scalar_type() == at::kLong &&
              row_dst.numel() == order.numel() && order.is_contiguous() && row_dst.is_contiguous() && n_tiles.numel() >= 2);
  TORCH_CHECK(tile_expert.scalar_type() == at::kInt && tile_row0.scalar_type() == at::kInt && tile_rows.scalar_type() == at::kInt &&
              n_tiles.scalar_type() == at::kInt && tile_row0.numel() == tile_expert.numel() && tile_rows.numel() == tile_expert.numel());
  const int64_t* v = desc.data_ptr<int64_t>();
  c10::cuda::CUDAGuard guard(order.device());
  MmbEpRecvParams p{};
  p.recv_meta = reinterpret_cast<const int*>(v[0]);
  p.recv_cnt = reinterpret_cast<const int*>(v[1]);
  p.flags = reinterpret_cast<const unsigned*>(v[2]);
  p.step = reinterpret_cast<const unsigned*>(v[3]);
  p.status = reinterpret_cast<int*>(v[4]);
  p.ret_peer = reinterpret_cast<const long long*>(v[5]);
  p.ep = (int)ep;
  p.cap = (int)cap;
  p.H = (int)H;
  p.E_local = (int)E_local;
  p.token_tile = (int)token_tile;
  p.max_tiles = (int)tile_expert.numel();
  p.order = order.data_ptr<int>();
  p.row_dst = reinterpret_cast<long long*>(row_dst.data_ptr<int64_t>());
  p.tile_expert = tile_expert.data_ptr<int>();
  p.tile_row0 = tile_row0.data_ptr<int>();
  p.tile_rows = tile_rows.data_ptr<int>();
  p.n_tiles = n_tiles.data_ptr<int>();
  p.n_rows_max = (int)order.numel();
  check(mmb_ep_recv_group(&p, cur_stream()), "ep_recv_group");
}

// desc [2] = peer_flags table (device array of ep pointers), step
void ep_signal(const Tensor& desc, int64_t ep) {
  TORCH_CHECK(!desc.is_cuda() && desc.scalar_type() == at::kLong && desc.numel() == 2);
  const int64_t* v = desc.data_ptr<int64_t>();
  check(mmb_ep_signal(reinterpret_cast<unsigned* const*>(v[0]), reinterpret_cast<const unsigned*>(v[1]), (int)ep, cur_stream()), "ep_signal");
}

// desc [4] = ret_y, flags, step, status
void ep_combine(const Tensor& desc, const Tensor& ids, const Tensor& weights, const OptT& add0, const OptT& add1, Tensor out, int64_t ep) {
  check_bf16(out, "out");
  TORCH_CHECK(!desc.is_cuda() && desc.scalar_type() == at::kLong && desc.numel() == 4);
  TORCH_CHECK(out.dim() == 2 && out.is_contiguous() && ids.scalar_type() == at::kInt && ids.is_contiguous() && ids.dim() == 2 &&
              ids.size(0) == out.size(0) && weights.scalar_type() == at::kFloat && weights.is_contiguous() && weights.numel() == ids.numel());
  if (add0.has_value() && add0->defined()) TORCH_CHECK(add0->is_contiguous() && add0->scalar_type() == at::kBFloat16 && add0->numel() == out.numel());
  if (add1.has_value() && add1->defined()) TORCH_CHECK(add1->is_contiguous() && add1->scalar_type() == at::kBFloat16 && add1->numel() == out.numel());
  const int64_t* v = desc.data_ptr<int64_t>();
  c10::cuda::CUDAGuard guard(out.device());
  MmbEpCombineParams p{};
  p.ret_y = reinterpret_cast<const void*>(v[0]);
  p.flags = reinterpret_cast<const unsigned*>(v[1]);
  p.step = reinterpret_cast<const unsigned*>(v[2]);
  p.status = reinterpret_cast<int*>(v[3]);
  p.ids = ids.data_ptr<int>();
  p.weights = weights.data_ptr<float>();
  p.add0 = cptr(add0);
  p.add1 = cptr(add1);
  p.out = out.data_ptr();
  p.T = (int)out.size(0);
  p.topk = (int)ids.size(1);
  p.N = (int)out.size(1);
  p.ep = (int)ep;
  check(mmb_ep_combine(&p, cur_stream()), "ep_combine");
}

void bf16_gemm_impl(const Tensor& x, const Tensor& w, Tensor out, Tensor status, const Tensor* ag);
void bf16_gemm(const Tensor& x, const Tensor& w, Tensor out, Tensor status) { bf16_gemm_impl(x, w, out, status, nullptr); }
void bf16_gemm_ag(const Tensor& x, const Tensor& w, Tensor out, Tensor status, const Tensor& ag) {
  TORCH_CHECK(out.dim() == 2, "the fused all-gather covers unbatched problems");
  bf16_gemm_impl(x, w, out, status, &ag);
}
void bf16_gemm_impl(const Tensor& x, const Tensor& w, Tensor out, Tensor status, const Tensor* ag) {
  // x [B?, M, K], w [B?, N, K] -> out [B?, M, N]; 2-D operands are shared across the batch
  check_bf16(x, "x");
  check_bf16(w, "w");
  TORCH_CHECK(x.stride(-1) == 1 && w.stride(-1) == 1 && out.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  MmbBf16GemmParams p{};
  p.x = x.data_ptr();
  p.w = w.data_ptr();
  p.out = out.data_ptr();
  p.M = (int)x.size(-2);
  p.N = (int)w.size(-2);
  p.K = (int)x.size(-1);
  p.ldx = (int)x.stride(-2);
  p.ldw = (int)w.stride(-2);
  p.ldo = (int)out.size(-1);
  p.out_f32 = out.scalar_type() == at::kFloat;
  p.batch = out.dim() == 3 ? (int)out.size(0) : 1;
  p.x_batch_stride = x.dim() == 3 ? x.stride(0) : 0;
  p.w_batch_stride = w.dim() == 3 ? w.stride(0) : 0;
  p.out_batch_stride = out.dim() == 3 ? out.stride(0) : 0;
  p.status = status.data_ptr<int>();
  if (ag != nullptr) p.ag = ag_from(*ag);
  check(mmb_bf16_gemm(&p, cur_stream()), "bf16_gemm");
}

}  // namespace

// ------------------------------------------------------------------------------------------------ secondary kernels
void hadamard(const Tensor& x, Tensor out, int64_t block) {
  check_bf16(x, "x");
  TORCH_CHECK(x.is_contiguous() && out.is_contiguous() && out.numel() == x.numel());
  c10::cuda::CUDAGuard guard(x.device());
  const int dim = (int)x.size(-1);
  check(mmb_hadamard(x.data_ptr(), out.data_ptr(), (int)(x.numel() / dim), dim, (int)block, cur_stream()), "hadamard");
}

void gptq_block(Tensor W, Tensor Q, Tensor E, const Tensor& Hinv, const Tensor& col_scale, const Tensor& grid, Tensor err_rows,
                int64_t i1, int64_t B) {
  for (const Tensor* t : std::initializer_list<const Tensor*>{&W, &Q, &E, &Hinv, &col_scale, &grid, &err_rows})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat, "gptq_block: fp32 CUDA tensors expected");
  TORCH_CHECK(W.dim() == 2 && W.stride(1) == 1 && Q.sizes() == W.sizes() && Q.stride(1) == 1 && Q.stride(0) == W.stride(0));
  TORCH_CHECK(col_scale.sizes() == W.sizes() && col_scale.stride(1) == 1 && col_scale.stride(0) == W.stride(0));
  TORCH_CHECK(Hinv.dim() == 2 && Hinv.stride(1) == 1 && Hinv.size(0) == W.size(1) && Hinv.size(1) == W.size(1));
  TORCH_CHECK(i1 >= 0 && B >= 1 && i1 + B <= W.size(1));
  TORCH_CHECK(E.is_contiguous() && E.size(0) == W.size(0) && E.size(1) == B && grid.is_contiguous());
  TORCH_CHECK(err_rows.is_contiguous() && err_rows.numel() == W.size(0));
  c10::cuda::CUDAGuard guard(W.device());
  check(mmb_gptq_block(W.data_ptr<float>(), Q.data_ptr<float>(), E.data_ptr<float>(), Hinv.data_ptr<float>(),
                       col_scale.data_ptr<float>(), grid.data_ptr<float>(), err_rows.data_ptr<float>(), (int)grid.numel(),
                       (int)W.size(0), (long)W.stride(0), (long)Hinv.stride(0), (int)i1, (int)B, cur_stream()), "gptq_block");
}

void fp4_quantize_pack(const Tensor& w, Tensor packed, Tensor scales, int64_t group_size) {
  TORCH_CHECK(w.is_cuda() && w.dim() == 2 && w.is_contiguous(), "fp4_quantize_pack: contiguous 2-D CUDA weight expected");
  TORCH_CHECK(w.scalar_type() == at::kFloat || w.scalar_type() == at::kBFloat16, "fp4_quantize_pack: fp32 or bf16 weight");
  TORCH_CHECK(w.size(1) % group_size == 0 && w.size(1) % 8 == 0);
  TORCH_CHECK(packed.is_contiguous() && packed.scalar_type() == at::kInt && packed.numel() == w.numel() / 8);
  TORCH_CHECK(scales.is_contiguous() && scales.scalar_type() == at::kHalf && scales.numel() == w.numel() / group_size);
  c10::cuda::CUDAGuard guard(w.device());
  check(mmb_fp4_quantize_pack(w.data_ptr(), w.scalar_type() == at::kBFloat16, (uint32_t*)packed.data_ptr(), scales.data_ptr(),
                              (long)w.size(0), (int)w.size(1), (int)group_size, cur_stream()), "fp4_quantize_pack");
}

void trellis_dequant(const Tensor& codes, const Tensor& scales, const Tensor& su, const Tensor& sv, Tensor out, int64_t bits,
                     int64_t group_size) {
  TORCH_CHECK(codes.scalar_type() == at::kByte && codes.is_contiguous() && scales.scalar_type() == at::kFloat && scales.is_contiguous());
  TORCH_CHECK(su.scalar_type() == at::kFloat && sv.scalar_type() == at::kFloat && out.scalar_type() == at::kBFloat16 && out.is_contiguous());
  const int out_f = (int)out.size(0), in_f = (int)out.size(1);
  TORCH_CHECK(codes.numel() >= (int64_t)((out_f + 15) / 16) * ((in_f + 15) / 16) * 32 * bits, "trellis code blob too small");
  TORCH_CHECK(su.numel() == in_f && sv.numel() == out_f && scales.size(1) == out_f);
  c10::cuda::CUDAGuard guard(codes.device());
  check(mmb_trellis_dequant(codes.data_ptr<uint8_t>(), scales.data_ptr<float>(), su.data_ptr<float>(), sv.data_ptr<float>(),
                            out.data_ptr(), out_f, in_f, (int)bits, (int)group_size, cur_stream()),
        "trellis_dequant");
}

void trellis_gemv(const Tensor& x, const Tensor& codes, const Tensor& scales, const Tensor& su, const Tensor& sv, Tensor y,
                  int64_t bits, int64_t group_size) {
  check_bf16(x, "x");
  TORCH_CHECK(codes.scalar_type() == at::kByte && codes.is_contiguous() && scales.is_contiguous() && x.stride(1) == 1 && y.stride(1) == 1);
  const int out_f = (int)y.size(1), in_f = (int)x.size(1);
  TORCH_CHECK(codes.numel() >= (int64_t)((out_f + 15) / 16) * ((in_f + 15) / 16) * 32 * bits, "trellis code blob too small");
  TORCH_CHECK(su.numel() == in_f && sv.numel() == out_f && scales.size(1) == out_f);
  c10::cuda::CUDAGuard guard(x.device());
  for (int64_t m0 = 0; m0 < x.size(0); m0 += 4) {
    const int m = (int)std::min<int64_t>(4, x.size(0) - m0);
    check(mmb_trellis_gemv((const char*)x.data_ptr() + m0 * x.stride(0) * 2, codes.data_ptr<uint8_t>(), scales.data_ptr<float>(),
                           su.data_ptr<float>(), sv.data_ptr<float>(), (char*)y.data_ptr() + m0 * y.stride(0) * 2, m, out_f, in_f,
                           (int)bits, (int)group_size, (int)x.stride(0), (int)y.stride(0), cur_stream()),
          "trellis_gemv");
  }
}

// mats: int64 CUDA tensor [n_experts * 3, 6] laid out like MmbTrellisMat (4 pointers, then out | in << 32, bits | gs << 32)
void trellis_moe(const Tensor& x, const Tensor& mats, const Tensor& ids, const Tensor& wts, Tensor h, Tensor y, int64_t hidden,
                 int64_t inter) {
  check_bf16(x, "x");
  check_bf16(h, "h");
  static_assert(sizeof(MmbTrellisMat) == 48, "descriptor rows are six 64-bit words");
  TORCH_CHECK(mats.is_cuda() && mats.scalar_type() == at::kLong && mats.is_contiguous() && mats.dim() == 2 && mats.size(1) == 6);
  TORCH_CHECK(ids.scalar_type() == at::kInt && ids.is_contiguous() && ids.dim() == 2 && wts.scalar_type() == at::kFloat && wts.is_contiguous() &&
              wts.numel() == ids.numel());
  const int T = (int)ids.size(0), topk = (int)ids.size(1);
  TORCH_CHECK(x.size(0) == T && x.stride(1) == 1 && x.size(1) >= hidden);
  TORCH_CHECK(h.is_contiguous() && h.size(0) == (int64_t)T * topk && h.size(1) == inter);
  TORCH_CHECK(y.scalar_type() == at::kFloat && y.is_contiguous() && y.size(0) == (int64_t)T * topk && y.size(1) == hidden);
  c10::cuda::CUDAGuard guard(x.device());
  check(mmb_trellis_moe(x.data_ptr(), reinterpret_cast<const MmbTrellisMat*>(mats.data_ptr<int64_t>()), ids.data_ptr<int>(),
                        wts.data_ptr<float>(), h.data_ptr(), y.data_ptr<float>(), T, topk, (int)hidden, (int)inter, (int)x.stride(0),
                        cur_stream()),
        "trellis_moe");
}

// Codebook weights on the tensor cores for more than 8 rows: look-up, zero point and group scale applied inside the GEMM's
// main loop (gemm_sm100.cu, weight format 3).
void codebook_gemm(const Tensor& x, const Tensor& codes, const Tensor& scales, const OptT& zeros, const Tensor& lut, Tensor out,
                   int64_t in_f, int64_t group_size, int64_t bits, Tensor status) {
  check_bf16(x, "x");
  check_bf16(out, "out");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && x.size(1) == in_f && out.is_contiguous() && out.size(0) == x.size(0));
  TORCH_CHECK(codes.is_cuda() && codes.scalar_type() == at::kByte && codes.is_contiguous() && codes.dim() == 2 &&
              codes.size(1) * 8 == in_f * bits && out.size(1) == codes.size(0));
  TORCH_CHECK(scales.scalar_type() == at::kHalf && scales.is_contiguous() && lut.scalar_type() == at::kFloat && lut.numel() == 256 && lut.is_cuda());
  TORCH_CHECK(group_size >= 32 && (group_size & (group_size - 1)) == 0 && in_f % group_size == 0 && in_f % 64 == 0,
              "codebook_gemm: group size must be a power of two >= 32 dividing the input width (a multiple of 64)");
  TORCH_CHECK(scales.numel() == codes.size(0) * (in_f / group_size));
  if (zeros.has_value() && zeros->defined()) TORCH_CHECK(zeros->scalar_type() == at::kHalf && zeros->is_contiguous() && zeros->numel() == scales.numel());
  c10::cuda::CUDAGuard guard(x.device());
  MmbFp4GemmParams p{};
  p.x = x.data_ptr();
  p.qw = codes.data_ptr();
  p.sc = scales.data_ptr();
  p.out = out.data_ptr();
  p.M = (int)x.size(0);
  p.N = (int)codes.size(0);
  p.K = (int)in_f;
  p.Kx = (int)in_f;
  p.ldo = (int)out.stride(0);
  int sh = 0;
  while ((1ll << sh) < group_size) ++sh;
  p.gs_shift = sh;
  p.status = status.data_ptr<int>();
  p.cb_zeros = cptr(zeros);
  p.cb_lut = lut.data_ptr<float>();
  p.cb_bits = (int)bits;
  check(mmb_codebook_gemm(&p, cur_stream()), "codebook_gemm");
}

// 2:4 sparse FP4 weights on the tensor cores (gemm_sm100.cu, weight format 4): codes uint8 [N, K / 4], meta uint8 [N, K / 8],
// scales fp16 [N, K / group].
void sparse24_gemm(const Tensor& x, const Tensor& codes, const Tensor& meta, const Tensor& scales, Tensor out, int64_t in_f,
                   int64_t group_size, Tensor status) {
  check_bf16(x, "x");
  check_bf16(out, "out");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && x.size(1) == in_f && out.is_contiguous() && out.size(0) == x.size(0));
  TORCH_CHECK(codes.is_cuda() && codes.scalar_type() == at::kByte && codes.is_contiguous() && codes.dim() == 2 && codes.size(1) * 4 == in_f &&
              out.size(1) == codes.size(0));
  TORCH_CHECK(meta.is_cuda() && meta.scalar_type() == at::kByte && meta.is_contiguous() && meta.size(0) == codes.size(0) && meta.size(1) * 8 == in_f);
  TORCH_CHECK(scales.scalar_type() == at::kHalf && scales.is_contiguous() && scales.numel() == codes.size(0) * (in_f / group_size));
  TORCH_CHECK(group_size >= 32 && (group_size & (group_size - 1)) == 0 && in_f % group_size == 0 && in_f % 64 == 0,
              "sparse24_gemm: group size must be a power of two >= 32 dividing the input width (a multiple of 64)");
  c10::cuda::CUDAGuard guard(x.device());
  MmbFp4GemmParams p{};
  p.x = x.data_ptr();
  p.qw = codes.data_ptr();
  p.sp_meta = meta.data_ptr();
  p.sc = scales.data_ptr();
  p.out = out.data_ptr();
  p.M = (int)x.size(0);
  p.N = (int)codes.size(0);
  p.K = (int)in_f;
  p.Kx = (int)in_f;
  p.ldo = (int)out.stride(0);
  int sh = 0;
  while ((1ll << sh) < group_size) ++sh;
  p.gs_shift = sh;
  p.status = status.data_ptr<int>();
  check(mmb_sparse24_gemm(&p, cur_stream()), "sparse24_gemm");
}

void codebook_gemv(const Tensor& x, const Tensor& codes, const Tensor& scales, const OptT& zeros, const Tensor& lut, Tensor y,
                   int64_t in_f, int64_t group_size, int64_t bits) {
  check_bf16(x, "x");
  TORCH_CHECK(codes.scalar_type() == at::kByte && codes.is_contiguous() && scales.scalar_type() == at::kHalf && scales.is_contiguous());
  TORCH_CHECK(lut.scalar_type() == at::kFloat && lut.numel() == 256 && x.stride(1) == 1 && y.stride(1) == 1 && x.size(0) <= 8);
  TORCH_CHECK(codes.size(1) * 8 == in_f * bits && x.size(1) >= in_f);
  c10::cuda::CUDAGuard guard(x.device());
  check(mmb_codebook_gemv_bits(x.data_ptr(), codes.data_ptr<uint8_t>(), scales.data_ptr(), cptr(zeros), lut.data_ptr<float>(),
                               y.data_ptr(), (int)x.size(0), (int)codes.size(0), (int)in_f, (int)group_size, (int)bits,
                               (int)x.stride(0), (int)y.stride(0), cur_stream()),
        "codebook_gemv");
}

void vision_preprocess(const Tensor& images, Tensor out, int64_t out_h, int64_t out_w, int64_t patch, std::vector<double> mean,
                       std::vector<double> stdv) {
  TORCH_CHECK(images.scalar_type() == at::kByte && images.is_contiguous() && images.dim() == 4 && images.size(3) == 3);
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.is_contiguous() && mean.size() == 3 && stdv.size() == 3);
  TORCH_CHECK(out.numel() == images.size(0) * 3 * out_h * out_w);
  const float m[3] = {(float)mean[0], (float)mean[1], (float)mean[2]}, sd[3] = {(float)stdv[0], (float)stdv[1], (float)stdv[2]};
  c10::cuda::CUDAGuard guard(images.device());
  check(mmb_vision_preprocess(images.data_ptr<uint8_t>(), out.data_ptr(), (int)images.size(0), (int)images.size(1), (int)images.size(2),
                              (int)out_h, (int)out_w, (int)patch, m, sd, cur_stream()),
        "vision_preprocess");
}

// crop = {y, x, h, w} of the source rectangle; mode 0 bilinear, 1 bicubic, 2 nearest; merge: patch grouping (1 = row major)
void vision_preprocess_ex(const Tensor& images, Tensor out, std::vector<int64_t> crop, int64_t out_h, int64_t out_w, int64_t patch,
                          int64_t merge, int64_t mode, std::vector<double> mean, std::vector<double> stdv) {
  TORCH_CHECK(images.scalar_type() == at::kByte && images.is_contiguous() && images.dim() == 4 && images.size(3) == 3);
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.is_contiguous() && mean.size() == 3 && stdv.size() == 3 && crop.size() == 4);
  TORCH_CHECK(out.numel() == images.size(0) * 3 * out_h * out_w);
  const float m[3] = {(float)mean[0], (float)mean[1], (float)mean[2]}, sd[3] = {(float)stdv[0], (float)stdv[1], (float)stdv[2]};
  c10::cuda::CUDAGuard guard(images.device());
  check(mmb_vision_preprocess_ex(images.data_ptr<uint8_t>(), out.data_ptr(), (int)images.size(0), (int)images.size(1), (int)images.size(2),
                                 (int)crop[0], (int)crop[1], (int)crop[2], (int)crop[3], (int)out_h, (int)out_w, (int)patch, (int)merge,
                                 (int)mode, m, sd, cur_stream()),
        "vision_preprocess_ex");
}
void channel_stats(const Tensor& images, Tensor out) {
  TORCH_CHECK(images.scalar_type() == at::kByte && images.is_contiguous() && images.dim() == 4 && images.size(3) == 3);
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.is_contiguous() && out.numel() == images.size(0) * 6);
  c10::cuda::CUDAGuard guard(images.device());
  check(mmb_channel_stats(images.data_ptr<uint8_t>(), out.data_ptr<float>(), (int)images.size(0), (int)images.size(1), (int)images.size(2),
                          cur_stream()),
        "channel_stats");
}
// LayerNorm over the last axis: out = (x - mean) * rstd * w + b (bf16 in / out, fp32 statistics); optional residual `delta`
// added first (resid_out receives x + delta).
void layernorm(const Tensor& x, const OptT& delta, const OptT& w, const OptT& b, Tensor out, const OptT& resid_out, double eps) {
  check_bf16(x, "x");
  check_bf16(out, "out");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && out.stride(1) == 1 && out.size(0) == x.size(0) && out.size(1) == x.size(1));
  c10::cuda::CUDAGuard guard(x.device());
  check(mmb_layernorm(x.data_ptr(), cptr(delta), cptr(w), cptr(b), out.data_ptr(), mptr(resid_out), (int)x.size(0), (int)x.size(1),
                      (int)x.stride(0), (int)out.stride(0), (float)eps, cur_stream()),
        "layernorm");
}

void spec_verify(const Tensor& p_target, const Tensor& p_draft, const Tensor& draft, const Tensor& u, const Tensor& u_res,
                 Tensor out_tokens, Tensor out_accepted) {
  TORCH_CHECK(p_target.scalar_type() == at::kFloat && p_draft.scalar_type() == at::kFloat && p_target.is_contiguous() && p_draft.is_contiguous());
  TORCH_CHECK(draft.scalar_type() == at::kLong && draft.is_contiguous() && u.scalar_type() == at::kFloat && u_res.scalar_type() == at::kFloat);
  TORCH_CHECK(out_tokens.scalar_type() == at::kLong && out_accepted.scalar_type() == at::kInt);
  const int B = (int)draft.size(0), K = (int)draft.size(1), V = (int)p_target.size(2);
  TORCH_CHECK(p_target.size(0) == B && p_target.size(1) == K + 1 && p_draft.size(1) == K && p_draft.size(2) == V);
  TORCH_CHECK(u.numel() == (int64_t)B * K && u_res.numel() == B && out_tokens.numel() == (int64_t)B * (K + 1) && out_accepted.numel() == B);
  c10::cuda::CUDAGuard guard(p_target.device());
  check(mmb_spec_verify(p_target.data_ptr<float>(), p_draft.data_ptr<float>(), draft.data_ptr<int64_t>(), u.data_ptr<float>(),
                        u_res.data_ptr<float>(), out_tokens.data_ptr<int64_t>(), out_accepted.data_ptr<int>(), B, K, V, cur_stream()),
        "spec_verify");
}

void gated_delta_step(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& g, const Tensor& beta, Tensor state, Tensor out,
                      double scale) {
  check_bf16(q, "q");
  check_bf16(k, "k");
  check_bf16(v, "v");
  TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && state.is_contiguous() && out.is_contiguous());
  TORCH_CHECK(g.scalar_type() == at::kFloat && beta.scalar_type() == at::kFloat && state.scalar_type() == at::kFloat);
  const int B = (int)q.size(0), H = (int)q.size(1), dk = (int)q.size(2), dv = (int)v.size(2);
  TORCH_CHECK(state.numel() == (int64_t)B * H * dk * dv && g.numel() == (int64_t)B * H && beta.numel() == (int64_t)B * H);
  c10::cuda::CUDAGuard guard(q.device());
  check(mmb_gated_delta_step(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr<float>(), beta.data_ptr<float>(), state.data_ptr<float>(),
                             out.data_ptr(), B, H, dk, dv, (float)scale, cur_stream()),
        "gated_delta_step");
}

static void check_f32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), name, " must be a contiguous CUDA fp32 tensor");
}
// r, k [B, T, H, dk], v [B, T, H, dv], w [B, T, H, dk] or [H, dk], u [H, dk], state [B, H, dk, dv] (in place), out [B, T, H, dv]
void wkv_scan(const Tensor& r, const Tensor& k, const Tensor& v, const Tensor& w, const Tensor& u, Tensor state, Tensor out) {
  for (const Tensor* t : {&r, &k, &v, &w, &u, (const Tensor*)&state, (const Tensor*)&out}) check_f32(*t, "wkv tensor");
  TORCH_CHECK(r.dim() == 4 && v.dim() == 4 && state.dim() == 4);
  const int B = (int)r.size(0), T = (int)r.size(1), H = (int)r.size(2), dk = (int)r.size(3), dv = (int)v.size(3);
  TORCH_CHECK(state.size(0) == B && state.size(1) == H && state.size(2) == dk && state.size(3) == dv && u.numel() == (int64_t)H * dk);
  const bool per_token = w.dim() == 4;
  TORCH_CHECK(per_token ? w.numel() == r.numel() : w.numel() == (int64_t)H * dk);
  c10::cuda::CUDAGuard guard(r.device());
  check(mmb_wkv(r.data_ptr<float>(), k.data_ptr<float>(), v.data_ptr<float>(), w.data_ptr<float>(), u.data_ptr<float>(), state.data_ptr<float>(),
                out.data_ptr<float>(), B, T, H, dk, dv, per_token ? (long long)T * H * dk : 0, per_token ? (long long)H * dk : 0, cur_stream()),
        "wkv_scan");
}
void gated_delta_scan(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& g, const Tensor& beta, Tensor state, Tensor out,
                      double scale) {
  for (const Tensor* t : {&q, &k, &v, &g, &beta, (const Tensor*)&state, (const Tensor*)&out}) check_f32(*t, "gated_delta tensor");
  const int B = (int)q.size(0), T = (int)q.size(1), H = (int)q.size(2), dk = (int)q.size(3), dv = (int)v.size(3);
  TORCH_CHECK(state.numel() == (int64_t)B * H * dk * dv && g.numel() == (int64_t)B * T * H && beta.numel() == g.numel());
  c10::cuda::CUDAGuard guard(q.device());
  check(mmb_gated_delta_scan(q.data_ptr<float>(), k.data_ptr<float>(), v.data_ptr<float>(), g.data_ptr<float>(), beta.data_ptr<float>(),
                             state.data_ptr<float>(), out.data_ptr<float>(), B, T, H, dk, dv, (float)scale, cur_stream()),
        "gated_delta_scan");
}
void selective_scan(const Tensor& x, const Tensor& dt, const Tensor& A, const Tensor& Bm, const Tensor& Cm, const OptT& Dskip, Tensor state,
                    Tensor y) {
  for (const Tensor* t : {&x, &dt, &A, &Bm, &Cm, (const Tensor*)&state, (const Tensor*)&y}) check_f32(*t, "selective_scan tensor");
  const int B = (int)x.size(0), T = (int)x.size(1), D = (int)x.size(2), N = (int)A.size(1);
  TORCH_CHECK(state.numel() == (int64_t)B * D * N && Bm.numel() == (int64_t)B * T * N && Cm.numel() == Bm.numel());
  const float* dsk = nullptr;
  if (Dskip.has_value() && Dskip->defined()) {
    check_f32(*Dskip, "Dskip");
    dsk = Dskip->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(x.device());
  check(mmb_selective_scan(x.data_ptr<float>(), dt.data_ptr<float>(), A.data_ptr<float>(), Bm.data_ptr<float>(), Cm.data_ptr<float>(), dsk,
                           state.data_ptr<float>(), y.data_ptr<float>(), B, T, D, N, cur_stream()),
        "selective_scan");
}

void selective_scan_step(const Tensor& x, const Tensor& dt, const Tensor& A, const Tensor& Bm, const Tensor& Cm, const OptT& Dskip,
                         Tensor state, Tensor y) {
  check_bf16(x, "x");
  TORCH_CHECK(x.is_contiguous() && dt.is_contiguous() && A.is_contiguous() && Bm.is_contiguous() && Cm.is_contiguous() && state.is_contiguous());
  TORCH_CHECK(dt.scalar_type() == at::kFloat && A.scalar_type() == at::kFloat && Bm.scalar_type() == at::kFloat && Cm.scalar_type() == at::kFloat &&
              state.scalar_type() == at::kFloat);
  const int B = (int)x.size(0), D = (int)x.size(1), N = (int)A.size(1);
  TORCH_CHECK(state.numel() == (int64_t)B * D * N && A.size(0) == D && Bm.numel() == (int64_t)B * N);
  c10::cuda::CUDAGuard guard(x.device());
  check(mmb_selective_scan_step(x.data_ptr(), dt.data_ptr<float>(), A.data_ptr<float>(), Bm.data_ptr<float>(), Cm.data_ptr<float>(),
                                (const float*)cptr(Dskip), state.data_ptr<float>(), y.data_ptr(), B, D, N, cur_stream()),
        "selective_scan_step");
}

// q [T, Hq, D], out [T, Hq, D] (any strides with unit inner stride); contiguous mode: k, v [N, Hk, D] + cu_k; paged mode:
// k, v pools [slots, Hk, D] + block_tables + ctx_lens.
void prefill_attention(const Tensor& q, const Tensor& k, const Tensor& v, Tensor out, const Tensor& cu_q, const OptT& cu_k,
                       const OptT& block_tables, const OptT& ctx_lens, int64_t block_size, int64_t max_q, double scale, int64_t window,
                       bool causal, int64_t sinks, const OptT& tree_mask, const OptT& block_mask) {
  check_bf16(q, "q");
  check_bf16(k, "k");
  check_bf16(v, "v");
  check_bf16(out, "out");
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3 && out.dim() == 3);
  TORCH_CHECK(q.stride(2) == 1 && k.stride(2) == 1 && v.stride(2) == 1 && out.stride(2) == 1);
  TORCH_CHECK(cu_q.scalar_type() == at::kInt && cu_q.is_contiguous() && q.size(2) == k.size(2) && v.size(2) == q.size(2));
  c10::cuda::CUDAGuard guard(q.device());
  MmbPrefillAttnParams p{};
  p.q = q.data_ptr();
  p.k = k.data_ptr();
  p.v = v.data_ptr();
  p.out = out.data_ptr();
  p.q_tok_stride = q.stride(0);
  p.q_head_stride = q.stride(1);
  p.k_tok_stride = k.stride(0);
  p.k_head_stride = k.stride(1);
  p.v_tok_stride = v.stride(0);
  p.v_head_stride = v.stride(1);
  p.o_tok_stride = out.stride(0);
  p.o_head_stride = out.stride(1);
  p.cu_q = cu_q.data_ptr<int>();
  p.cu_k = (cu_k.has_value() && cu_k->defined()) ? cu_k->data_ptr<int>() : nullptr;
  if (block_tables.has_value() && block_tables->defined()) {
    TORCH_CHECK(block_tables->scalar_type() == at::kInt && block_tables->is_contiguous() && ctx_lens.has_value() && ctx_lens->scalar_type() == at::kInt);
    p.block_tables = block_tables->data_ptr<int>();
    p.ctx_lens = ctx_lens->data_ptr<int>();
    p.max_blocks = (int)block_tables->size(1);
  }
  p.block_size = (int)block_size;
  p.B = (int)cu_q.numel() - 1;
  p.Hq = (int)q.size(1);
  p.Hk = (int)k.size(1);
  p.D = (int)q.size(2);
  p.max_q = (int)max_q;
  p.scale = (float)scale;
  p.window = (int)window;
  p.causal = causal ? 1 : 0;
  p.sinks = (int)sinks;
  if (tree_mask.has_value() && tree_mask->defined()) {
    TORCH_CHECK(tree_mask->scalar_type() == at::kByte && tree_mask->dim() == 2 && tree_mask->is_contiguous() && tree_mask->is_cuda() &&
                tree_mask->size(0) == q.size(0) && tree_mask->size(1) >= max_q);
    p.tree_mask = tree_mask->data_ptr<unsigned char>();
    p.tree_ld = (int)tree_mask->size(1);
  }
  if (block_mask.has_value() && block_mask->defined()) {
    TORCH_CHECK(block_mask->scalar_type() == at::kByte && block_mask->dim() == 3 && block_mask->is_contiguous() && block_mask->is_cuda() &&
                (block_mask->size(0) == 1 || block_mask->size(0) == q.size(1)) && block_mask->size(1) == (max_q + 127) / 128);
    p.block_mask = block_mask->data_ptr<unsigned char>();
    p.block_heads = (int)block_mask->size(0);
    p.n_kblocks = (int)block_mask->size(2);
  }
  check(mmb_prefill_attention(&p, cur_stream()), "prefill_attention");
}

void moe_group(const Tensor& ids, int64_t E, int64_t token_tile, Tensor order, Tensor inv, Tensor tile_expert, Tensor tile_row0,
               Tensor tile_rows, Tensor n_tiles) {
  TORCH_CHECK(ids.scalar_type() == at::kInt && ids.is_contiguous() && order.scalar_type() == at::kInt && inv.scalar_type() == at::kInt);
  TORCH_CHECK(tile_expert.scalar_type() == at::kInt && tile_row0.scalar_type() == at::kInt && tile_rows.scalar_type() == at::kInt &&
              n_tiles.scalar_type() == at::kInt);
  TORCH_CHECK(order.numel() == ids.numel() && inv.numel() == ids.numel() && tile_row0.numel() == tile_expert.numel() &&
              tile_rows.numel() == tile_expert.numel());
  c10::cuda::CUDAGuard guard(ids.device());
  check(mmb_moe_group(ids.data_ptr<int>(), (int)ids.numel(), (int)E, (int)token_tile, (int)tile_expert.numel(), order.data_ptr<int>(),
                      inv.data_ptr<int>(), tile_expert.data_ptr<int>(), tile_row0.data_ptr<int>(), tile_rows.data_ptr<int>(),
                      n_tiles.data_ptr<int>(), cur_stream()),
        "moe_group");
}

void moe_gather_impl(const Tensor& x, const Tensor& order, Tensor xs, int64_t topk, const int* n_dev);
void moe_gather(const Tensor& x, const Tensor& order, Tensor xs, int64_t topk) { moe_gather_impl(x, order, xs, topk, nullptr); }
// Gathers only the first `n_rows[idx]` rows (a count that lives on the device, e.g. the rows an expert owner received).
void moe_gather_n(const Tensor& x, const Tensor& order, Tensor xs, int64_t topk, const Tensor& n_rows, int64_t idx) {
  TORCH_CHECK(n_rows.is_cuda() && n_rows.scalar_type() == at::kInt && idx >= 0 && idx < n_rows.numel());
  moe_gather_impl(x, order, xs, topk, n_rows.data_ptr<int>() + idx);
}
void moe_gather_impl(const Tensor& x, const Tensor& order, Tensor xs, int64_t topk, const int* n_dev) {
  check_bf16(x, "x");
  check_bf16(xs, "xs");
  TORCH_CHECK(x.stride(1) == 1 && xs.is_contiguous() && order.scalar_type() == at::kInt && xs.size(0) == order.numel() && xs.size(1) <= x.size(1));
  c10::cuda::CUDAGuard guard(x.device());
  check(mmb_moe_gather(x.data_ptr(), order.data_ptr<int>(), xs.data_ptr(), (int)order.numel(), (int)topk, (int)xs.size(1), (int)x.stride(0),
                       n_dev, cur_stream()),
        "moe_gather");
}

void moe_combine(const Tensor& y, const Tensor& inv, const OptT& add0, const OptT& add1, Tensor out, int64_t topk) {
  check_bf16(y, "y");
  check_bf16(out, "out");
  TORCH_CHECK(y.is_contiguous() && out.is_contiguous() && inv.scalar_type() == at::kInt && inv.numel() == out.size(0) * topk);
  if (add0.has_value() && add0->defined()) TORCH_CHECK(add0->is_contiguous() && add0->scalar_type() == at::kBFloat16);
  if (add1.has_value() && add1->defined()) TORCH_CHECK(add1->is_contiguous() && add1->scalar_type() == at::kBFloat16);
  c10::cuda::CUDAGuard guard(y.device());
  check(mmb_moe_combine(y.data_ptr(), inv.data_ptr<int>(), cptr(add0), cptr(add1), out.data_ptr(), (int)out.size(0), (int)topk, (int)out.size(1),
                        cur_stream()),
        "moe_combine");
}

// Causal prefill attention of one sequence on the tcgen05 path.  q [t, Hq, D], k [n, Hk, D] (last dim contiguous),
// vt [Hk, D, n_pad] contiguous, out [t, Hq, D]; status: device int tensor (first word receives a code after a timeout).
void fmha_prefill(const Tensor& q, const Tensor& k, const Tensor& vt, Tensor out, int64_t n, double scale, Tensor status,
                  int64_t window) {
  check_bf16(q, "q");
  check_bf16(k, "k");
  check_bf16(vt, "vt");
  check_bf16(out, "out");
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && vt.dim() == 3 && out.dim() == 3 && q.stride(2) == 1 && k.stride(2) == 1 && out.stride(2) == 1 &&
              vt.is_contiguous());
  TORCH_CHECK(k.size(2) == q.size(2) && vt.size(1) == q.size(2) && vt.size(0) == k.size(1) && out.size(0) == q.size(0) &&
              out.size(1) == q.size(1) && out.size(2) == q.size(2) && k.size(0) >= n && vt.size(2) >= n);
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard guard(q.device());
  MmbFmhaPrefillParams p{};
  p.q = q.data_ptr();
  p.k = k.data_ptr();
  p.vt = vt.data_ptr();
  p.out = out.data_ptr();
  p.t = (int)q.size(0);
  p.n = (int)n;
  p.n_pad = (int)vt.size(2);
  p.Hq = (int)q.size(1);
  p.Hk = (int)k.size(1);
  p.D = (int)q.size(2);
  p.q_tok_stride = q.stride(0);
  p.q_head_stride = q.stride(1);
  p.k_tok_stride = k.stride(0);
  p.k_head_stride = k.stride(1);
  p.o_tok_stride = out.stride(0);
  p.o_head_stride = out.stride(1);
  p.scale = (float)scale;
  p.window = (int)window;
  p.status = status.data_ptr<int>();
  check(mmb_fmha_prefill(&p, cur_stream()), "fmha_prefill");
}

// In-switch all-reduce of the first `n` fp32 elements of a symmetric buffer.  desc (CPU int64 [6]): multicast address of the
// data, device table of the peers' flag bases, local flags, step word, counter, status word.
void mc_all_reduce(const Tensor& desc, int64_t n, int64_t tp, int64_t rank, const Tensor& anchor) {
  TORCH_CHECK(!desc.is_cuda() && desc.scalar_type() == at::kLong && desc.numel() == 6 && anchor.is_cuda());
  const int64_t* v = desc.data_ptr<int64_t>();
  c10::cuda::CUDAGuard guard(anchor.device());
  MmbMcAllReduceParams p{};
  p.mc = reinterpret_cast<float*>(v[0]);
  p.peer_flags = reinterpret_cast<unsigned* const*>(v[1]);
  p.local_flags = reinterpret_cast<const unsigned*>(v[2]);
  p.step = reinterpret_cast<unsigned*>(v[3]);
  p.counter = reinterpret_cast<unsigned*>(v[4]);
  p.status = reinterpret_cast<int*>(v[5]);
  p.n = n;
  p.tp = (int)tp;
  p.rank = (int)rank;
  check(mmb_mc_all_reduce(&p, cur_stream()), "mc_all_reduce");
}

// ---- symmetric-memory allocator (symm_vmm.cpp): thin pass-throughs; ids and file descriptors are plain integers
int64_t vmm_available() { return mmb_vmm_available(); }
int64_t vmm_create(int64_t dev, int64_t bytes) { return mmb_vmm_create((int)dev, bytes); }
int64_t vmm_export_fd(int64_t id) { return mmb_vmm_export_fd(id); }
int64_t vmm_import_fd(int64_t fd, int64_t bytes, int64_t dev) { return mmb_vmm_import_fd((int)fd, bytes, (int)dev); }
int64_t vmm_ptr(int64_t id) { return mmb_vmm_ptr(id); }
int64_t vmm_size(int64_t id) { return mmb_vmm_size(id); }
int64_t vmm_free(int64_t id) { return mmb_vmm_free(id); }
int64_t mc_create(int64_t n_dev, int64_t bytes) { return mmb_mc_create((int)n_dev, bytes); }
int64_t mc_export_fd(int64_t id) { return mmb_mc_export_fd(id); }
int64_t mc_import_fd(int64_t fd, int64_t n_dev, int64_t bytes) { return mmb_mc_import_fd((int)fd, (int)n_dev, bytes); }
int64_t mc_add_device(int64_t mc, int64_t dev) { return mmb_mc_add_device(mc, (int)dev); }
int64_t mc_bind(int64_t mc, int64_t mem) { return mmb_mc_bind(mc, mem); }
int64_t mc_map(int64_t mc, int64_t dev) { return mmb_mc_map(mc, (int)dev); }
int64_t mc_unbind(int64_t mc, int64_t dev, int64_t mem) { return mmb_mc_unbind(mc, (int)dev, mem); }
void vmm_close_fd(int64_t fd) { mmb_close_fd((int)fd); }
// Device-to-device copy between raw addresses (a mapped peer allocation and a local tensor) on the current stream of `dev`,
// the device the mappings were made for.
void vmm_copy(int64_t dst, int64_t src, int64_t nbytes, int64_t dev) {
  TORCH_CHECK(dst != 0 && src != 0 && nbytes > 0);
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)dev);
  check((int)cudaMemcpyAsync(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), (size_t)nbytes, cudaMemcpyDeviceToDevice,
                             cur_stream()),
        "vmm_copy");
}
// uint8 tensor over a mapped allocation (the allocation outlives the tensor: it is freed explicitly by id)
Tensor vmm_tensor(int64_t id, int64_t nbytes, int64_t dev) {
  const int64_t p = mmb_vmm_ptr(id);
  TORCH_CHECK(p != 0 && nbytes > 0 && nbytes <= mmb_vmm_size(id), "vmm_tensor: unknown allocation or size out of range");
  return torch::from_blob(reinterpret_cast<void*>(p), {nbytes}, [](void*) {},
                          torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, (int)dev));
}

TORCH_LIBRARY(mmb200, m) {
  m.def("fmha_prefill", &fmha_prefill);
  m.def("fp4_gemm_grouped", &fp4_gemm_grouped);
  m.def("bf16_gemm", &bf16_gemm);
  m.def("fp4_gemv", &fp4_gemv);
  m.def("fp4_moe_gemv", &fp4_moe_gemv);
  m.def("fp4_grouped_gemv", &fp4_grouped_gemv);
  m.def("bf16_gemv", &bf16_gemv);
  m.def("rmsnorm", &rmsnorm);
  m.def("silu_mul", &silu_mul);
  m.def("add", &add);
  m.def("mc_all_reduce", &mc_all_reduce);
  m.def("vmm_available", &vmm_available);
  m.def("vmm_create", &vmm_create);
  m.def("vmm_export_fd", &vmm_export_fd);
  m.def("vmm_import_fd", &vmm_import_fd);
  m.def("vmm_ptr", &vmm_ptr);
  m.def("vmm_size", &vmm_size);
  m.def("vmm_free", &vmm_free);
  m.def("vmm_tensor", &vmm_tensor);
  m.def("vmm_copy", &vmm_copy);
  m.def("vmm_close_fd", &vmm_close_fd);
  m.def("mc_create", &mc_create);
  m.def("mc_export_fd", &mc_export_fd);
  m.def("mc_import_fd", &mc_import_fd);
  m.def("mc_add_device", &mc_add_device);
  m.def("mc_bind", &mc_bind);
  m.def("mc_map", &mc_map);
  m.def("mc_unbind", &mc_unbind);
  m.def("embedding", &embedding);
  m.def("rope", &rope);
  m.def("qk_norm_rope_cache", &qk_norm_rope_cache);
  m.def("mla_prep", &mla_prep);
  m.def("paged_decode", &paged_decode);
  m.def("decode_chain", &decode_chain);
  m.def("decode_chain_param_bytes", &decode_chain_param_bytes);
  m.def("set_status_word", &set_status_word);
  m.def("decode_merge", &decode_merge);
  m.def("moe_router", &moe_router);
  m.def("moe_select", &moe_select);
  m.def("sample", &sample);
  m.def("argmax", &argmax);
  m.def("tp_argmax", &tp_argmax);
  m.def("fp4_gemm", &fp4_gemm);
  m.def("fp4_gemm_swiglu", &fp4_gemm_swiglu);
  m.def("trellis_gemm", &trellis_gemm);
  m.def("fp4_gemm_grouped_swiglu", &fp4_gemm_grouped_swiglu);
  m.def("fp4_gemm_rs", &fp4_gemm_rs);
  m.def("tp_rs_finish", &tp_rs_finish);
  m.def("tp_rs_finish_norm", &tp_rs_finish_norm);
  m.def("fp4_gemm_ag", &fp4_gemm_ag);
  m.def("bf16_gemm_ag", &bf16_gemm_ag);
  m.def("tp_wait", &tp_wait);
  m.def("hadamard", &hadamard);
  m.def("gptq_block", &gptq_block);
  m.def("fp4_quantize_pack", &fp4_quantize_pack);
  m.def("trellis_dequant", &trellis_dequant);
  m.def("trellis_gemv", &trellis_gemv);
  m.def("trellis_moe", &trellis_moe);
  m.def("codebook_gemv", &codebook_gemv);
  m.def("codebook_gemm", &codebook_gemm);
  m.def("sparse24_gemm", &sparse24_gemm);
  m.def("vision_preprocess", &vision_preprocess);
  m.def("vision_preprocess_ex", &vision_preprocess_ex);
  m.def("channel_stats", &channel_stats);
  m.def("layernorm", &layernorm);
  m.def("spec_verify", &spec_verify);
  m.def("fp4_gemm_grouped_scatter", &fp4_gemm_grouped_scatter);
  m.def("ep_dispatch", &ep_dispatch);
  m.def("ep_recv_group", &ep_recv_group);
  m.def("ep_signal", &ep_signal);
  m.def("ep_combine", &ep_combine);
  m.def("moe_group", &moe_group);
  m.def("moe_gather", &moe_gather);
  m.def("moe_gather_n", &moe_gather_n);
  m.def("moe_combine", &moe_combine);
  m.def("prefill_attention", &prefill_attention);
  m.def("qk_norm_rope_cache_fp8", &qk_norm_rope_cache_fp8);
  m.def("kv_fp8_gather", &kv_fp8_gather);
  m.def("mla_prep_fp8", &mla_prep_fp8);
  m.def("paged_decode_fp8", &paged_decode_fp8);
  m.def("gated_delta_step", &gated_delta_step);
  m.def("selective_scan_step", &selective_scan_step);
  m.def("wkv_scan", &wkv_scan);
  m.def("gated_delta_scan", &gated_delta_scan);
  m.def("selective_scan", &selective_scan);
}
