// C ABI of the kernel library: plain structs + extern "C" launchers.
// Every launcher takes raw device pointers and a stream, launches asynchronously and
// returns a cudaError_t value as int (0 = success).  No launcher allocates memory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ----------------------------------------------------------------------------- tensor-parallel exchange
// Optional in-kernel exchange of row-parallel partial sums over NVLink peer memory (see tp_comm.cuh).
// `in`: this kernel consumes the sum of tp partial slots as its residual delta.
// `out`: this kernel produces a partial and pushes it into every peer's receive buffer.
typedef struct {
  const float* in_buf;              // local fp32 [tp][in_slot_stride] (null = no consumption)
  const unsigned* in_flags;         // local [tp]
  long long in_slot_stride;
  float* const* out_peer_slots;     // device array [tp] (null = no production)
  unsigned* const* out_peer_flags;  // device array [tp]
  unsigned* out_counter;            // local, zero between launches
  const unsigned* step;             // device scalar, incremented once per decode step
  int* status;                      // optional error word
  int tp;
  float* out_mc_slot;               // optional: this rank's slot through the multicast (NVLS) mapping of the receive buffers;
                                    // when set, one multimem store per value replaces the tp peer stores
} MmbTpExchange;

// ----------------------------------------------------------------------------- FP4 small-M GEMV
// Weights are in the device tile layout: int32 [N/16][K/64][32][4]; scales fp16 [N/16][K/gs][8][2].
typedef struct {
  const void* qw;            // tile-layout weights (expert 0 for MoE banks)
  const void* sc;            // tile-layout scales
  const void* x;             // bf16 activations
  const void* delta;         // optional bf16, added to x before the norm (same ld as x)
  const void* norm_w;        // optional bf16 [Kx] RMSNorm weight applied to (x + delta)
  void* resid_out;           // optional bf16 [M, Kx]: receives x + delta (written by blockIdx.x == 0)
  void* out;                 // bf16 output
  const void* bias;          // optional bf16 [N]
  const void* out_add;       // optional bf16, added to the output (same ld as out)
  int M, N, K, Kx;           // tokens, logical rows, padded K (multiple of 64), logical K
  int ldx, ldo;              // leading dimensions in elements
  int gs_shift;              // log2(group size); group size is a power of two >= 16
  float eps;
  int act;                   // 0 = none, 1 = rows [0,N/2) are gate, [N/2,N) are up: out[:, n] = silu(g) * u
  int mode;                  // 0 dense, 1 MoE gate-up (one CTA column per (token, slot)), 2 MoE down, 3 grouped MoE (tile list)
  const int* expert_ids;     // [M, topk] routed expert per slot (negative = skip)
  const float* expert_w;     // [M, topk] routing weights (mode 2)
  int topk, n_shared;        // slots per token = topk + n_shared; shared expert j has index shared_base + j
  int shared_base;
  long long expert_stride_q; // distance between experts in 16-byte units
  long long expert_stride_s; // distance between experts in 4-byte units
  MmbTpExchange tpx;         // all-zero = single GPU
  // mode 3: grouped MoE over a device-built tile list (rows of the work are sorted by expert).  Tile j covers sorted rows
  // tile_row0[j] .. + tile_rows[j] (<= 8) of expert tile_expert[j]; *n_tiles tiles are valid.  x is used as is (no add /
  // norm).  row_order (optional) holds the flat (token * order_div + slot) pair of every sorted row: with order_div > 0
  // the input row is gathered from x[pair / order_div], and with expert_w set the output row is scaled by
  // expert_w[pair] (routing weight of the down projection).
  const int* tile_expert;
  const int* tile_row0;
  const int* tile_rows;
  const int* n_tiles;
  const int* row_order;
  int order_div;
  int max_tiles;
  int grouped_wpt, grouped_upi;   // 0 = chosen by the launcher; warps per unit (1, 2, 4, 8) and units per item and group
} MmbFp4GemvParams;

int mmb_fp4_gemv(const MmbFp4GemvParams* p, cudaStream_t stream);

// bf16 weights [N, K] row major, x bf16 [M, ldx] (M <= 8 per CTA row), out fp32 or bf16.
typedef struct {
  const void* w;
  const void* x;
  const void* delta;         // optional, added to x
  const void* norm_w;        // optional RMSNorm weight
  void* out;
  int M, N, K, ldx, ldo;
  float eps;
  int out_f32;
  MmbTpExchange tpx;         // consumer side only
} MmbBf16GemvParams;
int mmb_bf16_gemv(const MmbBf16GemvParams* p, cudaStream_t stream);

// ----------------------------------------------------------------------------- elementwise
int mmb_rmsnorm(const void* x, const void* delta, const void* w, void* out, void* resid_out, int rows, int dim,
                int ldx, int ldo, float eps, cudaStream_t stream);
// LayerNorm over the last axis (bf16 in / out, fp32 statistics): out = ((x + delta) - mean) * rstd * w + b; w, b, delta and
// resid_out optional (resid_out receives x + delta).
int mmb_layernorm(const void* x, const void* delta, const void* w, const void* b, void* out, void* resid_out, int rows, int dim, int ldx,
                  int ldo, float eps, cudaStream_t stream);
int mmb_silu_mul(const void* gate_up, void* out, int rows, int inter, cudaStream_t stream);
int mmb_add(const void* a, const void* b, void* out, long long n, cudaStream_t stream);
int mmb_embedding(const void* table, const int64_t* ids, void* out, int n, int dim, cudaStream_t stream);
// RoPE on q [T, Hq, D] and k [T, Hk, D] in place.  interleaved = 1 rotates pairs (2i, 2i+1), else (i, i+D/2).
int mmb_rope(void* q, void* k, const int* positions, const float* inv_freq, int T, int Hq, int Hk, int D,
             int rot_dim, int ldq, int ldk, int interleaved, float mscale, cudaStream_t stream);
// Per-head RMSNorm (Qwen3 q/k norm) fused with RoPE, then K/V scatter into a paged pool.
// Quantized variant of the K / V scatter: pools of 8- or 4-bit codes plus one fp32 scale per (slot, head); `kv_fmt`: 0 FP8
// E4M3, 1 INT8, 2 FP4 E2M1, 3 INT4 (kv_quant.cuh; the 4-bit formats hold two values per byte, rows of D / 2 bytes).
int mmb_qk_norm_rope_cache_fp8(void* q, const void* k, const void* v, const void* qn_w, const void* kn_w, const int* positions,
                               const float* inv_freq, const int64_t* slots, void* k_pool, void* v_pool, float* k_scale,
                               float* v_scale, int T, int Hq, int Hk, int D, int ldqkv, float eps, int interleaved, int kv_fmt,
                               cudaStream_t stream);
// Paged FP8 rows -> contiguous bf16 rows (prompt passes over a quantized cache): out[cu_k[b] + t, h, :] = pool row of token t
// of sequence b times its scale.
int mmb_kv_fp8_gather(const void* pool, const float* scale, const int* block_tables, const int* ctx_lens, const int* cu_k,
                      void* out, int B, int Hkv, int D, int block_size, int max_blocks, int max_ctx, int kv_fmt, cudaStream_t stream);
int mmb_qk_norm_rope_cache(void* q, const void* k, const void* v, const void* qn_w, const void* kn_w,
                           const int* positions, const float* inv_freq, const int64_t* slots, void* k_pool,
                           void* v_pool, int T, int Hq, int Hk, int D, int ldqkv, float eps, int interleaved,
                           cudaStream_t stream);

// ----------------------------------------------------------------------------- MLA
// Per token: q_nope [H, dn] absorbed through W_ukT [H, R, dn] into q_full[:, :R]; RoPE(q_rope) into
// q_full[:, R:]; and (block H) c_kv RMSNorm + RoPE(k_rope) scattered into the paged latent cache.
typedef struct {
  const void* q;            // bf16 [T, H, dn + dr]
  const void* kva;          // bf16 [T, ld_kva]: [c_kv (R) | k_rope (dr)]
  const void* w_ukT;        // bf16 [H, R, dn]
  const void* kv_norm_w;    // bf16 [R]
  const int* positions;     // [T]
  const float* inv_freq;    // [dr/2]
  const int64_t* slots;     // [T] flat slot (block * block_size + offset) in the latent cache; negative = skip
  void* q_full;             // bf16 [T, H, R + dr]
  void* cache;              // bf16 [num_slots, R + dr]
  int T, H, dn, dr, R, ld_q, ld_kva;
  float eps, mscale;
  int interleaved;
  int skip_absorb;          // 1: leave q_full[:, :, :R] untouched (prefill uses the non-absorbed form), only RoPE + cache write
  float* cache_scale;       // quantized cache: cache holds codes [num_slots, (R + dr) or (R + dr) / 2 bytes], cache_scale fp32 [num_slots]
  int cache_fmt;            // format of a quantized cache (0 FP8 E4M3, 1 INT8, 2 FP4 E2M1, 3 INT4)
} MmbMlaPrepParams;
int mmb_mla_prep(const MmbMlaPrepParams* p, cudaStream_t stream);

// Paged decode attention with grouped heads sharing one KV head (MLA: all heads, K = latent, V = K[:, :dv]).
typedef struct {
  const void* q;            // bf16 [B, Hq, dqk]
  const void* k_pool;       // bf16 [num_slots, Hkv, dqk]  (slot major)
  const void* v_pool;       // bf16 [num_slots, Hkv, dv] or null when V is the first dv columns of K
  const int* block_tables;  // [B, max_blocks]
  const int* ctx_lens;      // [B]
  float* part_o;            // fp32 [B, Hq, splits, dv]
  float* part_ml;           // fp32 [B, Hq, splits, 2] (running max, sum)
  int B, Hq, Hkv, dqk, dv, block_size, max_blocks, splits;
  float scale;
  int window;               // 0 = full; >0 = attend to the last `window` tokens only
  int* status;              // optional device word: set non-zero when a bounded wait inside the kernel expired
  // FP8 (E4M3) pools: k_pool / v_pool hold one byte per element and k_scale / v_scale fp32 [num_slots, Hkv] the scale of
  // every (token, head) row; rows are expanded to bf16 in shared memory after they land.  Null scales = bf16 pools.
  const float* k_scale;
  const float* v_scale;
  int kv_fmt;               // with scales: 0 FP8 E4M3, 1 INT8, 2 FP4 E2M1, 3 INT4 (4-bit rows hold dqk / 2 and dv / 2 bytes)
} MmbPagedDecodeParams;
int mmb_paged_decode(const MmbPagedDecodeParams* p, cudaStream_t stream);
// Merge the split partials; optional per-head up projection W_uv [Hq, dvo, dv] (MLA), output bf16 [B, Hq, dvo or dv].
int mmb_decode_merge(const float* part_o, const float* part_ml, const void* w_uv, void* out, int B, int Hq, int dv,
                     int dvo, int splits, cudaStream_t stream);

// ----------------------------------------------------------------------------- MoE router
typedef struct {
  const void* w;             // bf16 [E, K] router weight
  const void* x;             // bf16 [T, K]
  const void* delta;         // optional
  const void* norm_w;        // optional
  void* resid_out;           // optional: x + delta
  const float* bias;         // optional e_score_correction_bias [E] (sigmoid mode)
  int* ids;                  // [T, topk]
  float* weights;            // [T, topk]
  float* logits_out;         // optional fp32 [T, E]
  int* counts;               // optional [E] histogram (atomicAdd)
  int T, E, K, topk;
  float eps;
  int scoring;               // 0 softmax -> topk -> renorm(optional), 1 sigmoid (+bias for choice) -> topk -> renorm
  int renorm;
  float routed_scale;
  int n_group, topk_group;   // grouped top-k (DeepSeek/GLM); n_group <= 1 disables
  MmbTpExchange tpx;         // consumer side only
} MmbRouterParams;
int mmb_moe_router(const MmbRouterParams* p, cudaStream_t stream);
// Selection only: gate logits fp32 [T, E] are given (computed by a GEMM); uses the scoring / top-k fields of `p`.
int mmb_moe_select(const MmbRouterParams* p, const float* logits_in, cudaStream_t stream);

// ----------------------------------------------------------------------------- sampling
typedef struct {
  const float* logits;       // [B, V]
  int64_t* out_ids;          // [B]
  float* out_logprob;        // optional [B]
  const float* temperature;  // optional [B] (null or <= 0 = greedy)
  const int* top_k;          // optional [B] (<= 0 disables)
  const float* top_p;        // optional [B] (>= 1 disables)
  const float* min_p;        // optional [B]
  const int64_t* history;    // optional [B, hist_len] token ids for the repetition penalty (negative = pad)
  const float* rep_penalty;  // optional [B]
  int B, V, hist_len;
  unsigned long long seed, offset;
  const int64_t* offset_dev; // optional device scalar added to offset (lets a captured graph advance the RNG)
  const int64_t* seed_dev;   // optional per-row seeds [B] on the device (replace `seed`)
} MmbSampleParams;
int mmb_sample(const MmbSampleParams* p, cudaStream_t stream);
int mmb_argmax(const float* logits, int64_t* out, int B, int V, cudaStream_t stream);
// Vocab-parallel greedy head (tensor parallel): logits [B, Vloc] is this rank's vocabulary shard.
int mmb_tp_argmax(const float* logits, int64_t* out, int B, int Vloc, int vocab_offset, const MmbTpExchange* x,
                  cudaStream_t stream);

#ifdef __cplusplus
}
#endif
