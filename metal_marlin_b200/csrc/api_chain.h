// Decode chain: everything between two attention calls of a batch-1..8 decode step in ONE persistent launch.
//
// A decode layer of an MLA + MoE model is a chain of small dependent matrix-vector products; launched kernel by kernel
// each link pays a launch, a drain and a first-byte latency that together exceed its memory time several times over.
// This kernel runs the links as phases of one grid (one CTA per SM, 16 warps) separated by grid-wide barriers:
//
//   A  o_proj            attn_o [B, nh * dv]          -> delta_attn [B, H]
//   B  router logits     h_mid = h_in + delta_attn, RMSNorm(post_norm); gate logits [B, E]; the shared experts' gate|up rows
//   C  routed gate|up    top-k of the logits (every CTA selects for itself), SwiGLU       -> hmid [B, S, I]
//   D  down              weighted sum over the slots                                      -> delta_mlp [B, H]
//   E  q_a | kv_a        h_out = h_mid + delta_mlp, RMSNorm(in_norm)                      -> a [B, q_lora + R + dr]
//   F  q_b               RMSNorm(q_a) -> q [B, nh * (dn + dr)];  one CTA: RMSNorm(c_kv) | RoPE(k_rope) -> latent cache
//   G  absorb            q_nope through W_uk^T per head, RoPE(q_rope)                     -> q_full [B, nh, R + dr]
//
// Dense-MLP layers replace B..D by gate|up (SwiGLU) and down.  `phases` selects which links a launch runs (the first launch
// of a step runs E..G only, the last one A..D only).  Every barrier wait is bounded; on expiry a code (300 + phase) goes to
// the status word, an abort flag releases the other CTAs and the kernel returns.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  const void* q;             // tile-layout FP4 words (expert 0 of a bank)
  const void* s;             // tile-layout fp16 group scales
  int N, K, gs_shift;        // rows, columns (multiple of 64), log2(group size) (>= 6)
  long long stride_q;        // bank: distance between experts in 16-byte units (0 for a single matrix)
  long long stride_s;        // bank: distance between experts in 4-byte units
} MmbChainMat;

enum { MMB_CHAIN_A = 1, MMB_CHAIN_B = 2, MMB_CHAIN_C = 4, MMB_CHAIN_D = 8, MMB_CHAIN_E = 16, MMB_CHAIN_F = 32, MMB_CHAIN_G = 64 };

typedef struct {
  int B, H, phases;
  float eps;
  // ---- A
  const void* attn_o;        // bf16 [B, o.K]
  MmbChainMat o;
  void* delta_attn;          // bf16 [B, H]
  // ---- B..D
  const void* h_in;          // bf16 [B, H]
  void* h_mid;               // bf16 [B, H]
  const void* post_norm;     // bf16 [H]
  int moe;                   // 1: routed experts + shared experts; 0: dense MLP (gate_up / down are single matrices)
  const void* router_w;      // bf16 [E, H]
  const float* router_bias;  // fp32 [E] or null
  int E, topk, n_shared, scoring, renorm, n_group, topk_group;
  float routed_scale;
  float* logits;             // fp32 [B, E] scratch
  int* ids;                  // int32 [B, topk] out (also read back by phase C / D)
  float* weights;            // fp32 [B, topk] out
  MmbChainMat gate_up;       // N = 2 * I (gate rows, then up rows)
  MmbChainMat down;          // N = H, K = I
  void* hmid;                // bf16 [B, S, I] (S = topk + n_shared; dense: S = 1)
  void* delta_mlp;           // bf16 [B, H]
  // ---- E..G (next layer's attention prologue)
  void* h_out;               // bf16 [B, H]
  const void* in_norm;       // bf16 [H]
  MmbChainMat qa_kva;        // N = q_lora + R + dr
  void* a_out;               // bf16 [B, qa_kva.N]
  int q_lora;
  const void* q_a_norm;      // bf16 [q_lora]
  MmbChainMat q_b;           // N = nh * (dn + dr), K = q_lora
  void* q_out;               // bf16 [B, q_b.N]
  const void* kv_norm;       // bf16 [R]
  const void* w_ukT;         // bf16 [nh, R, dn]
  int nh, dn, dr, R;
  const int* positions;      // [B]
  const float* inv_freq;     // [dr / 2]
  const long long* slots;    // [B] cache slot of the new token (negative: not cached)
  void* cache;               // bf16 [num_slots, R + dr]
  float mscale;
  int interleaved;
  void* q_full;              // bf16 [B, nh, R + dr]
  // ---- synchronisation
  unsigned* sync;            // device words [4], zero between launches: arrival counter, exit counter, abort flag, spare
  int* status;               // optional status word (300 + phase index when a barrier wait ran out)
  int stage_k;               // widest staged row (host: max K over the phases that run); sizes the dynamic shared memory
  // Byte ranges requested into L2 when the launch ends (weights the kernels after it read first: W_uv of the attention
  // that follows, o_proj of the next launch).  Null / 0: none.
  const void* pf_ptr[2];
  long long pf_bytes[2];
} MmbChainParams;

// Launches the chain on min(#SMs, co-resident limit) CTAs (cooperative launch).  Returns a cudaError_t as int.
int mmb_decode_chain(const MmbChainParams* p, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
