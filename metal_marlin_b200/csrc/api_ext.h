// C entry points of the secondary kernels: trellis (2-8 bit codebook) weights, Hadamard rotation, generic
// group-quantized GEMV (INT4 / INT8 / FP8 / NF4 / sub-4-bit), vision preprocessing, speculative verification.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Orthonormal Walsh-Hadamard transform of consecutive `block`-wide slices (block a power of two, 2..1024) of every
// row of x bf16 [rows, dim]; out may alias x.
int mmb_hadamard(const void* x, void* out, int rows, int dim, int block, cudaStream_t stream);

// GPTQ over one lazy block of columns [i1, i1 + B), B <= 128: for every row and every column in order, quantize
// W[r, c] to grid[k] * col_scale[r, c] (nearest grid value, ties to the lower one; grid sorted, 2..256 values), store it in
// Q, store err = (w - q) / Hinv[c, c] in E [out_f, B] and subtract err * Hinv[c, c'] from the later columns c' of the
// block.  W, Q, col_scale fp32 with row stride ldw; Hinv fp32 upper Cholesky factor of the inverse Hessian, row stride ldh;
// err_rows fp32 [out_f] accumulates the squared quantization error of each row.  Plain fp32 roundings, no fused
// multiply-add, so the result equals the PyTorch loop bit for bit.
int mmb_gptq_block(float* W, float* Q, float* E, const float* Hinv, const float* col_scale, const float* grid,
                   float* err_rows, int n_grid, int out_f, long ldw, long ldh, int i1, int B, cudaStream_t stream);
// Round-to-nearest E2M1 quantization of w [out_f, in_f] (fp32, or bf16 when w_is_bf16) with one fp16 scale = absmax / 6
// per group of group_size (8..128, a power of two) input columns, packed eight codes per word along the input axis:
// packed uint32 [out_f, in_f / 8], scales fp16 [out_f, in_f / group_size].
int mmb_fp4_quantize_pack(const void* w, int w_is_bf16, uint32_t* packed, void* scales, long out_f, int in_f, int group_size,
                          cudaStream_t stream);

// Trellis weights.  `codes`: the 16x16-tile bit stream without its header byte ([tiles_out][tiles_in][32 * bits]
// bytes, codes LSB first, code index local_out * 16 + local_in); scales fp32 [n_groups, out]; su fp32 [in];
// sv fp32 [out].  W[o, i] = (code - (2^bits - 1) / 2) * 1.24371088 * scales[i / gs, o] * sv[o] * su[i].
int mmb_trellis_dequant(const uint8_t* codes, const float* scales, const float* su, const float* sv, void* out_bf16,
                        int out_f, int in_f, int bits, int group_size, cudaStream_t stream);
// y bf16 [M, out] = x bf16 [M, in] W^T for M <= 4 (decode), straight from the bit stream.
// One trellis matrix as the MoE kernels see it (device pointers; 48 bytes, built once per expert bank).
typedef struct {
  const uint8_t* codes;     // header-less tile bit stream
  const float* scales;      // [in / gs, out]
  const float* su;          // [in]
  const float* sv;          // [out]
  int out_f, in_f, bits, gs;
} MmbTrellisMat;
// Routed experts of a trellis MoE layer for T <= a few tokens: mats[e * 3 + {0, 1, 2}] = gate, up, down of expert e (any
// bits 2..8 per matrix); ids int32 [T, topk] (negative = skip), wts fp32 [T, topk]; h bf16 [T * topk, inter] scratch;
// y fp32 [T * topk, hidden] receives w * down(silu(gate(x)) * up(x)) per slot (x already normalized).
int mmb_trellis_moe(const void* x, const MmbTrellisMat* mats, const int* ids, const float* wts, void* h, float* y, int T, int topk,
                    int hidden, int inter, int ldx, cudaStream_t stream);
int mmb_trellis_gemv(const void* x, const uint8_t* codes, const float* scales, const float* su, const float* sv, void* y,
                     int M, int out_f, int in_f, int bits, int group_size, int ldx, int ldy, cudaStream_t stream);

// Group-quantized GEMV for the integer / codebook formats: codes uint8 [out, in] (one code per byte on the device),
// scales fp16 [out, in / gs], optional zeros fp16 [out, in / gs], `lut` fp32 [256] maps a code to its value before
// scaling (identity for integers, the E4M3 / NF4 / NF3 tables otherwise).  w = (lut[code] - zero) * scale.
// y bf16 [M, out] = x bf16 [M, in] W^T, M <= 8.  `bits` in {2, 4, 8}: codes packed LSB-first along the input axis.
int mmb_codebook_gemv_bits(const void* x, const uint8_t* codes, const void* scales, const void* zeros, const float* lut, void* y,
                           int M, int out_f, int in_f, int group_size, int bits, int ldx, int ldy, cudaStream_t stream);
// the 8-bit (one code per byte) form
int mmb_codebook_gemv(const void* x, const uint8_t* codes, const void* scales, const void* zeros, const float* lut, void* y,
                      int M, int out_f, int in_f, int group_size, int ldx, int ldy, cudaStream_t stream);

// Vision preprocessing: bilinear resize of uint8 HWC images [B, H, W, 3] to [out_h, out_w], per-channel
// (x / 255 - mean) / std, written either as bf16 CHW [B, 3, out_h, out_w] (patch == 0) or as flattened patches
// bf16 [B, (out_h / patch) * (out_w / patch), 3 * patch * patch] (channel-major inside a patch).
// General image preprocessing: crop rectangle, resampling mode (0 bilinear, 1 bicubic, 2 nearest), normalisation, CHW or
// patch output, patches optionally ordered by merge x merge groups.
int mmb_vision_preprocess_ex(const uint8_t* images, void* out, int B, int H, int W, int crop_y, int crop_x, int crop_h, int crop_w,
                             int out_h, int out_w, int patch, int merge, int mode, const float* mean3, const float* std3, cudaStream_t stream);
// fp32 [B, 3, 2]: mean and standard deviation of pixel / 255 per image and channel.
int mmb_channel_stats(const uint8_t* images, float* out, int B, int H, int W, cudaStream_t stream);
int mmb_vision_preprocess(const uint8_t* images, void* out, int B, int H, int W, int out_h, int out_w, int patch,
                          const float* mean3, const float* std3, cudaStream_t stream);

// Speculative verification (rejection sampling).  Per sequence b and draft position j < K: accept while
// u[b, j] < p_target[b, j, tok] / p_draft[b, j, tok]; at the first rejection sample from normalize(max(p_target -
// p_draft, 0)) with u_resample[b]; when all K are accepted sample the bonus token from p_target[b, K].
// p_target fp32 [B, K + 1, V], p_draft fp32 [B, K, V], draft int64 [B, K]; out_tokens int64 [B, K + 1] (-1 padded),
// out_accepted int32 [B].
int mmb_spec_verify(const float* p_target, const float* p_draft, const int64_t* draft, const float* u, const float* u_resample,
                    int64_t* out_tokens, int* out_accepted, int B, int K, int V, cudaStream_t stream);

// Recurrent layers, one decode step.  Gated delta rule: q, k bf16 [B, H, dk], v bf16 [B, H, dv], g (log decay) and beta fp32
// [B, H], state fp32 [B, H, dk, dv] updated in place, out bf16 [B, H, dv].
int mmb_gated_delta_step(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state, void* out,
                         int B, int H, int dk, int dv, float scale, cudaStream_t stream);
// Mamba selective scan: x bf16 [B, D], dt fp32 [B, D] (after softplus), A fp32 [D, N] (negative), Bm / Cm fp32 [B, N], optional
// skip Dskip fp32 [D], state fp32 [B, D, N] updated in place, y bf16 [B, D].
// Whole-sequence scans (recurrent_scan.cu); every tensor fp32 and contiguous, the state is updated in place.
//   WKV: r, k [B, T, H, dk], v [B, T, H, dv], u [H, dk], w addressed as w[b * w_bstride + t * w_tstride + h * dk + i]
//   (v6: per-token decay, strides T * H * dk and H * dk; v5: per-head decay, both strides 0), state [B, H, dk, dv].
int mmb_wkv(const float* r, const float* k, const float* v, const float* w, const float* u, float* state, float* out, int B, int T,
            int H, int dk, int dv, long long w_bstride, long long w_tstride, cudaStream_t stream);
int mmb_gated_delta_scan(const float* q, const float* k, const float* v, const float* g, const float* beta, float* state, float* out,
                         int B, int T, int H, int dk, int dv, float scale, cudaStream_t stream);
int mmb_selective_scan(const float* x, const float* dt, const float* A, const float* Bm, const float* Cm, const float* Dskip,
                       float* state, float* y, int B, int T, int D, int N, cudaStream_t stream);
int mmb_selective_scan_step(const void* x, const float* dt, const float* A, const float* Bm, const float* Cm, const float* Dskip,
                            float* state, void* y, int B, int D, int N, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
// Prefill (multi-query) attention with online softmax, causal / sliding-window (+ global tokens) / tree / block-sparse
// masks, grouped KV heads and variable
// sequence lengths.  Queries of sequence b are rows cu_q[b] .. cu_q[b + 1] of q and attend to that sequence's keys:
// either contiguous rows cu_k[b] .. cu_k[b + 1] of k / v, or (cu_k == null) the paged pool addressed through
// block_tables [B, max_blocks] with ctx_lens[b] keys.  The q rows are the LAST q_len positions of the kv_len keys.
// All strides in elements.  D == DV in {64, 128, 256}.
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  long long q_tok_stride, q_head_stride, k_tok_stride, k_head_stride, v_tok_stride, v_head_stride, o_tok_stride, o_head_stride;
  const int* cu_q;
  const int* cu_k;
  const int* block_tables;
  const int* ctx_lens;
  int max_blocks, block_size;
  int B, Hq, Hk, D, max_q;
  float scale;
  int window;      // 0 = none; > 0: a query sees the last `window` keys up to its own position
  int causal;
  // further mask modes (all optional, combined with the above by AND):
  int sinks;                        // with a window: the first `sinks` keys stay visible to every query (global tokens)
  const unsigned char* tree_mask;   // [total q rows][tree_ld]: query row i sees key q_off + j iff tree_mask[i][j] != 0; keys
  int tree_ld;                      //   before q_off (the committed context) stay visible (speculative token trees)
  const unsigned char* block_mask;  // [block_heads (1 or Hq)][ceil(max_q / 128)][n_kblocks]: 128-query x 64-key blocks
  int block_heads, n_kblocks;       //   with a zero byte are skipped entirely (block-sparse attention)
} MmbPrefillAttnParams;
int mmb_prefill_attention(const MmbPrefillAttnParams* p, cudaStream_t stream);
#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
// MoE dispatch helpers (see moe_dispatch.cu).  ids int32 [n = T * topk]; order / inv int32 [n]; tile arrays int32 [max_tiles].
int mmb_moe_group(const int* ids, int n, int E, int token_tile, int max_tiles, int* order, int* inv, int* tile_expert, int* tile_row0,
                  int* tile_rows, int* n_tiles, cudaStream_t stream);
// n_dev: optional device int; only the first min(n, *n_dev) rows are gathered (the rest of xs is left as it is)
int mmb_moe_gather(const void* x, const int* order, void* xs, int n, int topk, int K, int ldx, const int* n_dev, cudaStream_t stream);
int mmb_moe_combine(const void* y, const int* inv, const void* add0, const void* add1, void* out, int T, int topk, int N, cudaStream_t stream);
#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
// Expert-parallel token exchange over peer memory (see ep_comm.cu).  Every rank owns, in memory all peers can address:
//   recv_x    bf16 [ep][cap][H]   rows sent by rank src land in region src
//   recv_meta int  [ep][cap][2]   (local expert id, pair index t * topk + slot at the sender)
//   recv_cnt  int  [ep]           rows rank src sent this step
//   ret_y     bf16 [cap][H]       expert outputs of this rank's own pairs, written by the expert owners
//   flags     u32  [2][ep]        [0][src] dispatch of src arrived, [1][dst] returns of dst arrived (step numbers)
typedef struct {
  const void* x;                   // bf16 [T, H] local tokens (already normalized)
  int ldx;
  const int* ids;                  // int32 [T, topk] global expert ids, negative = dropped
  int T, topk, H;
  int experts_per_rank, ep, rank, cap;
  void* const* peer_recv_x;        // device arrays [ep]: bases on rank d
  int* const* peer_recv_meta;
  int* const* peer_recv_cnt;
  unsigned* const* peer_flags;     // flags[0][rank] on rank d
  int* send_cnt;                   // local int [ep], zero before and after the launch
  unsigned* counter;               // local CTA completion counter, zero before and after
  const unsigned* step;
  int* status;                     // 120: more than cap rows for one destination
} MmbEpDispatchParams;
int mmb_ep_dispatch(const MmbEpDispatchParams* p, cudaStream_t stream);

typedef struct {
  const int* recv_meta;            // local
  const int* recv_cnt;
  const unsigned* flags;           // local flags[0][*]
  const unsigned* step;
  int* status;                     // 121 + src: dispatch of rank src did not arrive within the limit
  int ep, cap, H, E_local, token_tile, max_tiles;
  const long long* ret_peer;       // device [ep]: address of ret_y on rank src
  int* order;                      // [ep * cap]: sorted position -> row of recv_x (-1 padded)
  long long* row_dst;              // [ep * cap]: sorted position -> address of the row's slot in the sender's ret_y (0 padded)
  int* tile_expert;
  int* tile_row0;
  int* tile_rows;
  int* n_tiles;                    // [2]: tiles, rows received in all
  int n_rows_max;                  // length of order / row_dst (0: ep * cap).  More rows than this: status 120, no tile is run
} MmbEpRecvParams;
int mmb_ep_recv_group(const MmbEpRecvParams* p, cudaStream_t stream);

// Publishes `step` in flags[1][rank] of every peer after everything earlier in the stream (the down projection whose
// epilogue stored into the peers' ret_y) is complete.
int mmb_ep_signal(unsigned* const* peer_flags, const unsigned* step, int ep, cudaStream_t stream);

typedef struct {
  const void* ret_y;               // local bf16 [T * topk, N]
  const int* ids;                  // [T, topk] (negative = dropped)
  const float* weights;            // fp32 [T, topk]
  const void* add0;                // optional bf16 [T, N]
  const void* add1;
  void* out;                       // bf16 [T, N]
  int T, topk, N, ep;
  const unsigned* flags;           // local flags[1][*]
  const unsigned* step;
  int* status;                     // 140 + dst: returns of rank dst did not arrive within the limit
} MmbEpCombineParams;
int mmb_ep_combine(const MmbEpCombineParams* p, cudaStream_t stream);
#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
// Causal prefill attention of ONE sequence on the tcgen05 tensor cores (see attention_fmha_sm100.cu).
// q [t, Hq, D], k [n, Hk, D] (element strides given), vt [Hk, D, n_pad] = V transposed per head with n_pad % 8 == 0 and
// zeros behind column n; out [t, Hq, D] bf16.  Query row i sits at key position n - t + i.  D is 128 or 256.
typedef struct {
  const void* q;
  const void* k;
  const void* vt;
  void* out;
  int t, n, n_pad, Hq, Hk, D;
  long long q_tok_stride, q_head_stride, k_tok_stride, k_head_stride, o_tok_stride, o_head_stride;
  float scale;
  int window;             // 0 = none; > 0: query position x sees the keys (x - window, x]
  int* status;            // device int: 31..36 after a bounded wait expired (producer, mma, softmax stages)
} MmbFmhaPrefillParams;
int mmb_fmha_prefill(const MmbFmhaPrefillParams* p, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
