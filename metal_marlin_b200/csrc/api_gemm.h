// C ABI of the tcgen05 (sm_100a) GEMM kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// All-gather fused into the GEMM's activation load: token row t of x is written into this GPU's memory by rank
// t / rows (peer stores of that rank's reduce kernel, see MmbRsFinishParams), which then publishes *step in flags[rank].
// The TMA producer of every CTA waits (bounded; on expiry the CTA aborts and status gets a code) for the owners of its
// token tile only, and token tiles are walked starting with this rank's own rows, so the transfer of the other
// ranks' rows overlaps the tiles that are already complete.
typedef struct {
  const unsigned* flags;    // local [tp] or null
  const unsigned* step;
  int tp, rank, rows;
} MmbAgWait;

// out[M, N] = x[M, Kx] * W^T with W in the FP4 device tile layout (see api.h).
// Grouped mode (MoE): tile_* describe, per token tile, which expert bank to use and which rows of
// the (expert-sorted) x / out it covers; all three arrays and n_tiles live in device memory so the
// host never waits for the routing result.
typedef struct {
  const void* x;            // bf16 [M, Kx] row major (16-byte aligned rows)
  const void* qw;           // tile-layout weights [(E,) N/16, K/64, 32, 4] int32
  const void* sc;           // tile-layout scales  [(E,) N/16, K/gs, 8, 2] fp16
  void* out;                // bf16 [M, ldo]
  int M, N, K, Kx, ldo;
  int gs_shift;
  int act;                  // 0 none; 1: rows [0,N/2) gate and [N/2,N) up are interleaved per 64-row half tile -> silu(g)*u
  int* status;              // device int[4]: [0] != 0 after a wait timed out (1 = producer, 2 = mma, 3 = dequant, 4 = epilogue)
  // grouped mode (all null/0 for a plain GEMM)
  const int* tile_expert;   // [max_tiles]
  const int* tile_row0;     // [max_tiles] first row of the tile in x / out
  const int* tile_rows;     // [max_tiles] valid rows in the tile (<= token tile)
  const int* n_tiles;       // device scalar
  int max_tiles;
  long long expert_stride_q;   // 16-byte units
  long long expert_stride_s;   // 4-byte units
  const float* row_scale;   // optional fp32 [M]: out row multiplied by it (routing weight)
  int token_tile;           // 0 = auto; else 32 / 64 / 128 / 256
  // Tensor-parallel reduce-scatter epilogue (row-parallel projection; all null / 0 on one GPU).  Token row t belongs
  // to rank t / rs_rows; this rank's fp32 partial of the row goes straight from the epilogue into slot `rs_rank` of
  // the owner's receive buffer fp32 [tp][rs_rows][N] (NVLink peer stores); the last CTA publishes the step number in
  // flag[rs_rank] on every peer.  `out` is not written in this mode.
  float* const* rs_peer_bufs;       // device array [tp]: base of rank r's receive buffer
  unsigned* const* rs_peer_flags;   // device array [tp]: flag[rs_rank] on rank r
  unsigned* rs_counter;             // local CTA completion counter (0 before and after the launch)
  const unsigned* rs_step;          // device scalar: current step number
  int rs_tp, rs_rank, rs_rows;
  MmbAgWait ag;                     // all-zero: x is complete when the kernel starts
  // Optional scatter epilogue (expert-parallel combine): row r of the result is stored as bf16 [N] at the address
  // out_rows[r] instead of out + r * ldo (0 = row not stored).  The addresses may lie in peer memory: the expert
  // outputs go straight from the epilogue into the token owners' return buffers over NVLink.
  const long long* out_rows;
  // Trellis weights (mmb_trellis_gemm): device table of matrix descriptors (see MmbTrellisMat in api_ext.h, 6 x int64 per
  // matrix), matrices per expert, and the first matrix of the projection (qw / sc / gs_shift are unused).
  const long long* tr_desc;
  int tr_stride, tr_first;
  // Codebook weights (mmb_codebook_gemm: INT8 / INT4 / INT2 with or without zero points, FP8, NF4 ...): qw = codes, row major
  // [N, K * bits / 8], LSB-first along K; sc = fp16 scales [N, K >> gs_shift]; w = (lut[code] - zero) * scale.
  const void* cb_zeros;     // fp16 [N, K >> gs_shift] or null
  const float* cb_lut;      // device float [256]
  int cb_bits;              // 2, 4 or 8
  // 2:4 sparse FP4 weights (mmb_sparse24_gemm): of every 4 consecutive input columns 2 are stored.  qw = E2M1 codes of the
  // kept values, row major [N, K / 4] bytes (two codes per byte, low nibble first); sp_meta = [N, K / 8] bytes, one nibble
  // per group of 4 columns (low nibble first): bits 0-1 position of the first kept value, bits 2-3 of the second; sc = fp16
  // scales [N, K >> gs_shift] over the dense columns.
  const void* sp_meta;
} MmbFp4GemmParams;

int mmb_fp4_gemm(const MmbFp4GemmParams* p, cudaStream_t stream);
// Same pipeline with trellis weights decoded inside the main loop (2..8 bits per matrix, mixed per expert and matrix).
int mmb_trellis_gemm(const MmbFp4GemmParams* p, cudaStream_t stream);
// Same pipeline with codebook weights (table look-up, zero point and group scale applied inside the main loop); plain mode only.
int mmb_codebook_gemm(const MmbFp4GemmParams* p, cudaStream_t stream);
// Same pipeline with 2:4 sparse FP4 weights: the kept values are scattered to their columns (zeros elsewhere) inside the main
// loop, so the matrix is read at 0.375 bytes per dense weight and no dense copy exists; plain mode only.
int mmb_sparse24_gemm(const MmbFp4GemmParams* p, cudaStream_t stream);

// out[M, N] = x[M, K] * W[N, K]^T, both bf16 row major (TMA for both operands), fp32 accumulate in TMEM.
// Batched over `batch` independent problems with element strides (0 = shared operand).
typedef struct {
  const void* x;
  const void* w;
  void* out;                // bf16 or fp32
  int M, N, K, ldo;
  int out_f32;
  int batch;
  long long x_batch_stride, w_batch_stride, out_batch_stride;   // elements
  int ldx, ldw;             // row strides in elements (multiples of 8)
  int* status;
  MmbAgWait ag;             // all-zero: x is complete when the kernel starts
} MmbBf16GemmParams;

int mmb_bf16_gemm(const MmbBf16GemmParams* p, cudaStream_t stream);

// Second half of the fused all-reduce of a row-parallel projection.  Waits (bounded) until every rank's partial of
// this rank's token rows has arrived, sums the tp slots in rank order, optionally adds a bf16 residual of the local
// rows, rounds to bf16 and stores the reduced rows into EVERY peer's gathered buffer bf16 [M, N] (all-gather by peer
// stores); the last CTA publishes the step in ag flag[rank] on every peer.
typedef struct {
  const float* in_buf;              // local fp32 [tp][rows][N]
  const unsigned* in_flags;         // local [tp]
  void* const* ag_peer_bufs;        // device array [tp]: base of rank r's gathered buffer
  unsigned* const* ag_peer_flags;   // device array [tp]: ag flag[rank] on rank r
  unsigned* counter;
  const unsigned* step;
  int* status;
  int tp, rank, rows, N, M;
  // Optional fused residual add + RMSNorm of the owned rows (sequence-parallel form of the layer boundary): with
  // norm_w set, h_new = bf16(resid + bf16(sum)) goes to every peer's ag_peer_bufs (the new residual stream) and
  // bf16(h_new * rstd * norm_w) to every peer's ag2_peer_bufs (the input of the next projection).
  const void* resid;                // bf16 [M, N] (only the owned rows are read) or null
  const void* norm_w;               // bf16 [N] or null
  void* const* ag2_peer_bufs;       // device array [tp] or null
  float eps;
} MmbRsFinishParams;
int mmb_tp_rs_finish(const MmbRsFinishParams* p, cudaStream_t stream);
// In-switch all-reduce of a symmetric fp32 buffer (tp_allreduce.cu): `mc` is the buffer's address through the NVSwitch
// multicast mapping, `peer_flags[r]` the base of rank r's flag words (arrive[tp] then done[tp]), `local_flags` this rank's.
typedef struct {
  float* mc;
  unsigned* const* peer_flags;      // device array [tp]
  const unsigned* local_flags;      // local [2 * tp]
  unsigned* step;                   // local device word, advanced by the kernel
  unsigned* counter;                // local CTA completion counter (0 before and after)
  int* status;
  long long n;                      // fp32 elements (multiple of 4)
  int tp, rank;
} MmbMcAllReduceParams;
int mmb_mc_all_reduce(const MmbMcAllReduceParams* p, cudaStream_t stream);
// Wait (bounded) until all tp ranks published `step` in `flags`; on expiry writes a code to `status`.
int mmb_tp_wait(const unsigned* flags, const unsigned* step, int* status, int tp, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
