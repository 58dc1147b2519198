"""Decoder-only transformer over the op layer: dense GQA (Llama / Qwen3), MLA + MoE
(GLM-4.7-Flash / DeepSeek) and GQA + MoE (Qwen3-MoE), always on a *paged* KV cache.

Parity: the reference's flagship model class ``MMFP4ForCausalLM`` is imported at
``metal_marlin/inference/mmfp4_pipeline.py:1843`` but absent from its tree; its layers are
``metal_marlin/layers/mmfp4_mla.py:149`` (MLA), ``metal_marlin/layers/mmfp4_moe.py:352`` (MoE),
``metal_marlin/layers/mmfp4_linear.py:600`` (linear) and, for dense models,
``metal_marlin/inference/pipeline.py:277-830`` (``MetalMarlinModel``).

Blackwell-first choices that differ from the reference:

* the residual stream is carried as ``(hidden, pending delta)``; the add and the RMSNorm that
  follow every sub-layer are fused into the *prologue* of the next weight-streaming kernel, so a
  decode layer is 9 launches (MLA + MoE) instead of ~40 dispatches;
* MLA decode uses the absorbed formulation on a post-norm / post-RoPE latent cache: the cache
  row is exactly what attention consumes (576 values), W_uk is applied to the query and W_uv to
  the merged output, so nothing is re-normalised or up-projected per cached token;
* the whole decode step (all layers, head, sampler) is captured in one CUDA graph.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from .. import ops
from ..ops import FP4ExpertBank, FP4Weight
from .config import ModelConfig


# ---------------------------------------------------------------------------------------------
# rotary frequencies (plain + YaRN)
# ---------------------------------------------------------------------------------------------
def rope_inv_freq(cfg: ModelConfig, rot_dim: int, device) -> Tuple[torch.Tensor, float]:
    """Returns (inv_freq fp32 [rot_dim/2], attention/mscale factor applied to cos and sin).
    YaRN follows the published NTK-by-parts rule.  Parity: reference ``metal_marlin/rope.py:44-250``."""
    base = float(cfg.rope_theta)
    idx = torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device)
    inv = 1.0 / (base ** (idx / rot_dim))
    rs = cfg.rope_scaling or {}
    kind = rs.get("rope_type", rs.get("type"))
    mscale = 1.0
    if kind == "linear":
        inv = inv / float(rs.get("factor", 1.0))
    elif kind == "yarn":
        factor = float(rs.get("factor", 1.0))
        orig = float(rs.get("original_max_position_embeddings", cfg.max_position_embeddings))
        beta_fast, beta_slow = float(rs.get("beta_fast", 32)), float(rs.get("beta_slow", 1))

        def corr_dim(n_rot):
            return (rot_dim * math.log(orig / (n_rot * 2 * math.pi))) / (2 * math.log(base))

        low = max(math.floor(corr_dim(beta_fast)), 0)
        high = min(math.ceil(corr_dim(beta_slow)), rot_dim - 1)
        ramp = ((torch.arange(rot_dim // 2, dtype=torch.float32, device=device) - low) / max(high - low, 1e-3)).clamp(0, 1)
        inv = inv / factor * ramp + inv * (1 - ramp)
        m, m_all = float(rs.get("mscale", 1.0)), float(rs.get("mscale_all_dim", 0.0))

        def ms(scale, mm):
            return 1.0 if scale <= 1 else 0.1 * mm * math.log(scale) + 1.0

        mscale = ms(factor, m) / ms(factor, m_all) if m_all else ms(factor, m)
    return inv.contiguous(), mscale


# ---------------------------------------------------------------------------------------------
# weights
# ---------------------------------------------------------------------------------------------
@dataclass
class LayerWeights:
    input_norm: torch.Tensor
    post_norm: torch.Tensor
    # GQA attention
    qkv: Optional[FP4Weight] = None
    qkv_bias: Optional[torch.Tensor] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    # MLA
    qa_kva: Optional[FP4Weight] = None        # rows [q_a (q_lora) | kv_a (kv_lora + rope)]  (or [q | kv_a] without q_lora)
    q_a_norm: Optional[torch.Tensor] = None
    q_b: Optional[FP4Weight] = None
    kv_a_norm: Optional[torch.Tensor] = None
    kv_b: Optional[FP4Weight] = None          # kept for prefill (non-absorbed) attention
    w_ukT: Optional[torch.Tensor] = None      # bf16 [H, R, dn]
    w_uv: Optional[torch.Tensor] = None       # bf16 [H, dv, R]
    kv_b_dense: Optional[torch.Tensor] = None  # bf16 [H * (dn + dv), R]: latent -> (k_nope | v) per head, for prefill
    o: Optional[FP4Weight] = None
    # dense MLP
    gate_up: Optional[FP4Weight] = None
    down: Optional[FP4Weight] = None
    # MoE
    router_w: Optional[torch.Tensor] = None
    router_bias: Optional[torch.Tensor] = None
    gate_up_bank: Optional[FP4ExpertBank] = None
    down_bank: Optional[FP4ExpertBank] = None
    # Gated DeltaNet (linear attention) mixer of hybrid stacks: in_proj rows [q | k | v | z | b | a], depthwise causal conv over
    # [q | k | v] (weights [C, K]), per-value-head decay parameters, gated RMSNorm weight [dv], out_proj
    lin_in: Optional[FP4Weight] = None
    lin_conv: Optional[torch.Tensor] = None
    lin_dt_bias: Optional[torch.Tensor] = None
    lin_A_log: Optional[torch.Tensor] = None
    lin_norm: Optional[torch.Tensor] = None
    lin_out: Optional[FP4Weight] = None
    # Mamba mixer of Jamba / Zamba style stacks: in_proj rows [x | z] (2 Di), depthwise causal conv [Di, K] + bias, x_proj rows
    # [dt (rank) | B (N) | C (N)], dt_proj [Di, rank] + bias, A_log [Di, N], D [Di], out_proj [H, Di]
    mamba_in: Optional[FP4Weight] = None
    mamba_conv: Optional[torch.Tensor] = None
    mamba_conv_b: Optional[torch.Tensor] = None
    mamba_x: Optional[FP4Weight] = None
    mamba_dt: Optional[torch.Tensor] = None
    mamba_dt_b: Optional[torch.Tensor] = None
    mamba_A_log: Optional[torch.Tensor] = None
    mamba_D: Optional[torch.Tensor] = None
    mamba_out: Optional[FP4Weight] = None
    # expert parallelism inside a tensor-parallel group: this rank's range of whole routed experts (0 = experts are width-sliced)
    ep_first: int = 0
    ep_local: int = 0
    ep_shared_local: int = 0


def absorb_kv_b(kv_b: FP4Weight, H: int, dn: int, dv: int, R: int, hadamard_block: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Split the dequantized kv_b projection ``[H * (dn + dv), R]`` into ``W_uk^T [H, R, dn]`` and
    ``W_uv [H, dv, R]`` (bf16) for absorbed-MLA decode.  Parity: reference
    ``metal_marlin/paged/mmfp4_paged_adapter.py:236-345``."""
    w = kv_b.dequantize(torch.float32)
    if hadamard_block:        # stored in a rotated input basis: W = W_rot . H
        from ..quant.hadamard import fwht
        w = fwht(w.reshape(w.shape[0], -1, hadamard_block)).reshape(w.shape)
    w = w.view(H, dn + dv, R)
    w_uk = w[:, :dn, :]
    return w_uk.transpose(1, 2).contiguous().to(torch.bfloat16), w[:, dn:, :].contiguous().to(torch.bfloat16)


# ---------------------------------------------------------------------------------------------
# paged KV storage
# ---------------------------------------------------------------------------------------------
class PagedKVStorage:
    """Device pools, one per layer.  MLA: ``[num_slots, R + dr]`` latent rows.  GQA: separate K and V
    pools ``[num_slots, Hkv, D]``.  A slot is ``block * block_size + offset``; block tables and slot
    mappings come from the host-side allocator (``kv/paged.py``)."""

    def __init__(self, cfg: ModelConfig, num_blocks: int, block_size: int, device, dtype=torch.bfloat16, kv_dtype: str = "bf16"):
        """``kv_dtype`` ``"fp8"`` / ``"int8"`` / ``"fp4"`` / ``"int4"``: pools of 8- or 4-bit codes with one scale per cached row
        (``ops.FP8KV``); written by the attention prologue kernels, expanded to bf16 inside the decode kernel."""
        self.cfg, self.num_blocks, self.block_size, self.kv_dtype = cfg, num_blocks, block_size, kv_dtype
        n_slots = num_blocks * block_size
        L = cfg.num_hidden_layers
        assert kv_dtype == "bf16" or kv_dtype in ops.KV_FORMATS, kv_dtype
        # hybrid stacks: recurrent (Gated DeltaNet) layers keep, per sequence, a convolution window and a state matrix instead
        # of cached keys.  The pools run parallel to the block pool and are addressed by the FIRST block of a sequence's block
        # table (unique among live sequences as long as blocks are not shared, which is why prefix sharing is off for them).
        self.rec = [None] * L
        if cfg.has_linear_layers:
            kd, vd = cfg.linear_num_key_heads * cfg.linear_key_head_dim, cfg.linear_num_value_heads * cfg.linear_value_head_dim
            for i in range(L):
                if cfg.layer_is_mamba(i):
                    self.rec[i] = (torch.zeros(num_blocks + 1, cfg.mamba_d_inner, cfg.mamba_d_conv - 1, dtype=torch.float32, device=device),
                                   torch.zeros(num_blocks + 1, cfg.mamba_d_inner, cfg.mamba_d_state, dtype=torch.float32, device=device))
                if cfg.layer_is_linear(i):
                    # one entry more than blocks: rows of a padded decode batch (slot -1) park their state there
                    self.rec[i] = (torch.zeros(num_blocks + 1, 2 * kd + vd, cfg.linear_conv_kernel_dim - 1, dtype=torch.float32, device=device),
                                   torch.zeros(num_blocks + 1, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim,
                                               dtype=torch.float32, device=device))
        if kv_dtype != "bf16":
            if cfg.is_mla:
                self.k = [ops.FP8KV(n_slots, (cfg.latent_dim,), device, kv_dtype) for _ in range(L)]
                self.v = [None] * L
            else:
                self.k = [ops.FP8KV(n_slots, (cfg.num_key_value_heads, cfg.dh), device, kv_dtype) for _ in range(L)]
                self.v = [ops.FP8KV(n_slots, (cfg.num_key_value_heads, cfg.dh), device, kv_dtype) for _ in range(L)]
        elif cfg.is_mla:
            self.k = [torch.zeros(n_slots, cfg.latent_dim, dtype=dtype, device=device) for _ in range(L)]
            self.v = [None] * L
        else:
            lin = [cfg.layer_is_recurrent(i) for i in range(L)]
            self.k = [None if lin[i] else torch.zeros(n_slots, cfg.num_key_value_heads, cfg.dh, dtype=dtype, device=device) for i in range(L)]
            self.v = [None if lin[i] else torch.zeros(n_slots, cfg.num_key_value_heads, cfg.dh, dtype=dtype, device=device) for i in range(L)]

    def snapshot_recurrent(self):
        """Copies of the recurrent-state pools (``None`` for a pure attention model).  A warm-up pass in front of a graph
        capture advances them - unlike cache rows, which a repeated pass rewrites with the same values - so the capture code
        restores them afterwards."""
        if not any(r is not None for r in self.rec):
            return None
        return [None if r is None else (r[0].clone(), r[1].clone()) for r in self.rec]

    def restore_recurrent(self, snap) -> None:
        if snap is None:
            return
        for r, s in zip(self.rec, snap):
            if r is not None:
                r[0].copy_(s[0])
                r[1].copy_(s[1])

    def bytes_per_token(self) -> int:
        cfg = self.cfg
        per = cfg.latent_dim if cfg.is_mla else 2 * cfg.num_key_value_heads * cfg.dh
        if self.kv_dtype != "bf16":       # one byte (or half a byte) per element + a 4-byte scale per row
            rows = 1 if cfg.is_mla else 2 * cfg.num_key_value_heads
            return ((per // 2 if self.kv_dtype in ("fp4", "int4") else per) + 4 * rows) * cfg.num_hidden_layers
        return per * 2 * cfg.num_hidden_layers


@dataclass
class BatchMeta:
    """Per-step batch description (all tensors on the model's device).

    ``positions [T] int32``, ``slots [T] int64`` (cache slot of every token, -1 = do not cache),
    ``block_tables [B, max_blocks] int32``, ``ctx_lens [B] int32`` (tokens visible to each sequence
    *including* this step's), ``cu_seqlens``: list of python ints delimiting the sequences inside
    the flattened token axis (prefill only), ``decode``: one token per sequence."""
    positions: torch.Tensor
    slots: torch.Tensor
    block_tables: torch.Tensor
    ctx_lens: torch.Tensor
    decode: bool = True
    cu_seqlens: Optional[List[int]] = None
    max_ctx: Optional[int] = None
    splits: Optional[int] = None
    ctx_lens_host: Optional[List[int]] = None
    attn_mask: Optional[torch.Tensor] = None     # [T, n_ctx] bool, single-sequence prefill only (tree verification)
    _dev_cache: Optional[dict] = None            # small device tensors derived from the host lists, built once per batch

    def dev_ints(self, key, values, device) -> torch.Tensor:
        """int32 device tensor of ``values``, cached under ``key``: a host list becomes a device tensor through a
        synchronous copy that drains the stream, so it must happen once per batch, not once per layer."""
        return self.cached(key, lambda: torch.tensor(list(values), dtype=torch.int32, device=device))

    def cached(self, key, make):
        """Per-batch memo for tensors every layer would otherwise rebuild (cache slots of a sequence, cumulative lengths)."""
        if self._dev_cache is None:
            self._dev_cache = {}
        t = self._dev_cache.get(key)
        if t is None:
            t = make()
            self._dev_cache[key] = t
        return t


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------
class Transformer:
    def __init__(self, cfg: ModelConfig, layers: List[LayerWeights], embed: torch.Tensor, final_norm: torch.Tensor,
                 lm_head: torch.Tensor):
        self.cfg = cfg
        self.layers = layers
        self.embed = embed
        self.final_norm = final_norm
        self.lm_head = lm_head
        self.device = embed.device
        rot = cfg.qk_rope_head_dim if cfg.is_mla else cfg.dh
        self.inv_freq, self.rope_mscale = rope_inv_freq(cfg, rot, self.device)
        self.scale = cfg.softmax_scale()
        self.mtp = None      # optional multi-token-prediction head (spec/mtp.py)
        # tensor parallelism (parallel/tp.py): a shard keeps only its local heads / vocabulary rows
        self._chain = None   # decode-chain runner (ops/chain.py); False once found unsupported for this model
        self.tp = None
        self.ep = None       # expert parallelism with replicated attention (parallel/ep.py::EPModelState)
        self.routing_hook = None     # optional callable(layer, expert_ids, router_probs)
        self.n_heads_local = cfg.num_attention_heads
        self.n_kv_heads_local = cfg.num_key_value_heads
        self.vocab_range = (0, cfg.vocab_size)

    # ------------------------------------------------------------------ tensor-parallel plumbing
    def _dargs(self, d) -> dict:
        """kwargs carrying the pending residual delta into the next op (tensor, or in-kernel exchange)."""
        if self.tp is not None:
            return self.tp.consume(d)
        return {"delta": d}

    def _norm_linear(self, h, d, W, norm_w, **kw):
        """``W(norm(h + d))`` and the new residual stream.  When ``d`` is a row-parallel projection whose partials sit
        with the row owners, the add and the norm run there on the owned rows only and the GEMM gathers while it
        loads (see ``parallel/tp.py``)."""
        eps = self.cfg.rms_norm_eps
        if self.tp is not None and getattr(d, "pending_rs", False):
            g = self.tp.finish_norm(d, h, norm_w, eps)
            return ops.linear(g.x, W, ag_wait=g, **kw), g.h
        new_h = torch.empty_like(h) if d is not None else None
        y = ops.linear(h, W, norm_w=norm_w, eps=eps, resid_out=new_h, **kw, **self._dargs(d))
        return y, (h if new_h is None else new_h)

    def _row_parallel(self, x, W, site: int):
        if self.tp is not None:
            return self.tp.row_parallel(x, W, site)
        return ops.linear(x, W)

    # ------------------------------------------------------------------ attention blocks
    def _attn_gqa(self, L: LayerWeights, li: int, h, d, kv: PagedKVStorage, meta: BatchMeta):
        cfg = self.cfg
        Hq, Hk, D = self.n_heads_local, self.n_kv_heads_local, cfg.dh
        T = h.shape[0]
        qkv, h = self._norm_linear(h, d, L.qkv, L.input_norm, bias=L.qkv_bias)
        q = qkv[:, : Hq * D]
        k = qkv[:, Hq * D: (Hq + Hk) * D]
        v = qkv[:, (Hq + Hk) * D:]
        ops.qk_norm_rope_cache(q, k, v, L.q_norm, L.k_norm, meta.positions, self.inv_freq, meta.slots, kv.k[li], kv.v[li],
                               Hq, Hk, D, cfg.rms_norm_eps, cfg.rope_interleave)
        if meta.decode:
            qc = q.contiguous().view(T, Hq, D)
            o = ops.paged_attention(qc, kv.k[li], kv.v[li], meta.block_tables, meta.ctx_lens, Hq=Hq, Hkv=Hk, dqk=D, dv=D,
                                    block_size=kv.block_size, scale=self.scale, window=cfg.sliding_window,
                                    splits=meta.splits, max_ctx=meta.max_ctx)
            o = o.reshape(T, Hq * D)
        else:
            o = self._prefill_attention_gqa(q.reshape(T, Hq, D), kv, li, meta)
        d = self._row_parallel(o, L.o, 2 * li)
        return h, d

    def _prefill_attention_gqa(self, q, kv: PagedKVStorage, li: int, meta: BatchMeta):
        """Causal attention of every prompt chunk against its sequence's cached keys (which already
        include this chunk).  Runs per sequence over gathered K/V."""
        cfg = self.cfg
        Hq, Hk, D = self.n_heads_local, self.n_kv_heads_local, cfg.dh
        out = torch.empty(q.shape[0], Hq * D, dtype=torch.bfloat16, device=q.device)
        bs = kv.block_size
        win = int(cfg.sliding_window or 0)

        def _first_key(t, n_ctx):
            # with a sliding window only the keys the chunk's first query can still see are gathered
            return max(0, n_ctx - t - win + 1) if win else 0

        def _rows(pool, b, lo, n_ctx):
            """bf16 rows ``[n_ctx - lo, Hk, D]`` of sequence ``b``'s cached keys or values (quantized pools are expanded by
            their gather kernel, with the window's leading rows cut off afterwards)."""
            if isinstance(pool, ops.FP8KV):
                cu_k = meta.cached(("cu_k1", n_ctx), lambda: torch.tensor([0, n_ctx], dtype=torch.int32, device=q.device))
                return ops.kv_fp8_rows(pool, meta.block_tables[b:b + 1], meta.ctx_lens[b:b + 1], cu_k, n_ctx, n_ctx, bs)[lo:]

            def _slots():
                tok = torch.arange(lo, n_ctx, device=q.device)
                return meta.block_tables[b, tok // bs].long() * bs + tok % bs
            return pool.view(-1, Hk, D)[meta.cached(("slots", b, lo, n_ctx), _slots)]

        if (meta.attn_mask is None and q.dtype == torch.bfloat16 and len(meta.cu_seqlens) == 2 and q.stride(2) == 1
                and ops.fmha_ok(q.shape[0], int(meta.ctx_lens_host[0]), D, D, q.device)):
            # one long sequence: its cache rows (this chunk included) gathered once, then the tcgen05 attention kernel
            n_ctx = int(meta.ctx_lens_host[0])
            lo = _first_key(q.shape[0], n_ctx)
            ops.fmha_prefill(q, _rows(kv.k[li], 0, lo, n_ctx), _rows(kv.v[li], 0, lo, n_ctx), out.view(-1, Hq, D), self.scale,
                             window=win)
            return out
        n_seq = len(meta.cu_seqlens) - 1
        if (meta.attn_mask is None and q.dtype == torch.bfloat16 and n_seq > 1 and q.stride(2) == 1
                and all(ops.fmha_ok(meta.cu_seqlens[b + 1] - meta.cu_seqlens[b], int(meta.ctx_lens_host[b]), D, D, q.device)
                        for b in range(n_seq))):
            # several long sequences: the tcgen05 attention kernel sequence by sequence (a launch per sequence costs
            # microseconds against the milliseconds of a prompt-size attention; the mma.sync kernel below is 4-5 x slower)
            for b in range(n_seq):
                s0, e0 = meta.cu_seqlens[b], meta.cu_seqlens[b + 1]
                n_ctx = int(meta.ctx_lens_host[b])
                lo = _first_key(e0 - s0, n_ctx)
                ops.fmha_prefill(q[s0:e0], _rows(kv.k[li], b, lo, n_ctx), _rows(kv.v[li], b, lo, n_ctx),
                                 out[s0:e0].view(-1, Hq, D), self.scale, window=win)
            return out
        if meta.attn_mask is None and q.dtype == torch.bfloat16:
            # one launch for all sequences: keys are read from the paged pool through the block table
            cu_q = meta.dev_ints("cu_q", meta.cu_seqlens, q.device)
            max_q = max(meta.cu_seqlens[i + 1] - meta.cu_seqlens[i] for i in range(len(meta.cu_seqlens) - 1))
            ops.prefill_attention(q, kv.k[li].view(-1, Hk, D), kv.v[li].view(-1, Hk, D), cu_q, block_tables=meta.block_tables,
                                  ctx_lens=meta.ctx_lens, block_size=bs, max_q=max_q, scale=self.scale, window=cfg.sliding_window,
                                  out=out.view(-1, Hq, D))
            return out
        if (meta.attn_mask is not None and q.dtype == torch.bfloat16 and len(meta.cu_seqlens) == 2 and q.is_cuda
                and D in ops.PREFILL_ATTN_DIMS and ops.native_available()):
            # token-tree verification: the committed context is fully visible, the last T keys through the given mask
            T = q.shape[0]
            n_ctx = int(meta.ctx_lens_host[0])
            tm = meta.attn_mask[:, n_ctx - T:].to(torch.uint8).contiguous()
            cu_q = meta.dev_ints("cu_q", meta.cu_seqlens, q.device)
            ops.prefill_attention(q, kv.k[li].view(-1, Hk, D), kv.v[li].view(-1, Hk, D), cu_q, block_tables=meta.block_tables,
                                  ctx_lens=meta.ctx_lens, block_size=bs, max_q=T, scale=self.scale, causal=False, tree_mask=tm,
                                  out=out.view(-1, Hq, D))
            return out
        for b in range(len(meta.cu_seqlens) - 1):
            s, e = meta.cu_seqlens[b], meta.cu_seqlens[b + 1]
            n_ctx = int(meta.ctx_lens_host[b])
            tok = torch.arange(n_ctx, device=q.device)
            slots = meta.block_tables[b, tok // bs].long() * bs + tok % bs
            K = kv.k[li][slots].transpose(0, 1).unsqueeze(0)       # [1, Hk, n, D]
            V = kv.v[li][slots].transpose(0, 1).unsqueeze(0)
            Q = q[s:e].transpose(0, 1).unsqueeze(0)                # [1, Hq, t, D]
            t = e - s
            mask = None
            if n_ctx != t or cfg.sliding_window:
                qpos = torch.arange(n_ctx - t, n_ctx, device=q.device).unsqueeze(1)
                kpos = tok.unsqueeze(0)
                mask = kpos <= qpos
                if cfg.sliding_window:
                    mask &= kpos > qpos - cfg.sliding_window
            if meta.attn_mask is not None:
                mask = meta.attn_mask
            o = F.scaled_dot_product_attention(Q, K, V, attn_mask=mask, is_causal=(mask is None), scale=self.scale,
                                               enable_gqa=(Hq != Hk))
            out[s:e] = o.squeeze(0).transpose(0, 1).reshape(t, Hq * D)
        return out

    def _attn_deltanet(self, L: LayerWeights, li: int, h, d, kv: PagedKVStorage, meta: BatchMeta):
        """Gated DeltaNet mixer (linear attention with the gated delta rule): ``in_proj -> causal depthwise conv + SiLU on
        [q | k | v] -> L2-normalised q, k -> S <- S exp(g) + k ((v - S^T k) beta)^T, o = S^T q -> RMSNorm(o) * silu(z) ->
        out_proj``.  The convolution window and the state matrix of every sequence live in ``kv.rec[li]`` at the index of
        the sequence's first cache block.  Prompt passes run the sequence-scan kernel per sequence (carrying the state from
        earlier chunks), decode steps the single-step kernel on the batch.  Parity: reference
        ``metal_marlin/kernels/qwen36_27b.py`` / ``src/qwen36_27b_decode.metal`` (DeltaNet decode path) and the DeltaNet
        fields of ``metal_marlin/trellis/config.py:75``."""
        from ..arch.deltanet import gated_delta_rule_chunked, gated_delta_step, l2norm
        cfg = self.cfg
        Hk, Hv, dk, dv, Kc = (cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim,
                              cfg.linear_conv_kernel_dim)
        kd, vd = Hk * dk, Hv * dv
        T = h.shape[0]
        proj, h = self._norm_linear(h, d, L.lin_in, L.input_norm)
        pf = proj.to(torch.float32)
        qkv, z, b, a = pf[:, : 2 * kd + vd], pf[:, 2 * kd + vd: 2 * kd + 2 * vd], pf[:, 2 * kd + 2 * vd: 2 * kd + 2 * vd + Hv], pf[:, 2 * kd + 2 * vd + Hv:]
        beta = torch.sigmoid(b)
        g = -torch.exp(L.lin_A_log.float()) * F.softplus(a + L.lin_dt_bias.float())
        conv_pool, state_pool = kv.rec[li]
        w = L.lin_conv.float()                                     # [C, Kc]
        first = meta.block_tables[:, 0].long()                     # pool index of every sequence
        if meta.decode:                                            # padding rows of a bucketed batch must not touch a live state
            first = torch.where(meta.slots >= 0, first, torch.full_like(first, conv_pool.shape[0] - 1))
        rep = Hv // Hk

        def heads(x_conv):
            q = l2norm(x_conv[..., :kd].reshape(*x_conv.shape[:-1], Hk, dk))
            k = l2norm(x_conv[..., kd: 2 * kd].reshape(*x_conv.shape[:-1], Hk, dk))
            v = x_conv[..., 2 * kd:].reshape(*x_conv.shape[:-1], Hv, dv)
            if rep > 1:
                q, k = q.repeat_interleave(rep, -2), k.repeat_interleave(rep, -2)
            return q, k, v

        if meta.decode:
            win = torch.cat([conv_pool.index_select(0, first), qkv.unsqueeze(-1)], -1)            # [B, C, Kc]
            xc = F.silu((win * w).sum(-1))
            conv_pool.index_copy_(0, first, win[..., 1:].contiguous())
            q, k, v = heads(xc)
            S = state_pool.index_select(0, first)
            o = gated_delta_step(q, k, v, g, beta, S, scale=dk ** -0.5).to(torch.float32)           # [B, Hv, dv]
            state_pool.index_copy_(0, first, S)
        else:
            o = torch.empty(T, Hv, dv, dtype=torch.float32, device=h.device)
            for bi in range(len(meta.cu_seqlens) - 1):
                s0, e0 = meta.cu_seqlens[bi], meta.cu_seqlens[bi + 1]
                t = e0 - s0
                idx = first[bi: bi + 1]
                fresh = int(meta.ctx_lens_host[bi]) == t                                            # the sequence starts in this pass
                hist = torch.zeros(1, 2 * kd + vd, Kc - 1, device=h.device) if fresh else conv_pool.index_select(0, idx)
                xin = torch.cat([hist[0], qkv[s0:e0].t()], -1)                                      # [C, Kc - 1 + t]
                xc = F.silu(F.conv1d(xin.unsqueeze(0), w.unsqueeze(1), groups=w.shape[0])[0].t())   # [t, C]
                conv_pool.index_copy_(0, idx, xin[:, -(Kc - 1):].unsqueeze(0).contiguous())
                q, k, v = heads(xc)
                S0 = None if fresh else state_pool.index_select(0, idx)
                os_, S = gated_delta_rule_chunked(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), g[s0:e0].unsqueeze(0), beta[s0:e0].unsqueeze(0),
                                                  S0, scale=dk ** -0.5)
                o[s0:e0] = os_[0].float()
                state_pool.index_copy_(0, idx, S.float())
        # gated RMSNorm per value head, then the output projection (the result is the pending residual delta)
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * L.lin_norm.float()
        o = (o * F.silu(z.reshape(T, Hv, dv))).reshape(T, vd).to(torch.bfloat16)
        return h, ops.linear(o, L.lin_out)

    def _attn_mamba(self, L: LayerWeights, li: int, h, d, kv: PagedKVStorage, meta: BatchMeta):
        """Mamba mixer (selective state space): ``in_proj -> [x | z]``, causal depthwise conv + SiLU on x, ``x_proj -> dt, B, C``,
        ``h_t = exp(dt_t A) h_{t-1} + dt_t B_t x_t``, ``y_t = C_t h_t + D x_t``, ``y * silu(z) -> out_proj``.  Convolution window and
        state per sequence live in ``kv.rec[li]`` like the DeltaNet state; prompt passes run the selective-scan kernel per
        sequence, decode steps the single-step kernel.  Parity: reference ``metal_marlin/architectures/mamba.py``,
        ``src/mamba_ssm.metal:204``."""
        from ..arch.mamba import selective_scan, selective_scan_step
        cfg = self.cfg
        Di, N, r, Kc = cfg.mamba_d_inner, cfg.mamba_d_state, cfg.mamba_rank, cfg.mamba_d_conv
        T = h.shape[0]
        xz, h = self._norm_linear(h, d, L.mamba_in, L.input_norm)
        xz = xz.to(torch.float32)
        x, z = xz[:, :Di], xz[:, Di:]
        conv_pool, state_pool = kv.rec[li]
        w, wb = L.mamba_conv.float(), L.mamba_conv_b.float()
        A = -torch.exp(L.mamba_A_log.float())
        first = meta.block_tables[:, 0].long()
        if meta.decode:
            first = torch.where(meta.slots >= 0, first, torch.full_like(first, conv_pool.shape[0] - 1))

        def ssm_inputs(xc):
            proj = ops.linear(xc.to(torch.bfloat16).contiguous(), L.mamba_x).to(torch.float32)
            dt = F.softplus(proj[:, :r] @ L.mamba_dt.float().t() + L.mamba_dt_b.float())
            return dt, proj[:, r: r + N], proj[:, r + N: r + 2 * N]

        if meta.decode:
            win = torch.cat([conv_pool.index_select(0, first), x.unsqueeze(-1)], -1)              # [B, Di, Kc]
            xc = F.silu((win * w).sum(-1) + wb)
            conv_pool.index_copy_(0, first, win[..., 1:].contiguous())
            dt, Bm, Cm = ssm_inputs(xc)
            S = state_pool.index_select(0, first)
            y = selective_scan_step(xc, dt, A, Bm, Cm, L.mamba_D.float(), S).to(torch.float32)
            state_pool.index_copy_(0, first, S)
        else:
            y = torch.empty(T, Di, dtype=torch.float32, device=h.device)
            for bi in range(len(meta.cu_seqlens) - 1):
                s0, e0 = meta.cu_seqlens[bi], meta.cu_seqlens[bi + 1]
                t = e0 - s0
                idx = first[bi: bi + 1]
                fresh = int(meta.ctx_lens_host[bi]) == t
                hist = torch.zeros(1, Di, Kc - 1, device=h.device) if fresh else conv_pool.index_select(0, idx)
                xin = torch.cat([hist[0], x[s0:e0].t()], -1)
                xc = F.silu(F.conv1d(xin.unsqueeze(0), w.unsqueeze(1), wb, groups=Di)[0].t())          # [t, Di]
                conv_pool.index_copy_(0, idx, xin[:, -(Kc - 1):].unsqueeze(0).contiguous())
                dt, Bm, Cm = ssm_inputs(xc)
                S0 = None if fresh else state_pool.index_select(0, idx)
                ys, S = selective_scan(xc.unsqueeze(0), dt.unsqueeze(0), A, Bm.unsqueeze(0), Cm.unsqueeze(0), L.mamba_D.float(), S0)
                y[s0:e0] = ys[0].float()
                state_pool.index_copy_(0, idx, S.float())
        y = (y * F.silu(z)).to(torch.bfloat16)
        return h, ops.linear(y, L.mamba_out)

    def _attn_mla(self, L: LayerWeights, li: int, h, d, kv: PagedKVStorage, meta: BatchMeta):
        cfg = self.cfg
        H, dn, dr, dv, R = self.n_heads_local, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        T = h.shape[0]
        a, h = self._norm_linear(h, d, L.qa_kva, L.input_norm)
        if L.q_b is not None:
            ql = cfg.q_lora_rank
            q = ops.linear(a[:, :ql], L.q_b, norm_w=L.q_a_norm, eps=cfg.rms_norm_eps)
            kva = a[:, ql:]
        else:
            ql = H * (dn + dr)
            q = a[:, :ql]
            kva = a[:, ql:]
        q_full = torch.empty(T, H, R + dr, dtype=torch.bfloat16, device=h.device)
        nonabsorbed = (not meta.decode) and L.kv_b_dense is not None and meta.attn_mask is None
        ops.mla_prep(q, kva, L.w_ukT, L.kv_a_norm, meta.positions, self.inv_freq, meta.slots, q_full, kv.k[li], H, dn, dr,
                     R, cfg.rms_norm_eps, self.rope_mscale, cfg.rope_interleave, skip_absorb=nonabsorbed)
        if meta.decode:
            o = ops.paged_attention(q_full, kv.k[li], None, meta.block_tables, meta.ctx_lens, Hq=H, Hkv=1, dqk=R + dr, dv=R,
                                    block_size=kv.block_size, scale=self.scale, splits=meta.splits, w_uv=L.w_uv,
                                    max_ctx=meta.max_ctx)
            o = o.reshape(T, H * dv)
        elif nonabsorbed:
            o = self._prefill_attention_mla_expanded(L, q.view(T, H, dn + dr), q_full, kv, li, meta)
        else:
            o = self._prefill_attention_mla(L, q_full, kv, li, meta)
        d = self._row_parallel(o, L.o, 2 * li)
        return h, d

    def _prefill_attention_mla_expanded(self, L: LayerWeights, q, q_full, kv: PagedKVStorage, li: int, meta: BatchMeta):
        """Non-absorbed causal prefill: the cached latent rows are lifted to per-head keys / values with one GEMM
        (``kv_b``), so attention runs with 256-wide heads instead of the 576 / 512-wide latent form - less than half
        the attention FLOPs and a head size the fused attention kernels support."""
        cfg = self.cfg
        H, dn, dr, dv, R = self.n_heads_local, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        out = torch.empty(q.shape[0], H * dv, dtype=torch.bfloat16, device=q.device)
        bs = kv.block_size
        for b in range(len(meta.cu_seqlens) - 1):
            s, e = meta.cu_seqlens[b], meta.cu_seqlens[b + 1]
            n_ctx = int(meta.ctx_lens_host[b])
            t = e - s
            def _slots(b=b, n_ctx=n_ctx):
                tok = torch.arange(n_ctx, device=q.device)
                return meta.block_tables[b, tok // bs].long() * bs + tok % bs
            slots = meta.cached(("slots", b, n_ctx), _slots)
            lat = kv.k[li][slots]                                           # [n, R + dr] post-norm | post-RoPE
            if R % 64 == 0 and ops.fmha_ok(t, n_ctx, dn + dr, dv, q.device):
                # tensor-core attention: keys per head from one GEMM, V^T per head straight from a second GEMM with the
                # operands swapped (W_v x c^T), so no transposition pass is needed
                n_pad = (n_ctx + 7) // 8 * 8
                c = torch.empty(n_pad, R, dtype=torch.bfloat16, device=q.device)
                c[:n_ctx].copy_(lat[:, :R])
                if n_pad > n_ctx:
                    c[n_ctx:].zero_()
                w_k, w_v = self._kv_b_split(L)
                k = torch.empty(n_ctx, H, dn + dr, dtype=torch.bfloat16, device=q.device)
                k[..., :dn].copy_(ops.bf16_gemm(c[:n_ctx], w_k).view(n_ctx, H, dn))
                k[..., dn:].copy_(lat[:, None, R:].expand(n_ctx, H, dr))
                vt = ops.bf16_gemm(w_v, c)                                  # [H, dv, n_pad]
                qq = torch.cat([q[s:e, :, :dn], q_full[s:e, :, R:]], -1)
                ops.fmha_prefill(qq, k, None, out[s:e].view(t, H, dv), self.scale, vt=vt)
                continue
            c = lat[:, :R].contiguous()
            kvx = (ops.bf16_gemm(c, L.kv_b_dense) if R % 64 == 0 else torch.matmul(c, L.kv_b_dense.t())).view(n_ctx, H, dn + dv)
            k = torch.cat([kvx[..., :dn], lat[:, None, R:].expand(n_ctx, H, dr)], -1)
            qq = torch.cat([q[s:e, :, :dn], q_full[s:e, :, R:]], -1)
            cu_q = meta.dev_ints(("cu_q1", b), [0, t], q.device)
            cu_k = meta.dev_ints(("cu_k1", b), [0, n_ctx], q.device)
            ops.prefill_attention(qq, k.contiguous(), kvx[..., dn:], cu_q, cu_k=cu_k, max_q=t, scale=self.scale,
                                  out=out[s:e].view(t, H, dv))
        return out

    def _kv_b_split(self, L: LayerWeights):
        """``kv_b`` split for the tensor-core prompt path: ``w_k [H * dn, R]`` (contiguous copy, made once per layer) and
        ``w_v [H, dv, R]`` (a strided view of the same matrix, the batched GEMM takes it as it is)."""
        sp = getattr(L, "_kv_b_split_cache", None)
        key = (L.kv_b_dense.data_ptr(), tuple(L.kv_b_dense.shape), self.n_heads_local)
        if sp is not None and sp[2] != key:        # a (sharded) copy of the layer carries another matrix (maybe at the same address)
            sp = None
        if sp is None:
            cfg = self.cfg
            H, dn, dv, R = self.n_heads_local, cfg.qk_nope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
            w = L.kv_b_dense.view(H, dn + dv, R)
            sp = (w[:, :dn, :].reshape(H * dn, R).contiguous(), w[:, dn:, :], key)
            L._kv_b_split_cache = sp
        return sp[0], sp[1]

    def _prefill_attention_mla(self, L: LayerWeights, q_full, kv: PagedKVStorage, li: int, meta: BatchMeta):
        """Absorbed-form causal prefill: scores and values live in the 576/512-d latent space, all heads
        share the latent keys (an MQA problem), then W_uv lifts the result to v_head_dim per head."""
        cfg = self.cfg
        H, dr, dv, R = self.n_heads_local, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        out = torch.empty(q_full.shape[0], H * dv, dtype=torch.bfloat16, device=q_full.device)
        bs = kv.block_size
        for b in range(len(meta.cu_seqlens) - 1):
            s, e = meta.cu_seqlens[b], meta.cu_seqlens[b + 1]
            n_ctx = int(meta.ctx_lens_host[b])
            t = e - s
            tok = torch.arange(n_ctx, device=q_full.device)
            slots = meta.block_tables[b, tok // bs].long() * bs + tok % bs
            lat = kv.k[li][slots]                                   # [n, R + dr]
            Q = q_full[s:e].transpose(0, 1).unsqueeze(0)            # [1, H, t, R + dr]
            Kt = lat.view(1, 1, n_ctx, R + dr)
            Vt = lat[:, :R].reshape(1, 1, n_ctx, R)
            mask = None
            if n_ctx != t:
                qpos = torch.arange(n_ctx - t, n_ctx, device=q_full.device).unsqueeze(1)
                mask = tok.unsqueeze(0) <= qpos
            if meta.attn_mask is not None:
                mask = meta.attn_mask
            o = F.scaled_dot_product_attention(Q, Kt.expand(1, H, n_ctx, R + dr), Vt.expand(1, H, n_ctx, R), attn_mask=mask,
                                               is_causal=(mask is None), scale=self.scale)
            o_lat = o.squeeze(0).transpose(0, 1).contiguous()       # [t, H, R]
            out[s:e] = torch.einsum("thr,hvr->thv", o_lat, L.w_uv).reshape(t, H * dv)
        return out

    # ------------------------------------------------------------------ MLP blocks
    def _mlp_dense(self, L: LayerWeights, li: int, h, d):
        cfg = self.cfg
        x, new_h = self._norm_linear(h, d, L.gate_up, L.post_norm, act=1)
        return new_h, self._row_parallel(x, L.down, 2 * li + 1)

    def _mlp_moe(self, L: LayerWeights, li: int, h, d, counts=None):
        cfg = self.cfg
        rkw = dict(bias=L.router_bias, topk=cfg.num_experts_per_tok, scoring=1 if cfg.scoring_func == "sigmoid" else 0,
                   renorm=cfg.norm_topk_prob, routed_scale=cfg.routed_scaling_factor, n_group=cfg.n_group,
                   topk_group=cfg.topk_group, counts=counts)
        if self.tp is not None and getattr(d, "pending_rs", False):
            # sequence-parallel boundary: add + norm on the owned rows inside the reduce kernel; the gate GEMM gathers
            g = self.tp.finish_norm(d, h, L.post_norm, cfg.rms_norm_eps)
            ids, wts = ops.moe_router(g.x, L.router_w, ag_wait=g, **rkw)
            if self.routing_hook is not None:
                self.routing_hook(li, ids, None)
            return g.h, self.tp.moe_row_parallel(g.x, {}, L, ids, wts, cfg, 2 * li + 1)
        new_h = torch.empty_like(h)
        ids, wts = ops.moe_router(h, L.router_w, norm_w=L.post_norm, eps=cfg.rms_norm_eps, resid_out=new_h, **self._dargs(d), **rkw)
        if self.routing_hook is not None:
            self.routing_hook(li, ids, None)       # analysis tools (expert-usage profiler); forces no sync by itself
        if self.tp is not None:
            return new_h, self.tp.moe_row_parallel(new_h, {"norm_w": L.post_norm, "eps": cfg.rms_norm_eps}, L, ids, wts, cfg,
                                                   2 * li + 1)
        if self.ep is not None:
            # every rank holds different tokens: rows travel to the ranks that own their experts and come back
            return new_h, self.ep.forward(li, new_h, ids, wts, norm_w=L.post_norm, eps=cfg.rms_norm_eps)
        out = ops.moe_forward(new_h, L.gate_up_bank, L.down_bank, ids, wts, n_shared=cfg.n_shared_experts,
                              shared_base=cfg.num_experts, norm_w=L.post_norm, eps=cfg.rms_norm_eps)
        return new_h, out

    def _use_chain(self, input_ids, kv, meta) -> bool:
        """Small decode batches of MLA models run the persistent decode-chain kernel (``ops/chain.py``): one launch between
        two attention calls instead of seven."""
        from ..ops import chain
        if self._chain is False or not input_ids.is_cuda or input_ids.shape[0] > chain.MAX_BATCH or self.routing_hook is not None:
            return False
        if ops._FORCE_REF or ops._capture is not None or isinstance(kv.k[0], ops.FP8KV) or meta.attn_mask is not None:
            return False
        if self._chain is None:
            self._chain = chain.DecodeChain(self) if (ops.native_available() and chain.model_supported(self)) else False
        return self._chain is not False

    # ------------------------------------------------------------------ full forward
    def forward_hidden(self, input_ids: torch.Tensor, kv: PagedKVStorage, meta: BatchMeta) -> Tuple[torch.Tensor, torch.Tensor]:
        """Runs all layers.  Returns (hidden, pending delta): the final residual add + norm is fused
        into the head projection."""
        if self.tp is not None:
            self.tp.begin_step()          # new exchange epoch: every in-kernel exchange site is used once per forward pass
        if meta.decode and self._use_chain(input_ids, kv, meta):
            return self._chain.step(input_ids, kv, meta)
        h = ops.embedding(self.embed, input_ids)
        d = None
        for li, L in enumerate(self.layers):
            if L.lin_in is not None:
                h, d = self._attn_deltanet(L, li, h, d, kv, meta)
            elif L.mamba_in is not None:
                h, d = self._attn_mamba(L, li, h, d, kv, meta)
            elif self.cfg.is_mla:
                h, d = self._attn_mla(L, li, h, d, kv, meta)
            else:
                h, d = self._attn_gqa(L, li, h, d, kv, meta)
            if L.router_w is not None:
                h, d = self._mlp_moe(L, li, h, d)
            else:
                h, d = self._mlp_dense(L, li, h, d)
        if getattr(d, "pending_rs", False):     # callers get a tensor (or a decode-path handle)
            d = self.tp.finish_plain(d)
        return h, d

    def logits(self, h, d, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """fp32 logits of the selected rows (default: all)."""
        if rows is not None and d is not None and not isinstance(d, torch.Tensor):
            # a short tensor-parallel pass leaves the last partial sums in the exchange buffers (the head kernel adds them
            # while it stages its input): run the head on all rows of the pass, then keep the requested ones
            lg = ops.bf16_linear(h, self.lm_head, norm_w=self.final_norm, eps=self.cfg.rms_norm_eps, out_dtype=torch.float32,
                                 **self._dargs(d))
            return lg.index_select(0, rows)
        if rows is not None:
            h = h.index_select(0, rows)
            d = d.index_select(0, rows) if d is not None else None
        return ops.bf16_linear(h, self.lm_head, norm_w=self.final_norm, eps=self.cfg.rms_norm_eps,
                               out_dtype=torch.float32, **self._dargs(d))

    def final_hidden(self, h, d) -> torch.Tensor:
        """Normalised last hidden state (input of the head / of MTP modules)."""
        return ops.rmsnorm(h, self.final_norm, self.cfg.rms_norm_eps, delta=d)

    def greedy(self, logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Arg-max token ids; with a vocabulary-sharded head the shards exchange (max, index) pairs."""
        if self.tp is not None and self.tp.tp > 1:
            return self.tp.greedy(logits, self.vocab_range[0], out=out)
        return ops.argmax(logits, out=out)

    def full_logits(self, logits: torch.Tensor) -> torch.Tensor:
        if self.tp is not None and self.tp.tp > 1:
            return self.tp.gather_logits(logits)
        return logits

    def forward(self, input_ids, kv: PagedKVStorage, meta: BatchMeta, last_only: bool = True) -> torch.Tensor:
        h, d = self.forward_hidden(input_ids, kv, meta)
        rows = None
        if not meta.decode and last_only and meta.cu_seqlens is not None:
            rows = torch.tensor([e - 1 for e in meta.cu_seqlens[1:]], device=h.device, dtype=torch.long)
        return self.logits(h, d, rows)

    def to(self, device) -> "Transformer":
        """Copy of the model on ``device`` (weights are moved as they are: no re-quantization, no kernel launch)."""
        import dataclasses
        device = torch.device(device)

        def mv(v):
            if isinstance(v, (FP4Weight, FP4ExpertBank, torch.Tensor)):
                return v.to(device)
            return v
        layers = [dataclasses.replace(L, **{f.name: mv(getattr(L, f.name)) for f in dataclasses.fields(L)}) for L in self.layers]
        head = self.embed.to(device) if self.lm_head is self.embed else self.lm_head.to(device)
        m = Transformer(self.cfg, layers, self.embed.to(device) if self.lm_head is not self.embed else head, self.final_norm.to(device), head)
        m.mtp = self.mtp
        return m

    # ------------------------------------------------------------------ accounting
    def weight_bytes(self) -> int:
        n = self.embed.numel() * 2 + (0 if self.lm_head is self.embed else self.lm_head.numel() * 2)
        for L in self.layers:
            for v in vars(L).values():
                if isinstance(v, (FP4Weight, FP4ExpertBank)):
                    n += v.nbytes()
                elif isinstance(v, torch.Tensor):
                    n += v.numel() * v.element_size()
        return n
