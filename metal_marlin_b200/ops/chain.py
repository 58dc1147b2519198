"""Decode chain: the links of a small-batch MLA decode step between two attention calls in one persistent launch
(``csrc/decode_chain.cu``, ``csrc/api_chain.h``).

A step of an MLA + MoE model then costs, per layer, the two attention launches (split-KV decode and merge) plus one chain
launch instead of nine kernels; inside the chain the phases (o_proj, router, expert gate|up, down, next layer's q_a|kv_a,
q_b + latent cache write, W_uk absorb + RoPE) are separated by grid barriers instead of launch boundaries.

Parity: the reference's lesson that launch count, not arithmetic, bounds batch-1 decode (``docs/optimization_status_final.md:56-70``)
and its fused decode shaders (``metal_marlin/shaders/attention_mla_fused.metal:189``, ``moe_fused_dispatch_shared_decode_fp4`` in
``src/moe_dispatch*.metal``).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch

from .weights import FP4ExpertBank, FP4Weight

PH_A, PH_B, PH_C, PH_D, PH_E, PH_F, PH_G = 1, 2, 4, 8, 16, 32, 64
MAX_BATCH = int(os.environ.get("MMB200_CHAIN_MAX_B", "4"))      # rows a launch stages per CTA (the kernel takes up to 8)
# Off unless asked for: measured on GLM-4.7-Flash at batch 1 the chain takes 63 us per layer boundary against 46 us for the seven
# stand-alone kernels it replaces (each of which already hides its launch behind the previous kernel and prefetches its
# weights before it waits); a phase here pays a grid barrier and a cold first weight load instead.
ENABLED = os.environ.get("MMB200_CHAIN", "0") == "1"


class _Mat(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("s", ctypes.c_void_p), ("N", ctypes.c_int), ("K", ctypes.c_int), ("gs_shift", ctypes.c_int),
                ("stride_q", ctypes.c_longlong), ("stride_s", ctypes.c_longlong)]


class _Params(ctypes.Structure):
    """Mirror of ``MmbChainParams`` (same field order; ctypes applies the C alignment rules)."""
    _fields_ = [
        ("B", ctypes.c_int), ("H", ctypes.c_int), ("phases", ctypes.c_int), ("eps", ctypes.c_float),
        ("attn_o", ctypes.c_void_p), ("o", _Mat), ("delta_attn", ctypes.c_void_p),
        ("h_in", ctypes.c_void_p), ("h_mid", ctypes.c_void_p), ("post_norm", ctypes.c_void_p), ("moe", ctypes.c_int),
        ("router_w", ctypes.c_void_p), ("router_bias", ctypes.c_void_p),
        ("E", ctypes.c_int), ("topk", ctypes.c_int), ("n_shared", ctypes.c_int), ("scoring", ctypes.c_int), ("renorm", ctypes.c_int),
        ("n_group", ctypes.c_int), ("topk_group", ctypes.c_int), ("routed_scale", ctypes.c_float),
        ("logits", ctypes.c_void_p), ("ids", ctypes.c_void_p), ("weights", ctypes.c_void_p),
        ("gate_up", _Mat), ("down", _Mat), ("hmid", ctypes.c_void_p), ("delta_mlp", ctypes.c_void_p),
        ("h_out", ctypes.c_void_p), ("in_norm", ctypes.c_void_p), ("qa_kva", _Mat), ("a_out", ctypes.c_void_p), ("q_lora", ctypes.c_int),
        ("q_a_norm", ctypes.c_void_p), ("q_b", _Mat), ("q_out", ctypes.c_void_p), ("kv_norm", ctypes.c_void_p), ("w_ukT", ctypes.c_void_p),
        ("nh", ctypes.c_int), ("dn", ctypes.c_int), ("dr", ctypes.c_int), ("R", ctypes.c_int),
        ("positions", ctypes.c_void_p), ("inv_freq", ctypes.c_void_p), ("slots", ctypes.c_void_p), ("cache", ctypes.c_void_p),
        ("mscale", ctypes.c_float), ("interleaved", ctypes.c_int), ("q_full", ctypes.c_void_p),
        ("sync", ctypes.c_void_p), ("status", ctypes.c_void_p), ("stage_k", ctypes.c_int),
        ("pf_ptr", ctypes.c_void_p * 2), ("pf_bytes", ctypes.c_longlong * 2),
    ]


def _mat(W) -> _Mat:
    m = _Mat()
    if W is None:
        return m
    m.q, m.s = W.qtile.data_ptr(), W.stile.data_ptr()
    m.N, m.K = W.out_features, (W.qtile.shape[-3]) * 64
    m.gs_shift = int(W.group_size).bit_length() - 1
    if isinstance(W, FP4ExpertBank):
        m.stride_q = W.qtile.stride(0) // 4
        m.stride_s = W.stile.stride(0) // 2
    return m


def _mat_ok(W) -> bool:
    return (W is not None and isinstance(W, (FP4Weight, FP4ExpertBank)) and not getattr(W, "is_generic", False) and W.group_size >= 64
            and (W.group_size & (W.group_size - 1)) == 0 and not getattr(W, "hadamard_block", 0) and W.in_features == W.qtile.shape[-3] * 64)


def model_supported(model) -> bool:
    """Whether every layer of ``model`` fits the chain kernel (MLA with a q_lora bottleneck, FP4 matrices with groups of 64+,
    bf16 latent cache, routed experts with at most 16 slots per token)."""
    cfg = model.cfg
    if not (ENABLED and cfg.is_mla and cfg.q_lora_rank and model.tp is None and model.ep is None and model.device.type == "cuda"):
        return False
    if cfg.kv_lora_rank > 512 or cfg.qk_nope_head_dim > 256 or cfg.qk_nope_head_dim % 8 or cfg.hidden_size % 64 or cfg.q_lora_rank % 64:
        return False
    if cfg.is_moe and (cfg.num_experts > 512 or cfg.num_experts_per_tok + cfg.n_shared_experts > 16):
        return False
    for L in model.layers:
        mats = [L.o, L.qa_kva, L.q_b] + ([L.gate_up_bank, L.down_bank] if L.router_w is not None else [L.gate_up, L.down])
        if not all(_mat_ok(m) for m in mats) or L.w_ukT is None:
            return False
    return True


class DecodeChain:
    """Per-model runner.  ``step(model, input_ids, kv, meta)`` returns ``(hidden, pending delta)`` like
    ``Transformer.forward_hidden``; buffers and launch descriptors are built once per batch size and token-state tensors."""

    def __init__(self, model):
        self.model = model
        self._state: Dict[tuple, dict] = {}
        n = int(torch.ops.mmb200.decode_chain_param_bytes())
        if n != ctypes.sizeof(_Params):
            raise RuntimeError(f"decode chain descriptor: the library expects {n} bytes, the Python mirror has {ctypes.sizeof(_Params)}")

    def _build(self, B: int, kv, meta) -> dict:
        from . import gemm_status
        m, cfg, dev = self.model, self.model.cfg, self.model.device
        H, nh, dn, dr, R = cfg.hidden_size, m.n_heads_local, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.kv_lora_rank
        bf = dict(dtype=torch.bfloat16, device=dev)
        S_max = max([(cfg.num_experts_per_tok + cfg.n_shared_experts) * cfg.moe_intermediate_size if L.router_w is not None
                     else L.gate_up.out_features // 2 for L in m.layers])
        st = {
            "h": [torch.empty(B, H, **bf) for _ in range(3)],            # in / mid / out, rotating
            "delta_attn": torch.empty(B, H, **bf), "delta_mlp": torch.empty(B, H, **bf),
            "hmid": torch.empty(B, S_max, **bf), "a": torch.empty(B, cfg.q_lora_rank + R + dr, **bf),
            "q": torch.empty(B, nh * (dn + dr), **bf), "q_full": torch.empty(B, nh, R + dr, **bf),
            "attn_o": torch.empty(B, nh * cfg.v_head_dim, **bf),
            "logits": torch.empty(B, max(1, cfg.num_experts), dtype=torch.float32, device=dev),
            "ids": torch.zeros(B, max(1, cfg.num_experts_per_tok), dtype=torch.int32, device=dev),
            "weights": torch.zeros(B, max(1, cfg.num_experts_per_tok), dtype=torch.float32, device=dev),
            "sync": torch.zeros(4, dtype=torch.int32, device=dev),
            "status": gemm_status(dev),
        }
        descs = []
        nL = len(m.layers)
        for i in range(nL + 1):
            # launch i runs the MLP side of layer i - 1 (A..D) and the attention prologue of layer i (E..G)
            p = _Params()
            p.B, p.H, p.eps = B, H, cfg.rms_norm_eps
            phases = 0
            # rotation: launch i reads h_in = X, writes h_mid = st["h"][1], h_out = Y; X / Y alternate between h[0] and h[2]
            h_in, h_mid, h_out = (st["h"][0], st["h"][1], st["h"][2]) if i % 2 == 1 else (st["h"][2], st["h"][1], st["h"][0])
            p.h_in, p.h_mid, p.h_out = h_in.data_ptr(), h_mid.data_ptr(), h_out.data_ptr()
            stage_k = H
            if i >= 1:
                L = m.layers[i - 1]
                phases |= PH_A | PH_B | PH_D
                p.attn_o, p.o, p.delta_attn = st["attn_o"].data_ptr(), _mat(L.o), st["delta_attn"].data_ptr()
                p.post_norm = L.post_norm.data_ptr()
                p.hmid, p.delta_mlp = st["hmid"].data_ptr(), st["delta_mlp"].data_ptr()
                stage_k = max(stage_k, p.o.K)
                if L.router_w is not None:
                    phases |= PH_C
                    p.moe = 1
                    p.router_w = L.router_w.data_ptr()
                    p.router_bias = L.router_bias.data_ptr() if L.router_bias is not None else None
                    p.E, p.topk, p.n_shared = cfg.num_experts, cfg.num_experts_per_tok, cfg.n_shared_experts
                    p.scoring, p.renorm = (1 if cfg.scoring_func == "sigmoid" else 0), (1 if cfg.norm_topk_prob else 0)
                    p.n_group, p.topk_group, p.routed_scale = cfg.n_group, cfg.topk_group, cfg.routed_scaling_factor
                    p.logits, p.ids, p.weights = st["logits"].data_ptr(), st["ids"].data_ptr(), st["weights"].data_ptr()
                    p.gate_up, p.down = _mat(L.gate_up_bank), _mat(L.down_bank)
                    stage_k = max(stage_k, (p.topk + p.n_shared) * (p.gate_up.N // 2))
                else:
                    p.moe = 0
                    p.gate_up, p.down = _mat(L.gate_up), _mat(L.down)
                    stage_k = max(stage_k, p.gate_up.N // 2)
            else:
                # first launch of a step: the embedding row is the residual stream, nothing is pending
                p.h_mid = h_in.data_ptr()          # phase E reads h_mid (+ delta_mlp, absent here) and writes h_out
                p.delta_mlp = None
            if i < nL:
                L = m.layers[i]
                phases |= PH_E | PH_F | PH_G
                p.in_norm, p.qa_kva, p.a_out = L.input_norm.data_ptr(), _mat(L.qa_kva), st["a"].data_ptr()
                p.q_lora, p.q_a_norm, p.q_b, p.q_out = cfg.q_lora_rank, L.q_a_norm.data_ptr(), _mat(L.q_b), st["q"].data_ptr()
                p.kv_norm, p.w_ukT = L.kv_a_norm.data_ptr(), L.w_ukT.data_ptr()
                p.nh, p.dn, p.dr, p.R = nh, dn, dr, R
                p.positions, p.inv_freq, p.slots = meta.positions.data_ptr(), m.inv_freq.data_ptr(), meta.slots.data_ptr()
                p.cache = kv.k[i].data_ptr()
                p.mscale, p.interleaved = float(m.rope_mscale), 1 if cfg.rope_interleave else 0
                p.q_full = st["q_full"].data_ptr()
                stage_k = max(stage_k, p.q_b.K)
                # what runs next: the attention of layer i (W_uv in its merge kernel), then launch i + 1 (o_proj of layer i)
                p.pf_ptr[0], p.pf_bytes[0] = L.w_uv.data_ptr(), L.w_uv.numel() * 2
                p.pf_ptr[1], p.pf_bytes[1] = L.o.qtile.data_ptr(), L.o.qtile.numel() * 4
            p.phases = phases
            p.sync, p.status = st["sync"].data_ptr(), st["status"].data_ptr()
            p.stage_k = (stage_k + 63) // 64 * 64
            descs.append(torch.frombuffer(bytearray(bytes(p)), dtype=torch.uint8).clone())
        st["descs"] = descs
        return st

    def step(self, input_ids, kv, meta):
        from . import K, embedding, paged_attention
        m, cfg = self.model, self.model.cfg
        B = input_ids.shape[0]
        key = (B, meta.positions.data_ptr(), meta.slots.data_ptr(), kv.k[0].data_ptr())
        st = self._state.get(key)
        if st is None:
            st = self._build(B, kv, meta)
            self._state[key] = st
        nL = len(m.layers)
        nh, dv, R, dr = m.n_heads_local, cfg.v_head_dim, cfg.kv_lora_rank, cfg.qk_rope_head_dim
        # the embedding row goes into the buffer launch 0 reads as its residual stream
        embedding(m.embed, input_ids, out=st["h"][2])
        anchor = st["sync"]
        K.mmb200.decode_chain(st["descs"][0], anchor)
        for i in range(nL):
            paged_attention(st["q_full"], kv.k[i], None, meta.block_tables, meta.ctx_lens, Hq=nh, Hkv=1, dqk=R + dr, dv=R,
                            block_size=kv.block_size, scale=m.scale, splits=meta.splits, w_uv=m.layers[i].w_uv, max_ctx=meta.max_ctx,
                            out=st["attn_o"].view(B, nh, dv))
            K.mmb200.decode_chain(st["descs"][i + 1], anchor)
        # after the last launch: h_mid holds the residual stream, delta_mlp the pending MLP output
        return st["h"][1], st["delta_mlp"]
