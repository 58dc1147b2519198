"""Weight sources: build a :class:`Transformer` from a checkpoint directory (MMFP4 / marlin_fp4,
sharded or single-file, HF tensor names) or from a seeded random initialisation that is RTN-quantized
on the target device (synthetic benchmarks; no checkpoint on disk).

Parity: reference ``metal_marlin/model_utils.py:502`` (``load_prequantized_mmfp4_model``),
``metal_marlin/_quantized_weights.py:272`` (expert alias table) and
``metal_marlin/mmfp4_loader.py:1248`` (``get_quantized_weight``).
"""
from __future__ import annotations

import zlib
from typing import List, Optional

import torch

from ..formats import fp4 as fp4fmt
from ..ops import FP4ExpertBank, FP4Weight
from .config import ModelConfig
from .transformer import LayerWeights, Transformer, absorb_kv_b


class RandomSource:
    """Deterministic random weights: every tensor is drawn from its own generator seeded by
    ``crc32(name) ^ seed`` so layer order and sharding do not change the values."""

    def __init__(self, cfg: ModelConfig, device, seed: int = 0, std: float = 0.02):
        self.cfg, self.device, self.seed, self.std = cfg, torch.device(device), seed, std

    def _gen(self, name: str) -> torch.Generator:
        g = torch.Generator(device=self.device)
        g.manual_seed((zlib.crc32(name.encode()) ^ self.seed) & 0x7FFFFFFF)
        return g

    def float(self, name: str, *shape, std: Optional[float] = None) -> torch.Tensor:
        return torch.randn(*shape, generator=self._gen(name), device=self.device, dtype=torch.float32) * (std or self.std)

    def dense(self, name: str, *shape, std: Optional[float] = None) -> torch.Tensor:
        return self.float(name, *shape, std=std).to(torch.bfloat16)

    def norm(self, name: str, dim: int) -> torch.Tensor:
        return (1.0 + 0.05 * torch.randn(dim, generator=self._gen(name), device=self.device)).to(torch.bfloat16)

    def linear(self, name: str, out_f: int, in_f: int) -> FP4Weight:
        return FP4Weight.from_float(self.float(name, out_f, in_f), self.cfg.group_size)

    def linear_cat(self, names: List[str], outs: List[int], in_f: int) -> FP4Weight:
        return FP4Weight.concat_rows([self.linear(n, o, in_f) for n, o in zip(names, outs)])

    def bank(self, name: str, n: int, out_f: int, in_f: int, parts: int = 1) -> FP4ExpertBank:
        """``n`` experts of ``parts`` row-stacked matrices (gate|up) each; quantized in one batched pass."""
        gs = fp4fmt.pick_group_size(in_f, self.cfg.group_size)
        chunk = max(1, min(n, (1 << 28) // max(1, out_f * parts * in_f)))
        qs, ss = [], []
        for e0 in range(0, n, chunk):
            ne = min(chunk, n - e0)
            w = self.float(f"{name}.{e0}", ne * parts * out_f, in_f)
            codes, scales = fp4fmt.quantize_codes(w, gs)
            del w
            q, s, _ = fp4fmt.to_tile_layout(codes, scales)
            qs.append(q.view(ne, parts * out_f // 16, *q.shape[1:]))
            ss.append(s.view(ne, parts * out_f // 16, *s.shape[1:]))
        return FP4ExpertBank(torch.cat(qs), torch.cat(ss), parts * out_f, in_f, gs)


class CheckpointSource:
    """Reads HF-named tensors from an MMFP4 or marlin_fp4 checkpoint directory."""

    def __init__(self, cfg: ModelConfig, path: str, device):
        from ..formats.mmfp4_loader import MMFP4ModelLoader
        self.cfg, self.device = cfg, torch.device(device)
        self.loader = MMFP4ModelLoader(path)

    def _q(self, name: str) -> FP4Weight:
        packed, scales, layout = self.loader.get_quantized_weight(name)
        if layout == "marlin_fp4":
            return FP4Weight.from_marlin_fp4(packed, scales, device=self.device)
        return FP4Weight.from_mmfp4(packed, scales, device=self.device)

    def has(self, name: str) -> bool:
        return self.loader.has_tensor(name)

    def linear(self, name: str, out_f: int, in_f: int) -> FP4Weight:
        if self.loader.is_quantized(name):
            w = self._q(name)
        else:
            w = FP4Weight.from_float(self.loader.load_tensor(name + ".weight").to(self.device), self.cfg.group_size)
        assert (w.out_features, w.in_features) == (out_f, in_f), (name, w.out_features, w.in_features, out_f, in_f)
        w.names = [(name + ".weight", out_f)]
        # MR-GPTQ checkpoints store the weight in a block-Hadamard-rotated input basis; the op layer rotates the activation
        w.hadamard_block = self.loader.get_hadamard_block_size(name)
        return w

    def linear_cat(self, names, outs, in_f) -> FP4Weight:
        parts = [self.linear(n, o, in_f) for n, o in zip(names, outs)]
        blocks = {p.hadamard_block for p in parts}
        if len(blocks) != 1:
            raise ValueError(f"projections fused over one input must share one rotation, got blocks {sorted(blocks)} for {names}")
        w = FP4Weight.concat_rows(parts)
        w.hadamard_block = blocks.pop()
        return w

    def dense(self, name: str, *shape, std=None) -> torch.Tensor:
        t = self.loader.load_tensor(name).to(self.device, torch.bfloat16)
        assert tuple(t.shape) == tuple(shape), (name, t.shape, shape)
        return t

    def norm(self, name: str, dim: int) -> torch.Tensor:
        return self.dense(name, dim)

    def float(self, name: str, *shape, std=None) -> torch.Tensor:
        return self.loader.load_tensor(name).to(self.device, torch.float32)


def _unrotate(w: torch.Tensor, block: int) -> torch.Tensor:
    """Dense copy of a weight stored in the rotated basis: ``W = W_rot . H`` (H block-diagonal, orthonormal, symmetric)."""
    if not block:
        return w
    from ..quant.hadamard import fwht
    return fwht(w.reshape(w.shape[0], -1, block)).reshape(w.shape)


def _bank_block(ws) -> int:
    blocks = {getattr(w, "hadamard_block", 0) for w in ws}
    if len(blocks) != 1:
        raise ValueError(f"the experts of one bank must share one rotation, got blocks {sorted(blocks)}")
    return blocks.pop()


def _expert_names(prefix: str, e: int):
    return [f"{prefix}.experts.{e}.gate_proj", f"{prefix}.experts.{e}.up_proj"], f"{prefix}.experts.{e}.down_proj"


def build_layer(cfg: ModelConfig, src, i: int) -> LayerWeights:
    p = f"model.layers.{i}"
    H = cfg.hidden_size
    L = LayerWeights(input_norm=src.norm(f"{p}.input_layernorm.weight", H),
                     post_norm=src.norm(f"{p}.post_attention_layernorm.weight", H))
    a = f"{p}.self_attn"
    if cfg.layer_is_mamba(i):
        mm = f"{p}.mamba"
        Di, N, r = cfg.mamba_d_inner, cfg.mamba_d_state, cfg.mamba_rank
        if Di % 16 or (r + 2 * N) % 16:
            raise ValueError("mamba: the inner width and dt_rank + 2 * d_state must be multiples of 16 (weight tile rows)")
        L.mamba_in = src.linear(f"{mm}.in_proj", 2 * Di, H)
        L.mamba_conv = src.float(f"{mm}.conv1d.weight", Di, cfg.mamba_d_conv, std=0.2).to(torch.float32).reshape(Di, cfg.mamba_d_conv).contiguous()
        L.mamba_conv_b = src.float(f"{mm}.conv1d.bias", Di, std=0.05).to(torch.float32)
        L.mamba_x = src.linear(f"{mm}.x_proj", r + 2 * N, Di)
        L.mamba_dt = src.float(f"{mm}.dt_proj.weight", Di, r, std=0.1).to(torch.float32)
        L.mamba_dt_b = src.float(f"{mm}.dt_proj.bias", Di, std=0.5).to(torch.float32)
        L.mamba_A_log = src.float(f"{mm}.A_log", Di, N, std=0.5).to(torch.float32)
        L.mamba_D = src.float(f"{mm}.D", Di, std=0.5).to(torch.float32)
        L.mamba_out = src.linear(f"{mm}.out_proj", H, Di)
    elif cfg.layer_is_linear(i):
        la = f"{p}.linear_attn"
        Hk, Hv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
        kd, vd = Hk * dk, Hv * dv
        if (2 * Hv) % 16 or kd % 16 or vd % 16:
            raise ValueError("linear attention: 2 x value heads and the key / value widths must be multiples of 16 (weight tile rows)")
        if isinstance(src, RandomSource) or src.has(f"{la}.in_proj_q.weight"):
            L.lin_in = src.linear_cat([f"{la}.in_proj_q", f"{la}.in_proj_k", f"{la}.in_proj_v", f"{la}.in_proj_z", f"{la}.in_proj_ba"],
                                      [kd, kd, vd, vd, 2 * Hv], H)
        else:
            raise ValueError(f"{la}: the checkpoint must store the input projection as in_proj_q / _k / _v / _z / _ba (rows in that "
                             "order); interleaved in_proj_qkvz tensors are split by the converter")
        L.lin_conv = src.float(f"{la}.conv1d.weight", 2 * kd + vd, cfg.linear_conv_kernel_dim, std=0.2).to(torch.float32) \
            .reshape(2 * kd + vd, cfg.linear_conv_kernel_dim).contiguous()          # checkpoints hold [C, 1, K]
        L.lin_dt_bias = src.float(f"{la}.dt_bias", Hv, std=0.5).to(torch.float32)
        L.lin_A_log = src.float(f"{la}.A_log", Hv, std=0.5).to(torch.float32)
        L.lin_norm = src.norm(f"{la}.norm.weight", dv)
        L.lin_out = src.linear(f"{la}.out_proj", H, vd)
    elif cfg.is_mla:
        nh, dn, dr, dv, R = cfg.num_attention_heads, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        if cfg.q_lora_rank:
            L.qa_kva = src.linear_cat([f"{a}.q_a_proj", f"{a}.kv_a_proj_with_mqa"], [cfg.q_lora_rank, R + dr], H)
            L.q_a_norm = src.norm(f"{a}.q_a_layernorm.weight", cfg.q_lora_rank)
            L.q_b = src.linear(f"{a}.q_b_proj", nh * (dn + dr), cfg.q_lora_rank)
        else:
            L.qa_kva = src.linear_cat([f"{a}.q_proj", f"{a}.kv_a_proj_with_mqa"], [nh * (dn + dr), R + dr], H)
        L.kv_a_norm = src.norm(f"{a}.kv_a_layernorm.weight", R)
        L.kv_b = src.linear(f"{a}.kv_b_proj", nh * (dn + dv), R)
        hb = getattr(L.kv_b, "hadamard_block", 0)
        L.w_ukT, L.w_uv = absorb_kv_b(L.kv_b, nh, dn, dv, R, hadamard_block=hb)
        L.kv_b_dense = _unrotate(L.kv_b.dequantize(torch.float32), hb).to(torch.bfloat16).contiguous()      # prefill lifts latent rows to per-head K / V with it
        L.kv_b = None      # the absorbed copies serve decode
        L.o = src.linear(f"{a}.o_proj", H, nh * dv)
    else:
        Hq, Hk, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.dh
        L.qkv = src.linear_cat([f"{a}.q_proj", f"{a}.k_proj", f"{a}.v_proj"], [Hq * D, Hk * D, Hk * D], H)
        if cfg.attention_bias:
            L.qkv_bias = torch.cat([src.dense(f"{a}.{n}_proj.bias", d) for n, d in
                                    (("q", Hq * D), ("k", Hk * D), ("v", Hk * D))])
        if cfg.qk_norm:
            L.q_norm = src.norm(f"{a}.q_norm.weight", D)
            L.k_norm = src.norm(f"{a}.k_norm.weight", D)
        L.o = src.linear(f"{a}.o_proj", H, Hq * D)
    m = f"{p}.mlp"
    if cfg.layer_is_moe(i):
        E, I, ns = cfg.num_experts, cfg.moe_intermediate_size, cfg.n_shared_experts
        L.router_w = src.dense(f"{m}.gate.weight", E, H)
        if cfg.router_bias:
            L.router_bias = (src.float(f"{m}.gate.e_score_correction_bias", E, std=0.01)).to(torch.float32).contiguous()
        if isinstance(src, RandomSource):
            L.gate_up_bank = src.bank(f"{m}.experts.gate_up", E + ns, I, H, parts=2)
            L.down_bank = src.bank(f"{m}.experts.down", E + ns, H, I)
        elif hasattr(src, "expert_banks"):
            L.gate_up_bank, L.down_bank = src.expert_banks(m, E, I, H, ns)
        else:
            gus, dws = [], []
            for e in range(E):
                gu_names, d_name = _expert_names(m, e)
                gus.append(src.linear_cat(gu_names, [I, I], H))
                dws.append(src.linear(d_name, H, I))
            if ns:
                # HF stores the shared experts as one MLP of width ns * I; split it into ns experts
                sg = src.linear(f"{m}.shared_experts.gate_proj", ns * I, H)
                su = src.linear(f"{m}.shared_experts.up_proj", ns * I, H)
                sd = src.linear(f"{m}.shared_experts.down_proj", H, ns * I)
                sdc, sds = sd.codes_scales()
                for j in range(ns):
                    gcs, ucs = sg.codes_scales(), su.codes_scales()
                    sl = slice(j * I, (j + 1) * I)
                    gu = FP4Weight.concat_rows([FP4Weight.from_codes(gcs[0][sl], gcs[1][sl]),
                                                FP4Weight.from_codes(ucs[0][sl], ucs[1][sl])])
                    gu.names = (sg.names or []) + (su.names or [])        # calibration: same input as the whole shared MLP
                    gu.hadamard_block = sg.hadamard_block
                    gus.append(gu)
                    gper = I // sd.group_size
                    dw = FP4Weight.from_codes(sdc[:, sl].contiguous(), sds[:, j * gper:(j + 1) * gper].contiguous())
                    assert not sd.hadamard_block or I % sd.hadamard_block == 0, "shared-expert width must be a multiple of the rotation block"
                    dw.hadamard_block = sd.hadamard_block
                    dw.names = sd.names if ns == 1 else None            # a column slice of the shared down matrix has no Hessian of its own
                    dws.append(dw)
            L.gate_up_bank = FP4ExpertBank.from_weights(gus)
            L.down_bank = FP4ExpertBank.from_weights(dws)
            L.gate_up_bank.hadamard_block, L.down_bank.hadamard_block = _bank_block(gus), _bank_block(dws)
    else:
        I = cfg.intermediate_size
        L.gate_up = src.linear_cat([f"{m}.gate_proj", f"{m}.up_proj"], [I, I], H)
        L.down = src.linear(f"{m}.down_proj", H, I)
    return L


def build_transformer(cfg: ModelConfig, src) -> Transformer:
    embed = src.dense("model.embed_tokens.weight", cfg.vocab_size, cfg.hidden_size)
    layers = [build_layer(cfg, src, i) for i in range(cfg.num_hidden_layers)]
    final_norm = src.norm("model.norm.weight", cfg.hidden_size)
    tied = cfg.tie_word_embeddings or (not isinstance(src, RandomSource) and not src.has("lm_head.weight"))
    lm_head = embed if tied else src.dense("lm_head.weight", cfg.vocab_size, cfg.hidden_size)
    return Transformer(cfg, layers, embed, final_norm, lm_head)


def random_transformer(cfg: ModelConfig, device="cpu", seed: int = 0) -> Transformer:
    return build_transformer(cfg, RandomSource(cfg, device, seed))
