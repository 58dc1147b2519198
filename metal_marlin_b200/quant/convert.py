"""Whole-checkpoint conversion: HF float safetensors -> ``marlin_fp4`` / ``mmfp4`` checkpoints,
and synthetic (random-init) checkpoint writers for the benchmark architectures.

Parity: reference ``metal_marlin/hf_loader.py:323`` (``should_quantize_tensor``), ``:424-606``
(``convert_model_to_fp4``: tensor ``name`` = packed uint32 ``[in/8, out]``, ``name.scales``,
``name.group_size``, verbatim copy of everything else, ``quantization_config.json``), ``:963``
(layer-wise streaming conversion); ``metal_marlin/mr_gptq.py:1115-1135`` and
``scripts/quantize_glm47_flash_mmfp4_cuda.py:323-375`` (MMFP4 shards + index + report).
"""
from __future__ import annotations

import json
import os
import shutil
import time
from typing import Callable, Dict, Iterable, Iterator, Optional, Tuple

import torch

from ..formats import fp4 as fp4fmt
from ..formats.safetensors_io import SafetensorsFile, save_file

SKIP_PATTERNS = ("embed", "norm", "lm_head", "shared_head.head", "output", "bias", "dt_proj", "a_log")      # vocabulary heads (also those of MTP modules) stay bf16
COPY_FILES = ("config.json", "tokenizer.json", "tokenizer_config.json", "tokenizer.model", "special_tokens_map.json",
              "generation_config.json", "vocab.json", "merges.txt", "chat_template.jinja")


def should_quantize_tensor(name: str, tensor: torch.Tensor, extra_skip: Iterable[str] = ()) -> bool:
    """2-D, name contains "weight", not an embedding / norm / head / bias, input dim divisible by 8."""
    if tensor.dim() != 2 or "weight" not in name:
        return False
    low = name.lower()
    if any(p in low for p in SKIP_PATTERNS) or any(p in low for p in extra_skip):
        return False
    if low.endswith("mlp.gate.weight"):        # MoE router stays in high precision
        return False
    return tensor.shape[1] % 8 == 0


def iter_safetensors_weights(model_dir: str) -> Iterator[Tuple[str, torch.Tensor]]:
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            wm = json.load(f)["weight_map"]
        files = sorted(set(wm.values()))
    else:
        files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    for fn in files:
        with SafetensorsFile(os.path.join(model_dir, fn)) as f:
            for k in list(f.keys()):
                yield k, f.get_tensor(k)


def _copy_aux(src: str, dst: str) -> None:
    for fn in COPY_FILES:
        p = os.path.join(src, fn)
        if os.path.exists(p):
            shutil.copy(p, os.path.join(dst, fn))


def quantize_named_tensors(tensors: Iterable[Tuple[str, torch.Tensor]], fmt: str, group_size: int,
                           device: str = "cpu", quantize_fn: Optional[Callable] = None, hadamard_block: int = 0,
                           extra_skip: Iterable[str] = ()) -> Iterator[Tuple[str, Dict[str, torch.Tensor], Dict[str, str], Optional[dict]]]:
    """For each input tensor yields (name, tensors-to-write, dtype-overrides, report-entry)."""
    for name, t in tensors:
        if not should_quantize_tensor(name, t, extra_skip):
            yield name, {name: t}, {}, None
            continue
        gs = fp4fmt.pick_group_size(t.shape[1], group_size)
        w = t.to(device=device, dtype=torch.float32)
        rot = hadamard_block if (hadamard_block and w.shape[1] % hadamard_block == 0) else 0
        if rot:      # quantize in the rotated input basis (W . H); readers rotate the activation: y = (W H)(H x)
            from .hadamard import fwht
            w = fwht(w.reshape(w.shape[0], -1, rot)).reshape(w.shape)
        if quantize_fn is not None:
            codes, scales = quantize_fn(name, w, gs)
        else:
            codes, scales = fp4fmt.quantize_codes(w, gs)
        err = float((fp4fmt.dequantize_codes(codes, scales) - w).pow(2).mean().sqrt() / w.pow(2).mean().sqrt().clamp_min(1e-12))
        if fmt == "marlin_fp4":
            packed, sc = fp4fmt.pack_marlin_fp4(codes, scales)
        else:
            packed, sc = fp4fmt.pack_mmfp4(codes, scales)
        # both reference writers key the side tensors off the full tensor name: "<name>.scales", "<name>.group_size"
        out = {name: packed.cpu(), name + ".scales": sc.cpu(), name + ".group_size": torch.tensor([gs], dtype=torch.int32)}
        if rot:
            out[name + ".hadamard_block_size"] = torch.tensor([rot], dtype=torch.int32)
        yield name, out, {name: "U32"}, {"name": name, "shape": list(t.shape), "group_size": gs, "rel_rmse": err}


def convert_model(model_dir: str, out_dir: str, fmt: str = "marlin_fp4", group_size: int = 128, device: str = "cpu",
                  shard_bytes: int = 4 << 30, quantize_fn: Optional[Callable] = None, verbose: bool = False,
                  hadamard_block: int = 0, tensors: Optional[Iterable[Tuple[str, torch.Tensor]]] = None,
                  extra_skip: Iterable[str] = ()) -> dict:
    """Stream a float HF checkpoint into a quantized one.  ``fmt``: ``marlin_fp4`` (single
    ``model.safetensors``) or ``mmfp4`` (shards + ``model.safetensors.index.json``).  ``tensors``: take the ``(name, tensor)``
    stream from the caller instead of the safetensors files of ``model_dir`` (importers that de-quantize another format);
    ``extra_skip``: lower-case name fragments of further tensors to keep unquantized."""
    os.makedirs(out_dir, exist_ok=True)
    t0 = time.time()
    report, weight_map = [], {}
    shard, shard_dt, shard_sz, shard_no = {}, {}, 0, 1
    single = fmt == "marlin_fp4"

    def flush():
        nonlocal shard, shard_dt, shard_sz, shard_no
        if not shard:
            return
        fn = "model.safetensors" if single else f"model-{shard_no:05d}.safetensors"
        save_file(shard, os.path.join(out_dir, fn), metadata={"format": "pt"}, dtype_overrides=shard_dt)
        for k in shard:
            weight_map[k] = fn
        shard, shard_dt, shard_sz = {}, {}, 0
        shard_no += 1

    n_q = n_total = 0
    for name, outs, dts, rep in quantize_named_tensors(tensors if tensors is not None else iter_safetensors_weights(model_dir), fmt, group_size, device, quantize_fn,
                                                         hadamard_block, tuple(extra_skip)):
        n_total += 1
        if rep is not None:
            n_q += 1
            report.append(rep)
            if verbose:
                print(f"  {name}: rel_rmse {rep['rel_rmse']:.4f}")
        for k, v in outs.items():
            shard[k] = v
            shard_sz += v.numel() * v.element_size()
        shard_dt.update(dts)
        if not single and shard_sz >= shard_bytes:
            flush()
    flush()
    fmt_name = "marlin_fp4" if single else "mmfp4_e2m1_marlin"
    qc = {"format": fmt_name, "group_size": group_size, "bits": 4, "quant_method": "rtn" if quantize_fn is None else "custom"}
    with open(os.path.join(out_dir, "quantization_config.json"), "w") as f:
        json.dump(qc, f, indent=1)
    if not single:
        with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"format": fmt_name}, "weight_map": weight_map}, f)
        with open(os.path.join(out_dir, "quantization_report.json"), "w") as f:
            json.dump({"layers": report, "seconds": time.time() - t0}, f)
    _copy_aux(model_dir, out_dir)
    cfgp = os.path.join(out_dir, "config.json")
    if os.path.exists(cfgp):
        with open(cfgp) as f:
            cfg = json.load(f)
        cfg["quantization_config"] = qc
        with open(cfgp, "w") as f:
            json.dump(cfg, f, indent=1)
    mean_err = sum(r["rel_rmse"] for r in report) / max(1, len(report))
    return {"quantized": n_q, "tensors": n_total, "mean_rel_rmse": mean_err, "seconds": time.time() - t0}


def convert_model_to_fp4(model_dir: str, out_dir: str, group_size: int = 128, **kw) -> dict:
    return convert_model(model_dir, out_dir, "marlin_fp4", group_size, **kw)


def convert_model_to_mmfp4(model_dir: str, out_dir: str, group_size: int = 128, **kw) -> dict:
    return convert_model(model_dir, out_dir, "mmfp4", group_size, **kw)


# ---------------------------------------------------------------------------------------------
# synthetic float checkpoints with HF tensor names (tests, demos, benchmark fixtures)
# ---------------------------------------------------------------------------------------------
def random_hf_state(cfg, seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    H = cfg.hidden_size

    def w(*shape):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    def n(dim):
        return (1.0 + 0.05 * torch.randn(dim, generator=g)).to(torch.bfloat16)

    sd = {"model.embed_tokens.weight": w(cfg.vocab_size, H), "model.norm.weight": n(H)}
    if not cfg.tie_word_embeddings:
        sd["lm_head.weight"] = w(cfg.vocab_size, H)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        sd[f"{p}.input_layernorm.weight"] = n(H)
        sd[f"{p}.post_attention_layernorm.weight"] = n(H)
        a = f"{p}.self_attn"
        if cfg.layer_is_mamba(i):
            mm = f"{p}.mamba"
            Di, N, r = cfg.mamba_d_inner, cfg.mamba_d_state, cfg.mamba_rank
            sd[f"{mm}.in_proj.weight"] = w(2 * Di, H)
            sd[f"{mm}.conv1d.weight"] = (torch.randn(Di, 1, cfg.mamba_d_conv, generator=g) * 0.2).to(torch.bfloat16)
            sd[f"{mm}.conv1d.bias"] = torch.randn(Di, generator=g) * 0.05
            sd[f"{mm}.x_proj.weight"] = w(r + 2 * N, Di)
            sd[f"{mm}.dt_proj.weight"] = torch.randn(Di, r, generator=g) * 0.1
            sd[f"{mm}.dt_proj.bias"] = torch.randn(Di, generator=g) * 0.5
            sd[f"{mm}.A_log"] = torch.randn(Di, N, generator=g) * 0.5
            sd[f"{mm}.D"] = torch.randn(Di, generator=g) * 0.5
            sd[f"{mm}.out_proj.weight"] = w(H, Di)
        elif cfg.layer_is_linear(i):
            la = f"{p}.linear_attn"
            kd, vd, Hv = cfg.linear_num_key_heads * cfg.linear_key_head_dim, cfg.linear_num_value_heads * cfg.linear_value_head_dim, cfg.linear_num_value_heads
            for nm, rows in (("in_proj_q", kd), ("in_proj_k", kd), ("in_proj_v", vd), ("in_proj_z", vd), ("in_proj_ba", 2 * Hv)):
                sd[f"{la}.{nm}.weight"] = w(rows, H)
            sd[f"{la}.conv1d.weight"] = (torch.randn(2 * kd + vd, 1, cfg.linear_conv_kernel_dim, generator=g) * 0.2).to(torch.bfloat16)
            sd[f"{la}.dt_bias"] = torch.randn(Hv, generator=g) * 0.5
            sd[f"{la}.A_log"] = torch.randn(Hv, generator=g) * 0.5
            sd[f"{la}.norm.weight"] = n(cfg.linear_value_head_dim)
            sd[f"{la}.out_proj.weight"] = w(H, vd)
        elif cfg.is_mla:
            nh, dn, dr, dv, R = cfg.num_attention_heads, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
            if cfg.q_lora_rank:
                sd[f"{a}.q_a_proj.weight"] = w(cfg.q_lora_rank, H)
                sd[f"{a}.q_a_layernorm.weight"] = n(cfg.q_lora_rank)
                sd[f"{a}.q_b_proj.weight"] = w(nh * (dn + dr), cfg.q_lora_rank)
            else:
                sd[f"{a}.q_proj.weight"] = w(nh * (dn + dr), H)
            sd[f"{a}.kv_a_proj_with_mqa.weight"] = w(R + dr, H)
            sd[f"{a}.kv_a_layernorm.weight"] = n(R)
            sd[f"{a}.kv_b_proj.weight"] = w(nh * (dn + dv), R)
            sd[f"{a}.o_proj.weight"] = w(H, nh * dv)
        else:
            Hq, Hk, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.dh
            sd[f"{a}.q_proj.weight"] = w(Hq * D, H)
            sd[f"{a}.k_proj.weight"] = w(Hk * D, H)
            sd[f"{a}.v_proj.weight"] = w(Hk * D, H)
            sd[f"{a}.o_proj.weight"] = w(H, Hq * D)
            if cfg.qk_norm:
                sd[f"{a}.q_norm.weight"] = n(D)
                sd[f"{a}.k_norm.weight"] = n(D)
        m = f"{p}.mlp"
        if cfg.layer_is_moe(i):
            I = cfg.moe_intermediate_size
            sd[f"{m}.gate.weight"] = w(cfg.num_experts, H)
            if cfg.router_bias:
                sd[f"{m}.gate.e_score_correction_bias"] = torch.randn(cfg.num_experts, generator=g) * 0.01
            for e in range(cfg.num_experts):
                sd[f"{m}.experts.{e}.gate_proj.weight"] = w(I, H)
                sd[f"{m}.experts.{e}.up_proj.weight"] = w(I, H)
                sd[f"{m}.experts.{e}.down_proj.weight"] = w(H, I)
            if cfg.n_shared_experts:
                Is = I * cfg.n_shared_experts
                sd[f"{m}.shared_experts.gate_proj.weight"] = w(Is, H)
                sd[f"{m}.shared_experts.up_proj.weight"] = w(Is, H)
                sd[f"{m}.shared_experts.down_proj.weight"] = w(H, Is)
        else:
            I = cfg.intermediate_size
            sd[f"{m}.gate_proj.weight"] = w(I, H)
            sd[f"{m}.up_proj.weight"] = w(I, H)
            sd[f"{m}.down_proj.weight"] = w(H, I)
    return sd


def save_random_checkpoint(cfg, out_dir: str, fmt: str = "mmfp4", seed: int = 0, float_dir: Optional[str] = None,
                           hadamard_block: int = 0) -> dict:
    """Write a random-init float checkpoint (HF names) and quantize it to ``fmt`` in ``out_dir``.  With
    ``hadamard_block`` every quantized matrix is stored in the block-Hadamard-rotated input basis (as MR-GPTQ writes
    them), with a ``<name>.hadamard_block_size`` tensor beside it."""
    float_dir = float_dir or os.path.join(out_dir, "_float")
    os.makedirs(float_dir, exist_ok=True)
    save_file(random_hf_state(cfg, seed), os.path.join(float_dir, "model.safetensors"), metadata={"format": "pt"})
    cfg.save_pretrained(float_dir)
    info = convert_model(float_dir, out_dir, fmt, cfg.group_size, hadamard_block=hadamard_block)
    shutil.rmtree(float_dir, ignore_errors=True)
    return info
