"""Offline quantization driver behind ``metal-marlin quantize``.

Parity: reference ``metal_marlin/hf_loader.py:963`` (``convert_model_to_fp4``) / ``:1355`` (MMFP4 writer) for
round-to-nearest, and ``metal_marlin/mr_gptq.py:686-974`` for the calibrated methods: run calibration text
through the model, accumulate the input Hessian of every quantized projection (one per expert for MoE banks),
then re-quantize every tensor with GPTQ / MR-GPTQ / AWQ and write the same checkpoint formats.  Calibration
activations come from a round-to-nearest FP4 copy of the model running on this engine's own kernels.
"""
from __future__ import annotations

import json
import os
import shutil
import tempfile
import time
from typing import Dict, Optional

import torch

from .. import ops
from ..formats import fp4 as fp4fmt
from . import awq as awq_mod
from . import gptq as gptq_mod
from .calibration import HessianCollector, load_calibration_tokens
from .convert import convert_model, iter_safetensors_weights, should_quantize_tensor, _copy_aux
from .mixed_precision import policy_for

_FP4_FORMATS = {"fp4": "marlin_fp4", "marlin_fp4": "marlin_fp4", "mmfp4": "mmfp4"}


def collect_hessians(model_dir_fp4: str, calibration: str = "synthetic", num_samples: int = 32, seq_len: int = 512,
                     device: Optional[str] = None, keep_inputs: int = 0) -> HessianCollector:
    """Run calibration sequences through the FP4 model at ``model_dir_fp4`` and accumulate ``X^T X`` per checkpoint
    tensor name.  ``keep_inputs`` > 0 also keeps that many input rows per tensor (AWQ needs activations)."""
    from ..models.mmfp4_causal_lm import MMFP4ForCausalLM
    lm = MMFP4ForCausalLM.from_pretrained(model_dir_fp4, device=device)
    tok = None
    try:
        from ..inference.tokenizer import load_tokenizer
        tok = load_tokenizer(model_dir_fp4)
    except Exception:
        tok = None
    max_len = min(seq_len, lm.config.max_position_embeddings)
    if isinstance(calibration, str):
        seqs = load_calibration_tokens(calibration, tok, lm.config.vocab_size, num_samples, max_len)
    else:            # token sequences from the caller (lists or tensors of ids)
        seqs = [[int(t) for t in torch.as_tensor(s).reshape(-1)[:max_len]] for s in calibration][:num_samples]
    col = HessianCollector()
    col.inputs: Dict[str, torch.Tensor] = {}

    def keep(name, x):
        if keep_inputs and name not in col.inputs:
            col.inputs[name] = x[:keep_inputs].detach().to(torch.float32).cpu()

    def hook(kind, W, x, ids):
        if W.names is None:
            return
        if kind == "linear":
            for name, _rows in W.names:            # fused matrices share one input
                col.add(name, x)
                keep(name, x)
            return
        flat_x = x.reshape(-1, x.shape[-1]) if kind == "moe_down" else None
        for e in ids.unique().tolist():
            if e < 0 or e >= len(W.names):
                continue
            if kind == "moe_gate_up":
                rows = x[(ids == e).any(1)]
            else:
                rows = flat_x[(ids == e).reshape(-1)]
            for name, _rows in W.names[e]:
                col.add(name, rows)
                keep(name, rows)

    ops.set_capture(hook)
    try:
        with torch.no_grad():
            for s in seqs:
                lm.forward_logits(s)
    finally:
        ops.set_capture(None)
    return col


def _generic_group_writer(model_dir: str, out_dir: str, fmt: str, group_size: int, mixed_preset: Optional[str], device: str) -> dict:
    """Formats other than FP4: packed codes ``<name>`` (uint8 bit stream) + ``<name>.scales`` (+ ``<name>.zeros``)."""
    from ..formats.safetensors_io import save_file
    from .rtn import pack_bits, quantize
    os.makedirs(out_dir, exist_ok=True)
    tensors, n_q, errs = {}, 0, []
    for name, t in iter_safetensors_weights(model_dir):
        pol_fmt, gs = fmt, group_size
        if mixed_preset:
            pol = policy_for(name, mixed_preset)
            pol_fmt, gs = (None, 0) if pol.fmt == "keep" else (pol.fmt if pol.fmt != "fp4" or fmt == "fp4" else fmt, pol.group_size)
        if pol_fmt is None or not should_quantize_tensor(name, t):
            tensors[name] = t
            continue
        q = quantize(t.to(device=device, dtype=torch.float32), pol_fmt, fp4fmt.pick_group_size(t.shape[1], gs))
        tensors[name] = pack_bits(q.codes.cpu(), q.bits)
        tensors[name + ".scales"] = q.scales.cpu()
        if q.zeros is not None:
            tensors[name + ".zeros"] = q.zeros.cpu()
        tensors[name + ".group_size"] = torch.tensor([q.group_size], dtype=torch.int32)
        tensors[name + ".shape"] = torch.tensor(list(t.shape), dtype=torch.int32)
        errs.append(float((q.dequantize().cpu() - t.float()).pow(2).mean().sqrt() / t.float().pow(2).mean().sqrt().clamp_min(1e-12)))
        n_q += 1
    save_file(tensors, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(out_dir, "quantization_config.json"), "w") as f:
        json.dump({"format": f"marlin_{fmt}", "group_size": group_size, "quant_method": "rtn", "mixed_preset": mixed_preset}, f)
    _copy_aux(model_dir, out_dir)
    return {"quantized": n_q, "tensors": len(tensors), "mean_rel_rmse": sum(errs) / max(1, len(errs))}


class _HessianView:
    """``name -> Hessian`` mapping over a collector (only ``get`` is needed by the writers)."""

    def __init__(self, col):
        self.col = col

    def get(self, name, default=None):
        H = self.col.get(name)
        return default if H is None else H


def quantize_checkpoint(model_dir: str, out_dir: str, fmt: str = "mmfp4", method: str = "rtn", group_size: int = 128,
                        bits: Optional[int] = None, calibration: str = "synthetic", num_samples: int = 32, seq_len: int = 512,
                        mixed_preset: Optional[str] = None, device: Optional[str] = None, act_order: bool = False,
                        target_bpw: Optional[float] = None) -> dict:
    """``fmt="trellis-v2"`` with ``method="ldlq"`` is the EXL3-style pipeline: Hessians of every layer input from calibration
    text, LDL error feedback per matrix, and (with ``target_bpw``) sensitivity-driven mixed bit widths."""
    t0 = time.time()
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    if fmt == "trellis-v2":
        from ..formats.trellis import quantize_model_trellis
        hess = None
        if method in ("ldlq", "exl3"):
            tmp = tempfile.mkdtemp(prefix="mmb200_rtn_")
            try:
                convert_model(model_dir, tmp, "mmfp4", group_size, device=device)
                col = collect_hessians(tmp, calibration, num_samples, seq_len, device)
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
            hess = _HessianView(col)
        elif method != "rtn":
            raise ValueError(f"method {method!r} does not write trellis containers; use rtn or ldlq")
        stats = quantize_model_trellis(model_dir, out_dir, bits=bits or 4, group_size=group_size, device=device, hessians=hess,
                                       target_bpw=target_bpw)
        stats["method"] = "ldlq" if hess is not None else "rtn"
        stats["seconds"] = time.time() - t0
        return stats
    if fmt not in _FP4_FORMATS:
        if method != "rtn":
            raise ValueError(f"method {method!r} writes FP4 formats only; use --format fp4 / mmfp4")
        stats = _generic_group_writer(model_dir, out_dir, fmt, group_size, mixed_preset, device)
        stats["seconds"] = time.time() - t0
        return stats
    ck_fmt = _FP4_FORMATS[fmt]

    def gs_for(name, default):
        if mixed_preset:
            pol = policy_for(name, mixed_preset)
            if pol.fmt == "fp4":
                return pol.group_size
        return default

    if method == "rtn":
        fn = None
        if mixed_preset:
            fn = lambda name, w, gs: fp4fmt.quantize_codes(w, fp4fmt.pick_group_size(w.shape[1], gs_for(name, gs)))
        stats = convert_model(model_dir, out_dir, ck_fmt, group_size, device=device, quantize_fn=fn)
        stats["method"] = "rtn"
        return stats
    # calibrated methods: activations from a round-to-nearest copy
    tmp = tempfile.mkdtemp(prefix="mmb200_rtn_")
    try:
        convert_model(model_dir, tmp, "mmfp4", group_size, device=device)
        col = collect_hessians(tmp, calibration, num_samples, seq_len, device, keep_inputs=256 if method == "awq" else 0)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    state = gptq_mod.ResumableState(out_dir) if os.path.isdir(out_dir) else None
    os.makedirs(out_dir, exist_ok=True)
    state = state or gptq_mod.ResumableState(out_dir)
    info = {"with_hessian": 0, "rtn_fallback": 0, "rotated": 0}

    if method == "awq":
        # whole-checkpoint AWQ: one scale per (RMSNorm -> projections) group, folded into the projections' input channels
        # and out of the norm's weight, so the result is an ordinary weights-only checkpoint
        from ..formats.safetensors_io import SafetensorsFile
        where = {}
        for fn in sorted(os.listdir(model_dir)):
            if fn.endswith(".safetensors"):
                with SafetensorsFile(os.path.join(model_dir, fn)) as sf:
                    for k in sf.keys():
                        where[k] = os.path.join(model_dir, fn)

        def get_w(n):
            with SafetensorsFile(where[n]) as sf:
                return sf.get_tensor(n).to(torch.float32)

        plan = awq_mod.awq_plan(where.keys(), get_w, lambda n: getattr(col, "inputs", {}).get(n), "fp4", group_size)
        stats = convert_model(model_dir, out_dir, ck_fmt, group_size, device=device,
                              tensors=awq_mod.apply_awq_plan(iter_safetensors_weights(model_dir), plan))
        stats.update(method="awq", awq_groups=len(plan), awq_scaled_tensors=sum(len(g["consumers"]) for g in plan.values()),
                     awq_mean_gain=(sum(g["mse_rtn"] / max(g["mse"], 1e-30) for g in plan.values()) / max(1, len(plan))),
                     calibration_tokens=sum(col.n.values()) // max(1, len(col.n)))
        return stats

    def qfn(name, w, gs):
        gs = fp4fmt.pick_group_size(w.shape[1], gs_for(name, gs))
        H = col.get(name)
        if H is None:
            info["rtn_fallback"] += 1
            return fp4fmt.quantize_codes(w, gs)
        H = H.to(w.device)
        if method == "gptq":
            wq, scales, st = gptq_mod.gptq_quantize(w, H, gptq_mod.GPTQConfig("fp4", gs, act_order=act_order))
        else:
            # weights-only checkpoints carry no runtime rotation, so the rotation gate is held closed here; the
            # rotated variant is available through quant.gptq.mr_gptq_quantize + layers.HadamardLinear
            wq, scales, st = gptq_mod.mr_gptq_quantize(w, H, gptq_mod.MRGPTQConfig("fp4", gs, act_order=act_order, force_rotation=False))
        info["with_hessian"] += 1
        state.mark(name, st)
        qt = gptq_mod.to_quantized_tensor(wq, scales, "fp4", gs)
        return qt.codes, qt.scales

    stats = convert_model(model_dir, out_dir, ck_fmt, group_size, device=device, quantize_fn=qfn)
    stats.update(info)
    stats["method"] = method
    stats["calibration_tokens"] = sum(col.n.values()) // max(1, len(col.n))
    return stats
