"""Parity checks of ``.qmi4`` INT4 artifacts through the kernels that serve them: a random activation goes through the
artifact's INT4 layer (the code-table GEMV / GEMM path) and selected output columns are compared with an oracle computed
straight from the packed words in float64 — an independent restatement of ``w = (nibble - zero) * scale``.

Checks mirror the blocks of a hybrid decoder layer: projections alone, the dense MLP (gate | up -> SwiGLU -> down), the
full-attention block for one token (q with its output gate, k, v, then the output projection of ``sigmoid(gate) * v`` — a
single token attends to itself, so the soft-max is the identity), the linear-attention block's projections with its output
projection, and the LM head.

Parity: reference ``qwen36_27b_validation.py`` (``ArtifactParityResult`` :52, ``validate_layer0_qkvb_artifacts`` :304,
``validate_layer0_mlp_artifacts`` :365, ``validate_layer0_full_attention_artifacts`` :460, ``validate_layer0_linear_block_artifacts`` :551,
``validate_layer0_lm_head_artifacts`` :640).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import qmi4


@dataclass(frozen=True)
class ArtifactParityResult:
    role: str
    checked_columns: Tuple[int, ...]
    max_abs_error: float
    max_rel_error: float

    def within(self, atol: float, rtol: float) -> bool:
        return self.max_abs_error <= atol or self.max_rel_error <= rtol


@dataclass
class BlockValidation:
    """Results of one block check, with the norms of the activations that went through it."""
    manifest_dir: str
    block: str
    results: List[ArtifactParityResult] = field(default_factory=list)
    norms: Dict[str, float] = field(default_factory=dict)

    @property
    def max_abs_error(self) -> float:
        return max((r.max_abs_error for r in self.results), default=0.0)

    @property
    def max_rel_error(self) -> float:
        return max((r.max_rel_error for r in self.results), default=0.0)

    def by_role(self) -> Dict[str, ArtifactParityResult]:
        return {r.role: r for r in self.results}

    def assert_within(self, *, atol: float, rtol: float) -> None:
        """A role fails when it is outside BOTH tolerances."""
        for r in self.results:
            if not r.within(atol, rtol):
                raise AssertionError(f"{self.block}: {r.role} parity failed: max_abs_error={r.max_abs_error:.6g} > {atol}, "
                                     f"max_rel_error={r.max_rel_error:.6g} > {rtol}")


def sample_columns(out_features: int, max_columns: int) -> Tuple[int, ...]:
    """All columns when few; else the first, middle and last plus an even stride, ``max_columns`` at most."""
    if max_columns <= 0:
        raise ValueError("max_columns must be positive")
    if out_features <= max_columns:
        return tuple(range(out_features))
    picks = {0, out_features // 2, out_features - 1}
    stride = out_features / max(1, max_columns - 3)
    picks.update(min(out_features - 1, int(i * stride)) for i in range(max_columns - 3))
    return tuple(sorted(picks))[:max_columns]


def oracle_columns(hidden: torch.Tensor, t: qmi4.Qmi4Tensor, columns: Sequence[int]) -> torch.Tensor:
    """``hidden [in] . W[:, columns]`` from the packed container in float64 (``W [in, out]`` in the container's orientation)."""
    cols = torch.as_tensor(list(columns), dtype=torch.long)
    words = t.qweight[:, cols].to(torch.int64) & 0xFFFFFFFF                                    # [packed_k, C]
    shifts = (torch.arange(8, dtype=torch.int64) * 4).view(1, 8, 1)
    nib = ((words.unsqueeze(1) >> shifts) & 0xF).reshape(-1, cols.numel())[: t.in_features].double()
    g = torch.arange(t.in_features) // t.group_size
    w = (nib - t.zeros[:, cols].double()[g]) * t.scales[:, cols].double()[g]
    return (hidden.detach().cpu().double().reshape(1, -1) @ w).reshape(-1)


def compare(role: str, hidden: torch.Tensor, t: qmi4.Qmi4Tensor, actual: torch.Tensor, max_columns: int) -> ArtifactParityResult:
    cols = sample_columns(t.out_features, max_columns)
    want = oracle_columns(hidden, t, cols)
    got = actual.detach().cpu().double().reshape(-1)[list(cols)]
    err = (got - want).abs()
    rel = err / want.abs().clamp_min(1e-6)
    return ArtifactParityResult(role, cols, float(err.max()) if err.numel() else 0.0, float(rel.max()) if rel.numel() else 0.0)


class _Layer:
    """The artifacts of one layer (or the global ones) with their INT4 layers on ``device``."""

    def __init__(self, manifest_dir: str, layer: Optional[int], device=None, shapes=None):
        self.dir = manifest_dir
        m = qmi4.read_manifest(os.path.join(manifest_dir, "manifest.json"), shapes)
        self.tensors = {a.role: qmi4.load_artifact(manifest_dir, a) for a in m.tensors if a.layer_index == layer}
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self._lin: Dict[str, object] = {}

    def need(self, roles: Sequence[str]) -> None:
        missing = [r for r in roles if r not in self.tensors]
        if missing:
            raise KeyError(f"{self.dir}: the manifest has no artifacts for {missing}")

    def run(self, role: str, x: torch.Tensor) -> torch.Tensor:
        lin = self._lin.get(role)
        if lin is None:
            lin = self._lin[role] = self.tensors[role].to_linear(self.device)
        xin = x.reshape(1, -1).to(self.device)
        y = lin(xin.to(torch.bfloat16) if self.device.type == "cuda" else xin.float())
        return y.float().reshape(-1).cpu()

    def act(self, x: torch.Tensor) -> torch.Tensor:
        """The activation as the kernel sees it (bf16 on the GPU), so that the oracle takes the same input."""
        return x.to(torch.bfloat16).float() if self.device.type == "cuda" else x.float()


def _hidden(n: int, seed: int) -> torch.Tensor:
    return torch.randn(n, generator=torch.Generator().manual_seed(seed)) * 0.5


def validate_projections(manifest_dir: str, layer: Optional[int] = 0, roles: Optional[Sequence[str]] = None, max_columns: int = 64, seed: int = 0,
                         device=None, shapes=None) -> BlockValidation:
    """Every named role (default: all of the layer's roles that read the hidden state) on one random hidden vector."""
    L = _Layer(manifest_dir, layer, device, shapes)
    if roles is None:
        roles = [r for r in L.tensors if not r.endswith(("_out", "_o", "mlp_down"))]
    L.need(roles)
    out = BlockValidation(manifest_dir, "projections")
    for r in roles:
        x = L.act(_hidden(L.tensors[r].in_features, seed))
        out.norms[r] = float(x.norm())
        out.results.append(compare(r, x, L.tensors[r], L.run(r, x), max_columns))
    return out


def validate_mlp(manifest_dir: str, layer: Optional[int] = 0, max_columns: int = 64, seed: int = 0, device=None, shapes=None) -> BlockValidation:
    L = _Layer(manifest_dir, layer, device, shapes)
    L.need(qmi4.DENSE_MLP_ROLES)
    x = L.act(_hidden(L.tensors["mlp_gate"].in_features, seed))
    gate, up = L.run("mlp_gate", x), L.run("mlp_up", x)
    inter = L.act(torch.nn.functional.silu(gate) * up)
    out = BlockValidation(manifest_dir, "mlp", norms={"hidden": float(x.norm()), "intermediate": float(inter.norm())})
    out.results += [compare("mlp_gate", x, L.tensors["mlp_gate"], gate, max_columns), compare("mlp_up", x, L.tensors["mlp_up"], up, max_columns),
                    compare("mlp_down", inter, L.tensors["mlp_down"], L.run("mlp_down", inter), max_columns)]
    return out


def validate_full_attention(manifest_dir: str, layer: Optional[int] = 3, max_columns: int = 64, seed: int = 0, device=None, shapes=None,
                            kv_heads: int = 1) -> BlockValidation:
    """One token: ``q`` (query and, when the projection is twice the output projection's input, its output gate), ``k``, ``v``; the
    token attends to itself, so the attention output is ``v`` repeated over the query heads of its group, gated; then ``o``."""
    L = _Layer(manifest_dir, layer, device, shapes)
    L.need(qmi4.FULL_ATTENTION_ROLES)
    x = L.act(_hidden(L.tensors["full_attn_q"].in_features, seed))
    q, k, v = (L.run(r, x) for r in ("full_attn_q", "full_attn_k", "full_attn_v"))
    o_in = L.tensors["full_attn_o"].in_features
    reps = o_in // v.numel()
    if reps * v.numel() != o_in:
        raise ValueError(f"output projection input {o_in} is not a multiple of the value width {v.numel()}")
    if v.numel() % kv_heads:
        raise ValueError(f"value width {v.numel()} is not a multiple of kv_heads={kv_heads}")
    ctx = v.reshape(kv_heads, -1).repeat_interleave(reps, 0).reshape(-1)      # each query head reads the key / value head of its group
    if q.numel() == 2 * o_in:                                  # [query | gate]
        ctx = ctx * torch.sigmoid(q[o_in:])
    ctx = L.act(ctx)
    out = BlockValidation(manifest_dir, "full_attention", norms={"hidden": float(x.norm()), "context": float(ctx.norm())})
    out.results += [compare(r, x, L.tensors[r], y, max_columns) for r, y in (("full_attn_q", q), ("full_attn_k", k), ("full_attn_v", v))]
    out.results.append(compare("full_attn_o", ctx, L.tensors["full_attn_o"], L.run("full_attn_o", ctx), max_columns))
    return out


def validate_linear_block(manifest_dir: str, layer: Optional[int] = 0, max_columns: int = 64, seed: int = 0, device=None, shapes=None
                          ) -> BlockValidation:
    """The linear-attention block's input projections on one hidden vector, and its output projection on ``v * silu(z)`` (the
    gated value path of a first token, whose recurrent state is still empty)."""
    L = _Layer(manifest_dir, layer, device, shapes)
    L.need(qmi4.LINEAR_ATTENTION_ROLES)
    x = L.act(_hidden(L.tensors["linear_attn_q"].in_features, seed))
    ys = {r: L.run(r, x) for r in qmi4.LINEAR_ATTENTION_ROLES if r != "linear_attn_out"}
    core = L.act(ys["linear_attn_v"] * torch.nn.functional.silu(ys["linear_attn_z"]))
    out = BlockValidation(manifest_dir, "linear_block", norms={"hidden": float(x.norm()), "core": float(core.norm())})
    out.results += [compare(r, x, L.tensors[r], y, max_columns) for r, y in ys.items()]
    out.results.append(compare("linear_attn_out", core, L.tensors["linear_attn_out"], L.run("linear_attn_out", core), max_columns))
    return out


def validate_lm_head(manifest_dir: str, max_columns: int = 128, seed: int = 0, device=None, shapes=None) -> BlockValidation:
    L = _Layer(manifest_dir, None, device, shapes)
    L.need(("lm_head",))
    x = L.act(_hidden(L.tensors["lm_head"].in_features, seed))
    y = L.run("lm_head", x)
    out = BlockValidation(manifest_dir, "lm_head", norms={"hidden": float(x.norm()), "logits": float(y.norm())})
    out.results.append(compare("lm_head", x, L.tensors["lm_head"], y, max_columns))
    return out


def validate_all(manifest_dir: str, linear_layer: Optional[int] = 0, attention_layer: Optional[int] = 3, max_columns: int = 64, device=None,
                 shapes=None) -> Dict[str, BlockValidation]:
    """Every block check the manifest has the artifacts for."""
    m = qmi4.read_manifest(os.path.join(manifest_dir, "manifest.json"), shapes)
    have = {(a.layer_index, a.role) for a in m.tensors}
    out: Dict[str, BlockValidation] = {}
    for layer in sorted({l for l, _ in have if l is not None}):
        if all((layer, r) in have for r in qmi4.DENSE_MLP_ROLES) and "mlp" not in out:
            out["mlp"] = validate_mlp(manifest_dir, layer, max_columns, device=device, shapes=shapes)
    if all((linear_layer, r) in have for r in qmi4.LINEAR_ATTENTION_ROLES):
        out["linear_block"] = validate_linear_block(manifest_dir, linear_layer, max_columns, device=device, shapes=shapes)
    if all((attention_layer, r) in have for r in qmi4.FULL_ATTENTION_ROLES):
        out["full_attention"] = validate_full_attention(manifest_dir, attention_layer, max_columns, device=device, shapes=shapes)
    if (None, "lm_head") in have:
        out["lm_head"] = validate_lm_head(manifest_dir, max_columns, device=device, shapes=shapes)
    return out
