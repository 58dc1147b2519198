"""Routing profile of a mixture-of-experts model: per-layer expert load (counts, rank distribution, probability moments,
balance measures), which experts fire together, how well a layer's routing is predicted by the layer before it, hot / cold /
dead experts and prefetch recommendations, a JSON report and a heat-map image.

Streaming by design: ``record_routing`` folds each batch into fixed-size count tensors (``[E]``, ``[E, K]``, ``[E, E]``) with
``bincount`` / one-hot products — on the device the ids live on — so memory does not grow with the number of tokens profiled.
Between consecutive layers of one forward pass (same token order, same token count) it also accumulates the ``[E, E]``
transition counts that the predictability estimate uses.  ``profile_model`` drives it from an engine model through the
operator capture hook.

Parity: reference ``analysis/moe_routing.py`` (``ExpertLoadStats`` :44, ``ExpertCooccurrence`` :79, ``LayerRoutingProfile`` :107,
``RoutingPredictability`` :147, ``MoERoutingProfiler`` :173 with ``record_routing`` / ``layer_profiles`` / ``cooccurrence`` /
``predictability`` / ``get_hot_experts`` / ``get_cold_experts`` / ``get_dead_experts`` / ``get_prefetch_recommendations`` /
``generate_report`` / ``save_report`` / ``print_summary`` / ``plot_routing_heatmap``; ``analyze_routing_from_file`` :868;
``simulate_routing_for_model`` :917).
"""
from __future__ import annotations

import json
import math
import os
import threading
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class ExpertLoadStats:
    expert_id: int
    total_activations: int = 0
    activation_rate: float = 0.0             # share of all routing decisions of the layer
    avg_probability: float = 0.0
    std_probability: float = 0.0
    rank_distribution: Dict[int, int] = field(default_factory=dict)
    is_hot: bool = False
    is_cold: bool = False
    is_dead: bool = False

    @property
    def primary_selection_rate(self) -> float:
        return self.rank_distribution.get(0, 0) / self.total_activations if self.total_activations else 0.0


@dataclass
class ExpertCooccurrence:
    num_experts: int
    cooccurrence_matrix: Optional[np.ndarray] = None      # [E, E] symmetric counts, zero diagonal
    conditional_probs: Optional[np.ndarray] = None        # [i, j] = P(j selected | i selected)
    top_pairs: List[Tuple[int, int, int]] = field(default_factory=list)

    def __post_init__(self):
        if self.cooccurrence_matrix is None:
            self.cooccurrence_matrix = np.zeros((self.num_experts, self.num_experts), dtype=np.int64)


@dataclass
class LayerRoutingProfile:
    layer_idx: int
    expert_stats: Dict[int, ExpertLoadStats] = field(default_factory=dict)
    total_tokens: int = 0
    load_balance_cv: float = 0.0
    entropy: float = 0.0                     # of the load distribution, in bits
    gini_coefficient: float = 0.0
    active_experts: int = 0
    dead_experts: int = 0

    def get_hot_experts(self, threshold: Optional[float] = None) -> List[int]:
        if threshold is None:
            return [e for e, s in self.expert_stats.items() if s.is_hot]
        mean = 1.0 / max(1, len(self.expert_stats))
        return [e for e, s in self.expert_stats.items() if s.activation_rate > threshold * mean]

    def get_cold_experts(self, threshold: Optional[float] = None) -> List[int]:
        if threshold is None:
            return [e for e, s in self.expert_stats.items() if s.is_cold]
        mean = 1.0 / max(1, len(self.expert_stats))
        return [e for e, s in self.expert_stats.items() if 0 < s.activation_rate < threshold * mean]

    def get_dead_experts(self) -> List[int]:
        return [e for e, s in self.expert_stats.items() if s.is_dead]


@dataclass
class RoutingPredictability:
    num_layers: int
    layer_correlations: Optional[np.ndarray] = None       # [L, L]: correlation of the layers' load vectors
    predictable_from_layer: int = -1
    avg_prediction_accuracy: float = 0.0
    per_layer_accuracy: Dict[int, float] = field(default_factory=dict)

    def __post_init__(self):
        if self.layer_correlations is None:
            self.layer_correlations = np.zeros((self.num_layers, self.num_layers), dtype=np.float32)


def gini(x: np.ndarray) -> float:
    x = np.sort(np.asarray(x, dtype=np.float64))
    n, s = x.size, x.sum()
    if n == 0 or s <= 0:
        return 0.0
    return float((2 * np.arange(1, n + 1) - n - 1).dot(x) / (n * s))


class MoERoutingProfiler:
    def __init__(self, num_experts: int, num_layers: int, top_k: int = 2, hot_threshold: float = 1.5, cold_threshold: float = 0.5,
                 predictability_threshold: float = 0.5):
        self.num_experts, self.num_layers, self.top_k = num_experts, num_layers, top_k
        self.hot_threshold, self.cold_threshold, self.predictability_threshold = hot_threshold, cold_threshold, predictability_threshold
        E, L, K = num_experts, num_layers, top_k
        self._counts = torch.zeros(L, E, dtype=torch.int64)
        self._rank = torch.zeros(L, E, K, dtype=torch.int64)
        self._psum = torch.zeros(L, E, dtype=torch.float64)
        self._psq = torch.zeros(L, E, dtype=torch.float64)
        self._pcount = torch.zeros(L, E, dtype=torch.int64)
        self._tokens = [0] * L
        self._cooc = torch.zeros(E, E, dtype=torch.int64)
        self._trans: Dict[int, torch.Tensor] = {}            # layer l -> [E, E] counts: expert of layer l-1 (row) with expert of layer l (column)
        self._last: Optional[Tuple[int, torch.Tensor]] = None
        self._lock = threading.Lock()
        self._cache: Dict[str, Any] = {}

    # ------------------------------------------------------------------ recording
    def record_routing(self, layer_idx: int, expert_ids, expert_probs=None) -> None:
        """``expert_ids [tokens, top_k]`` (a flat vector is cut into rows of ``top_k``; negative ids are ignored), ``expert_probs`` of
        the same shape or None."""
        if not 0 <= layer_idx < self.num_layers:
            raise ValueError(f"layer_idx {layer_idx} out of range [0, {self.num_layers})")
        ids = torch.as_tensor(np.asarray(expert_ids) if not isinstance(expert_ids, torch.Tensor) else expert_ids).long()
        ids = ids.reshape(-1, self.top_k) if ids.dim() == 1 else ids.reshape(-1, ids.shape[-1])
        K = min(ids.shape[1], self.top_k)
        E = self.num_experts
        if ids.numel() and int(ids.max()) >= E:
            raise ValueError(f"expert id {int(ids.max())} out of range [0, {E})")
        valid = ids >= 0
        safe = ids.clamp_min(0)
        ones = valid.to(torch.int64)
        rank = torch.zeros(E, self.top_k, dtype=torch.int64, device=ids.device)
        for k in range(K):
            rank[:, k] = torch.bincount(safe[:, k], weights=None if valid[:, k].all() else ones[:, k].double(), minlength=E).long()[:E]
        hot = torch.zeros(ids.shape[0], E, dtype=torch.float32, device=ids.device)
        hot.scatter_add_(1, safe, valid.float())
        hot.clamp_(max=1.0)
        cooc = (hot.t() @ hot).round().long()
        trans = None
        with self._lock:
            prev = self._last
            if prev is not None and prev[0] == layer_idx - 1 and prev[1].shape[0] == hot.shape[0] and prev[1].device == hot.device:
                trans = (prev[1].t() @ hot).round().long().cpu()
            self._last = (layer_idx, hot)
            self._counts[layer_idx] += rank.sum(1).cpu()
            self._rank[layer_idx] += rank.cpu()
            self._tokens[layer_idx] += ids.shape[0]
            c = cooc.cpu()
            c.fill_diagonal_(0)
            self._cooc += c
            if trans is not None:
                self._trans[layer_idx] = self._trans.get(layer_idx, torch.zeros(E, E, dtype=torch.int64)) + trans
            if expert_probs is not None:
                p = torch.as_tensor(np.asarray(expert_probs) if not isinstance(expert_probs, torch.Tensor) else expert_probs).to(ids.device)
                p = p.reshape(ids.shape).double() * valid
                flat = safe.reshape(-1)
                self._psum[layer_idx] += torch.zeros(E, dtype=torch.float64, device=ids.device).scatter_add_(0, flat, p.reshape(-1)).cpu()
                self._psq[layer_idx] += torch.zeros(E, dtype=torch.float64, device=ids.device).scatter_add_(0, flat, (p * p).reshape(-1)).cpu()
                self._pcount[layer_idx] += torch.zeros(E, dtype=torch.int64, device=ids.device).scatter_add_(0, flat, ones.reshape(-1)).cpu()
            self._cache.clear()

    def end_pass(self) -> None:
        """Forget the previous layer's tokens (call between forward passes when layer 0 does not follow the last layer)."""
        with self._lock:
            self._last = None

    # ------------------------------------------------------------------ results
    @property
    def layer_profiles(self) -> Dict[int, LayerRoutingProfile]:
        if "profiles" not in self._cache:
            out = {}
            E = self.num_experts
            for l in range(self.num_layers):
                counts = self._counts[l].numpy().astype(np.float64)
                total = counts.sum()
                prof = LayerRoutingProfile(l, total_tokens=self._tokens[l])
                if total > 0:
                    rate = counts / total
                    mean = 1.0 / E
                    nz = rate[rate > 0]
                    prof.load_balance_cv = float(counts.std() / counts.mean())
                    prof.entropy = float(-(nz * np.log2(nz)).sum())
                    prof.gini_coefficient = gini(counts)
                    prof.active_experts = int((counts > 0).sum())
                    prof.dead_experts = E - prof.active_experts
                    for e in range(E):
                        n = int(self._pcount[l, e])
                        avg = float(self._psum[l, e]) / n if n else 0.0
                        var = max(0.0, float(self._psq[l, e]) / n - avg * avg) if n else 0.0
                        prof.expert_stats[e] = ExpertLoadStats(
                            e, int(counts[e]), float(rate[e]), avg, math.sqrt(var), {k: int(self._rank[l, e, k]) for k in range(self.top_k)},
                            is_hot=rate[e] > self.hot_threshold * mean, is_cold=0 < rate[e] < self.cold_threshold * mean, is_dead=counts[e] == 0)
                out[l] = prof
            self._cache["profiles"] = out
        return self._cache["profiles"]

    @property
    def cooccurrence(self) -> ExpertCooccurrence:
        if "cooc" not in self._cache:
            m = self._cooc.numpy().copy()
            sel = self._counts.sum(0).numpy().astype(np.float64)         # how often each expert was selected (any layer)
            cond = np.divide(m, sel[:, None], out=np.zeros(m.shape, dtype=np.float64), where=sel[:, None] > 0)
            iu = np.triu_indices(self.num_experts, 1)
            order = np.argsort(-m[iu], kind="stable")[:20]
            pairs = [(int(iu[0][i]), int(iu[1][i]), int(m[iu][i])) for i in order if m[iu][i] > 0]
            self._cache["cooc"] = ExpertCooccurrence(self.num_experts, m, cond.astype(np.float32), pairs)
        return self._cache["cooc"]

    @property
    def predictability(self) -> RoutingPredictability:
        """``per_layer_accuracy[l]``: expected share of layer ``l``'s selected experts that are among the ``top_k`` most likely
        successors of an expert selected at layer ``l - 1`` (from the transition counts; 1.0 = the previous layer decides the next).
        ``predictable_from_layer``: first layer from which every later measured layer is above the threshold."""
        if "pred" not in self._cache:
            L = self.num_layers
            loads = self._counts.numpy().astype(np.float64)
            corr = np.zeros((L, L), dtype=np.float32)
            live = [l for l in range(L) if loads[l].std() > 0]
            if len(live) > 1:
                c = np.corrcoef(loads[live])
                for a, la in enumerate(live):
                    for b, lb in enumerate(live):
                        corr[la, lb] = c[a, b]
            acc: Dict[int, float] = {}
            for l, T in sorted(self._trans.items()):
                t = T.numpy().astype(np.float64)
                rows = t.sum(1)
                if rows.sum() <= 0:
                    continue
                k = min(self.top_k, t.shape[1])
                best = -np.sort(-t, axis=1)[:, :k].sum(1)                 # mass of the k most likely successors of each source expert
                acc[l] = float(best.sum() / rows.sum())
            start = -1
            for l in sorted(acc):
                if all(acc[m] >= self.predictability_threshold for m in acc if m >= l):
                    start = l - 1
                    break
            self._cache["pred"] = RoutingPredictability(L, corr, start, float(np.mean(list(acc.values()))) if acc else 0.0, acc)
        return self._cache["pred"]

    def _collect(self, which: str, layer_idx: Optional[int]) -> List[int]:
        profs = self.layer_profiles
        if layer_idx is not None:
            return getattr(profs[layer_idx], which)()
        sets = [set(getattr(p, which)()) for p in profs.values() if p.total_tokens]
        if not sets:
            return []
        # hot / cold anywhere; dead only when dead in every profiled layer
        return sorted(set.intersection(*sets) if which == "get_dead_experts" else set.union(*sets))

    def get_hot_experts(self, layer_idx: Optional[int] = None) -> List[int]:
        return self._collect("get_hot_experts", layer_idx)

    def get_cold_experts(self, layer_idx: Optional[int] = None) -> List[int]:
        return self._collect("get_cold_experts", layer_idx)

    def get_dead_experts(self, layer_idx: Optional[int] = None) -> List[int]:
        return self._collect("get_dead_experts", layer_idx)

    def get_prefetch_recommendations(self, layer_idx: int, num_experts: int = 4, given_previous: Optional[Sequence[int]] = None) -> List[int]:
        """The experts of ``layer_idx`` most worth having resident: by load, or — with the experts just selected at the layer
        before — by the transition counts from those experts."""
        if given_previous is not None and layer_idx in self._trans:
            score = self._trans[layer_idx][list(given_previous)].sum(0).double()
            if float(score.sum()) > 0:
                return torch.argsort(score, descending=True, stable=True)[:num_experts].tolist()
        return torch.argsort(self._counts[layer_idx], descending=True, stable=True)[:num_experts].tolist()

    # ------------------------------------------------------------------ reports
    def generate_report(self) -> Dict[str, Any]:
        profs, co, pr = self.layer_profiles, self.cooccurrence, self.predictability
        layers = {}
        for l, p in profs.items():
            if not p.total_tokens:
                continue
            layers[str(l)] = {"total_tokens": p.total_tokens, "load_balance_cv": p.load_balance_cv, "entropy": p.entropy, "max_entropy": math.log2(self.num_experts),
                              "gini_coefficient": p.gini_coefficient, "active_experts": p.active_experts, "dead_experts": p.dead_experts,
                              "hot_experts": p.get_hot_experts(), "cold_experts": p.get_cold_experts(), "dead_expert_ids": p.get_dead_experts(),
                              "top_experts": [{"expert_id": s.expert_id, "activation_rate": s.activation_rate, "avg_probability": s.avg_probability,
                                               "primary_selection_rate": s.primary_selection_rate}
                                              for s in sorted(p.expert_stats.values(), key=lambda s: -s.activation_rate)[:8]]}
        cvs = [v["load_balance_cv"] for v in layers.values()]
        return {"config": {"num_experts": self.num_experts, "num_layers": self.num_layers, "top_k": self.top_k, "hot_threshold": self.hot_threshold,
                           "cold_threshold": self.cold_threshold},
                "summary": {"layers_profiled": len(layers), "tokens_per_layer": max(self._tokens) if self._tokens else 0,
                            "mean_load_balance_cv": float(np.mean(cvs)) if cvs else 0.0, "hot_experts": self.get_hot_experts(),
                            "dead_experts_all_layers": self.get_dead_experts()},
                "layers": layers,
                "cooccurrence": {"top_pairs": [{"experts": [a, b], "count": c} for a, b, c in co.top_pairs]},
                "predictability": {"predictable_from_layer": pr.predictable_from_layer, "avg_prediction_accuracy": pr.avg_prediction_accuracy,
                                   "per_layer_accuracy": {str(k): v for k, v in pr.per_layer_accuracy.items()}}}

    def save_report(self, path: str) -> None:
        os.makedirs(os.path.dirname(os.path.abspath(str(path))), exist_ok=True)
        with open(path, "w") as f:
            json.dump(self.generate_report(), f, indent=1)

    def summary_text(self) -> str:
        r = self.generate_report()
        s = r["summary"]
        lines = [f"MoE routing: {self.num_layers} layers x {self.num_experts} experts, top-{self.top_k}; {s['layers_profiled']} layers profiled, "
                 f"{s['tokens_per_layer']} tokens", f"mean load CV {s['mean_load_balance_cv']:.3f}; hot {len(s['hot_experts'])}, dead everywhere {len(s['dead_experts_all_layers'])}"]
        for l, v in r["layers"].items():
            lines.append(f"  layer {l:>3}: CV {v['load_balance_cv']:.3f}  entropy {v['entropy']:.2f}/{v['max_entropy']:.2f}  gini {v['gini_coefficient']:.3f}  "
                         f"active {v['active_experts']}  hot {len(v['hot_experts'])}  dead {v['dead_experts']}")
        p = r["predictability"]
        lines.append(f"next-layer prediction accuracy {p['avg_prediction_accuracy']:.3f}; predictable from layer {p['predictable_from_layer']}")
        return "\n".join(lines)

    def print_summary(self) -> None:
        print(self.summary_text())

    def plot_routing_heatmap(self, path: Optional[str] = None, cell: int = 6) -> np.ndarray:
        """Layers (rows) by experts (columns), colour = load relative to the uniform share (black 0, through red and yellow to
        white at 3x and above).  Returns the ``[L * cell, E * cell, 3]`` uint8 image and writes it (PNG through Pillow when the
        name ends in ``.png``, else binary PPM)."""
        loads = self._counts.numpy().astype(np.float64)
        tot = loads.sum(1, keepdims=True)
        rel = np.divide(loads * self.num_experts, tot, out=np.zeros_like(loads), where=tot > 0)
        v = np.clip(rel / 3.0, 0, 1)
        rgb = np.stack([np.clip(3 * v, 0, 1), np.clip(3 * v - 1, 0, 1), np.clip(3 * v - 2, 0, 1)], -1)
        img = (np.kron(rgb, np.ones((cell, cell, 1))) * 255).astype(np.uint8)
        if path is not None:
            os.makedirs(os.path.dirname(os.path.abspath(str(path))), exist_ok=True)
            if str(path).lower().endswith(".png"):
                from PIL import Image
                Image.fromarray(img).save(path)
            else:
                with open(path, "wb") as f:
                    f.write(f"P6 {img.shape[1]} {img.shape[0]} 255\n".encode() + img.tobytes())
        return img


def analyze_routing_from_file(routing_log_path: str, num_experts: int, num_layers: int, top_k: int, output_dir: Optional[str] = None) -> MoERoutingProfiler:
    """JSON lines ``{"layer": l, "expert_ids": [[..], ..], "probs": [[..], ..]}`` -> profiler; with ``output_dir`` also
    ``routing_report.json`` and ``routing_heatmap.png`` there."""
    prof = MoERoutingProfiler(num_experts, num_layers, top_k)
    with open(routing_log_path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            prof.record_routing(int(rec["layer"]), np.asarray(rec["expert_ids"]), np.asarray(rec["probs"]) if rec.get("probs") is not None else None)
    if output_dir:
        prof.save_report(os.path.join(output_dir, "routing_report.json"))
        prof.plot_routing_heatmap(os.path.join(output_dir, "routing_heatmap.png"))
    return prof


SIMULATED_MODELS = {"qwen3_30b": dict(num_experts=128, num_layers=48, top_k=8), "mixtral": dict(num_experts=8, num_layers=32, top_k=2),
                    "glm47": dict(num_experts=64, num_layers=40, top_k=2), "glm47_flash": dict(num_experts=64, num_layers=46, top_k=4),
                    "deepseek_moe": dict(num_experts=64, num_layers=28, top_k=6)}


def simulate_routing_for_model(model_name: str, num_samples: int = 1000, seed: int = 42, layer_coupling: float = 0.5) -> MoERoutingProfiler:
    """Synthetic routing with the traits of real routers: a skewed popularity per layer (a quarter of the experts favoured,
    a twentieth nearly dead in every fifth layer) and token logits that carry over from layer to layer with weight
    ``layer_coupling`` (what makes the next layer predictable)."""
    if model_name not in SIMULATED_MODELS:
        raise ValueError(f"unknown model {model_name!r}; options: {sorted(SIMULATED_MODELS)}")
    cfg = SIMULATED_MODELS[model_name]
    E, L, K = cfg["num_experts"], cfg["num_layers"], cfg["top_k"]
    g = torch.Generator().manual_seed(seed)
    prof = MoERoutingProfiler(**cfg)
    token = torch.randn(num_samples, E, generator=g)
    for l in range(L):
        base = torch.randn(E, generator=g) * 0.5
        fav = torch.randperm(E, generator=g)[: max(1, E // 4)]
        base[fav] += 1.0
        if l % 5 == 0:
            base[torch.randperm(E, generator=g)[: max(1, E // 20)]] -= 12.0
        token = layer_coupling * token + (1 - layer_coupling) * torch.randn(num_samples, E, generator=g)
        p = torch.softmax(base + token, -1)
        w, ids = p.topk(K, -1)
        prof.record_routing(l, ids, w / w.sum(-1, keepdim=True))
    prof.end_pass()
    return prof


def profile_model(lm, token_sequences: Sequence[Sequence[int]], profiler: Optional[MoERoutingProfiler] = None) -> MoERoutingProfiler:
    """Run token sequences through an engine model and record the routing of every MoE layer (through the operator capture
    hook; MoE layers are numbered in order of appearance — by the expert bank's tensor names when it has them, else by position in the pass)."""
    from .. import ops
    from ..formats.mmfp4_loader import extract_layer_index
    cfg = lm.config
    moe_layers: Dict[int, int] = {}
    if profiler is None:
        n_moe = sum(1 for i in range(cfg.num_hidden_layers) if cfg.layer_is_moe(i))
        profiler = MoERoutingProfiler(cfg.num_experts, max(1, n_moe), cfg.num_experts_per_tok)

    seen = [0]                                      # MoE layers met so far in the current pass

    def hook(kind, W, x, ids):
        if kind != "moe_gate_up":
            return
        names = getattr(W, "names", None)
        layer = extract_layer_index(names[0][0][0]) if names else None
        slot = moe_layers.setdefault(layer, len(moe_layers)) if layer is not None else seen[0]
        seen[0] += 1
        if slot < profiler.num_layers:
            sel = ids[:, : profiler.top_k]                         # shared experts, when appended, come after the routed ones
            profiler.record_routing(slot, sel.masked_fill(sel >= profiler.num_experts, -1))

    ops.set_capture(hook)
    try:
        with torch.no_grad():
            for s in token_sequences:
                seen[0] = 0
                lm.forward_logits(list(s))
                profiler.end_pass()
    finally:
        ops.set_capture(None)
    return profiler


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="MoE routing analysis from a routing log (JSON lines) or a simulated model")
    ap.add_argument("--log")
    ap.add_argument("--simulate", choices=sorted(SIMULATED_MODELS))
    ap.add_argument("--num-experts", type=int)
    ap.add_argument("--num-layers", type=int)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--samples", type=int, default=1000)
    ap.add_argument("--output-dir")
    a = ap.parse_args(argv)
    if a.simulate:
        prof = simulate_routing_for_model(a.simulate, a.samples)
        if a.output_dir:
            prof.save_report(os.path.join(a.output_dir, "routing_report.json"))
            prof.plot_routing_heatmap(os.path.join(a.output_dir, "routing_heatmap.png"))
    elif a.log and a.num_experts and a.num_layers:
        prof = analyze_routing_from_file(a.log, a.num_experts, a.num_layers, a.top_k, a.output_dir)
    else:
        ap.error("give --simulate, or --log with --num-experts and --num-layers")
    prof.print_summary()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
