"""Draft token sources for speculative decoding.

Parity: reference ``metal_marlin/speculative/draft.py``: ``DraftModel`` ABC ``:64``, ``SmallModelDraft``
``:102``, ``NGramDraft`` ``:272`` (online n-gram table), ``EagleHead`` ``:459/:550`` (tree drafts);
``metal_marlin/speculative/mtp_draft.py:17`` / ``metal_marlin/layers/mmfp4_mtp_head.py:39`` (multi-token
prediction heads sharing the target's lm_head).
"""
from __future__ import annotations

import abc
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch


@dataclass
class DraftOutput:
    tokens: List[int]
    probs: Optional[torch.Tensor] = None          # [K, V] draft distributions (None = deterministic draft)
    parents: Optional[List[int]] = None           # tree drafts: parent index of every node (-1 = context)


class DraftModel(abc.ABC):
    @abc.abstractmethod
    def propose(self, context: Sequence[int], k: int, hidden: Optional[torch.Tensor] = None) -> DraftOutput:
        ...

    def observe(self, context: Sequence[int]) -> None:
        """Feed accepted tokens back (online drafts learn from them)."""

    def reset(self) -> None:
        pass


class NGramDraft(DraftModel):
    """Prompt-lookup / online n-gram table: the longest suffix seen before predicts what followed it."""

    def __init__(self, max_n: int = 4, min_n: int = 1):
        self.max_n, self.min_n = max_n, min_n
        self.table: Dict[Tuple[int, ...], Dict[int, int]] = defaultdict(lambda: defaultdict(int))
        self._seen = 0

    def reset(self) -> None:
        self.table.clear()
        self._seen = 0

    def observe(self, context: Sequence[int]) -> None:
        ctx = list(context)
        for i in range(max(self._seen, 1), len(ctx)):
            for n in range(self.min_n, self.max_n + 1):
                if i - n < 0:
                    break
                self.table[tuple(ctx[i - n:i])][ctx[i]] += 1
        self._seen = len(ctx)

    def _next(self, ctx: List[int]) -> Optional[int]:
        for n in range(min(self.max_n, len(ctx)), self.min_n - 1, -1):
            nxt = self.table.get(tuple(ctx[-n:]))
            if nxt:
                return max(nxt.items(), key=lambda kv: (kv[1], -kv[0]))[0]
        return None

    def propose(self, context, k, hidden=None) -> DraftOutput:
        self.observe(context)
        ctx, out = list(context), []
        for _ in range(k):
            t = self._next(ctx)
            if t is None:
                break
            out.append(t)
            ctx.append(t)
        return DraftOutput(out)


class SmallModelDraft(DraftModel):
    """A smaller causal LM with the target's vocabulary drafts ``k`` tokens autoregressively.  It keeps
    its own paged cache and only prefills the tokens it has not seen yet."""

    def __init__(self, lm, max_len: int = 8192, block_size: int = 16, temperature: float = 0.0):
        from ..models.mmfp4_causal_lm import prefill
        self.lm, self._prefill = lm, prefill
        self.block_size = block_size
        self.nb = -(-max_len // block_size)
        self.kv = lm.new_cache(self.nb, block_size)
        self.bt = torch.arange(self.nb, dtype=torch.int32).view(1, self.nb)
        self.cached: List[int] = []
        self.temperature = temperature

    def reset(self) -> None:
        self.cached = []

    @torch.no_grad()
    def propose(self, context, k, hidden=None) -> DraftOutput:
        ctx = list(context)
        common = 0
        for a, b in zip(self.cached, ctx):
            if a != b:
                break
            common += 1
        common = min(common, len(ctx) - 1)
        toks, probs = [], []
        cur = ctx
        for _ in range(k):
            lg = self._prefill(self.lm.model, self.kv, [cur], self.bt, start=[common])[0]
            if self.temperature > 0:
                p = torch.softmax(lg / self.temperature, -1)
                t = int(torch.multinomial(p.cpu(), 1))
                probs.append(p)
            else:
                t = int(lg.argmax())
            common = len(cur)
            toks.append(t)
            cur = cur + [t]
        self.cached = cur[:-1]
        return DraftOutput(toks, torch.stack(probs) if probs else None)


class MTPHead:
    """Multi-token-prediction module: depth ``d`` maps the target's final hidden state (plus the embedding
    of the last drafted token) to a hidden state whose head projection predicts token ``t + d + 1``.

    Per depth: an optional ``[H, 2H]`` bf16 fusion projection (``proj``; input = ``[norm_h(hidden) | norm_e(embedding)]``), an
    optional output norm, and either its own vocabulary head ``[V, H]`` (``heads``) or the target's ``lm_head``.  Random
    initialisation gives the projections only; :meth:`from_checkpoint` reads whatever the checkpoint carries:

    * GLM style (``model.layers.<L + d>.shared_head.head.weight``): a vocabulary head per depth applied to the target's
      hidden state - no fusion projection;
    * DeepSeek-V3 style (``model.layers.<L + d>.{eh_proj, enorm, hnorm, shared_head.norm, shared_head.head}``): fusion
      projection + norms + head (the module's transformer block is not run: the draft is one projection deep)."""

    def __init__(self, model, depth: int = 4, seed: int = 0, std: float = 0.02, random_init: bool = True):
        H = model.cfg.hidden_size
        self.model, self.depth = model, depth
        self.proj: List[Optional[torch.Tensor]] = [None] * depth
        self.heads: List[Optional[torch.Tensor]] = [None] * depth
        self.enorm: List[Optional[torch.Tensor]] = [None] * depth
        self.hnorm: List[Optional[torch.Tensor]] = [None] * depth
        self.out_norm: List[Optional[torch.Tensor]] = [None] * depth
        self.source = "random"
        if random_init:
            g = torch.Generator(device="cpu").manual_seed(seed)
            self.proj = [(torch.randn(H, 2 * H, generator=g) * std).to(torch.bfloat16).to(model.device) for _ in range(depth)]

    @classmethod
    def from_checkpoint(cls, model, loader, depth: Optional[int] = None) -> Optional["MTPHead"]:
        """Build the head from the tensors of ``loader`` (``has_tensor`` / ``load_tensor``); ``None`` if it has none."""
        cfg = model.cfg
        L, H, V = cfg.num_hidden_layers, cfg.hidden_size, cfg.vocab_size
        want = depth or getattr(cfg, "num_nextn_predict_layers", 0) or 1
        dev = model.device

        def get(key, shape=None):
            if not loader.has_tensor(key):
                return None
            t = loader.load_tensor(key)
            base = key[: -len(".weight")] if key.endswith(".weight") else key
            if not torch.is_floating_point(t) and hasattr(loader, "is_quantized") and loader.is_quantized(base):
                # a converter quantized the matrix with the rest of the model: draft heads are small, keep them as bf16
                from ..ops.weights import FP4Weight
                packed, scales, layout = loader.get_quantized_weight(base)
                w = FP4Weight.from_marlin_fp4(packed, scales, "cpu") if layout == "marlin_fp4" else FP4Weight.from_mmfp4(packed, scales, "cpu")
                t = w.dequantize(torch.float32)
            if not torch.is_floating_point(t):
                return None
            if shape is not None:
                if tuple(t.shape) == tuple(shape[::-1]) and len(shape) == 2 and shape[0] != shape[1]:
                    t = t.t()
                if tuple(t.shape) != tuple(shape):
                    return None
            return t.to(dev, torch.bfloat16).contiguous()

        found = []
        for li in list(range(L, L + want)) + [L - 1]:                  # the modules follow the decoder stack
            pre = f"model.layers.{li}."
            ent = {"proj": get(pre + "eh_proj.weight", (H, 2 * H)), "enorm": get(pre + "enorm.weight", (H,)),
                   "hnorm": get(pre + "hnorm.weight", (H,)), "out_norm": get(pre + "shared_head.norm.weight", (H,)),
                   "head": get(pre + "shared_head.head.weight", (V, H))}
            if ent["proj"] is not None or ent["head"] is not None:
                found.append(ent)
            if len(found) >= want:
                break
        if not found:
            return None
        self = cls(model, len(found), random_init=False)
        for d, ent in enumerate(found):
            self.proj[d], self.enorm[d], self.hnorm[d] = ent["proj"], ent["enorm"], ent["hnorm"]
            self.out_norm[d], self.heads[d] = ent["out_norm"], ent["head"]
        self.source = "checkpoint"
        return self

    def _norm(self, x: torch.Tensor, w: Optional[torch.Tensor]) -> torch.Tensor:
        if w is None:
            return x
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.model.cfg.rms_norm_eps) * w.float()).to(torch.bfloat16)

    def step(self, d: int, h: torch.Tensor, tok: int):
        """One depth: ``(next hidden [1, H] bf16, logits [V] fp32)``."""
        m = self.model
        if self.proj[d] is not None:
            e = m.embed[tok].reshape(1, -1)
            x = torch.cat([self._norm(h, self.hnorm[d]), self._norm(e, self.enorm[d])], -1)
            h = torch.nn.functional.linear(x.float(), self.proj[d].float()).to(torch.bfloat16)
        hn = self._norm(h, self.out_norm[d])
        head = self.heads[d] if self.heads[d] is not None else m.lm_head
        return h, torch.nn.functional.linear(hn.float(), head.float())[0]

    @torch.no_grad()
    def draft(self, hidden: torch.Tensor, last_token: int, k: int) -> List[int]:
        h = hidden.reshape(1, -1).to(torch.bfloat16)
        tok = last_token
        out = []
        for d in range(min(k, self.depth)):
            h, lg = self.step(d, h, tok)
            tok = int(lg.argmax(-1))
            out.append(tok)
        return out


class MTPDraft(DraftModel):
    def __init__(self, model, depth: int = 4, seed: int = 0):
        if model.mtp is None:
            model.mtp = MTPHead(model, depth, seed)
        self.head = model.mtp

    def propose(self, context, k, hidden=None) -> DraftOutput:
        if hidden is None:
            return DraftOutput([])
        return DraftOutput(self.head.draft(hidden, context[-1], k))


class EagleDraft(DraftModel):
    """EAGLE-style tree draft: a light autoregressive head expands the ``width`` most likely continuations
    per level for ``depth`` levels; the tree is verified in one target pass with a tree attention mask."""

    def __init__(self, model, width: int = 3, depth: int = 3, seed: int = 0, head: Optional[MTPHead] = None):
        self.model, self.width = model, width
        self.head = head if head is not None else MTPHead(model, depth, seed + 17)
        self.depth = min(depth, self.head.depth)

    @classmethod
    def from_checkpoint(cls, model, path: str, width: int = 3, depth: int = 3) -> "EagleDraft":
        """Draft head from a safetensors file (or a directory holding ``model.safetensors``).  Understood layouts:
        ``fc.weight [H, 2H]`` (the fusion layer of published EAGLE heads, shared by every depth; ``fc.bias`` is folded in when
        the checkpoint has one, and its own ``lm_head.weight`` / ``norm.weight`` are used if present) and the per-depth
        ``heads.<d>.weight [V, H]`` / ``proj.<d>.weight [H, 2H]`` tensors :meth:`save` writes."""
        import os
        from ..formats.safetensors_io import load_file
        fn = os.path.join(path, "model.safetensors") if os.path.isdir(path) else path
        sd = load_file(fn)
        H, V, dev = model.cfg.hidden_size, model.cfg.vocab_size, model.device
        bf = lambda t: t.to(dev, torch.bfloat16).contiguous()
        n = max([int(k.split(".")[1]) + 1 for k in sd if k.startswith(("heads.", "proj."))] + [0])
        head = MTPHead(model, n or depth, random_init=False)
        if "fc.weight" in sd and tuple(sd["fc.weight"].shape) == (H, 2 * H):
            for d in range(head.depth):
                head.proj[d] = bf(sd["fc.weight"])
                if "lm_head.weight" in sd and tuple(sd["lm_head.weight"].shape) == (V, H):
                    head.heads[d] = bf(sd["lm_head.weight"])
                if "norm.weight" in sd:
                    head.out_norm[d] = bf(sd["norm.weight"])
        for d in range(head.depth):
            if f"proj.{d}.weight" in sd:
                head.proj[d] = bf(sd[f"proj.{d}.weight"])
            if f"heads.{d}.weight" in sd:
                head.heads[d] = bf(sd[f"heads.{d}.weight"])
        if all(p is None and h is None for p, h in zip(head.proj, head.heads)):
            raise ValueError(f"{fn} holds no draft-head tensors (fc.weight, proj.<d>.weight or heads.<d>.weight)")
        head.source = "checkpoint"
        return cls(model, width, depth, head=head)

    def save(self, path: str) -> None:
        from ..formats.safetensors_io import save_file
        sd = {}
        for d in range(self.head.depth):
            if self.head.proj[d] is not None:
                sd[f"proj.{d}.weight"] = self.head.proj[d].cpu()
            if self.head.heads[d] is not None:
                sd[f"heads.{d}.weight"] = self.head.heads[d].cpu()
        save_file(sd, path)

    @torch.no_grad()
    def propose(self, context, k, hidden=None) -> DraftOutput:
        if hidden is None:
            return DraftOutput([], parents=[])
        m = self.model
        tokens, parents = [], []
        frontier = [(-1, hidden.reshape(1, -1).to(torch.bfloat16), context[-1])]
        for d in range(self.depth):
            nxt = []
            for parent, h, tok in frontier:
                hh, lg = self.head.step(d, h, tok)
                top = lg.topk(self.width if d == 0 else 1).indices.tolist()
                for t in top:
                    tokens.append(t)
                    parents.append(parent)
                    nxt.append((len(tokens) - 1, hh, t))
            frontier = nxt
            if len(tokens) >= max(k, 1) * self.width:
                break
        return DraftOutput(tokens, parents=parents)
