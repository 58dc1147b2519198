"""Decode sessions: static device buffers + one CUDA graph per batch shape.

Parity: the reference's allocation- and sync-free decode loop
(``metal_marlin/inference/mmfp4_pipeline.py:428`` ``_optimized_generate``: every buffer
pre-allocated at ``:577-659``, EOS polled every 8 tokens at ``:732``) and its batch
dispatcher ``cpp/src/batch_dispatch.mm`` (queue many kernels, commit once).  On Blackwell the
"commit once" primitive is a CUDA graph of the whole step: embedding, every layer, head,
sampler and the bookkeeping that advances positions / cache slots, so consecutive steps need
no host work at all; the host only copies the chosen token ids back when it wants them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import ops
from ..models.transformer import BatchMeta, PagedKVStorage, Transformer


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    seed: int = 0


class DecodeSession:
    """Fixed-batch decode over a paged cache.

    The caller owns block allocation: ``block_tables`` must cover every position the session will
    write.  ``step()`` consumes ``self.ids`` (current token of each sequence) and leaves the sampled
    next tokens in ``self.ids`` / ``self.out_ids`` and, when ``record`` is on, in ``self.history``.
    """

    def __init__(self, model: Transformer, kv: PagedKVStorage, batch: int, max_blocks_per_seq: int,
                 max_new_tokens: int = 0, use_graph: Optional[bool] = None, max_ctx: Optional[int] = None):
        self.model, self.kv, self.B = model, kv, batch
        dev = model.device
        self.device = dev
        self.ids = torch.zeros(batch, dtype=torch.int64, device=dev)
        self.out_ids = torch.zeros(batch, dtype=torch.int64, device=dev)
        self.positions = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.slots = torch.zeros(batch, dtype=torch.int64, device=dev)
        self.block_tables = torch.zeros(batch, max_blocks_per_seq, dtype=torch.int32, device=dev)
        self.ctx_lens = torch.ones(batch, dtype=torch.int32, device=dev)
        self.active = torch.ones(batch, dtype=torch.bool, device=dev)
        self.temperature = torch.zeros(batch, dtype=torch.float32, device=dev)
        self.top_k = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.top_p = torch.ones(batch, dtype=torch.float32, device=dev)
        self.min_p = torch.zeros(batch, dtype=torch.float32, device=dev)
        self.rep_penalty = torch.ones(batch, dtype=torch.float32, device=dev)
        self.logprob = torch.zeros(batch, dtype=torch.float32, device=dev)
        self.step_idx = torch.zeros(1, dtype=torch.int64, device=dev)
        self.seed = 0
        self.max_new = max_new_tokens
        self.history = torch.full((batch, max(1, max_new_tokens)), -1, dtype=torch.int64, device=dev)
        self.use_sampler_filters = False
        self.use_history_penalty = False
        self.max_ctx = max_ctx or max_blocks_per_seq * kv.block_size
        cfg = model.cfg
        self.splits = ops.default_splits(batch, 1 if cfg.is_mla else cfg.num_key_value_heads, self.max_ctx,
                                         mla_latent=cfg.is_mla and cfg.latent_dim == 576 and getattr(kv, "kv_dtype", "bf16") == "bf16")
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.use_graph = (dev.type == "cuda") if use_graph is None else use_graph
        self.launches_per_step = 0
        self.logits: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ host-side setup
    def set_sampling(self, params: Sequence[SamplingParams]) -> None:
        assert len(params) == self.B
        self.temperature.copy_(torch.tensor([p.temperature for p in params], dtype=torch.float32))
        self.top_k.copy_(torch.tensor([p.top_k for p in params], dtype=torch.int32))
        self.top_p.copy_(torch.tensor([p.top_p for p in params], dtype=torch.float32))
        self.min_p.copy_(torch.tensor([p.min_p for p in params], dtype=torch.float32))
        self.rep_penalty.copy_(torch.tensor([p.repetition_penalty for p in params], dtype=torch.float32))
        self.seed = params[0].seed
        new_filters = any(p.temperature > 0 for p in params)
        new_hist = any(p.repetition_penalty != 1.0 for p in params)
        if (new_filters, new_hist) != (self.use_sampler_filters, self.use_history_penalty):
            self.graph = None    # the captured step bakes in which sampler inputs exist
        self.use_sampler_filters, self.use_history_penalty = new_filters, new_hist

    def set_state(self, ids: torch.Tensor, positions: Sequence[int], block_tables: torch.Tensor) -> None:
        """``positions[b]`` = index of the token in ``ids[b]`` inside its sequence."""
        bs = self.kv.block_size
        self.ids.copy_(ids.to(self.device))
        pos = torch.as_tensor(list(positions), dtype=torch.int32)
        self.positions.copy_(pos)
        self.ctx_lens.copy_(pos + 1)
        nb = block_tables.shape[1]
        self.block_tables.zero_()
        self.block_tables[:, :nb].copy_(block_tables.to(self.device))
        p64 = self.positions.long()
        self.slots.copy_(self.block_tables.gather(1, (p64 // bs).unsqueeze(1)).squeeze(1).long() * bs + p64 % bs)
        self.step_idx.zero_()
        self.history.fill_(-1)

    # ------------------------------------------------------------------ one step
    def _step_body(self) -> None:
        meta = BatchMeta(positions=self.positions, slots=self.slots, block_tables=self.block_tables,
                         ctx_lens=self.ctx_lens, decode=True, max_ctx=self.max_ctx, splits=self.splits)
        logits = self.model.forward(self.ids, self.kv, meta)      # (a tensor-parallel model opens its exchange epoch itself)
        self.logits = logits
        if self.use_sampler_filters or self.use_history_penalty:
            logits = self.model.full_logits(logits)
            ops.sample(logits, temperature=self.temperature, top_k=self.top_k, top_p=self.top_p, min_p=self.min_p,
                       history=self.history if self.use_history_penalty else None,
                       rep_penalty=self.rep_penalty if self.use_history_penalty else None,
                       seed=self.seed, offset=0, offset_dev=self.step_idx, out=self.out_ids, out_logprob=self.logprob)
        else:
            self.model.greedy(logits, out=self.out_ids)
        # bookkeeping on device: next token, position, cache slot, history
        bs = self.kv.block_size
        self.ids.copy_(self.out_ids)
        if self.max_new > 0:
            self.history.scatter_(1, self.step_idx.expand(self.B, 1).clamp(max=self.history.shape[1] - 1),
                                  self.out_ids.unsqueeze(1))
        self.step_idx += 1
        self.positions += 1
        self.ctx_lens += 1
        p64 = self.positions.long()
        blk = self.block_tables.gather(1, (p64 // bs).clamp(max=self.block_tables.shape[1] - 1).unsqueeze(1)).squeeze(1)
        self.slots.copy_(blk.long() * bs + p64 % bs)

    def capture(self, warmup: int = 2) -> None:
        """Capture the step in a CUDA graph (state is saved and restored around the warm-up runs)."""
        if self.device.type != "cuda":
            return
        saved = [t.clone() for t in (self.ids, self.positions, self.slots, self.ctx_lens, self.step_idx, self.history)]
        rec = self.kv.snapshot_recurrent() if hasattr(self.kv, "snapshot_recurrent") else None
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            for _ in range(warmup):
                self._step_body()
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        for dst, src in zip((self.ids, self.positions, self.slots, self.ctx_lens, self.step_idx, self.history), saved):
            dst.copy_(src)
        if rec is not None:
            self.kv.restore_recurrent(rec)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._step_body()
        for dst, src in zip((self.ids, self.positions, self.slots, self.ctx_lens, self.step_idx, self.history), saved):
            dst.copy_(src)
        self.graph = g

    def step(self) -> torch.Tensor:
        if self.use_graph and self.device.type == "cuda":
            if self.graph is None:
                self.capture()
            self.graph.replay()
        else:
            self._step_body()
        return self.out_ids

    def run(self, n_steps: int, eos_ids: Optional[Sequence[int]] = None, poll_every: int = 8) -> torch.Tensor:
        """Run ``n_steps`` decode steps; with ``eos_ids`` the host polls the history every
        ``poll_every`` steps and stops once every sequence has produced an EOS.  Returns
        ``history[:, :steps_run]`` (device tensor)."""
        done = 0
        eos = torch.tensor(list(eos_ids), device=self.device) if eos_ids else None
        while done < n_steps:
            self.step()
            done += 1
            if eos is not None and (done % poll_every == 0 or done == n_steps):
                h = self.history[:, :done]
                if bool(torch.isin(h, eos).any(dim=1).all()):
                    break
        return self.history[:, :done]
