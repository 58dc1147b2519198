"""``MMFP4ForCausalLM``: the user-facing causal LM (load, prefill, generate).

Parity: the class the reference imports at ``metal_marlin/inference/mmfp4_pipeline.py:1843``
(``MMFP4ForCausalLM.from_pretrained``) and ``metal_marlin/cli.py:1780``; generation mirrors
``metal_marlin/inference/mmfp4_pipeline.py:428`` (prefill, then a sync-free decode loop) and
chunked prefill from ``metal_marlin/inference/prefill.py:174`` (chunk 2048).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..engine.session import DecodeSession, SamplingParams
from .config import ModelConfig, get_preset
from .loading import CheckpointSource, RandomSource, build_transformer
from .transformer import BatchMeta, PagedKVStorage, Transformer


def prefill(model: Transformer, kv: PagedKVStorage, seqs: Sequence[Sequence[int]], block_tables: torch.Tensor,
            start: Optional[Sequence[int]] = None, chunk_tokens: int = 4096, max_batch_tokens: int = 32768) -> torch.Tensor:
    """Write the prompts into the paged cache and return fp32 logits of each sequence's last token.

    Sequences are processed in chunks of at most ``chunk_tokens`` (chunked prefill); chunks of
    different sequences are flattened into one varlen batch of at most ``max_batch_tokens``.
    ``start[b]`` tokens of sequence ``b`` are assumed to be cached already (prefix reuse)."""
    dev = model.device
    bs = kv.block_size
    B = len(seqs)
    # parallel models bound a pass: the expert-parallel exchange by its receive regions, the tensor-parallel prompt path by
    # the size of its reduce-scatter / gather buffers
    ep, tp = getattr(model, "ep", None), getattr(model, "tp", None)
    if ep is not None:
        max_batch_tokens = min(max_batch_tokens, ep.max_tokens())
    if tp is not None and getattr(tp, "tp", 1) > 1:
        from ..parallel.tp import FUSED_GEMM_MAX_TOKENS
        max_batch_tokens = min(max_batch_tokens, FUSED_GEMM_MAX_TOKENS)
    chunk_tokens = min(chunk_tokens, max_batch_tokens)
    done = list(start) if start is not None else [0] * B
    last_logits = None       # [B, vocab] (or the rank's vocabulary shard under tensor parallelism)
    pending = [b for b in range(B) if done[b] < len(seqs[b])]
    while pending:
        batch, ntok = [], 0
        for b in list(pending):
            n = min(chunk_tokens, len(seqs[b]) - done[b])
            if batch and ntok + n > max_batch_tokens:
                break
            batch.append((b, done[b], n))
            ntok += n
        ids, pos, cu, ctx, rows = [], [], [0], [], []
        for b, s, n in batch:
            ids.extend(seqs[b][s:s + n])
            pos.extend(range(s, s + n))
            cu.append(cu[-1] + n)
            ctx.append(s + n)
            rows.append(b)
        ids_t = torch.tensor(ids, dtype=torch.int64, device=dev)
        pos_t = torch.tensor(pos, dtype=torch.int32, device=dev)
        bt = block_tables[rows].to(dev)
        # slot of every token: its sequence's block table looked up at position // block_size
        row_of_tok = torch.repeat_interleave(torch.arange(len(batch), device=dev),
                                             torch.tensor([n for _, _, n in batch], device=dev))
        p64 = pos_t.long()
        slots = bt[row_of_tok, p64 // bs].long() * bs + p64 % bs
        meta = BatchMeta(positions=pos_t, slots=slots, block_tables=bt.to(torch.int32).contiguous(),
                         ctx_lens=torch.tensor(ctx, dtype=torch.int32, device=dev), decode=False, cu_seqlens=cu,
                         ctx_lens_host=ctx)
        lg = model.forward(ids_t, kv, meta, last_only=True)
        if last_logits is None:
            last_logits = torch.zeros(B, lg.shape[1], dtype=torch.float32, device=dev)
        for j, (b, s, n) in enumerate(batch):
            done[b] = s + n
            if done[b] >= len(seqs[b]):
                last_logits[b] = lg[j]
                pending.remove(b)
    return last_logits


class MMFP4ForCausalLM:
    def __init__(self, model: Transformer):
        self.model = model
        self.config: ModelConfig = model.cfg
        self.device = model.device

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_pretrained(cls, path: str, device: Optional[str] = None) -> "MMFP4ForCausalLM":
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        cfg = ModelConfig.from_pretrained(path)
        src = CheckpointSource(cfg, path, device)
        lm = cls(build_transformer(cfg, src))
        # multi-token-prediction modules stored after the decoder stack become the model's draft head
        # (reference: metal_marlin/model_utils.py:416 _load_mtp_head_from_checkpoint)
        from ..spec.draft import MTPHead
        lm.model.mtp = MTPHead.from_checkpoint(lm.model, src.loader)
        return lm

    @classmethod
    def from_config(cls, cfg, device: Optional[str] = None, seed: int = 0) -> "MMFP4ForCausalLM":
        """Random-init model quantized to MMFP4 on ``device`` (synthetic workloads)."""
        if isinstance(cfg, str):
            cfg = get_preset(cfg)
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        return cls(build_transformer(cfg, RandomSource(cfg, device, seed)))

    def to(self, device) -> "MMFP4ForCausalLM":
        return MMFP4ForCausalLM(self.model.to(device))

    # ------------------------------------------------------------------ cache helpers
    def new_cache(self, num_blocks: int, block_size: int = 16, kv_dtype: str = "bf16") -> PagedKVStorage:
        return PagedKVStorage(self.config, num_blocks, block_size, self.device, kv_dtype=kv_dtype)

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 32,
                 sampling: Optional[Sequence[SamplingParams]] = None, eos_token_id=None, block_size: int = 16,
                 kv: Optional[PagedKVStorage] = None, use_graph: Optional[bool] = None,
                 return_session: bool = False):
        """Greedy / sampled generation for a batch of token-id prompts.  Returns a list of lists with the
        newly generated ids (truncated after the first EOS)."""
        B = len(prompts)
        max_len = max(len(p) for p in prompts) + max_new_tokens
        nb = (max_len + block_size - 1) // block_size
        if kv is None:
            kv = self.new_cache(B * nb, block_size)
        block_tables = torch.arange(B * nb, dtype=torch.int32).view(B, nb)
        logits = prefill(self.model, kv, prompts, block_tables)
        sess = DecodeSession(self.model, kv, B, nb, max_new_tokens=max_new_tokens, use_graph=use_graph)
        if sampling is None:
            sampling = [SamplingParams()] * B
        sess.set_sampling(sampling)
        # first token comes from the prefill logits (same sampler, no history yet)
        from .. import ops
        first = ops.sample(logits, temperature=sess.temperature, top_k=sess.top_k, top_p=sess.top_p, min_p=sess.min_p,
                           seed=sess.seed, offset=1 << 40) if sess.use_sampler_filters else ops.argmax(logits)
        sess.set_state(first, [len(p) for p in prompts], block_tables)
        eos = None
        if eos_token_id is not None:
            eos = [eos_token_id] if isinstance(eos_token_id, int) else list(eos_token_id)
        out = [[int(t)] for t in first.tolist()]
        if max_new_tokens > 1:
            hist = sess.run(max_new_tokens - 1, eos_ids=eos).tolist()
            for b in range(B):
                out[b].extend(hist[b])
        if eos:
            for b in range(B):
                for i, t in enumerate(out[b]):
                    if t in eos:
                        out[b] = out[b][: i + 1]
                        break
        if return_session:
            return out, sess
        return out

    @torch.no_grad()
    def forward_logits(self, token_ids: Sequence[int], block_size: int = 16) -> torch.Tensor:
        """fp32 logits for every position of one sequence (perplexity / evaluation)."""
        T = len(token_ids)
        nb = (T + block_size - 1) // block_size
        kv = self.new_cache(nb, block_size)
        dev = self.device
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        meta = BatchMeta(positions=pos, slots=pos.long(), block_tables=torch.arange(nb, dtype=torch.int32, device=dev).view(1, nb),
                         ctx_lens=torch.tensor([T], dtype=torch.int32, device=dev), decode=False, cu_seqlens=[0, T],
                         ctx_lens_host=[T])
        return self.model.forward(torch.tensor(list(token_ids), dtype=torch.int64, device=dev), kv, meta, last_only=False)
