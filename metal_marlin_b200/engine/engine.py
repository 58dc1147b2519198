"""Serving engine: scheduler + paged cache + model runner, driven by ``step()`` (synchronously or
from a background thread).

Parity: the loop the reference sketches but never wires to its HTTP server
(``metal_marlin/serving/continuous_batch.py:550,614`` + ``metal_marlin/serving/runner.py:157``
``BatchedModelRunner.execute`` + ``metal_marlin/serving/continuous_engine.py:129``).  Differences by
design: the KV scatter is one kernel instead of a per-token python loop (runner.py:562); decode
batches replay a CUDA graph per batch-size bucket with inputs staged through pinned host buffers;
sampling happens on the device and only token ids cross PCIe.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from ..kv.paged import PagedKVCache
from ..models.transformer import BatchMeta, PagedKVStorage, Transformer
from .request import GenerationRequest, RequestStatus, RunningRequest, SchedulerOutput
from .scheduler import BatchScheduler, SchedulerConfig
from .session import SamplingParams
from ..parallel.health import raise_for_status


@dataclass
class EngineConfig:
    num_kv_blocks: int = 512
    block_size: int = 16
    kv_cache_dtype: str = "bf16"       # "fp8" / "int8" (half the cache bytes), "fp4" / "int4" (a quarter): codes + one scale per cached row
    max_model_len: int = 4096
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 2048
    max_prefill_tokens: int = 1024
    max_chunk: int = 512
    enable_prefix_cache: bool = True
    use_cuda_graphs: bool = True
    request_timeout_s: float = 60.0
    graph_buckets: Sequence[int] = (1, 2, 4, 8, 16, 32, 64)
    scheduler_policy: str = "priority"   # "priority" (continuous batching with priorities) | "fcfs" | "shortest_first" | "longest_first"
    preemption_mode: str = "recompute"   # "swap": a preempted sequence keeps its cache rows in pinned host memory and resumes from them
    swap_space_blocks: int = 0           # host blocks for swapped sequences (0 with "swap": as many as ``num_kv_blocks``)
    adaptive_prefill_budget: bool = False   # shrink the prompt-token budget under memory pressure / after an out-of-memory error, regrow later


HISTORY_LEN = 256      # most recent tokens (prompt tail + generated) the repetition penalty looks at


class PrefillBudget:
    """Memory-aware prompt-token budget of an engine.  Before every iteration the free device memory (what the driver
    reports plus what the caching allocator holds unused) is compared with the transient memory a prompt pass of the
    current budget needs: below 1.25 x the need the scheduler's ``max_prefill_tokens`` is halved (never below ``floor``),
    above 2 x the need of a budget a quarter larger it grows back toward the configured value.  A prompt pass that still
    runs out of memory halves it at once and its chunks are planned again.  Activations of a prompt pass scale with its token
    count, so this is the batch-size knob that matters once the cache itself is a fixed pool; a device that is simply full of
    pre-allocated pools is not pressure by this measure.

    Parity: reference ``metal_marlin/inference/mmfp4_pipeline.py:2735`` (``_dynamic_batch``: shrink on pressure, recover
    gradually, per-request memory estimate) and ``metal_marlin/memory/memory_pressure.py``."""

    def __init__(self, scheduler_cfg, need_fn, free_fn=None, floor: int = 128):
        self.cfg = scheduler_cfg
        self.ceiling = scheduler_cfg.max_prefill_tokens
        self.floor = min(floor, self.ceiling)
        self.need_fn = need_fn                       # tokens -> bytes a prompt pass of that many tokens allocates
        self.free_fn = free_fn or self._device_free
        self.shrinks = self.ooms = 0

    @staticmethod
    def _device_free() -> int:
        if not torch.cuda.is_available():
            return 1 << 62
        free, _total = torch.cuda.mem_get_info()
        return free + torch.cuda.memory_reserved() - torch.cuda.memory_allocated()

    @property
    def value(self) -> int:
        return self.cfg.max_prefill_tokens

    def _set(self, v: int) -> int:
        self.cfg.max_prefill_tokens = max(self.floor, min(self.ceiling, int(v)))
        return self.cfg.max_prefill_tokens

    def before_iteration(self) -> int:
        free = self.free_fn()
        if free < 1.25 * self.need_fn(self.value):
            if self.value > self.floor:
                self.shrinks += 1
            return self._set(self.value // 2)
        if self.value < self.ceiling:
            grown = min(self.ceiling, self.value + max(16, self.value // 4))
            if free > 2.0 * self.need_fn(grown):
                return self._set(grown)
        return self.value

    def on_oom(self) -> int:
        self.ooms += 1
        return self._set(self.value // 2)

    def stats(self) -> dict:
        return {"max_prefill_tokens": self.value, "configured": self.ceiling, "shrinks": self.shrinks, "ooms": self.ooms}


def _packed(specs, pin: bool, device=None):
    """One byte buffer holding several named arrays (16-byte aligned segments), so a whole decode batch crosses PCIe (or is
    broadcast to tensor-parallel followers) as a single copy.  ``specs``: ``(name, dtype, shape)``.  Returns
    ``(buffer, {name: view})``."""
    off, segs = 0, []
    for name, dt, shape in specs:
        n = 1
        for d in shape:
            n *= d
        nbytes = n * torch.empty(0, dtype=dt).element_size()
        segs.append((name, dt, shape, off, nbytes))
        off += (nbytes + 15) // 16 * 16
    buf = torch.zeros(off, dtype=torch.uint8, pin_memory=pin) if device is None else torch.zeros(off, dtype=torch.uint8, device=device)
    return buf, {name: buf[o:o + nb].view(dt).view(*shape) for name, dt, shape, o, nb in segs}


class _DecodeBucket:
    """Static buffers (+ optional CUDA graph) for decode batches padded to ``B`` rows.  All per-step inputs live in one
    packed host buffer and one packed device buffer; the device status word of the bounded in-kernel waits comes back in
    the same trip as the sampled ids."""

    def __init__(self, model: Transformer, kv: PagedKVStorage, B: int, max_blocks: int, use_graph: bool):
        dev = model.device
        self.model, self.kv, self.B, self.dev = model, kv, B, dev
        pin = dev.type == "cuda"
        specs = [("ids", torch.int64, (B,)), ("slots", torch.int64, (B,)), ("seeds", torch.int64, (B,)),
                 ("pos", torch.int32, (B,)), ("ctx", torch.int32, (B,)), ("topk", torch.int32, (B,)),
                 ("bt", torch.int32, (B, max_blocks)), ("f", torch.float32, (4, B))]     # f: temperature, top_p, min_p, rep_penalty
        self.h_buf, h = _packed(specs, pin)
        self.d_buf, d = _packed(specs, False, dev)
        self.h_ids, self.h_slots, self.h_seeds, self.h_pos, self.h_ctx = h["ids"], h["slots"], h["seeds"], h["pos"], h["ctx"]
        self.h_topk, self.h_bt, self.h_f = h["topk"], h["bt"], h["f"]
        self.ids, self.slots, self.seeds, self.pos, self.ctx = d["ids"], d["slots"], d["seeds"], d["pos"], d["ctx"]
        self.topk, self.bt, self.f = d["topk"], d["bt"], d["f"]
        self.h_slots.fill_(-1)
        self.h_ctx.fill_(1)
        self.h_hist = torch.full((B, HISTORY_LEN), -1, dtype=torch.int64, pin_memory=pin)
        self.hist = torch.full((B, HISTORY_LEN), -1, dtype=torch.int64, device=dev)
        self.hist_dirty = False
        self.h_out = torch.zeros(B, dtype=torch.int64, pin_memory=pin)
        self.h_status = torch.zeros(4, dtype=torch.int32, pin_memory=pin)
        self.out = torch.zeros(B, dtype=torch.int64, device=dev)
        self.step_no = torch.zeros(1, dtype=torch.int64, device=dev)
        cfg = model.cfg
        self.max_ctx = max_blocks * kv.block_size
        self.splits = ops.default_splits(B, 1 if cfg.is_mla else cfg.num_key_value_heads, self.max_ctx,
                                         mla_latent=cfg.is_mla and cfg.latent_dim == 576 and getattr(self.kv, "kv_dtype", "bf16") == "bf16")
        self.use_graph = use_graph and dev.type == "cuda"
        ep = getattr(model, "ep", None)
        if ep is not None and ep.mode != "fused":
            self.use_graph = False       # the all-to-all baseline reads its split sizes on the host: not capturable
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.status = ops.gemm_status(dev)

    def _forward(self):
        meta = BatchMeta(positions=self.pos, slots=self.slots, block_tables=self.bt, ctx_lens=self.ctx, decode=True,
                         max_ctx=self.max_ctx, splits=self.splits)
        self.logits = self.model.forward(self.ids, self.kv, meta)

    def _sample(self):
        ops.sample(self.model.full_logits(self.logits), temperature=self.f[0], top_k=self.topk, top_p=self.f[1], min_p=self.f[2],
                   history=self.hist, rep_penalty=self.f[3], seed_dev=self.seeds, offset_dev=self.step_no, out=self.out)
        self.step_no += 1

    def _body(self):
        self._forward()
        self._sample()

    def upload(self) -> None:
        """Stage this step's inputs on the device: one copy of the packed buffer (+ the token history when a row uses a
        repetition penalty)."""
        self.d_buf.copy_(self.h_buf, non_blocking=True)
        if self.hist_dirty:
            self.hist.copy_(self.h_hist, non_blocking=True)
        self.hist_dirty = False

    def execute(self) -> torch.Tensor:
        # With a vocabulary-sharded head the sampler needs the logits of all ranks: that gather is a library collective and
        # stays outside the captured graph (the graph then holds this library's kernels only).
        split = getattr(self.model, "tp", None) is not None and self.model.tp.tp > 1
        if self.use_graph:
            if self.graph is None:
                rec = self.kv.snapshot_recurrent() if hasattr(self.kv, "snapshot_recurrent") else None
                s = torch.cuda.Stream(device=self.dev)
                s.wait_stream(torch.cuda.current_stream(self.dev))
                with torch.cuda.stream(s):
                    self._body()
                torch.cuda.current_stream(self.dev).wait_stream(s)
                torch.cuda.synchronize(self.dev)
                if rec is not None:
                    self.kv.restore_recurrent(rec)      # the warm-up pass advanced the recurrent states
                self.step_no.zero_()            # the warm-up pass must not advance the random stream
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph):
                    self._forward() if split else self._body()
                self.step_no.zero_()
            self.graph.replay()
            if split:
                self._sample()
        else:
            self._body()
        self.h_out.copy_(self.out, non_blocking=True)
        self.h_status.copy_(self.status, non_blocking=True)
        if self.dev.type == "cuda":
            torch.cuda.current_stream(self.dev).synchronize()
        code = int(self.h_status[0])
        if code:
            self.status.zero_()             # one expiry must not fail every later step
            self.h_status.zero_()
            ep = getattr(self.model, "ep", None)
            if code == 120 and ep is not None and getattr(ep, "capacity_policy", "error") == "drop":
                ep.overflow_steps += 1      # token dropping was asked for: the step stands without the rows that did not fit
            else:
                raise_for_status(code)
        return self.h_out

    def run(self) -> torch.Tensor:
        self.upload()
        return self.execute()


class LLMEngine:
    def __init__(self, model: Transformer, config: Optional[EngineConfig] = None, coordinator=None):
        """``coordinator`` (``engine/distributed.py``): set on the leading rank of a tensor-parallel group; it tells the
        other ranks which batch to run before this rank launches it, so all shards execute the same passes in step."""
        self.model = model
        self.cfg = config or EngineConfig()
        self.coordinator = coordinator
        self.spec = None             # speculative decoding inside the batch loop (enable_speculative)
        self.spec_proposed = 0
        self.spec_accepted = 0
        self.lockstep = None         # set by an expert-parallel group: passes are agreed between the ranks (engine/distributed.py)
        self._tracked: Dict[str, RunningRequest] = {}
        self._filler_block: Optional[int] = None
        c = self.cfg
        self.recurrent = bool(getattr(model.cfg, "has_linear_layers", False))
        if self.recurrent and c.enable_prefix_cache:
            # the recurrent state of a sequence is addressed by its first cache block and cannot be shared or truncated:
            # no prefix sharing (and no speculative roll-back, see enable_speculative) for hybrid stacks
            import dataclasses
            c = self.cfg = dataclasses.replace(c, enable_prefix_cache=False)
        self.kv = PagedKVStorage(model.cfg, c.num_kv_blocks, c.block_size, model.device, kv_dtype=c.kv_cache_dtype)
        self.cache = PagedKVCache(c.num_kv_blocks, c.block_size, enable_prefix_cache=c.enable_prefix_cache,
                                  copy_fn=self._copy_block)
        # swapping moves cache rows only: the recurrent state of a hybrid stack is addressed by a sequence's first block, and
        # the shards of a tensor-parallel group would each have to repeat the moves, so both fall back to recompute
        swap = c.preemption_mode == "swap" and not self.recurrent and coordinator is None
        self.swap_blocks = (c.swap_space_blocks or c.num_kv_blocks) if swap else 0
        self._swap_pools = None
        scfg = SchedulerConfig(max_num_seqs=c.max_num_seqs, max_num_batched_tokens=c.max_num_batched_tokens,
                               max_prefill_tokens=c.max_prefill_tokens, block_size=c.block_size, max_chunk=c.max_chunk,
                               max_model_len=c.max_model_len, preemption_mode="swap" if swap else "recompute",
                               swap_space_blocks=self.swap_blocks)
        if c.scheduler_policy == "priority":
            self.scheduler = BatchScheduler(scfg, self.cache)
        else:
            from .fcfs import FCFSScheduler, PrefillStrategy
            self.scheduler = FCFSScheduler(scfg, self.cache, prefill_strategy=PrefillStrategy(c.scheduler_policy))
        self.prefill_budget = None
        if c.adaptive_prefill_budget and coordinator is None:
            from ..inference.prefill import estimate_chunk_bytes
            self.prefill_budget = PrefillBudget(self.scheduler.cfg, lambda n: estimate_chunk_bytes(model.cfg, n, c.max_model_len))
        self.max_blocks = -(-c.max_model_len // c.block_size)
        self._buckets: Dict[int, _DecodeBucket] = {}
        self._lock = threading.RLock()
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self._wake = threading.Event()
        self.iterations = 0
        self.tokens_generated = 0
        self.last_error: Optional[str] = None

    # ------------------------------------------------------------------ cache plumbing
    def _copy_block(self, src: int, dst: int) -> None:
        bs = self.cfg.block_size
        for pool in (self.kv.k, self.kv.v):
            for t in pool:
                if t is not None:
                    ops.kv_copy_rows(t, slice(dst * bs, (dst + 1) * bs), slice(src * bs, (src + 1) * bs))

    def _host_pools(self):
        """Host mirrors of the cache pools (``swap_blocks`` blocks each, pinned on a CUDA engine), created at the first swap."""
        if self._swap_pools is None:
            n = self.swap_blocks * self.cfg.block_size
            pin = self.model.device.type == "cuda"

            def host(t):
                return torch.zeros(n, *t.shape[1:], dtype=t.dtype, pin_memory=pin)
            pools = []
            for group in (self.kv.k, self.kv.v):
                for t in group:
                    if t is None:
                        continue
                    pools.extend((d, host(d)) for d in ([t.data, t.scale] if isinstance(t, ops.FP8KV) else [t]))
            self._swap_pools = pools
        return self._swap_pools

    def _apply_swaps(self, out: SchedulerOutput) -> None:
        """Carry out the block moves the scheduler planned: all moves to the host first (their device blocks may be handed
        to another sequence in this very iteration, and to a sequence swapped in below), then the moves back."""
        bs = self.cfg.block_size
        dev = self.model.device
        ar = torch.arange(bs)

        def rows(blocks):
            return (torch.tensor(blocks, dtype=torch.int64).unsqueeze(1) * bs + ar).reshape(-1)
        pools = self._host_pools()
        for _rr, dev_blocks, host_blocks in out.swap_out:
            d, h = rows(dev_blocks).to(dev), rows(host_blocks)
            for dev_t, host_t in pools:
                host_t[h] = dev_t[d].to("cpu")
        for _rr, host_blocks, dev_blocks in out.swap_in:
            d, h = rows(dev_blocks).to(dev), rows(host_blocks)
            for dev_t, host_t in pools:
                dev_t[d] = host_t[h].to(dev, non_blocking=False)

    # ------------------------------------------------------------------ public API
    def add_request(self, req: GenerationRequest) -> RunningRequest:
        if req.timeout_s is None:
            req.timeout_s = self.cfg.request_timeout_s
        with self._lock:
            rr = self.scheduler.add_request(req)
            if self.lockstep is not None:
                self._tracked[rr.id] = rr
        self._wake.set()
        return rr

    def tracked(self) -> List[RunningRequest]:
        """Requests added since they were last untracked (an expert-parallel group reports their progress to the leader)."""
        return list(self._tracked.values())

    def untrack(self, request_id: str) -> None:
        self._tracked.pop(request_id, None)

    def fail_running(self, reason: str) -> None:
        """Fail every in-flight request (after a step raised) so the engine can carry on with new ones."""
        self.last_error = reason
        with self._lock:
            for rr in list(self.scheduler.running):
                rr.error = reason
                self.scheduler.running.remove(rr)
                self.cache.release(rr.id)
                rr.transition(RequestStatus.FAILED)

    def abort(self, request_id: str) -> bool:
        with self._lock:
            return self.scheduler.abort(request_id)

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    @torch.no_grad()
    def step(self) -> List[RunningRequest]:
        """One engine iteration.  Returns the requests that finished in it."""
        with self._lock:
            if self.iterations % 64 == 63 and not self.recurrent and self.coordinator is None and self.lockstep is None:
                self.cache.compact()         # packs the blocks in use when the free space has crumbled (rarely true)
            if self.prefill_budget is not None and self.lockstep is None and (
                    self.scheduler.num_waiting or any(r.status is RequestStatus.PREFILLING for r in self.scheduler.running)):
                self.prefill_budget.before_iteration()          # only iterations that can schedule prompt tokens pay the query
            out = self.scheduler.schedule()
            if out.swap_out or out.swap_in:
                self._apply_swaps(out)
            do_prefill, do_decode = bool(out.prefill), bool(out.decode)
            n_pre = n_dec = 0
            if self.lockstep is not None:
                # expert-parallel group: a pass runs on every rank if any rank needs it (a rank without work runs a filler);
                # the ranks also learn the largest token count of each pass, which bounds the rows an expert owner receives
                mine_pre = sum(ch.length for ch in out.prefill)
                mine_dec = self._bucket_size(len(out.decode)) if out.decode else 0
                n_pre, n_dec = self.lockstep.agree(mine_pre, mine_dec)
                do_prefill, do_decode = n_pre > 0, n_dec > 0
            elif out.is_empty:
                return []
            sampled: Dict[str, int] = {}
            ep = getattr(self.model, "ep", None)
            if do_prefill:
                if ep is not None:
                    ep.pass_tokens = n_pre
                sampled.update(self._run_prefill(out) if out.prefill else self._filler_prefill())
            if do_decode:
                if ep is not None:
                    ep.pass_tokens = n_dec
                if self.spec is not None and out.decode and self.lockstep is None:
                    sampled.update(self._run_decode_speculative(out.decode))
                else:
                    sampled.update(self._run_decode(out.decode) if out.decode else self._filler_decode())
            if out.is_empty:
                return []
            finished = self.scheduler.step(out, sampled)
            self.iterations += 1
            self.tokens_generated += sum(len(v) if isinstance(v, (list, tuple)) else 1 for v in sampled.values())
            return finished

    def run_until_done(self, max_iters: int = 1 << 30) -> None:
        it = 0
        while self.has_work() and it < max_iters:
            self.step()
            it += 1

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16,
                 sampling: Optional[SamplingParams] = None, eos_ids: Sequence[int] = ()) -> List[List[int]]:
        rrs = [self.add_request(GenerationRequest(list(p), max_new_tokens, sampling or SamplingParams(), eos_ids))
               for p in prompts]
        if self._thread is None:
            self.run_until_done()
        else:
            for rr in rrs:
                rr.done.wait()
        return [rr.output_ids for rr in rrs]

    # ------------------------------------------------------------------ background loop
    def start(self) -> None:
        if self._thread is not None:
            return
        self._stop.clear()
        self._thread = threading.Thread(target=self._loop, name="mmb200-engine", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        self._wake.set()
        if self._thread is not None:
            self._thread.join(timeout=10)
            self._thread = None

    def _loop(self) -> None:
        while not self._stop.is_set():
            if not self.has_work():
                self._wake.wait(timeout=0.05)
                self._wake.clear()
                continue
            try:
                self.step()
            except Exception as e:      # fail every in-flight request rather than wedging the server
                self.fail_running(repr(e))

    # ------------------------------------------------------------------ model execution
    def _prefill_arrays(self, out: SchedulerOutput) -> Dict[str, list]:
        """Host description of a flattened prompt pass (token ids, positions, cache slots, block tables)."""
        ids: List[int] = []
        pos: List[int] = []
        slots: List[int] = []
        cu = [0]
        ctx = []
        tables = []
        for ch in out.prefill:
            rr = ch.request
            ids.extend(rr.all_ids[ch.start:ch.start + ch.length])
            pos.extend(range(ch.start, ch.start + ch.length))
            slots.extend(self.cache.table.slot_mapping(rr.id, ch.start, ch.length))
            cu.append(cu[-1] + ch.length)
            ctx.append(ch.start + ch.length)
            tables.append(self.cache.table.block_table(rr.id))
        width = max(len(t) for t in tables)
        return {"ids": ids, "pos": pos, "slots": slots, "cu": cu, "ctx": ctx,
                "tables": [t + [0] * (width - len(t)) for t in tables]}

    def _exec_prefill(self, a: Dict[str, list]) -> torch.Tensor:
        """Runs the prompt pass described by ``a`` on this rank's model shard; returns the full-vocabulary logits of the
        last token of every chunk (of every token when ``a["all_rows"]`` is set: speculative verification).  Every rank of
        a tensor-parallel group runs this with the same arrays."""
        dev = self.model.device
        meta = BatchMeta(positions=torch.tensor(a["pos"], dtype=torch.int32, device=dev),
                         slots=torch.tensor(a["slots"], dtype=torch.int64, device=dev),
                         block_tables=torch.tensor(a["tables"], dtype=torch.int32, device=dev),
                         ctx_lens=torch.tensor(a["ctx"], dtype=torch.int32, device=dev), decode=False, cu_seqlens=list(a["cu"]),
                         ctx_lens_host=list(a["ctx"]))
        logits = self.model.forward(torch.tensor(a["ids"], dtype=torch.int64, device=dev), self.kv, meta,
                                    last_only=not a.get("all_rows", 0))
        return self.model.full_logits(logits)

    def _run_prefill(self, out: SchedulerOutput) -> Dict[str, int]:
        arrays = self._prefill_arrays(out)
        if self.coordinator is not None:
            self.coordinator.announce_prefill(arrays)
        if self.prefill_budget is not None and self.lockstep is None:
            try:
                logits = self._exec_prefill(arrays)
            except torch.cuda.OutOfMemoryError:
                # the pass did not fit: give the allocator's cache back, halve the budget and plan these chunks again (their
                # progress is only recorded after a pass, so dropping them from this iteration's plan is the whole roll-back)
                torch.cuda.empty_cache()
                if sum(ch.length for ch in out.prefill) <= self.prefill_budget.floor:
                    raise
                self.prefill_budget.on_oom()
                out.prefill.clear()
                return {}
        else:
            logits = self._exec_prefill(arrays)
        # sample a first token only for requests whose prefill completes now and that have no output yet
        rows, reqs = [], []
        for j, ch in enumerate(out.prefill):
            rr = ch.request
            if ch.start + ch.length >= rr.prefill_target and not rr.output_ids:
                rows.append(j)
                reqs.append(rr)
        if not rows:
            self._check_device_status()
            return {}
        toks = self._sample(logits[rows].contiguous(), reqs)
        self._check_device_status()
        return {rr.id: int(t) for rr, t in zip(reqs, toks)}

    # ------------------------------------------------------------------ speculative decoding in the batch loop
    def enable_speculative(self, draft="ngram", num_speculative_tokens: int = 4, adaptive: bool = True, **draft_kw) -> None:
        """Every decoding request drafts up to ``num_speculative_tokens`` tokens per step (``draft``: ``"ngram"``, a callable
        ``request -> DraftModel``, or a small causal LM shared by all requests' drafts); one flattened target pass verifies
        the drafts of the whole batch (k + 1 positions per sequence, paged attention over each sequence's own context),
        accepted tokens are kept, the cache rows of rejected ones are given back.  Requests that sample with a temperature
        use rejection sampling against the draft distribution where the draft provides one, else fall back to one token."""
        if getattr(self, "recurrent", False):
            raise ValueError("speculative decoding needs a cache that can be rolled back; recurrent (linear attention) layers keep a state "
                             "that cannot")
        from ..spec.adaptive import AdaptiveSpeculationController
        from ..spec.draft import DraftModel, NGramDraft, SmallModelDraft
        if draft == "ngram":
            make = lambda rr: NGramDraft(**draft_kw)
        elif callable(draft) and not isinstance(draft, DraftModel):
            make = draft
        elif isinstance(draft, DraftModel):
            raise ValueError("pass a factory (request -> DraftModel): drafts keep per-request state")
        else:        # a small causal LM: every request gets its own draft cache over the shared weights
            make = lambda rr, lm=draft: SmallModelDraft(lm, max_len=self.cfg.max_model_len, block_size=self.cfg.block_size, **draft_kw)
        self.spec = {"make": make, "k": int(num_speculative_tokens),
                     "ctrl": (lambda: AdaptiveSpeculationController(depth=num_speculative_tokens)) if adaptive else None}

    def disable_speculative(self) -> None:
        self.spec = None

    def _run_decode_speculative(self, reqs: List[RunningRequest]) -> Dict[str, list]:
        from ..kv.paged import OutOfBlocks
        bs = self.cfg.block_size
        plan = []
        for rr in reqs:
            if not hasattr(rr, "draft") or rr.draft is None:
                rr.draft = self.spec["make"](rr)
                rr.spec_ctrl = self.spec["ctrl"]() if self.spec["ctrl"] else None
            n = self.cache.table.num_tokens(rr.id)              # includes the slot of this step's input token
            room = min(rr.req.max_new_tokens - len(rr.output_ids) - 1, self.cfg.max_model_len - n - 1)
            k = max(0, min(rr.spec_ctrl.depth if rr.spec_ctrl else self.spec["k"], room))
            sp = rr.req.sampling
            drafts: List[int] = []
            if k > 0 and sp.temperature <= 0 and sp.repetition_penalty == 1.0:
                prop = rr.draft.propose(rr.all_ids, k)
                drafts = [] if prop.parents is not None else list(prop.tokens)[:k]
            if drafts:
                try:
                    self.cache.append(rr.id, len(drafts))
                except OutOfBlocks:
                    drafts = []
            plan.append((rr, n, drafts))
        arrays = {"ids": [], "pos": [], "slots": [], "cu": [0], "ctx": [], "tables": [], "all_rows": 1}
        for rr, n, drafts in plan:
            t = 1 + len(drafts)
            arrays["ids"].extend([rr.output_ids[-1]] + drafts)
            arrays["pos"].extend(range(n - 1, n - 1 + t))
            arrays["slots"].extend(self.cache.table.slot_mapping(rr.id, n - 1, t))
            arrays["cu"].append(arrays["cu"][-1] + t)
            arrays["ctx"].append(n - 1 + t)
            arrays["tables"].append(self.cache.table.block_table(rr.id))
        width = max(len(t) for t in arrays["tables"])
        arrays["tables"] = [t + [0] * (width - len(t)) for t in arrays["tables"]]
        if self.coordinator is not None:
            self.coordinator.announce_prefill(arrays)
        logits = self._exec_prefill(arrays)                      # [sum(k_i + 1), V]
        self._check_device_status()
        # requests that sample draw their (single) token from their row; greedy rows are verified against the drafts
        target = ops.argmax(logits).tolist()
        out: Dict[str, list] = {}
        row = 0
        sampled_rows, sampled_reqs = [], []
        for rr, n, drafts in plan:
            t = 1 + len(drafts)
            if rr.req.sampling.temperature > 0 or rr.req.sampling.repetition_penalty != 1.0:
                sampled_rows.append(row)
                sampled_reqs.append(rr)
                row += t
                continue
            a = 0
            while a < len(drafts) and target[row + a] == drafts[a]:
                a += 1
            out[rr.id] = drafts[:a] + [target[row + a]]
            rr.spec_proposed += len(drafts)
            rr.spec_accepted += a
            self.spec_proposed += len(drafts)
            self.spec_accepted += a
            if rr.spec_ctrl is not None and drafts:
                rr.spec_ctrl.update(len(drafts), a)
            if a < len(drafts):                                  # give back the cache rows of the rejected drafts
                self.cache.table.truncate(rr.id, n + a)
            row += t
        if sampled_rows:
            toks = self._sample(logits[sampled_rows].contiguous(), sampled_reqs)
            for rr, tk in zip(sampled_reqs, toks):
                out[rr.id] = [int(tk)]
        return out

    def _sample(self, logits: torch.Tensor, reqs: List[RunningRequest]) -> List[int]:
        dev = logits.device
        sp = [r.req.sampling for r in reqs]
        if all(p.temperature <= 0 for p in sp):
            return ops.argmax(logits).tolist()
        t = torch.tensor([p.temperature for p in sp], dtype=torch.float32, device=dev)
        k = torch.tensor([p.top_k for p in sp], dtype=torch.int32, device=dev)
        tp = torch.tensor([p.top_p for p in sp], dtype=torch.float32, device=dev)
        mp = torch.tensor([p.min_p for p in sp], dtype=torch.float32, device=dev)
        seeds = torch.tensor([(int(p.seed) * 1000003 + len(r.output_ids)) & 0x7FFFFFFFFFFFFFFF for p, r in zip(sp, reqs)],
                             dtype=torch.int64, device=dev)
        hist = rp = None
        if any(p.repetition_penalty != 1.0 for p in sp):
            hist = torch.full((len(reqs), HISTORY_LEN), -1, dtype=torch.int64)
            for i, r in enumerate(reqs):
                tail = r.all_ids[-HISTORY_LEN:]
                hist[i, : len(tail)] = torch.tensor(tail, dtype=torch.int64)
            hist = hist.to(dev)
            rp = torch.tensor([p.repetition_penalty for p in sp], dtype=torch.float32, device=dev)
        return ops.sample(logits, temperature=t, top_k=k, top_p=tp, min_p=mp, history=hist, rep_penalty=rp, seed_dev=seeds).tolist()

    def _bucket_size(self, n: int) -> int:
        return next((b for b in self.cfg.graph_buckets if b >= n), n)

    def _bucket(self, n: int) -> _DecodeBucket:
        B = self._bucket_size(n)
        # an expert-parallel model sizes its expert passes by the group's largest decode batch: a captured step is valid
        # for that bound only, so it is part of the key
        ep = getattr(self.model, "ep", None)
        key = B if ep is None else (B, ep.pass_tokens)
        bk = self._buckets.get(key)
        if bk is None:
            bk = _DecodeBucket(self.model, self.kv, B, self.max_blocks, self.cfg.use_cuda_graphs)
            self._buckets[key] = bk
        return bk

    def _run_decode(self, reqs: List[RunningRequest]) -> Dict[str, int]:
        bk = self._bucket(len(reqs))
        bs = self.cfg.block_size
        bk.h_slots.fill_(-1)
        bk.h_ctx.fill_(1)
        bk.h_pos.zero_()
        bk.h_ids.zero_()
        bk.h_f.zero_()
        bk.h_f[1].fill_(1.0)
        bk.h_f[3].fill_(1.0)
        bk.h_topk.zero_()
        bk.h_seeds.zero_()
        for i, rr in enumerate(reqs):
            n = self.cache.table.num_tokens(rr.id)         # includes the slot appended for this step's input
            blocks = self.cache.table.block_table(rr.id)
            bk.h_ids[i] = rr.output_ids[-1]
            bk.h_pos[i] = n - 1
            bk.h_ctx[i] = n
            bk.h_slots[i] = blocks[(n - 1) // bs] * bs + (n - 1) % bs
            bk.h_bt[i, : len(blocks)] = torch.tensor(blocks, dtype=torch.int32)
            sp = rr.req.sampling
            bk.h_f[0, i], bk.h_f[1, i], bk.h_f[2, i], bk.h_f[3, i] = sp.temperature, sp.top_p, sp.min_p, sp.repetition_penalty
            bk.h_topk[i] = sp.top_k
            # a row's random stream depends on its own seed and on how many tokens it has produced, not on its batch slot
            bk.h_seeds[i] = (int(sp.seed) * 1000003 + len(rr.output_ids)) & 0x7FFFFFFFFFFFFFFF
            if sp.repetition_penalty != 1.0:
                tail = rr.all_ids[-HISTORY_LEN:]
                bk.h_hist[i].fill_(-1)
                bk.h_hist[i, : len(tail)] = torch.tensor(tail, dtype=torch.int64)
                bk.hist_dirty = True
        out = self._execute_decode(bk)
        return {rr.id: int(out[i]) for i, rr in enumerate(reqs)}

    # ------------------------------------------------------------------ filler passes (lockstep groups)
    def _filler_slot(self) -> int:
        """First slot of a cache block reserved for passes that exist only to keep an expert-parallel group in step."""
        if self._filler_block is None:
            self._filler_block = self.cache.alloc.allocate()
        return self._filler_block * self.cfg.block_size

    def _filler_prefill(self) -> Dict[str, int]:
        slot = self._filler_slot()
        self._exec_prefill({"ids": [0], "pos": [0], "slots": [slot], "cu": [0, 1], "ctx": [1], "tables": [[self._filler_block]]})
        self._check_device_status()
        return {}

    def _filler_decode(self) -> Dict[str, int]:
        bk = self._bucket(1)
        slot = self._filler_slot()
        bk.h_ids.zero_()
        bk.h_pos.zero_()
        bk.h_ctx.fill_(1)
        bk.h_slots.fill_(slot)
        bk.h_bt.zero_()
        bk.h_bt[:, 0] = self._filler_block
        bk.h_f.zero_()
        bk.h_f[1].fill_(1.0)
        bk.h_f[3].fill_(1.0)
        bk.h_topk.zero_()
        bk.run()
        return {}

    def _execute_decode(self, bk: _DecodeBucket) -> torch.Tensor:
        if self.coordinator is not None:
            self.coordinator.announce_decode(bk)
        return bk.run()

    def _check_device_status(self) -> None:
        """Host read of the device status word after a prompt pass (the pass already synchronised to sample)."""
        st = ops.gemm_status(self.model.device)
        code = int(st[0].item())
        if code:
            st.zero_()
            ep = getattr(self.model, "ep", None)
            if code == 120 and ep is not None and getattr(ep, "capacity_policy", "error") == "drop":
                ep.overflow_steps += 1       # token dropping was asked for: the step stands without the rows that did not fit
                return
            raise_for_status(code)

    # ------------------------------------------------------------------ introspection
    def stats(self) -> dict:
        s = self.scheduler.stats()
        s.update(iterations=self.iterations, tokens_generated=self.tokens_generated, last_error=self.last_error)
        if self.prefill_budget is not None:
            s["prefill_budget"] = self.prefill_budget.stats()
        if self.spec is not None:
            s.update(spec_proposed=self.spec_proposed, spec_accepted=self.spec_accepted,
                     spec_acceptance_rate=self.spec_accepted / max(1, self.spec_proposed))
        return s
