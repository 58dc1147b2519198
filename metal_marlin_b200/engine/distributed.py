"""Multi-GPU serving: one process per GPU (``torchrun``), three ways to spread a model over them.

* ``tp``: one model replica split over the ranks (``parallel/tp.py``: heads, MLP / expert widths and the vocabulary are
  sharded; partial sums meet inside the kernels over NVLink).  Rank 0 owns the scheduler and the HTTP front end; before
  it launches a prompt pass or a decode step it sends the batch description to the other ranks over a CPU (gloo) control
  group, so all shards launch the same kernels in the same order (:class:`TPCoordinator`, :func:`tp_follow`).
* ``tp`` + ``ep``: as above, but every rank keeps whole experts (its range of the routed experts) instead of a slice of
  every expert: tokens are replicated, a rank computes the experts it owns and the partial outputs meet like any other
  row-parallel sum.
* ``ep`` (attention data parallel, experts expert parallel): every rank holds the dense layers and serves its own
  requests; the MoE layers exchange token rows with the ranks that own the experts (``parallel/ep.py``).  Such an exchange
  needs every rank to run every forward pass, so the ranks step in lockstep: each step they agree (one small all-reduce on
  the control group) whether a prompt pass and / or a decode pass happens and a rank with nothing to do runs a one-token
  filler (:class:`EPLockstep`).  Rank 0 receives all requests and deals them to the ranks; sampled tokens travel back to
  rank 0 with the same control messages (:class:`EPEngineGroup`).
* ``dp``: independent replicas behind a request router (``serving/router.py``).

Parity: the reference simulates tensor parallelism inside one process (``metal_marlin/distributed/tensor_parallel.py:279-753``)
and has no multi-process serving; the scheduler / runner split follows ``metal_marlin/serving/continuous_batch.py:550``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .engine import EngineConfig, LLMEngine, _DecodeBucket
from .request import GenerationRequest, RequestStatus, RunningRequest
from .session import SamplingParams

KIND_STOP, KIND_PREFILL, KIND_DECODE = 0, 1, 2


@dataclass
class ParallelConfig:
    """How the ranks of the job are used.  ``tp * dp`` (or ``ep`` when attention is data parallel) must equal the world size."""
    tp: int = 1
    ep: int = 1
    dp: int = 1
    exchange: str = "fused"        # "fused": in-kernel NVLink exchange; "nccl": library collectives (baseline)

    @property
    def mode(self) -> str:
        if self.tp > 1 and self.ep > 1:
            return "tp+ep"
        if self.tp > 1:
            return "tp"
        if self.ep > 1:
            return "ep"
        return "dp" if self.dp > 1 else "single"

    @classmethod
    def parse(cls, tp: int = 1, ep: int = 1, dp: int = 1, world: Optional[int] = None, exchange: str = "fused") -> "ParallelConfig":
        world = world if world is not None else int(os.environ.get("WORLD_SIZE", "1"))
        pc = cls(max(1, tp), max(1, ep), max(1, dp), exchange)
        if pc.tp > 1 and pc.ep > 1 and pc.ep != pc.tp:
            raise ValueError("with tensor and expert parallelism together both span the same ranks (ep == tp)")
        need = pc.tp * pc.dp if pc.tp > 1 else max(pc.ep, 1) * pc.dp
        if pc.mode != "single" and need != world:
            raise ValueError(f"tp={pc.tp} ep={pc.ep} dp={pc.dp} needs {need} ranks, the job has {world}")
        return pc


def init_process_group(device: Optional[torch.device] = None, timeout_s: int = 180):
    """Joins the job described by the ``torchrun`` environment.  Returns ``(rank, world, device, control_group)``; the
    control group is a gloo group over all ranks for host-side messages (batch descriptions, request hand-over)."""
    import datetime
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if device is None:
        device = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        to = datetime.timedelta(seconds=timeout_s)
        if device.type == "cuda":
            dist.init_process_group("nccl", device_id=device, timeout=to)
        else:
            dist.init_process_group("gloo", timeout=to)
    ctrl = None
    if world > 1:
        # Host-side control messages.  A follower legitimately waits in a broadcast while the leader is idle, so the default
        # limit is long; MMB200_CTRL_TIMEOUT_S shortens it (tests, or deployments whose leader sends keep-alives).
        ctl_to = datetime.timedelta(seconds=int(os.environ.get("MMB200_CTRL_TIMEOUT_S", "1800")))
        ctrl = dist.new_group(backend="gloo", timeout=ctl_to) if device.type == "cuda" else dist.group.WORLD
    return rank, world, device, ctrl


def parallelize(model, pc: ParallelConfig, rank: int, device, max_tokens: int = 2048, group=None):
    """This rank's part of ``model`` under ``pc`` (every rank built or loaded the same full model)."""
    if pc.mode in ("single", "dp"):
        return model
    if pc.mode in ("tp", "tp+ep"):
        from ..parallel.tp import make_context, shard_transformer
        ctx = make_context(model.cfg, device, group=group, mode="fused" if pc.exchange == "fused" else "nccl")
        return shard_transformer(model, rank, pc.tp, ctx, expert_parallel=(pc.mode == "tp+ep"))
    from ..parallel.ep import shard_transformer_ep
    return shard_transformer_ep(model, rank, pc.ep, max_tokens, group=group, mode=pc.exchange)


# ---------------------------------------------------------------------------------------------------------------------
# tensor parallel: leader announces, followers replay
# ---------------------------------------------------------------------------------------------------------------------
class TPCoordinator:
    """Leader side of the control channel: tells the other shards what to run next."""

    def __init__(self, ctrl_group, leader: int = 0):
        self.group, self.leader = ctrl_group, leader

    def _header(self, *vals) -> None:
        h = torch.zeros(8, dtype=torch.int64)
        h[: len(vals)] = torch.tensor(vals, dtype=torch.int64)
        dist.broadcast(h, src=self.leader, group=self.group)

    def announce_prefill(self, a: Dict[str, list]) -> None:
        n_seq, width = len(a["ctx"]), len(a["tables"][0])
        flat = a["ids"] + a["pos"] + a["slots"] + a["cu"] + a["ctx"] + [b for t in a["tables"] for b in t]
        self._header(KIND_PREFILL, len(a["ids"]), n_seq, width, int(a.get("all_rows", 0)))
        dist.broadcast(torch.tensor(flat, dtype=torch.int64), src=self.leader, group=self.group)

    def announce_decode(self, bk: _DecodeBucket) -> None:
        self._header(KIND_DECODE, bk.B, 1 if bk.hist_dirty else 0)
        dist.broadcast(bk.h_buf, src=self.leader, group=self.group)
        if bk.hist_dirty:
            dist.broadcast(bk.h_hist, src=self.leader, group=self.group)

    def stop(self) -> None:
        self._header(KIND_STOP)


def unpack_prefill(flat: torch.Tensor, T: int, n_seq: int, width: int) -> Dict[str, list]:
    v = flat.tolist()
    o = 0
    out = {}
    for name, n in (("ids", T), ("pos", T), ("slots", T), ("cu", n_seq + 1), ("ctx", n_seq)):
        out[name] = v[o:o + n]
        o += n
    out["tables"] = [v[o + i * width: o + (i + 1) * width] for i in range(n_seq)]
    return out


def tp_follow(engine: LLMEngine, ctrl_group, leader: int = 0) -> int:
    """Follower loop of a tensor-parallel shard: replay every batch the leader announces until it says stop.  Returns the
    number of passes run."""
    n = 0
    with torch.no_grad():
        while True:
            h = torch.zeros(8, dtype=torch.int64)
            dist.broadcast(h, src=leader, group=ctrl_group)
            kind = int(h[0])
            if kind == KIND_STOP:
                return n
            if kind == KIND_PREFILL:
                T, n_seq, width = int(h[1]), int(h[2]), int(h[3])
                flat = torch.empty(3 * T + 2 * n_seq + 1 + n_seq * width, dtype=torch.int64)
                dist.broadcast(flat, src=leader, group=ctrl_group)
                arrays = unpack_prefill(flat, T, n_seq, width)
                arrays["all_rows"] = int(h[4])
                engine._exec_prefill(arrays)
                engine._check_device_status()
            elif kind == KIND_DECODE:
                bk = engine._bucket(int(h[1]))
                dist.broadcast(bk.h_buf, src=leader, group=ctrl_group)
                bk.hist_dirty = bool(int(h[2]))
                if bk.hist_dirty:
                    dist.broadcast(bk.h_hist, src=leader, group=ctrl_group)
                bk.run()
            n += 1


# ---------------------------------------------------------------------------------------------------------------------
# expert parallel with data-parallel attention: lockstep engines
# ---------------------------------------------------------------------------------------------------------------------
class EPLockstep:
    """Per-step agreement between the ranks of an expert-parallel group: a pass runs on every rank if any rank needs it."""

    def __init__(self, ctrl_group):
        self.group = ctrl_group

    def agree(self, prefill_tokens: int, decode_tokens: int):
        """Largest prompt-pass and decode-pass token counts over the ranks (0: nobody runs that pass)."""
        f = torch.tensor([int(prefill_tokens), int(decode_tokens)], dtype=torch.int64)
        dist.all_reduce(f, op=dist.ReduceOp.MAX, group=self.group)
        return int(f[0]), int(f[1])


def _req_to_wire(rid: str, req: GenerationRequest) -> dict:
    sp = req.sampling
    return {"id": rid, "prompt": list(req.prompt_ids), "max_new": req.max_new_tokens, "eos": list(req.eos_ids or ()),
            "sampling": [sp.temperature, sp.top_k, sp.top_p, sp.min_p, sp.repetition_penalty, sp.seed]}


def _req_from_wire(d: dict) -> GenerationRequest:
    t, k, p, mp, rp, seed = d["sampling"]
    return GenerationRequest(list(d["prompt"]), int(d["max_new"]), SamplingParams(t, int(k), p, mp, rp, int(seed)), tuple(d["eos"]),
                             request_id=d["id"])


class RemoteRequest:
    """Leader-side view of a request that another rank executes."""

    def __init__(self, rid: str, req: GenerationRequest, owner: int):
        import threading
        self.id, self.req, self.owner = rid, req, owner
        self.output_ids: List[int] = []
        self.status = RequestStatus.WAITING
        self.error: Optional[str] = None
        self.finish_reason: Optional[str] = None
        self.done = threading.Event()

    def deliver(self, token: Optional[int], finished: bool, failed: Optional[str]) -> None:
        if token is not None:
            self.output_ids.append(token)
            self.status = RequestStatus.RUNNING
            if self.req.on_token is not None:
                self.req.on_token(self.id, token)
        if failed:
            self.error, self.status = failed, RequestStatus.FAILED
            self.done.set()
        elif finished:
            self.status = RequestStatus.FINISHED
            eos = set(self.req.eos_ids or ())
            self.finish_reason = "stop" if (self.output_ids and self.output_ids[-1] in eos) else "length"
            self.done.set()


class EPEngineGroup:
    """One :class:`LLMEngine` per rank, stepped in lockstep.  The leader (rank 0 of the control group) takes requests
    through :meth:`submit` and deals them to the rank with the fewest open requests; every rank calls :meth:`step` in a
    loop (followers: :meth:`follow`)."""

    def __init__(self, engine: LLMEngine, ctrl_group, rank: int, world: int):
        self.engine, self.group, self.rank, self.world = engine, ctrl_group, rank, world
        engine.lockstep = EPLockstep(ctrl_group)
        self._pending: List[tuple] = []
        self._open = [0] * world
        self._remote: Dict[str, RemoteRequest] = {}
        self._local_seen: Dict[str, int] = {}
        self._stop = False
        self._n = 0

    # ------------------------------------------------------------------ leader API
    def submit(self, req: GenerationRequest):
        """Leader only.  Returns an object with ``output_ids`` / ``done`` / ``status`` (a :class:`RemoteRequest`)."""
        assert self.rank == 0
        self._n += 1
        rid = req.request_id or f"ep-{self._n}"
        owner = min(range(self.world), key=lambda r: self._open[r])
        self._open[owner] += 1
        rr = RemoteRequest(rid, req, owner)
        self._remote[rid] = rr
        self._pending.append((owner, _req_to_wire(rid, req)))
        return rr

    def shutdown(self) -> None:
        self._stop = True

    def abort(self, rid: str) -> bool:
        """Leader: stop reporting a request (its owner finishes it on its own; the tokens are dropped)."""
        rq = self._remote.get(rid)
        if rq is None:
            return False
        rq.req.on_token = None
        rq.status = RequestStatus.ABORTED
        rq.done.set()
        return True

    def has_work(self) -> bool:
        return bool(self._pending) or any(not r.done.is_set() for r in self._remote.values())

    # ------------------------------------------------------------------ one lockstep iteration (every rank)
    def step(self) -> bool:
        """Returns False once the leader asked every rank to stop."""
        msg = [None]
        if self.rank == 0:
            new = {}
            for owner, wire in self._pending:
                new.setdefault(owner, []).append(wire)
            self._pending = []
            msg = [{"stop": self._stop, "new": new}]
        dist.broadcast_object_list(msg, src=0, group=self.group)
        m = msg[0]
        if m["stop"]:
            return False
        for wire in m["new"].get(self.rank, []):
            self.engine.add_request(_req_from_wire(wire))
        err = None
        try:
            self.engine.step()
        except Exception as e:          # keep the group in step: report, fail the local requests, carry on
            err = repr(e)
            self.engine.fail_running(err)
        events = []
        for rr in list(self.engine.tracked()):
            seen = self._local_seen.get(rr.id, 0)
            new_toks = rr.output_ids[seen:]
            fin = rr.status in (RequestStatus.FINISHED, RequestStatus.FAILED, RequestStatus.ABORTED)
            if new_toks or fin:
                events.append((rr.id, new_toks, fin, rr.error))
                self._local_seen[rr.id] = len(rr.output_ids)
            if fin:
                self.engine.untrack(rr.id)
                self._local_seen.pop(rr.id, None)
        gathered = [None] * self.world if self.rank == 0 else None
        dist.gather_object(events, gathered, dst=0, group=self.group)
        if self.rank == 0:
            for r, evs in enumerate(gathered):
                for rid, toks, fin, error in evs:
                    rq = self._remote.get(rid)
                    if rq is None:
                        continue
                    for t in toks:
                        rq.deliver(t, False, None)
                    if fin:
                        rq.deliver(None, True, error)
                        self._open[r] -= 1
                        self._remote.pop(rid, None)
        return True

    def follow(self) -> None:
        while self.step():
            pass

    def run_until_done(self, max_iters: int = 1 << 30) -> None:
        """Leader: step until every submitted request has finished, then leave the others waiting for the next step."""
        it = 0
        while self.has_work() and it < max_iters:
            self.step()
            it += 1


# ---------------------------------------------------------------------------------------------------------------------
# one entry point for the pipeline / server / CLI
# ---------------------------------------------------------------------------------------------------------------------
class DistributedEngine:
    """The engine a multi-GPU job exposes on rank 0, with the surface of :class:`LLMEngine` (``add_request``, ``generate``,
    ``start`` / ``stop``, ``abort``, ``stats``) so pipelines and the HTTP server use it unchanged; the other ranks call
    :meth:`serve_forever`.  Built by :func:`build_engine`."""

    def __init__(self, engine: LLMEngine, pc: ParallelConfig, rank: int, world: int, ctrl_group):
        import threading
        self.engine, self.pc, self.rank, self.world, self.ctrl = engine, pc, rank, world, ctrl_group
        self.cfg = engine.cfg
        self.model = engine.model
        self.group: Optional[EPEngineGroup] = None
        self._thread: Optional["threading.Thread"] = None
        self._stop_evt = threading.Event()
        self._released = False
        if pc.mode == "ep":
            self.group = EPEngineGroup(engine, ctrl_group, rank, world)
        elif pc.mode in ("tp", "tp+ep") and rank == 0:
            engine.coordinator = TPCoordinator(ctrl_group, 0)

    @property
    def is_leader(self) -> bool:
        return self.rank == 0

    @property
    def last_error(self):
        return self.engine.last_error

    @property
    def iterations(self) -> int:
        return self.engine.iterations

    def serve_forever(self) -> None:
        """Ranks other than 0: execute what the leader decides until it stops the job."""
        if self.group is not None:
            self.group.follow()
        elif self.pc.mode in ("tp", "tp+ep"):
            tp_follow(self.engine, self.ctrl, 0)

    # ------------------------------------------------------------------ LLMEngine surface (leader)
    def add_request(self, req: GenerationRequest):
        assert self.is_leader
        return self.group.submit(req) if self.group is not None else self.engine.add_request(req)

    def abort(self, request_id: str) -> bool:
        return self.group.abort(request_id) if self.group is not None else self.engine.abort(request_id)

    def step(self):
        return self.group.step() if self.group is not None else self.engine.step()

    def has_work(self) -> bool:
        return self.group.has_work() if self.group is not None else self.engine.has_work()

    def run_until_done(self, max_iters: int = 1 << 30) -> None:
        if self.group is not None:
            self.group.run_until_done(max_iters)
        else:
            self.engine.run_until_done(max_iters)

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16, sampling: Optional[SamplingParams] = None,
                 eos_ids: Sequence[int] = ()) -> List[List[int]]:
        assert self.is_leader
        rrs = [self.add_request(GenerationRequest(list(p), max_new_tokens, sampling or SamplingParams(), eos_ids)) for p in prompts]
        if self._thread is None:
            self.run_until_done()
        for r in rrs:
            r.done.wait()
        failed = [r.error for r in rrs if getattr(r, "error", None)]
        if failed:
            raise RuntimeError(f"{len(failed)} request(s) failed: {failed[0]}")
        return [r.output_ids for r in rrs]

    def start(self) -> None:
        """Background stepping on the leader (the HTTP server and streaming calls use it)."""
        if self._thread is not None:
            return
        if self.group is None:
            self.engine.start()
            self._thread = self.engine._thread
            return
        import threading
        import time

        def loop():
            while not self._stop_evt.is_set():
                if not self.group.has_work():
                    time.sleep(0.002)       # idle: do not flood the control group with empty steps
                    continue
                self.group.step()
        self._stop_evt.clear()
        self._thread = threading.Thread(target=loop, name="mmb200-ep-leader", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        """Leader: stop stepping and release the other ranks (call once, when the job ends)."""
        if self.group is None:
            self.engine.stop()
        elif self._thread is not None:
            self._stop_evt.set()
            self._thread.join(timeout=30)
        self._thread = None
        if not self.is_leader or self._released:
            return
        self._released = True
        if self.group is not None:
            self.group.shutdown()
            self.group.step()
        elif self.engine.coordinator is not None:
            self.engine.coordinator.stop()

    def stats(self) -> dict:
        s = self.engine.stats()
        s.update(parallel=self.pc.mode, world=self.world)
        if self.group is not None:
            s["open_per_rank"] = list(self.group._open)
            s["waiting"] = s.get("waiting", 0) + len(self.group._pending)
        return s

    def check(self) -> int:
        m = self.engine.model
        if m.tp is not None:
            return m.tp.check()
        if m.ep is not None:
            return m.ep.check()
        return 0


def build_engine(model, engine_cfg: Optional[EngineConfig], pc: ParallelConfig, rank: int, world: int, device, ctrl_group) -> DistributedEngine:
    """Shard ``model`` for this rank and wrap it in the engine that matches ``pc``."""
    cfg = engine_cfg or EngineConfig()
    shard = parallelize(model, pc, rank, device, max_tokens=max(cfg.max_num_batched_tokens, max(cfg.graph_buckets)))
    eng = LLMEngine(shard, cfg)
    return DistributedEngine(eng, pc, rank, world, ctrl_group)
