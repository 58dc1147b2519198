"""Expert parallelism.

Two regimes:

* decode (few tokens, replicated on every rank of the group because attention is replicated or tensor parallel): no
  token ever moves.  Every rank runs the routed experts it owns for all tokens - remote experts are masked to id -1,
  which the MoE kernels skip - and the partial outputs are summed with the same in-kernel NVLink exchange the
  tensor-parallel row projections use (``csrc/tp_comm.cuh``): dispatch is implicit, combine is fused into the
  down-projection epilogue.
* prefill / large batches, every rank holding different tokens: tokens travel to the ranks owning their experts, run
  through the grouped tcgen05 expert GEMM there and come back.  ``forward_fused`` does the whole exchange inside our own
  kernels over NVLink peer memory (``csrc/ep_comm.cu``): sender warps store token rows straight into the owners' receive
  regions, the owner builds the GEMM tile list on the device once the senders' flags arrive, and the down projection's
  epilogue stores every output row directly into the token owner's return buffer; no collective call, no host
  synchronisation on the routing result.  ``forward_dispatch`` is the NCCL all-to-all baseline of the same thing.

Parity: reference ``metal_marlin/distributed/expert_parallel.py`` (simulated expert placement + dispatch / combine).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..ops.weights import FP4ExpertBank


def expert_range(num_experts: int, rank: int, ep: int) -> Tuple[int, int]:
    per = (num_experts + ep - 1) // ep
    return min(num_experts, rank * per), min(num_experts, (rank + 1) * per)


def shard_bank(bank: FP4ExpertBank, num_routed: int, n_shared: int, rank: int, ep: int) -> Tuple[FP4ExpertBank, int, int, int]:
    """Local bank = this rank's routed experts, followed by the shared experts on rank 0 only.  Returns
    ``(bank, first_expert, n_local_routed, n_local_shared)``."""
    e0, e1 = expert_range(num_routed, rank, ep)
    idx = list(range(e0, e1)) + (list(range(num_routed, num_routed + n_shared)) if rank == 0 else [])
    sel = torch.tensor(idx, dtype=torch.long, device=bank.qtile.device)
    local = FP4ExpertBank(bank.qtile.index_select(0, sel).contiguous(), bank.stile.index_select(0, sel).contiguous(),
                          bank.out_features, bank.in_features, bank.group_size)
    return local, e0, e1 - e0, (n_shared if rank == 0 else 0)


def localize_ids(ids: torch.Tensor, first: int, n_local: int) -> torch.Tensor:
    """Global expert ids -> local ids, -1 for experts other ranks own (no host sync)."""
    loc = ids.to(torch.int32) - first
    return torch.where((loc >= 0) & (loc < n_local), loc, torch.full_like(loc, -1))


class ExpertParallelMoE:
    """One MoE layer's experts sharded over the ranks of ``group``."""

    def __init__(self, gate_up: FP4ExpertBank, down: FP4ExpertBank, num_routed: int, n_shared: int, rank: int, ep: int, group=None):
        self.rank, self.ep, self.group = rank, ep, group
        self.num_routed = num_routed
        self.gate_up, self.first, self.n_local, self.n_shared_local = shard_bank(gate_up, num_routed, n_shared, rank, ep)
        self.down = shard_bank(down, num_routed, n_shared, rank, ep)[0]
        self.hidden = self.down.out_features

    def partial(self, x, ids, weights, *, norm_w=None, eps=1e-6, tpx=None):
        """This rank's share of the expert output for replicated tokens (sum over ranks = full MoE output)."""
        lid = localize_ids(ids, self.first, self.n_local)
        return ops.moe_forward(x, self.gate_up, self.down, lid, weights, n_shared=self.n_shared_local, shared_base=self.n_local,
                               norm_w=norm_w, eps=eps, tpx=tpx)

    def forward_replicated(self, x, ids, weights, *, norm_w=None, eps=1e-6):
        """Decode regime with a library collective (baseline; the fused path passes ``tpx`` to :meth:`partial`)."""
        y = self.partial(x, ids, weights, norm_w=norm_w, eps=eps).to(torch.float32)
        if self.ep > 1:
            dist.all_reduce(y, group=self.group)
        return y.to(torch.bfloat16)

    def forward_dispatch(self, x_local, ids_local, weights_local, *, norm_w=None, eps=1e-6):
        """Prefill regime: every rank holds different tokens ``x_local [T_r, H]``.  Tokens travel to expert owners and back."""
        ep, dev = self.ep, x_local.device
        xin = ops.rmsnorm(x_local, norm_w, eps) if norm_w is not None else x_local
        T, k = ids_local.shape
        flat_e = ids_local.reshape(-1).long()
        owner = torch.div(flat_e, (self.num_routed + ep - 1) // ep, rounding_mode="floor").clamp_(0, ep - 1)
        order = torch.argsort(owner, stable=True)
        send_counts = torch.bincount(owner, minlength=ep)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        tok = torch.div(order, k, rounding_mode="floor")
        send_x = xin.index_select(0, tok).contiguous()
        send_e = flat_e.index_select(0, order).contiguous()
        recv_x = torch.empty(sum(rc), xin.shape[1], dtype=xin.dtype, device=dev)
        recv_e = torch.empty(sum(rc), dtype=torch.long, device=dev)
        dist.all_to_all_single(recv_x, send_x, rc, sc, group=self.group)
        dist.all_to_all_single(recv_e, send_e, rc, sc, group=self.group)
        # local experts on the received (token, expert) pairs: one slot per row, weight 1 (weights applied at home)
        lid = localize_ids(recv_e.view(-1, 1), self.first, self.n_local)
        ones = torch.ones(recv_x.shape[0], 1, dtype=torch.float32, device=dev)
        y = ops.moe_forward(recv_x, self.gate_up, self.down, lid, ones) if recv_x.shape[0] else recv_x.new_zeros(0, self.hidden)
        back = torch.empty(send_x.shape[0], self.hidden, dtype=y.dtype, device=dev)
        dist.all_to_all_single(back, y.contiguous(), sc, rc, group=self.group)
        w_sorted = weights_local.reshape(-1).index_select(0, order).to(torch.float32)
        out = torch.zeros(T, self.hidden, dtype=torch.float32, device=dev)
        out.index_add_(0, tok, back.to(torch.float32) * w_sorted.unsqueeze(-1))
        return out.to(torch.bfloat16)


    def forward_fused(self, ex: "EPExchange", x_local, ids_local, weights_local, *, norm_w=None, eps=1e-6, add0=None, add1=None,
                      token_tile: int = 0, rows_bound: int = 0):
        """Same result as :meth:`forward_dispatch` (+ ``add0`` + ``add1``, e.g. the shared expert and the residual input)
        with the dispatch, the expert GEMMs and the combine chained on the device over peer memory."""
        if not (x_local.is_cuda and ops.native_available()):
            out = self.forward_dispatch(x_local, ids_local, weights_local, norm_w=norm_w, eps=eps).to(torch.float32)
            for a in (add0, add1):
                if a is not None:
                    out = out + a.to(torch.float32)
            return out.to(torch.bfloat16)
        st = self.fused_dispatch(ex, x_local, ids_local, weights_local, norm_w=norm_w, eps=eps)
        self.fused_experts(ex, expected_rows=ids_local.numel(), token_tile=token_tile, rows_bound=rows_bound)
        return self.fused_combine(ex, st, add0=add0, add1=add1)

    # The three phases of forward_fused, separately callable so that several emulated ranks on one GPU can be stepped phase
    # by phase (a kernel must never wait for a launch that comes after it in the same stream).
    def fused_dispatch(self, ex: "EPExchange", x_local, ids_local, weights_local, *, norm_w=None, eps=1e-6):
        """Phase 1 (token owner): normalise, then store every (token, slot) row into the expert owner's receive region."""
        T, k = ids_local.shape
        assert ex.ep == self.ep and ex.rank == self.rank and T * k <= ex.cap and x_local.shape[1] == ex.hidden
        xin = ops.rmsnorm(x_local, norm_w, eps) if norm_w is not None else x_local
        ids32 = ids_local.to(torch.int32).contiguous()
        ex.begin()
        per = (self.num_routed + self.ep - 1) // self.ep
        ops.K.mmb200.ep_dispatch(xin, ids32, ex.desc_dispatch, per, self.ep, self.rank, ex.cap)
        return ids32, weights_local.to(torch.float32).contiguous()

    def fused_experts(self, ex: "EPExchange", *, expected_rows: int, token_tile: int = 0, rows_bound: int = 0) -> None:
        """Phase 2 (expert owner): wait for the senders, group the received rows, run the experts, return the rows.
        ``rows_bound``: an upper bound of the (token, slot) rows ONE rank sends in this pass that every rank agrees on
        (0: the exchange capacity); the work arrays and the launch grids are sized by it, and a pass that receives more
        rows than ``ep * rows_bound`` runs no tile and raises status 120."""
        K = ops.K.mmb200
        dev = ex.local.device
        gu_b, dn_b = self.gate_up, self.down
        n = self.ep * (min(ex.cap, rows_bound) if rows_bound > 0 else ex.cap)
        if not token_tile:      # rows arrive from every rank: a local expert expects about expected_rows / n_local of them
            avg = expected_rows / max(1, self.n_local)
            token_tile = 32 if avg <= 24 else (64 if avg <= 48 else (128 if avg <= 160 else 256))
        max_tiles = n // token_tile + self.n_local + 1
        order = torch.empty(n, dtype=torch.int32, device=dev)
        row_dst = torch.empty(n, dtype=torch.int64, device=dev)
        t_e = torch.empty(max_tiles, dtype=torch.int32, device=dev)
        t_r0, t_rows = torch.empty_like(t_e), torch.empty_like(t_e)
        n_tiles = torch.empty(2, dtype=torch.int32, device=dev)      # [tiles, rows received]
        K.ep_recv_group(ex.desc_recv, self.ep, ex.cap, self.hidden, max(1, self.n_local), token_tile, order, row_dst, t_e, t_r0,
                        t_rows, n_tiles)
        st = ops.gemm_status(dev)
        xs = torch.empty(n, self.hidden, dtype=torch.bfloat16, device=dev)
        K.moe_gather_n(ex.recv_x, order, xs, 1, n_tiles, 1)      # only the rows that arrived, not the worst-case capacity
        self._run_local_experts(ex, xs, n, (t_e, t_r0, t_rows, n_tiles), token_tile, row_dst, st)
        K.ep_signal(ex.desc_signal, self.ep)

    def _run_local_experts(self, ex, xs, n, tiles, token_tile, row_dst, st) -> None:
        """Gate|up (SwiGLU) and down projection of the sorted rows; the down epilogue stores each row at ``row_dst``."""
        K = ops.K.mmb200
        dev = xs.device
        gu_b, dn_b = self.gate_up, self.down
        t_e, t_r0, t_rows, n_tiles = tiles
        h = torch.empty(n, gu_b.out_features // 2, dtype=torch.bfloat16, device=dev)
        if gu_b.out_features % 128 == 0:       # SwiGLU in the GEMM epilogue: only rows that a tile covers are touched
            K.fp4_gemm_grouped_swiglu(xs, gu_b.qtile, gu_b.stile, h, gu_b.out_features, gu_b.group_size, t_e, t_r0, t_rows, n_tiles,
                                      token_tile, st)
        else:
            gu = torch.empty(n, gu_b.out_features, dtype=torch.bfloat16, device=dev)
            K.fp4_gemm_grouped(xs, gu_b.qtile, gu_b.stile, gu, gu_b.out_features, gu_b.group_size, t_e, t_r0, t_rows, n_tiles, token_tile,
                               None, st)
            K.silu_mul(gu, h)
        # down projection: every output row goes from the epilogue into its token owner's return buffer
        K.fp4_gemm_grouped_scatter(h, dn_b.qtile, dn_b.stile, ex.ret_y[:1], dn_b.out_features, dn_b.group_size, t_e, t_r0, t_rows,
                                   n_tiles, token_tile, st, row_dst)

    def fused_combine(self, ex: "EPExchange", state, *, add0=None, add1=None):
        """Phase 3 (token owner): wait for the owners' returns, routing-weighted sum over the slots (+ adds)."""
        ids32, w32 = state
        out = torch.empty(ids32.shape[0], self.hidden, dtype=torch.bfloat16, device=ids32.device)
        ops.K.mmb200.ep_combine(ex.desc_combine, ids32, w32, None if add0 is None else add0.contiguous(),
                                None if add1 is None else add1.contiguous(), out, self.ep)
        return out


class GenericExpertParallelMoE(ExpertParallelMoE):
    """Expert parallelism over a bank of generic (trellis) experts: the rank keeps its range of the routed experts as they
    are (mixed bit widths per expert and matrix); the exchanged rows run through the grouped trellis GEMMs, whose codes are
    decoded inside the tensor-core main loop, with the same scatter epilogue into the token owners' return buffers."""

    def __init__(self, bank, num_routed: int, rank: int, ep: int, group=None):
        from ..ops.generic import GenericExpertBank, _trellis_desc
        self.rank, self.ep, self.group, self.num_routed = rank, ep, group, num_routed
        e0, e1 = expert_range(num_routed, rank, ep)
        self.first, self.n_local, self.n_shared_local = e0, e1 - e0, 0
        local = GenericExpertBank(bank.gate_up[e0:e1], bank.down[e0:e1])
        self.gate_up = self.down = local
        self.hidden = bank.in_features
        self.inter = bank.gate_up[0].out_features // 2
        self._desc_fn = _trellis_desc

    def _run_local_experts(self, ex, xs, n, tiles, token_tile, row_dst, st) -> None:
        desc = self._desc_fn(self.gate_up, self.n_local, xs.device)
        if desc is None or self.hidden % 64 or self.inter % 64:
            raise RuntimeError("the fused expert-parallel path needs uniformly trellis experts with widths that are multiples of 64")
        mats, H, I = desc
        h = ops.trellis_gemm(xs, mats, 2 * I, H, act=1, first=0, stride=3, tiles=tiles, token_tile=token_tile)
        ops.trellis_gemm(h, mats, H, I, act=0, first=2, stride=3, tiles=tiles, token_tile=token_tile, out=ex.ret_y[:1], out_rows=row_dst)


class EPExchange:
    """One rank's peer-addressable buffers for :meth:`ExpertParallelMoE.forward_fused` and the descriptors the kernels take.

    Layout of the allocation (identical on every rank): flag words ``u32 [2][ep]``, received row counts ``int [ep]``, local
    scratch words (send counters, CTA counter, step, status), ``recv_meta int [ep][cap][2]``, ``recv_x bf16 [ep][cap][H]``,
    ``ret_y bf16 [cap][H]`` with ``cap = max_tokens * topk`` (the worst case: every pair of a rank goes to one owner).
    One buffer serves every layer: a rank can only start the next layer's dispatch after its combine saw all return
    flags, i.e. after every owner finished reading the previous layer's rows."""

    OFF_FLAGS, OFF_CNT, OFF_SEND, OFF_COUNTER, OFF_STEP, OFF_STATUS, OFF_META = 0, 256, 512, 640, 644, 648, 1024

    @staticmethod
    def layout(ep: int, cap: int, hidden: int) -> Dict[str, int]:
        assert ep <= 32 and hidden % 8 == 0
        meta = EPExchange.OFF_META
        rx = (meta + ep * cap * 8 + 255) // 256 * 256
        ry = (rx + ep * cap * hidden * 2 + 255) // 256 * 256
        return {"meta": meta, "recv_x": rx, "ret_y": ry, "bytes": ry + cap * hidden * 2}

    def __init__(self, rank: int, ep: int, hidden: int, max_tokens: int, topk: int, local: torch.Tensor, peer_ptrs: Sequence[int]):
        self.rank, self.ep, self.hidden, self.cap = rank, ep, hidden, max_tokens * topk
        self.local, self.peer_ptrs = local, [int(p) for p in peer_ptrs]
        lay = self.layout(ep, self.cap, hidden)
        assert local.numel() >= lay["bytes"] and local.dtype == torch.uint8 and self.peer_ptrs[rank] == local.data_ptr()
        dev = local.device
        base = local.data_ptr()
        self.recv_x = local[lay["recv_x"]: lay["recv_x"] + ep * self.cap * hidden * 2].view(torch.bfloat16).view(ep * self.cap, hidden)
        self.ret_y = local[lay["ret_y"]: lay["ret_y"] + self.cap * hidden * 2].view(torch.bfloat16).view(self.cap, hidden)
        self.step = local[self.OFF_STEP: self.OFF_STEP + 4].view(torch.int32)
        self.status = local[self.OFF_STATUS: self.OFF_STATUS + 8].view(torch.int32)     # [code, wait limit in us (0: one second)]
        tbl = torch.tensor([[p + lay["recv_x"] for p in self.peer_ptrs],
                            [p + lay["meta"] for p in self.peer_ptrs],
                            [p + self.OFF_CNT for p in self.peer_ptrs],
                            [p + self.OFF_FLAGS + 4 * rank for p in self.peer_ptrs],                 # dispatch flag [0][rank] on d
                            [p + lay["ret_y"] for p in self.peer_ptrs],
                            [p + self.OFF_FLAGS + 4 * (ep + rank) for p in self.peer_ptrs]],        # return flag [1][rank] on s
                           dtype=torch.int64).to(dev)
        self._tbl = tbl
        row = lambda i: tbl.data_ptr() + i * ep * 8
        i64 = lambda *v: torch.tensor(list(v), dtype=torch.int64)
        self.desc_dispatch = i64(row(0), row(1), row(2), row(3), base + self.OFF_SEND, base + self.OFF_COUNTER, base + self.OFF_STEP,
                                 base + self.OFF_STATUS)
        self.desc_recv = i64(base + lay["meta"], base + self.OFF_CNT, base + self.OFF_FLAGS, base + self.OFF_STEP, base + self.OFF_STATUS,
                             row(4))
        self.desc_signal = i64(row(5), base + self.OFF_STEP)
        self.desc_combine = i64(base + lay["ret_y"], base + self.OFF_FLAGS + 4 * ep, base + self.OFF_STEP, base + self.OFF_STATUS)

    def begin(self) -> None:
        """Advance the exchange epoch (every rank, once per exchanged layer)."""
        self.step += 1

    def check(self) -> int:
        """0, or the code of the wait that gave up / the overflow (reads the device: call between steps)."""
        return int(self.status[0].item())

    def set_wait_limit_us(self, us: int) -> None:
        """Give up device-side waits of this exchange after ``us`` microseconds (0 restores the one-second default)."""
        self.status[1] = int(us)

    @classmethod
    def create(cls, hidden: int, max_tokens: int, topk: int, device, group=None) -> "EPExchange":
        """Allocates the buffers in symmetric memory of ``group`` (one rank per GPU)."""
        from .symm import SymmetricBuffer
        g = group if group is not None else dist.group.WORLD
        ep, rank = dist.get_world_size(g), dist.get_rank(g)
        buf = SymmetricBuffer(cls.layout(ep, max_tokens * topk, hidden)["bytes"], torch.device(device), g)
        ex = cls(rank, ep, hidden, max_tokens, topk, buf.local, buf.peer_ptrs)
        ex._buf = buf
        return ex

    @classmethod
    def emulated(cls, ep: int, hidden: int, max_tokens: int, topk: int, device) -> List["EPExchange"]:
        """All ``ep`` ranks' buffers on ONE device (tests, single-GPU bring-up).  The kernels of the emulated ranks must be
        launched phase by phase - every rank's dispatch, then every rank's expert pass, then every rank's combine - so
        that no launch ever waits for a later one."""
        nbytes = cls.layout(ep, max_tokens * topk, hidden)["bytes"]
        bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(ep)]
        ptrs = [b.data_ptr() for b in bufs]
        return [cls(r, ep, hidden, max_tokens, topk, bufs[r], ptrs) for r in range(ep)]


class EPModelState:
    """Expert parallelism of a whole model whose attention and dense layers are replicated (every rank serves its own
    sequences): per MoE layer the rank's routed experts (:class:`ExpertParallelMoE`) plus a local copy of the shared
    experts, and one :class:`EPExchange` that all layers use in turn.

    ``mode``: ``"fused"`` - dispatch, expert GEMMs and combine inside this library's kernels over peer memory;
    ``"nccl"`` - the all-to-all baseline (:meth:`ExpertParallelMoE.forward_dispatch`)."""

    def __init__(self, rank: int, ep: int, exchange: Optional[EPExchange], group=None, mode: str = "fused"):
        self.rank, self.ep, self.exchange, self.group, self.mode = rank, ep, exchange, group, mode
        self.layers: Dict[int, ExpertParallelMoE] = {}
        self.shared: Dict[int, Tuple[FP4ExpertBank, FP4ExpertBank]] = {}
        self.n_shared = 0
        # Most tokens ANY rank brings to the current forward pass, when the ranks know it (an engine group agrees on it every
        # step; ``uniform`` says every rank brings as many tokens as this one): the expert owners size their work by it
        # instead of by the exchange capacity.
        self.pass_tokens = 0
        self.uniform = False
        # What a receive-buffer overflow (device status 120: a rank was sent more rows than its region holds; the rows beyond it
        # are not computed) means to the engine: "error" fails the step's requests, "drop" accepts the loss of those expert
        # contributions (token dropping, as a capacity factor below the worst case implies) and counts the steps it happened in.
        self.capacity_policy = "error"
        self.overflow_steps = 0

    def add_layer(self, li: int, gate_up, down, num_routed: int, n_shared: int) -> None:
        self.n_shared = n_shared
        if getattr(gate_up, "is_generic", False):
            from ..ops.generic import GenericExpertBank
            self.layers[li] = GenericExpertParallelMoE(gate_up, num_routed, self.rank, self.ep, self.group)
            if n_shared:
                self.shared[li] = GenericExpertBank(gate_up.gate_up[num_routed:], gate_up.down[num_routed:])
            return
        moe = ExpertParallelMoE(gate_up, down, num_routed, 0, self.rank, self.ep, self.group)
        self.layers[li] = moe
        if n_shared:
            sel = torch.arange(num_routed, num_routed + n_shared, device=gate_up.qtile.device)
            pick = lambda b: FP4ExpertBank(b.qtile.index_select(0, sel).contiguous(), b.stile.index_select(0, sel).contiguous(),
                                           b.out_features, b.in_features, b.group_size)
            self.shared[li] = (pick(gate_up), pick(down))

    def max_tokens(self) -> int:
        return self.exchange.cap // max(1, self._topk) if self.exchange is not None else 1 << 30

    _topk = 1

    def forward(self, li: int, x, ids, weights, *, norm_w=None, eps=1e-6):
        """MoE output for this rank's tokens ``x [T, H]`` (un-normalised residual stream; ``norm_w`` is applied first)."""
        moe = self.layers[li]
        add0 = None
        if li in self.shared:
            xin = ops.rmsnorm(x, norm_w, eps) if norm_w is not None else x
            if isinstance(self.shared[li], tuple):
                gu, dn = self.shared[li]
                add0 = ops._shared_experts(xin, gu, dn, self.n_shared, 0)
            else:      # generic (trellis) shared experts: no routed slot, the bank's experts all act as shared ones
                from ..ops import generic
                bank = self.shared[li]
                none = torch.empty(x.shape[0], 0, dtype=torch.int32, device=x.device)
                add0 = generic._finish_shared(torch.zeros(x.shape[0], x.shape[1], dtype=torch.float32, device=x.device), xin, bank,
                                              len(bank.gate_up), 0, None)
        if self.mode == "fused" and self.exchange is not None and x.is_cuda:
            bound = ids.shape[0] if self.uniform else self.pass_tokens
            return moe.forward_fused(self.exchange, x, ids, weights, norm_w=norm_w, eps=eps, add0=add0, rows_bound=bound * ids.shape[1])
        out = moe.forward_dispatch(x, ids, weights, norm_w=norm_w, eps=eps)
        return out if add0 is None else (out.to(torch.float32) + add0.to(torch.float32)).to(out.dtype)

    def check(self) -> int:
        return self.exchange.check() if self.exchange is not None else 0


def shard_transformer_ep(model, rank: int, ep: int, max_tokens: int, group=None, mode: str = "fused"):
    """The rank's expert-parallel copy of ``model``: attention, dense MLPs, router and shared experts stay whole, the
    routed experts of every MoE layer are cut to this rank's range, and the model's MoE layers exchange tokens through one
    :class:`EPExchange` (``max_tokens`` = most tokens a rank brings to one forward pass)."""
    import copy
    from ..models.transformer import Transformer
    cfg = model.cfg
    dev = model.device
    ex = None
    if mode == "fused" and dev.type == "cuda" and ep > 1:
        ex = EPExchange.create(cfg.hidden_size, max_tokens, cfg.num_experts_per_tok, dev, group)
    st = EPModelState(rank, ep, ex, group, mode)
    st._topk = cfg.num_experts_per_tok
    layers = []
    for li, L in enumerate(model.layers):
        S = copy.copy(L)
        if L.router_w is not None:
            st.add_layer(li, L.gate_up_bank, L.down_bank, cfg.num_experts, cfg.n_shared_experts)
            S.gate_up_bank = S.down_bank = None      # only the rank's experts stay resident (inside ``st``)
        layers.append(S)
    m = Transformer(cfg, layers, model.embed, model.final_norm, model.lm_head)
    m.ep = st
    m.mtp = model.mtp
    return m
