"""Tensor parallelism over the GPUs of one node.

Sharding (per layer): attention heads are split across ranks (q_b / q / k / v rows, W_uk / W_uv, o_proj columns);
MLP and expert intermediate dimensions are split on quantization-group boundaries (gate/up rows, down columns);
the vocabulary is split for the LM head; small matrices (q_a | kv_a, router, norms, embeddings) are replicated so
no collective is needed for them, and the MLA latent cache is replicated (it is 576 values per token).

Two ways to combine the row-parallel partial sums:

* ``fused`` (decode, <= 16 tokens): the producing GEMV stores its partial directly into every peer's receive
  buffer over NVLink and the next kernel sums the tp slots while staging its input (``csrc/tp_comm.cuh``);
  no collective kernel is launched at all.  The LM head is vocabulary-parallel with an in-kernel exchange of
  (max, argmax) pairs.
* prefill (33 .. 8192 tokens): GEMM -> reduce-scatter -> all-gather -> GEMM without a collective call.  The tcgen05
  GEMM's epilogue scatters fp32 partials to the owners of the token rows; the owners' reduce kernel adds the
  residual, applies the next RMSNorm to its rows only (sequence-parallel layer boundary) and stores residual and
  normalized rows into every peer's gathered buffers; the next projection's GEMM waits per token tile, inside its
  TMA producer, for the owners of that tile and starts with this rank's own rows, so the gather overlaps the math.
* ``nccl`` (large batches and the baseline): ``torch.distributed.all_reduce`` on the partial.

Parity: reference ``metal_marlin/distributed/tensor_parallel.py:61-276`` (``ParallelMode``, ``shard_tensor``,
``TensorParallelLinear.from_marlin_linear`` ``:341``, column ``:515`` / row ``:546`` forward, simulated
collectives) and ``metal_marlin/distributed/verification.py:85-509`` (sharded-vs-unsharded equality).
"""
from __future__ import annotations

import copy
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..models.transformer import LayerWeights, Transformer
from .symm import SymmetricBuffer

FUSED_MAX_TOKENS = 16
FUSED_GEMM_MAX_TOKENS = 8192      # prefill chunks up to this many tokens use the GEMM -> reduce-scatter epilogue


def even_split(n: int, parts: int, unit: int = 1) -> List[Tuple[int, int]]:
    """Split ``n`` into ``parts`` contiguous ranges whose inner boundaries are multiples of ``unit``; a ragged
    tail (``n % unit``) goes to the last range."""
    u = n // unit
    assert u >= parts, (n, parts, unit)
    out = [((r * u) // parts * unit, ((r + 1) * u) // parts * unit) for r in range(parts)]
    out[-1] = (out[-1][0], n)
    return out


@dataclass
class TPPendingRS:
    """A row-parallel projection whose partials were scattered to the row owners by the GEMM epilogue; the reduce +
    gather kernel has not run yet, so the consumer can have its residual add and RMSNorm fused into it."""
    site: int
    rows: int
    pending_rs = True


@dataclass
class TPGathered:
    """Gathered (normalized activation, new residual) of a prefill site; ``wait`` is the CPU descriptor for the GEMM
    that consumes ``x`` first (per-tile wait inside its TMA producer)."""
    x: torch.Tensor
    h: torch.Tensor
    wait: torch.Tensor
    flags_desc: torch.Tensor

    def ensure(self):
        """Stand-alone bounded wait, for a first consumer that is not one of the GEMM kernels."""
        ops.K.mmb200.tp_wait(self.flags_desc)


@dataclass
class TPPartial:
    """Handle for "the sum over ranks of the partials of site ``site``" (not yet materialised)."""
    site: int
    rows: int


class TPContext:
    def __init__(self, rank: int, tp: int, device: torch.device, n_sites: int, hidden: int, group=None,
                 max_tokens: int = FUSED_MAX_TOKENS, mode: str = "fused"):
        self.rank, self.tp, self.device, self.mode = rank, tp, device, mode
        self.group = group
        self.hidden, self.max_tokens, self.n_sites = hidden, max_tokens, n_sites
        self.fused_ok = mode == "fused" and device.type == "cuda" and ops.native_available()
        self.slot = max_tokens * hidden                     # fp32 elements per (site, source rank)
        self.site_bytes = tp * self.slot * 4
        pair_bytes = tp * max_tokens * 2 * 4
        flags_off = n_sites * self.site_bytes + pair_bytes
        self.n_flag_sites = n_sites + 1
        total = flags_off + self.n_flag_sites * tp * 4
        self._desc_cache: Dict[Tuple[str, int, int], torch.Tensor] = {}
        self.use_multimem = False
        if not self.fused_ok:
            self.buf = None
            return
        self.buf = SymmetricBuffer(total, device, group)
        # NVSwitch multicast for the decode exchange (off when NVLS is switched off for the process, as the multi-rank failure
        # tests do: their ranks may leave while others still run)
        self.use_multimem = bool(self.buf.multicast_ptr) and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0" \
            and os.environ.get("MMB_TP_MULTIMEM", "1") != "0"
        self.pairs_off = n_sites * self.site_bytes
        self.flags_off = flags_off
        self.step = torch.zeros(1, dtype=torch.int32, device=device)
        self.counters = torch.zeros(self.n_flag_sites, dtype=torch.int32, device=device)
        self.status = ops.gemm_status(device)      # one status word per device: the engine reads it back with the sampled ids
        # per site: device arrays of peer addresses (my slot in every peer's buffer, my flag on every peer)
        slots = torch.empty(self.n_flag_sites, tp, dtype=torch.int64)
        flags = torch.empty(self.n_flag_sites, tp, dtype=torch.int64)
        for s in range(self.n_flag_sites):
            for r in range(tp):
                if s < n_sites:
                    slots[s, r] = self.buf.peer_addr(r, s * self.site_bytes + rank * self.slot * 4)
                else:
                    slots[s, r] = self.buf.peer_addr(r, self.pairs_off + rank * max_tokens * 2 * 4)
                flags[s, r] = self.buf.peer_addr(r, flags_off + (s * tp + rank) * 4)
        self.peer_slots = slots.to(device)
        self.peer_flags = flags.to(device)
        self._big = None       # prefill-size exchange buffers, created on first use

    # ------------------------------------------------------------------ prefill-size exchange (GEMM -> RS, then AG)
    def _big_buffers(self):
        """Two (ping-pong by site parity) receive buffers fp32 [tp][rows][hidden] and gathered buffers bf16
        [M][hidden], their flag words and the per-peer address tables.  Site s + 2 may reuse the buffers of site s:
        no rank can produce site s + 2 before it consumed site s + 1, which needs every rank's site s + 1 partial,
        which a rank only produces after it consumed site s."""
        if self._big is not None:
            return self._big
        tp, H, M = self.tp, self.hidden, FUSED_GEMM_MAX_TOKENS
        rows = (M + tp - 1) // tp
        rs_bytes = tp * rows * H * 4
        ag_bytes = 2 * M * H * 2                                  # reduced rows / new residual, and normalized rows
        flag_bytes = self.n_sites * 2 * tp * 4                   # [site][rs | ag][tp]: flags are per site, buffers ping-pong
        buf = SymmetricBuffer(2 * (rs_bytes + ag_bytes) + flag_bytes, self.device, self.group)
        self._big = {"buf": buf, "rows_max": rows, "rs_bytes": rs_bytes, "ag_bytes": ag_bytes, "flags_off": 2 * (rs_bytes + ag_bytes),
                     "tabs": {}, "counters": torch.zeros(2 * self.n_sites, dtype=torch.int32, device=self.device)}
        return self._big

    def _big_tables(self, site: int):
        big = self._big_buffers()
        t = big["tabs"].get(site)
        if t is None:
            buf, tp = big["buf"], self.tp
            par = site & 1
            rs_off = par * (big["rs_bytes"] + big["ag_bytes"])
            ag_off = rs_off + big["rs_bytes"]
            f_rs = big["flags_off"] + (site * 2 + 0) * tp * 4
            f_ag = big["flags_off"] + (site * 2 + 1) * tp * 4
            dev = self.device
            t = {
                "rs_bufs": torch.tensor([buf.peer_addr(r, rs_off) for r in range(tp)], dtype=torch.int64).to(dev),
                "rs_flags": torch.tensor([buf.peer_addr(r, f_rs + self.rank * 4) for r in range(tp)], dtype=torch.int64).to(dev),
                "ag_bufs": torch.tensor([buf.peer_addr(r, ag_off) for r in range(tp)], dtype=torch.int64).to(dev),
                "ag_flags": torch.tensor([buf.peer_addr(r, f_ag + self.rank * 4) for r in range(tp)], dtype=torch.int64).to(dev),
                "ag2_bufs": torch.tensor([buf.peer_addr(r, ag_off + big["ag_bytes"] // 2) for r in range(tp)], dtype=torch.int64).to(dev),
                "rs_local": buf.local.data_ptr() + rs_off, "ag_local_off": ag_off, "ag2_local_off": ag_off + big["ag_bytes"] // 2,
                "rs_flags_local": buf.local.data_ptr() + f_rs, "ag_flags_local": buf.local.data_ptr() + f_ag,
            }
            big["tabs"][site] = t
        return big, t

    def use_fused_gemm(self, n_tokens: int, W) -> bool:
        return (self.fused_ok and self.tp > 1 and ops.GEMV_MAX_M < n_tokens <= FUSED_GEMM_MAX_TOKENS and isinstance(W, ops.FP4Weight)
                and W.out_features == self.hidden and W.in_features % 64 == 0)

    def fused_gemm_rs(self, x, W, site: int) -> TPPendingRS:
        """First launch of the fused all-reduce: the tcgen05 GEMM whose epilogue scatters the fp32 partials to the
        owners of the token rows."""
        big, t = self._big_tables(site)
        M, tp = x.shape[0], self.tp
        rows = (M + tp - 1) // tp
        cnt = big["counters"]
        rs = torch.tensor([t["rs_bufs"].data_ptr(), t["rs_flags"].data_ptr(), cnt[site * 2:].data_ptr(), self.step.data_ptr(), tp, self.rank, rows],
                          dtype=torch.int64)
        xin = x if x.is_contiguous() and x.shape[1] == W.in_features else x[:, : W.in_features].contiguous()
        ops.K.mmb200.fp4_gemm_rs(xin, W.qtile, W.stile, W.out_features, W.group_size, ops.gemm_status(x.device), rs)
        return TPPendingRS(site, M)

    def _finish_desc(self, site: int, M: int):
        big, t = self._big_tables(site)
        tp, H = self.tp, self.hidden
        rows = (M + tp - 1) // tp
        cnt = big["counters"]
        fin = torch.tensor([t["rs_local"], t["rs_flags_local"], t["ag_bufs"].data_ptr(), t["ag_flags"].data_ptr(), cnt[site * 2 + 1:].data_ptr(),
                            self.step.data_ptr(), self.status.data_ptr(), tp, self.rank, rows, H, M], dtype=torch.int64)
        flags_desc = torch.tensor([t["ag_flags_local"], self.step.data_ptr(), self.status.data_ptr(), tp], dtype=torch.int64)
        return big, t, rows, fin, flags_desc

    def finish_plain(self, d: TPPendingRS) -> torch.Tensor:
        """Reduce + all-gather by peer stores + a bounded wait; returns the all-reduced projection output as a bf16
        ``[M, hidden]`` view of the gathered buffer."""
        M, H = d.rows, self.hidden
        big, t, rows, fin, flags_desc = self._finish_desc(d.site, M)
        ops.K.mmb200.tp_rs_finish(fin)
        ops.K.mmb200.tp_wait(flags_desc)
        off = t["ag_local_off"]
        return big["buf"].local[off: off + M * H * 2].view(torch.bfloat16).view(M, H)

    def finish_norm(self, d: TPPendingRS, h: torch.Tensor, norm_w: torch.Tensor, eps: float) -> TPGathered:
        """Reduce with the residual add and the next RMSNorm fused on the owned rows; residual and normalized rows are
        gathered by peer stores.  Nothing waits here: the first consumer does (see :class:`TPGathered`)."""
        M, H = d.rows, self.hidden
        big, t, rows, fin, flags_desc = self._finish_desc(d.site, M)
        ops.K.mmb200.tp_rs_finish_norm(fin, h.contiguous(), norm_w, t["ag2_bufs"].data_ptr(), eps)
        off, off2 = t["ag_local_off"], t["ag2_local_off"]
        loc = big["buf"].local
        wait = torch.tensor([t["ag_flags_local"], self.step.data_ptr(), self.tp, self.rank, rows], dtype=torch.int64)
        return TPGathered(x=loc[off2: off2 + M * H * 2].view(torch.bfloat16).view(M, H),
                          h=loc[off: off + M * H * 2].view(torch.bfloat16).view(M, H), wait=wait, flags_desc=flags_desc)

    def fused_gemm_all_reduce(self, x, W, site: int) -> torch.Tensor:
        """``all_reduce(x @ W^T)`` in three launches and no collective call (GEMM with scatter epilogue, reduce +
        gather, bounded wait)."""
        return self.finish_plain(self.fused_gemm_rs(x, W, site))

    # ------------------------------------------------------------------ descriptors (CPU int64[9])
    def _desc(self, kind: str, site: int, rows: int) -> torch.Tensor:
        key = (kind, site, rows)
        d = self._desc_cache.get(key)
        if d is None:
            base = self.buf.local.data_ptr()
            v = [0] * 10
            if kind == "in":
                v[0] = base + site * self.site_bytes
                v[1] = base + self.flags_off + site * self.tp * 4
                v[2] = self.slot
            elif kind == "out":
                v[3] = self.peer_slots[site].data_ptr()
                v[4] = self.peer_flags[site].data_ptr()
                v[5] = self.counters[site:].data_ptr()
                if self.use_multimem and site < self.n_sites:
                    # my slot of this site in EVERY rank's buffer through the multicast mapping: one multimem store per value
                    v[9] = self.buf.multicast_ptr + site * self.site_bytes + self.rank * self.slot * 4
            else:       # "pairs": vocabulary-parallel arg-max exchange (both directions)
                v[0] = base + self.pairs_off
                v[1] = base + self.flags_off + site * self.tp * 4
                v[2] = self.max_tokens * 2
                v[3] = self.peer_slots[site].data_ptr()
                v[4] = self.peer_flags[site].data_ptr()
            v[6] = self.step.data_ptr()
            v[7] = self.status.data_ptr()
            v[8] = self.tp
            d = torch.tensor(v, dtype=torch.int64)
            self._desc_cache[key] = d
        return d

    # ------------------------------------------------------------------ step bookkeeping
    def begin_step(self) -> None:
        """Advance the exchange epoch; must run (on every rank) once before each decode step's kernels."""
        if self.fused_ok:
            self.step += 1

    def use_fused(self, n_tokens: int) -> bool:
        return self.fused_ok and n_tokens <= self.max_tokens

    # ------------------------------------------------------------------ producers / consumers
    def row_parallel(self, x, W, site: int):
        """Row-parallel linear: returns a :class:`TPPartial` (fused) or the all-reduced tensor (nccl)."""
        M = x.shape[0]
        if self.use_fused(M):
            ops.linear(x, W, tpx=self._desc("out", site, M), out=self._dummy(M, W.out_features))
            return TPPartial(site, M)
        if self.use_fused_gemm(M, W):
            return self.fused_gemm_rs(x, W, site)
        y = ops.linear(x, W)
        return self.all_reduce(y)

    def moe_row_parallel(self, h, x_normed_args, L, ids, wts, cfg, site: int):
        T = ids.shape[0]
        n_shared, shared_base = cfg.n_shared_experts, cfg.num_experts
        if getattr(L, "ep_local", 0):
            # whole experts per rank: experts of other ranks become id -1, which the kernels skip; the partial outputs
            # of the ranks add up to the full MoE output exactly like the slices of a width-sharded expert
            from .ep import localize_ids
            ids = localize_ids(ids, L.ep_first, L.ep_local)
            n_shared, shared_base = L.ep_shared_local, L.ep_local
        if self.use_fused(T):
            hmid = ops.moe_gate_up(h, L.gate_up_bank, ids, n_shared=n_shared, shared_base=shared_base, **x_normed_args)
            ops.moe_down(hmid, L.down_bank, ids, wts, n_shared=n_shared, shared_base=shared_base,
                         tpx=self._desc("out", site, T), out=self._dummy(T, L.down_bank.out_features))
            return TPPartial(site, T)
        y = ops.moe_forward(h, L.gate_up_bank, L.down_bank, ids, wts, n_shared=n_shared, shared_base=shared_base, **x_normed_args)
        return self.all_reduce(y)

    def _dummy(self, m: int, n: int) -> torch.Tensor:
        key = ("dummy", m, n)
        t = self._desc_cache.get(key)
        if t is None:
            t = torch.empty(m, n, dtype=torch.bfloat16, device=self.device)
            self._desc_cache[key] = t
        return t

    def consume(self, d) -> dict:
        """kwargs for the consuming op: either a plain ``delta`` tensor or the in-kernel exchange descriptor."""
        if isinstance(d, TPPartial):
            return {"delta": None, "tpx": self._desc("in", d.site, d.rows)}
        if isinstance(d, TPPendingRS):
            return {"delta": self.finish_plain(d)}
        return {"delta": d}

    AR_MAX_ELEMS = 8192 * 4096          # fp32 elements of the in-switch all-reduce buffer (128 MiB per rank)

    def _ar_buffers(self):
        """Symmetric fp32 buffer + flag words of the in-switch all-reduce (``csrc/tp_allreduce.cu``), created on first use;
        ``None`` when the allocation has no NVSwitch multicast mapping (the collective library is used then)."""
        ar = getattr(self, "_ar", None)
        if ar is None:
            ar = False
            if self.fused_ok and self.use_multimem and self.tp > 1 and os.environ.get("MMB_TP_MC_ALLREDUCE", "1") != "0":
                nbytes = self.AR_MAX_ELEMS * 4
                buf = SymmetricBuffer(nbytes + 256, self.device, self.group)
                if buf.multicast_ptr:
                    flags_off = nbytes
                    table = torch.tensor([buf.peer_addr(r, flags_off) for r in range(self.tp)], dtype=torch.int64).to(self.device)
                    step = torch.zeros(1, dtype=torch.int32, device=self.device)
                    counter = torch.zeros(1, dtype=torch.int32, device=self.device)
                    desc = torch.tensor([buf.multicast_ptr, table.data_ptr(), buf.local.data_ptr() + flags_off, step.data_ptr(),
                                         counter.data_ptr(), self.status.data_ptr()], dtype=torch.int64)
                    ar = {"buf": buf, "data": buf.view(0, (self.AR_MAX_ELEMS,), torch.float32), "table": table, "step": step,
                          "counter": counter, "desc": desc}
            self._ar = ar
        return ar or None

    def all_reduce(self, y: torch.Tensor) -> torch.Tensor:
        """Sum of ``y`` over the tensor-parallel ranks.  With NVSwitch multicast: one kernel of this library
        (``multimem.ld_reduce`` + ``multimem.st`` on a symmetric fp32 copy, bounded flag waits, no collective call);
        otherwise ``torch.distributed.all_reduce``."""
        if self.tp <= 1:
            return y
        n = y.numel()
        ar = self._ar_buffers() if (y.is_cuda and n % 4 == 0 and n <= self.AR_MAX_ELEMS) else None
        if ar is not None:
            data = ar["data"][:n].view(y.shape)
            data.copy_(y)                                                   # cast to fp32 into this rank's symmetric copy
            ops.K.mmb200.mc_all_reduce(ar["desc"], n, self.tp, self.rank, data)
            return data.to(y.dtype)
        yf = y.to(torch.float32)
        dist.all_reduce(yf, group=self.group)
        return yf.to(y.dtype)

    def greedy(self, logits_local: torch.Tensor, vocab_offset: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Global arg-max of vocabulary-sharded logits."""
        B = logits_local.shape[0]
        if self.use_fused(B):
            return ops.tp_argmax(logits_local, vocab_offset, self._desc("pairs", self.n_sites, B), out=out)
        full = self.gather_logits(logits_local)
        r = full.argmax(-1)
        if out is not None:
            out.copy_(r)
            return out
        return r

    def gather_logits(self, logits_local: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(logits_local) for _ in range(self.tp)]
        dist.all_gather(parts, logits_local.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    def check(self) -> int:
        return int(self.status[0].item()) if self.fused_ok else 0


# ---------------------------------------------------------------------------------------------
# sharding
# ---------------------------------------------------------------------------------------------
def shard_layer(cfg, L: LayerWeights, rank: int, tp: int, expert_parallel: bool = False) -> Tuple[LayerWeights, dict]:
    """Returns the rank's shard of one layer and its local dimensions.  ``expert_parallel``: the routed experts are not
    sliced; the rank keeps its range of whole experts (and rank 0 the shared experts), see ``parallel/ep.py``."""
    S = copy.copy(L)
    info = {}
    if cfg.is_mla:
        H, dn, dr, dv = cfg.num_attention_heads, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        h0, h1 = even_split(H, tp)[rank]
        info["heads"] = h1 - h0
        dq = dn + dr
        if L.q_b is not None:
            S.q_b = L.q_b.slice_rows(h0 * dq, h1 * dq)
        else:
            # direct q projection fused with kv_a: keep q rows of the local heads + all kv_a rows
            nq = H * dq
            q = L.qa_kva.slice_rows(h0 * dq, h1 * dq)
            kv = L.qa_kva.slice_rows(nq, L.qa_kva.out_features)
            from ..ops import FP4Weight
            S.qa_kva = FP4Weight.concat_rows([q, kv])
        S.w_ukT = L.w_ukT[h0:h1].contiguous()
        S.w_uv = L.w_uv[h0:h1].contiguous()
        if L.kv_b_dense is not None:
            per = cfg.qk_nope_head_dim + cfg.v_head_dim
            S.kv_b_dense = L.kv_b_dense[h0 * per: h1 * per].contiguous()
        S.o = L.o.slice_cols(h0 * dv, h1 * dv)
    else:
        Hq, Hk, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.dh
        assert Hk % tp == 0 or tp % Hk == 0, "kv heads must divide (or be divided by) the tensor-parallel degree"
        kv_per = max(1, Hk // tp)
        k0 = (rank * Hk) // tp
        g = Hq // Hk
        q0, q1 = (rank * Hq) // tp, ((rank + 1) * Hq) // tp
        info["heads"], info["kv_heads"] = q1 - q0, kv_per
        from ..ops import FP4Weight
        S.qkv = FP4Weight.concat_rows([L.qkv.slice_rows(q0 * D, q1 * D),
                                       L.qkv.slice_rows((Hq + k0) * D, (Hq + k0 + kv_per) * D),
                                       L.qkv.slice_rows((Hq + Hk + k0) * D, (Hq + Hk + k0 + kv_per) * D)])
        if L.qkv_bias is not None:
            b = L.qkv_bias
            S.qkv_bias = torch.cat([b[q0 * D:q1 * D], b[(Hq + k0) * D:(Hq + k0 + kv_per) * D],
                                    b[(Hq + Hk + k0) * D:(Hq + Hk + k0 + kv_per) * D]]).contiguous()
        S.o = L.o.slice_cols(q0 * D, q1 * D)
        assert g >= 1
    if L.gate_up_bank is not None and expert_parallel:
        from .ep import shard_bank
        S.gate_up_bank, first, n_local, n_sh = shard_bank(L.gate_up_bank, cfg.num_experts, cfg.n_shared_experts, rank, tp)
        S.down_bank = shard_bank(L.down_bank, cfg.num_experts, cfg.n_shared_experts, rank, tp)[0]
        S.ep_first, S.ep_local, S.ep_shared_local = first, n_local, n_sh
        info["moe_inter"] = L.gate_up_bank.out_features // 2
    elif L.gate_up_bank is not None:
        I = L.gate_up_bank.out_features // 2
        unit = max(64, L.down_bank.group_size)
        i0, i1 = even_split(I, tp, unit)[rank]
        info["moe_inter"] = i1 - i0
        assert i1 > i0, "tensor-parallel degree exceeds the number of quantization groups of the expert width"
        S.gate_up_bank = L.gate_up_bank.slice_rows([(i0, i1), (I + i0, I + i1)])
        S.down_bank = L.down_bank.slice_cols(i0, i1)
    else:
        I = L.gate_up.out_features // 2
        unit = max(64, L.down.group_size)
        i0, i1 = even_split(I, tp, unit)[rank]
        from ..ops import FP4Weight
        S.gate_up = FP4Weight.concat_rows([L.gate_up.slice_rows(i0, i1), L.gate_up.slice_rows(I + i0, I + i1)])
        S.down = L.down.slice_cols(i0, i1)
    return S, info


def shard_transformer(model: Transformer, rank: int, tp: int, ctx: Optional[TPContext] = None,
                      expert_parallel: bool = False) -> Transformer:
    """Build the rank's tensor-parallel shard of ``model`` (weights are sliced, not re-quantized)."""
    cfg = model.cfg
    if getattr(cfg, "has_linear_layers", False):
        raise NotImplementedError("tensor parallelism over Gated DeltaNet layers is not implemented (serve hybrid stacks with --dp)")
    layers, infos = [], []
    for L in model.layers:
        S, info = shard_layer(cfg, L, rank, tp, expert_parallel)
        layers.append(S)
        infos.append(info)
    v0, v1 = even_split(cfg.vocab_size, tp)[rank]
    head = model.lm_head[v0:v1].contiguous()
    m = Transformer(cfg, layers, model.embed, model.final_norm, head)
    m.tp = ctx
    m.tp_rank, m.tp_size = rank, tp
    m.vocab_range = (v0, v1)
    m.n_heads_local = infos[0]["heads"]
    m.n_kv_heads_local = infos[0].get("kv_heads", 1)
    return m


def make_context(model_cfg, device, group=None, mode: str = "fused", max_tokens: int = FUSED_MAX_TOKENS) -> TPContext:
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    tp = dist.get_world_size(group) if dist.is_initialized() else 1
    return TPContext(rank, tp, device, 2 * model_cfg.num_hidden_layers, model_cfg.hidden_size, group, max_tokens, mode)
