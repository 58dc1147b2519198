"""Plain-PyTorch restatement of every native op (runs on CPU or GPU).

This is the numerics oracle for the CUDA kernels and the execution path on machines
without a GPU.  Math is fp32 with bf16 rounding at the same points where the kernels
store bf16, so kernel-vs-reference comparisons are tight.  Parity: the reference's
CPU fallbacks, e.g. ``metal_marlin/layers/mmfp4_linear.py:227`` (``_fast_dequant`` +
``F.linear``), ``metal_marlin/moe_dispatch.py:99`` (router softmax/top-k),
``metal_marlin/paged/mla_cache.py:717`` (``mla_attention`` numpy reference).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# Dtype of the dequantized weight copies and of the matrix products.  fp32 is the numerics oracle; the eager
# baseline (``baseline_eager.py``) switches to bf16 so its matrix products run as library bf16 GEMMs.
MATMUL_DTYPE = torch.float32


def _mm(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` in ``MATMUL_DTYPE``, returned as fp32."""
    if MATMUL_DTYPE == torch.float32:
        return x.to(torch.float32) @ w.to(torch.float32).t()
    return F.linear(x.to(MATMUL_DTYPE), w.to(MATMUL_DTYPE)).to(torch.float32)


def _bf(x: torch.Tensor) -> torch.Tensor:
    """Round to bf16 and come back to fp32."""
    return x.to(torch.bfloat16).to(torch.float32)


def add_norm(x, delta, norm_w, eps, resid_out=None):
    """Returns fp32 ``bf16(norm(bf16(x + delta)))`` (norm skipped when ``norm_w`` is None)."""
    s = x.to(torch.float32)
    if delta is not None:
        s = _bf(s + delta.to(torch.float32))
        if resid_out is not None:
            resid_out.copy_(s.to(resid_out.dtype))
    if norm_w is not None:
        rs = torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps)
        s = _bf(s * rs * norm_w.to(torch.float32))
    return s


def rmsnorm(x, w, eps, delta=None, resid_out=None, out=None):
    y = add_norm(x, delta, w if w is not None else torch.ones(x.shape[-1], device=x.device), eps, resid_out)
    y = y.to(torch.bfloat16)
    if out is not None:
        out.copy_(y)
        return out
    return y


def linear(x, W, *, delta=None, norm_w=None, eps=1e-6, resid_out=None, act=0, bias=None, out_add=None, out=None):
    xin = add_norm(x[:, : W.in_features], None if delta is None else delta[:, : W.in_features], norm_w, eps, resid_out)
    wd = W.dequantize(MATMUL_DTYPE, cache=True)
    y = _mm(xin, wd)
    if bias is not None:
        y = y + bias.to(torch.float32)
    if act == 1:
        half = W.out_features // 2
        y = F.silu(y[:, :half]) * y[:, half:]
    if out_add is not None:
        y = y + out_add.to(torch.float32)
    y = y.to(torch.bfloat16)
    if out is not None:
        out.copy_(y)
        return out
    return y


def bf16_linear(x, w, *, delta=None, norm_w=None, eps=1e-6, out_dtype=torch.bfloat16, out=None):
    xin = add_norm(x, delta, norm_w, eps)
    y = _mm(xin, w).to(out_dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def silu_mul(gu, out=None):
    inter = gu.shape[-1] // 2
    g = gu[..., :inter].to(torch.float32)
    u = gu[..., inter:].to(torch.float32)
    y = (F.silu(g) * u).to(torch.bfloat16)
    if out is not None:
        out.copy_(y)
        return out
    return y


def embedding(table, ids, out=None):
    y = table[ids.reshape(-1)]
    if out is not None:
        out.copy_(y)
        return out
    return y


def _rope_angles(positions, inv_freq):
    ang = positions.to(torch.float32).unsqueeze(-1) * inv_freq.to(torch.float32)     # [T, half]
    return ang.cos(), ang.sin()


def rope_rotate(x, cos, sin, interleaved: bool, mscale: float = 1.0):
    """x [T, H, rot_dim] fp32; cos/sin [T, half]."""
    c, s = cos.unsqueeze(1) * mscale, sin.unsqueeze(1) * mscale
    if interleaved:
        a, b = x[..., 0::2], x[..., 1::2]
        ra, rb = a * c - b * s, b * c + a * s
        return torch.stack([ra, rb], dim=-1).flatten(-2)
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def rope(q, k, positions, inv_freq, Hq, Hk, D, rot_dim, interleaved, mscale=1.0):
    """In place on q [T, Hq*D] (and k [T, Hk*D])."""
    cos, sin = _rope_angles(positions, inv_freq)
    for t, H in ((q, Hq), (k, Hk)):
        if t is None:
            continue
        T = t.shape[0]
        v = t.view(T, H, D)
        r = rope_rotate(v[..., :rot_dim].to(torch.float32), cos, sin, interleaved, mscale)
        v[..., :rot_dim] = r.to(t.dtype)
    return q, k


def qk_norm_rope_cache(q, k, v, qn_w, kn_w, positions, inv_freq, slots, k_pool, v_pool, Hq, Hk, D, eps, interleaved):
    T = q.shape[0]
    cos, sin = _rope_angles(positions, inv_freq)
    qv = q.view(T, Hq, D) if q.dim() == 2 else q
    qf = qv.to(torch.float32)
    kf = k.reshape(T, Hk, D).to(torch.float32)
    if qn_w is not None:
        qf = _bf(qf * torch.rsqrt(qf.pow(2).mean(-1, keepdim=True) + eps) * qn_w.to(torch.float32))
    if kn_w is not None:
        kf = _bf(kf * torch.rsqrt(kf.pow(2).mean(-1, keepdim=True) + eps) * kn_w.to(torch.float32))
    qr = rope_rotate(qf, cos, sin, interleaved)
    kr = rope_rotate(kf, cos, sin, interleaved)
    qv.copy_(qr.to(q.dtype))
    ok = slots >= 0
    if ok.any():
        k_pool.view(-1, Hk, D)[slots[ok]] = kr[ok].to(k_pool.dtype)
        v_pool.view(-1, Hk, D)[slots[ok]] = v.reshape(T, Hk, D)[ok].to(v_pool.dtype)
    return q


def mla_prep(q, kva, w_ukT, kv_norm_w, positions, inv_freq, slots, q_full, cache, H, dn, dr, R, eps, mscale, interleaved):
    T = positions.numel()
    qv = q.reshape(T, H, dn + dr).to(torch.float32)
    cos, sin = _rope_angles(positions, inv_freq)
    q_lat = torch.einsum("thd,hcd->thc", qv[..., :dn], w_ukT.to(torch.float32))
    q_rope = rope_rotate(qv[..., dn:], cos, sin, interleaved, mscale)
    q_full.view(T, H, R + dr)[..., :R] = q_lat.to(q_full.dtype)
    q_full.view(T, H, R + dr)[..., R:] = q_rope.to(q_full.dtype)
    kvf = kva[:, : R + dr].to(torch.float32)
    c = kvf[:, :R]
    c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * kv_norm_w.to(torch.float32)
    kr = rope_rotate(kvf[:, R:].unsqueeze(1), cos, sin, interleaved, mscale).squeeze(1)
    ok = slots >= 0
    lat = torch.cat([c, kr], -1).to(cache.dtype)
    if ok.any():
        cache.view(-1, R + dr)[slots[ok]] = lat[ok]
    return q_full


def paged_attention(q, k_pool, v_pool, block_tables, ctx_lens, Hq, Hkv, dqk, dv, block_size, scale, window=0):
    """Returns bf16 [B, Hq, dv].  ``v_pool`` None means V = K[..., :dv] (MLA latent)."""
    B = ctx_lens.numel()
    out = torch.zeros(B, Hq, dv, dtype=torch.float32, device=q.device)
    Gh = Hq // Hkv
    kp = k_pool.view(-1, Hkv, dqk)
    vp = v_pool.view(-1, Hkv, dv) if v_pool is not None else None
    for b in range(B):
        n = int(ctx_lens[b])
        if n == 0:
            continue
        lo = max(0, n - window) if window > 0 else 0
        tok = torch.arange(lo, n, device=q.device)
        slots = block_tables[b, tok // block_size].long() * block_size + (tok % block_size)
        K = kp[slots].to(torch.float32)                                   # [n, Hkv, dqk]
        V = vp[slots].to(torch.float32) if vp is not None else K[..., :dv]
        qb = q[b].view(Hkv, Gh, dqk).to(torch.float32)
        s = torch.einsum("hgd,nhd->hgn", qb, K) * scale
        p = torch.softmax(s, dim=-1)
        out[b] = torch.einsum("hgn,nhd->hgd", p, V).reshape(Hq, dv)
    return out.to(torch.bfloat16)


def mla_up(o_lat, w_uv):
    """o_lat bf16 [B, H, R], w_uv [H, dvo, R] -> bf16 [B, H, dvo]."""
    return torch.einsum("bhr,hvr->bhv", o_lat.to(torch.float32), w_uv.to(torch.float32)).to(torch.bfloat16)


def moe_router(x, w, *, delta=None, norm_w=None, eps=1e-6, resid_out=None, bias=None, topk=4, scoring=0, renorm=True,
               routed_scale=1.0, n_group=1, topk_group=1) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    xin = add_norm(x, delta, norm_w, eps, resid_out)
    logits = xin @ w.to(torch.float32).t()
    ids, wts = moe_select(logits, bias=bias, topk=topk, scoring=scoring, renorm=renorm, routed_scale=routed_scale, n_group=n_group,
                          topk_group=topk_group)
    return ids, wts, logits


def moe_select(logits, *, bias=None, topk=4, scoring=0, renorm=True, routed_scale=1.0, n_group=1, topk_group=1):
    """Scores, (grouped) top-k and weights from fp32 gate logits ``[T, E]``."""
    logits = logits.to(torch.float32)
    if scoring == 0:
        scores = torch.softmax(logits, dim=-1)
        choice = scores
    else:
        scores = torch.sigmoid(logits)
        choice = scores + (bias.to(torch.float32) if bias is not None else 0.0)
    T, E = logits.shape
    if n_group > 1 and topk_group < n_group:
        grp = choice.view(T, n_group, E // n_group)
        gscore = grp.topk(2, dim=-1).values.sum(-1)
        keep = torch.zeros_like(gscore, dtype=torch.bool)
        keep.scatter_(1, gscore.topk(topk_group, dim=-1).indices, True)
        choice = torch.where(keep.unsqueeze(-1).expand_as(grp), grp, torch.full_like(grp, float("-inf"))).reshape(T, E)
    ids = choice.topk(topk, dim=-1).indices
    wts = scores.gather(1, ids)
    if renorm:
        wts = wts / (wts.sum(-1, keepdim=True) + 1e-20)
    wts = wts * routed_scale
    return ids.to(torch.int32), wts.to(torch.float32)


def moe_gate_up(x, bank, ids, *, n_shared=0, shared_base=0, norm_w=None, eps=1e-6, out=None):
    """x [T, K] -> [T * S, I] with S = topk + n_shared; bank rows are [gate (I) | up (I)]."""
    T, topk = ids.shape
    S = topk + n_shared
    xin = add_norm(x[:, : bank.in_features], None, norm_w, eps)
    W = bank.dequantize(MATMUL_DTYPE, cache=True)                     # [E, 2I, K]
    inter = bank.out_features // 2
    e_all = torch.cat([ids.long(), torch.arange(shared_base, shared_base + n_shared, device=x.device)
                       .expand(T, n_shared)], 1) if n_shared else ids.long()
    res = torch.zeros(T, S, inter, dtype=torch.float32, device=x.device)
    for e in e_all.unique().tolist():
        if e < 0:
            continue
        tt, ss = (e_all == e).nonzero(as_tuple=True)
        y = _mm(xin[tt], W[e])
        res[tt, ss] = F.silu(y[:, :inter]) * y[:, inter:]
    res = res.to(torch.bfloat16).view(T * S, inter)
    if out is not None:
        out.copy_(res)
        return out
    return res


def moe_down(h, bank, ids, weights, *, n_shared=0, shared_base=0, out_add=None, out=None):
    """h [T * S, I] -> [T, H] = sum_s w[t, s] * (W_d[e(t, s)] h[t, s])."""
    T, topk = ids.shape
    S = topk + n_shared
    W = bank.dequantize(MATMUL_DTYPE, cache=True)
    hv = h.view(T, S, -1)[..., : bank.in_features].to(torch.float32)
    e_all = torch.cat([ids.long(), torch.arange(shared_base, shared_base + n_shared, device=h.device)
                       .expand(T, n_shared)], 1) if n_shared else ids.long()
    w_all = torch.cat([weights.to(torch.float32), torch.ones(T, n_shared, device=h.device)], 1) if n_shared \
        else weights.to(torch.float32)
    y = torch.zeros(T, bank.out_features, dtype=torch.float32, device=h.device)
    for e in e_all.unique().tolist():
        if e < 0:
            continue
        tt, ss = (e_all == e).nonzero(as_tuple=True)
        y.index_add_(0, tt, _mm(hv[tt, ss], W[e]) * w_all[tt, ss].unsqueeze(-1))
    if out_add is not None:
        y = y + out_add.to(torch.float32)
    y = y.to(torch.bfloat16)
    if out is not None:
        out.copy_(y)
        return out
    return y


def sample(logits, *, temperature=None, top_k=None, top_p=None, min_p=None, history=None, rep_penalty=None,
           generator: Optional[torch.Generator] = None):
    """Row-wise sampling with the same filter order as the kernel.  Returns (ids int64 [B], logprob fp32 [B])."""
    B, V = logits.shape
    lg = logits.to(torch.float32).clone()
    if history is not None and rep_penalty is not None:
        for b in range(B):
            h = history[b]
            h = h[(h >= 0) & (h < V)].unique()
            rp = float(rep_penalty[b])
            v = lg[b, h]
            lg[b, h] = torch.where(v > 0, v / rp, v * rp)
    ids = torch.empty(B, dtype=torch.int64, device=logits.device)
    lps = torch.empty(B, dtype=torch.float32, device=logits.device)
    for b in range(B):
        t = float(temperature[b]) if temperature is not None else 0.0
        row = lg[b]
        if t <= 0:
            ids[b] = int(row.argmax())
            lps[b] = torch.log_softmax(row, -1)[ids[b]]
            continue
        row = row / t
        logp_full = torch.log_softmax(row, -1)
        k = int(top_k[b]) if top_k is not None else 0
        p = float(top_p[b]) if top_p is not None else 1.0
        mp = float(min_p[b]) if min_p is not None else 0.0
        sv, si = torch.sort(row, descending=True, stable=True)
        n_keep = V
        if k > 0:
            n_keep = min(k, V)
        probs = torch.softmax(sv[:n_keep], -1) if k > 0 else torch.softmax(sv, -1)[:n_keep]
        if p < 1.0:
            cum = probs.cumsum(-1)
            n_keep = min(n_keep, int((cum < p).sum()) + 1)
        if mp > 0:
            n_keep = max(1, min(n_keep, int((sv[:n_keep] - sv[0] >= math.log(mp)).sum())))
        pr = torch.softmax(sv[:n_keep], -1)
        j = int(torch.multinomial(pr, 1, generator=generator))
        ids[b] = si[j]
        lps[b] = logp_full[si[j]]
    return ids, lps


# ---------------------------------------------------------------------------------------------------------------
# secondary ops
# ---------------------------------------------------------------------------------------------------------------
def unpack_lsb(codes: torch.Tensor, bits: int, n: int) -> torch.Tensor:
    """``uint8 [rows, n * bits / 8]`` packed LSB-first -> ``int64 [rows, n]``."""
    if bits == 8:
        return codes.long()[:, :n]
    per = 8 // bits
    sh = torch.arange(per, device=codes.device) * bits
    return ((codes.long().unsqueeze(-1) >> sh) & ((1 << bits) - 1)).reshape(codes.shape[0], -1)[:, :n]


def codebook_dequant(codes, scales, zeros, lut, in_f: int, group_size: int, bits: int = 8) -> torch.Tensor:
    c = unpack_lsb(codes, bits, in_f)
    v = lut.to(torch.float32)[c]
    out_f = c.shape[0]
    g = v.view(out_f, in_f // group_size, group_size)
    if zeros is not None:
        g = g - zeros.to(torch.float32).unsqueeze(-1)
    return (g * scales.to(torch.float32).unsqueeze(-1)).reshape(out_f, in_f)


def vision_preprocess(images, out_h, out_w, patch, mean, std):
    x = images.permute(0, 3, 1, 2).to(torch.float32)
    x = F.interpolate(x, size=(out_h, out_w), mode="bilinear", align_corners=False)
    m = torch.tensor(mean, device=x.device).view(1, 3, 1, 1)
    s = torch.tensor(std, device=x.device).view(1, 3, 1, 1)
    x = (x / 255.0 - m) / s
    if patch:
        B = x.shape[0]
        x = x.view(B, 3, out_h // patch, patch, out_w // patch, patch).permute(0, 2, 4, 1, 3, 5).reshape(B, -1, 3 * patch * patch)
    return x.to(torch.bfloat16)


def vision_preprocess_ex(images, out_h, out_w, crop, patch, merge, resample, mean, std):
    """Crop rectangle -> resample (bilinear / bicubic / nearest, half-pixel centres) -> normalise -> CHW or patches."""
    y0, x0, ch, cw = crop
    x = images[:, y0:y0 + ch, x0:x0 + cw].permute(0, 3, 1, 2).to(torch.float32)
    if resample == "nearest":
        iy = ((torch.arange(out_h, device=x.device).float() + 0.5) * ch / out_h).floor().long().clamp(0, ch - 1)
        ix = ((torch.arange(out_w, device=x.device).float() + 0.5) * cw / out_w).floor().long().clamp(0, cw - 1)
        x = x[:, :, iy][:, :, :, ix]
    else:
        x = F.interpolate(x, size=(out_h, out_w), mode=resample, align_corners=False)
    m = torch.tensor(mean, device=x.device).view(1, 3, 1, 1)
    s = torch.tensor(std, device=x.device).view(1, 3, 1, 1)
    x = (x / 255.0 - m) / s
    if patch:
        B = x.shape[0]
        ph, pw = out_h // patch, out_w // patch
        x = x.view(B, 3, ph, patch, pw, patch).permute(0, 2, 4, 1, 3, 5)           # [B, ph, pw, 3, p, p]
        if merge > 1:
            x = x.reshape(B, ph // merge, merge, pw // merge, merge, 3, patch, patch).permute(0, 1, 3, 2, 4, 5, 6, 7)
        x = x.reshape(B, ph * pw, 3 * patch * patch)
    return x.to(torch.bfloat16)


def spec_verify(p_target, p_draft, draft, u, u_resample):
    B, K1, V = p_target.shape
    K = K1 - 1
    toks = torch.full((B, K1), -1, dtype=torch.int64, device=p_target.device)
    acc = torch.zeros(B, dtype=torch.int32, device=p_target.device)
    for b in range(B):
        n = 0
        while n < K:
            t = int(draft[b, n])
            q, p = float(p_draft[b, n, t]), float(p_target[b, n, t])
            ratio = min(1.0, p / q) if q > 0 else 1.0
            if not float(u[b, n]) < ratio:
                break
            n += 1
        w = p_target[b, n].to(torch.float64)
        if n < K:
            r = (w - p_draft[b, n].to(torch.float64)).clamp_min(0)
            w = r if float(r.sum()) > 0 else w
        cdf = torch.cumsum(w, 0)
        target = float(u_resample[b]) * float(cdf[-1])
        idx = int(torch.searchsorted(cdf, torch.tensor(target, dtype=cdf.dtype, device=cdf.device), right=True))
        idx = min(idx, V - 1)
        toks[b, :n] = draft[b, :n]
        toks[b, n] = idx
        acc[b] = n
    return toks, acc


def prefill_attention(q, k, v, cu_q, cu_k, block_tables, ctx_lens, block_size, scale, window, causal, out, sinks=0, tree_mask=None,
                      block_mask=None):
    T, Hq, D = q.shape
    Hk = k.shape[1]
    cq = cu_q.tolist()
    for b in range(len(cq) - 1):
        s, e = cq[b], cq[b + 1]
        t = e - s
        if t == 0:
            continue
        if cu_k is not None:
            ck = cu_k.tolist()
            kb, vb = k[ck[b]:ck[b + 1]], v[ck[b]:ck[b + 1]]
        else:
            n = int(ctx_lens[b])
            tok = torch.arange(n, device=q.device)
            slots = block_tables[b, tok // block_size].long() * block_size + tok % block_size
            kb, vb = k[slots], v[slots]
        n = kb.shape[0]
        qf = q[s:e].to(torch.float32).transpose(0, 1)                                 # [Hq, t, D]
        kf = kb.to(torch.float32).transpose(0, 1).repeat_interleave(Hq // Hk, 0)
        vf = vb.to(torch.float32).transpose(0, 1).repeat_interleave(Hq // Hk, 0)
        sc = qf @ kf.transpose(-1, -2) * scale
        qpos = torch.arange(n - t, n, device=q.device)[:, None]
        kpos = torch.arange(n, device=q.device)[None, :]
        ok = torch.ones(t, n, dtype=torch.bool, device=q.device)
        if causal:
            ok &= kpos <= qpos
        if window and window > 0:
            ok &= (kpos > qpos - window) | (kpos < (sinks or 0))
        if tree_mask is not None:
            tm = torch.ones(t, n, dtype=torch.bool, device=q.device)
            tm[:, n - t:] = tree_mask[s:e, :t].bool()
            ok &= tm
        ok = ok.unsqueeze(0).expand(Hq, t, n)
        if block_mask is not None:
            qb = torch.arange(t, device=q.device) // 128
            kb_i = torch.arange(n, device=q.device) // 64
            bm = block_mask.bool()
            inside = kb_i < bm.shape[2]
            sel = bm[:, qb][:, :, kb_i.clamp_max(bm.shape[2] - 1)] & inside[None, None, :]
            ok = ok & sel.expand(Hq, t, n)
        sc = sc.masked_fill(~ok, float("-inf"))
        pr = torch.softmax(sc, -1)
        pr = torch.where(ok.any(-1, keepdim=True), pr, torch.zeros_like(pr))       # rows that see nothing give zeros
        out[s:e] = (pr @ vf).transpose(0, 1).to(out.dtype)
    return out


def sparse24_dequant(codes, meta, scales, in_f: int, group_size: int) -> torch.Tensor:
    """Dense fp32 ``[out, in]`` matrix of a 2:4 sparse FP4 weight: ``codes uint8 [out, in / 4]`` (two E2M1 codes per byte, low
    nibble first: the kept values of one group of four columns), ``meta uint8 [out, in / 8]`` (one nibble per group, low nibble
    first: bits 0-1 column of the first kept value, bits 2-3 of the second), ``scales fp16 [out, in / group_size]``."""
    from .._compat import get_e2m1_torch_table
    out_f = codes.shape[0]
    tab = get_e2m1_torch_table(codes.device, torch.float32)
    c = codes.long()
    vals = torch.stack([tab[c & 15], tab[c >> 4]], -1)                       # [out, in / 4, 2]
    m = meta.long()
    nib = torch.stack([m & 15, m >> 4], -1).reshape(out_f, in_f // 4)          # [out, groups]
    pos = torch.stack([nib & 3, nib >> 2], -1)                                  # [out, groups, 2]
    dense = torch.zeros(out_f, in_f // 4, 4, dtype=torch.float32, device=codes.device)
    dense.scatter_(2, pos, vals)
    dense = dense.view(out_f, in_f)
    return dense * scales.to(torch.float32).repeat_interleave(group_size, 1)
