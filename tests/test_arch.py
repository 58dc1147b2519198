"""Recurrent layer families and hybrid layouts (reference: tests/test_mamba.py, test_rwkv.py, test_hybrid.py,
test_qwen36_deltanet.py)."""
import pytest
import torch

from metal_marlin_b200 import arch


def test_gated_delta_chunked_matches_recurrence_and_step():
    torch.manual_seed(0)
    B, T, H, dk, dv = 2, 37, 3, 16, 24
    q, k = arch.l2norm(torch.randn(B, T, H, dk)), arch.l2norm(torch.randn(B, T, H, dk))
    v = torch.randn(B, T, H, dv)
    g = -torch.rand(B, T, H) * 0.3
    beta = torch.rand(B, T, H)
    o_ref, S_ref = arch.gated_delta_rule_recurrent(q, k, v, g, beta)
    o_chk, S_chk = arch.gated_delta_rule_chunked(q, k, v, g, beta, chunk=8)
    torch.testing.assert_close(o_chk, o_ref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(S_chk, S_ref, rtol=1e-4, atol=1e-4)
    # prefill the first 30 tokens in chunks, then step the rest one token at a time
    _, S = arch.gated_delta_rule_chunked(q[:, :30], k[:, :30], v[:, :30], g[:, :30], beta[:, :30], chunk=16)
    outs = [arch.gated_delta_step(q[:, t], k[:, t], v[:, t], g[:, t], beta[:, t], S) for t in range(30, T)]
    torch.testing.assert_close(torch.stack(outs, 1), o_ref[:, 30:], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(S, S_ref, rtol=1e-4, atol=1e-4)


def test_mamba_block_forward_equals_stepping():
    cfg = arch.MambaConfig(d_model=32, d_state=8, d_conv=4, expand=2)
    blk = arch.MambaBlock.random(cfg, seed=1)
    u = torch.randn(2, 11, 32)
    y_full, _ = blk.forward(u)
    y_a, st = blk.forward(u[:, :6])
    ys = [y_a]
    for t in range(6, 11):
        y_t, st = blk.step(u[:, t], st)
        ys.append(y_t[:, None])
    torch.testing.assert_close(torch.cat(ys, 1), y_full, rtol=1e-4, atol=1e-5)
    x, dt = torch.randn(2, 5, 16), torch.rand(2, 5, 16) * 0.1
    A, Bm, Cm = -torch.rand(16, 4), torch.randn(2, 5, 4), torch.randn(2, 5, 4)
    y, h = arch.selective_scan(x, dt, A, Bm, Cm, torch.ones(16))
    st = torch.zeros(2, 16, 4)
    ys = [arch.selective_scan_step(x[:, t], dt[:, t], A, Bm[:, t], Cm[:, t], torch.ones(16), st) for t in range(5)]
    torch.testing.assert_close(torch.stack(ys, 1), y, rtol=1e-5, atol=1e-6)
    y2, h2 = arch.mamba2_scan(torch.randn(1, 4, 2, 8), torch.rand(1, 4, 2) * 0.1, -torch.rand(2), torch.randn(1, 4, 4), torch.randn(1, 4, 4))
    assert y2.shape == (1, 4, 2, 8) and h2.shape == (1, 2, 8, 4)


def test_rwkv_wkv_state_carry():
    torch.manual_seed(2)
    B, T, H, dk, dv = 1, 9, 2, 8, 8
    r, k, v = torch.randn(B, T, H, dk), torch.randn(B, T, H, dk) * 0.3, torch.randn(B, T, H, dv)
    w, u = torch.rand(H, dk) * 0.5 + 0.4, torch.randn(H, dk) * 0.1
    o, S = arch.wkv5(r, k, v, w, u)
    o1, S1 = arch.wkv5(r[:, :4], k[:, :4], v[:, :4], w, u)
    o2, S2 = arch.wkv5(r[:, 4:], k[:, 4:], v[:, 4:], w, u, S1)
    torch.testing.assert_close(torch.cat([o1, o2], 1), o, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(S2, S, rtol=1e-5, atol=1e-6)
    o6, _ = arch.wkv6(r, k, v, w[None, None].expand(B, T, H, dk), u)
    torch.testing.assert_close(o6, o)


def test_hybrid_layouts():
    j = arch.jamba_layout(16)
    assert [i for i, l in enumerate(j) if l.mixer == "attention"] == [4, 12] and j[1].mlp == "moe" and j[0].mlp == "dense"
    q = arch.qwen35_layout(8)
    assert [l.mixer for l in q] == ["deltanet"] * 3 + ["attention"] + ["deltanet"] * 3 + ["attention"] and arch.kv_layers(q) == [3, 7]
    z = arch.zamba_layout(12, 6)
    assert arch.kv_layers(z) == [5, 11]
    lt = arch.layout_from_config({"num_hidden_layers": 4, "layer_types": ["linear_attention", "linear_attention", "linear_attention", "full_attention"],
                                  "num_experts": 8})
    assert [l.mixer for l in lt] == ["deltanet", "deltanet", "deltanet", "attention"] and lt[0].mlp == "moe"
    assert arch.layout_from_config({"num_hidden_layers": 8, "full_attention_interval": 4}) == arch.qwen35_layout(8, 4, False)


@pytest.mark.gpu
def test_recurrent_step_kernels_gpu():
    torch.manual_seed(3)
    dev = "cuda"
    B, H, dk, dv = 3, 4, 128, 128
    q, k = arch.l2norm(torch.randn(B, H, dk, device=dev)).bfloat16(), arch.l2norm(torch.randn(B, H, dk, device=dev)).bfloat16()
    v = torch.randn(B, H, dv, device=dev).bfloat16()
    g, beta = -torch.rand(B, H, device=dev) * 0.3, torch.rand(B, H, device=dev)
    S0 = torch.randn(B, H, dk, dv, device=dev) * 0.1
    S_gpu = S0.clone()
    o = arch.gated_delta_step(q, k, v, g, beta, S_gpu)
    o_ref, S_ref = arch.gated_delta_rule_recurrent(q[:, None].float().cpu(), k[:, None].float().cpu(), v[:, None].float().cpu(), g[:, None].cpu(),
                                                   beta[:, None].cpu(), S0.cpu())
    torch.testing.assert_close(o.float().cpu(), o_ref[:, 0], rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(S_gpu.cpu(), S_ref, rtol=1e-3, atol=1e-3)
    Di, N = 700, 16
    x, dt = torch.randn(B, Di, device=dev).bfloat16(), torch.rand(B, Di, device=dev) * 0.1
    A, Bm, Cm, D = -torch.rand(Di, N, device=dev), torch.randn(B, N, device=dev), torch.randn(B, N, device=dev), torch.ones(Di, device=dev)
    st0 = torch.randn(B, Di, N, device=dev) * 0.1
    st = st0.clone()
    y = arch.selective_scan_step(x, dt, A, Bm, Cm, D, st)
    y_ref, h_ref = arch.selective_scan(x[:, None].float().cpu(), dt[:, None].cpu(), A.cpu(), Bm[:, None].cpu(), Cm[:, None].cpu(), D.cpu(), st0.cpu())
    torch.testing.assert_close(y.float().cpu(), y_ref[:, 0], rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(st.cpu(), h_ref, rtol=1e-3, atol=1e-3)


@pytest.mark.gpu
def test_sequence_scan_kernels_match_token_loops():
    """Whole-sequence scan kernels (state in registers, one launch over all tokens) against the PyTorch token loops:
    RWKV v5 / v6 WKV, Mamba selective scan, gated delta rule; with and without an initial state."""
    import torch
    from metal_marlin_b200 import ops
    from metal_marlin_b200.arch import deltanet as dn
    from metal_marlin_b200.arch import mamba as mb
    from metal_marlin_b200.arch import rwkv
    dev = "cuda"
    torch.manual_seed(0)
    B, T, H, dk, dv = 2, 37, 3, 64, 64
    r, k = torch.randn(B, T, H, dk, device=dev) * 0.5, torch.randn(B, T, H, dk, device=dev) * 0.5
    v = torch.randn(B, T, H, dv, device=dev)
    w6 = torch.rand(B, T, H, dk, device=dev) * 0.5 + 0.4
    w5, u = torch.rand(H, dk, device=dev) * 0.5 + 0.4, torch.randn(H, dk, device=dev) * 0.3
    s0 = torch.randn(B, H, dk, dv, device=dev) * 0.1
    for fn, w in ((rwkv.wkv6, w6), (rwkv.wkv5, w5)):
        for st in (None, s0):
            o, S = fn(r, k, v, w, u, st)
            with ops.force_reference():
                o_ref, S_ref = fn(r, k, v, w, u, st)
            torch.testing.assert_close(o, o_ref, rtol=2e-4, atol=2e-4)
            torch.testing.assert_close(S, S_ref, rtol=2e-4, atol=2e-4)
    # selective scan
    Di, N = 200, 16
    x, dt = torch.randn(B, T, Di, device=dev), torch.rand(B, T, Di, device=dev) * 0.1
    A = -torch.rand(Di, N, device=dev)
    Bm, Cm, D = torch.randn(B, T, N, device=dev), torch.randn(B, T, N, device=dev), torch.randn(Di, device=dev)
    h0 = torch.randn(B, Di, N, device=dev) * 0.1
    for st in (None, h0):
        y, h = mb.selective_scan(x, dt, A, Bm, Cm, D, st)
        with ops.force_reference():
            y_ref, h_ref = mb.selective_scan(x, dt, A, Bm, Cm, D, st)
        torch.testing.assert_close(y, y_ref, rtol=2e-4, atol=2e-4)
        torch.testing.assert_close(h, h_ref, rtol=2e-4, atol=2e-4)
    # gated delta rule
    dk2, dv2 = 64, 128
    q, kk = torch.randn(B, T, H, dk2, device=dev), dn.l2norm(torch.randn(B, T, H, dk2, device=dev))
    vv = torch.randn(B, T, H, dv2, device=dev)
    g, beta = -torch.rand(B, T, H, device=dev) * 0.2, torch.rand(B, T, H, device=dev)
    o, S = dn.gated_delta_rule_chunked(q, kk, vv, g, beta)
    o_ref, S_ref = dn.gated_delta_rule_recurrent(q, kk, vv, g, beta)
    torch.testing.assert_close(o, o_ref, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(S, S_ref, rtol=1e-3, atol=1e-3)
