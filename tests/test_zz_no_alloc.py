"""The allocation-free C entry point for paged decode attention (``csrc/attention_noalloc.h``), called through
ctypes on raw device pointers: it must agree with the regular op (which takes its split-KV workspace from the
caller) and with the PyTorch fp32 restatement, on two calls in a row, and must refuse sizes beyond its built-in
scratch.  Collected last so that it also runs after every other GPU test has used the device."""
import ctypes
import math
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from metal_marlin_b200 import _build
    _build.load(require=True)                      # the package's own loader: fails loudly when the .so is missing
    import metal_marlin_b200
    path = os.path.join(os.path.dirname(metal_marlin_b200.__file__), "_C.so")
    lib = ctypes.CDLL(path)
    fn = lib.mmb_paged_attention_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 9 + [ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
    lib.mmb_paged_attention_noalloc_error.restype = ctypes.c_char_p
    lib.mmb_paged_attention_noalloc_limits.argtypes = [ctypes.POINTER(ctypes.c_longlong)] * 2
    return lib


def _call(lib, q, kp, vp, bt, cl, w_uv, out, Hq, Hkv, dqk, dv, dvo, bs, splits, scale, window=0):
    ptr = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.mmb_paged_attention_noalloc(ptr(q), ptr(kp), ptr(vp), ptr(bt), ptr(cl), ptr(w_uv), ptr(out), cl.numel(), Hq, Hkv,
                                           dqk, dv, dvo, bs, bt.shape[1], splits, ctypes.c_float(scale), window, stream)


def _setup(ctxs, bs, n_blocks, dev):
    g = torch.Generator().manual_seed(3)
    perm = torch.randperm(n_blocks, generator=g).to(torch.int32)
    maxb = max((c + bs - 1) // bs for c in ctxs)
    bt = torch.zeros(len(ctxs), maxb, dtype=torch.int32)
    used = 0
    for b, c in enumerate(ctxs):
        nb = (c + bs - 1) // bs
        bt[b, :nb] = perm[used:used + nb]
        used += nb
    return bt.to(dev), torch.tensor(ctxs, dtype=torch.int32, device=dev)


def _bf(*shape, scale=1.0, dev="cuda"):
    return (torch.randn(*shape, device=dev) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("case", ["mla", "gqa"])
def test_noalloc_matches_regular_entry_point_twice(case):
    from metal_marlin_b200 import ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(11)
    lib = _lib()
    bs = 16
    if case == "mla":
        H, Hkv, R, dr, dvo = 20, 1, 512, 64, 256
        ctxs = [1, 100, 1500]
        dqk, dv = R + dr, R
        w_uv = _bf(H, dvo, R, scale=0.05)
        scale = 1.0 / math.sqrt(256)
    else:
        H, Hkv, dqk, dv, dvo = 32, 8, 128, 128, 128
        ctxs = [63, 700, 129, 1024]
        w_uv = None
        scale = dqk ** -0.5
    n_blocks = sum((c + bs - 1) // bs for c in ctxs) + 4
    bt, cl = _setup(ctxs, bs, n_blocks, dev)
    kp = _bf(n_blocks * bs, Hkv, dqk, scale=0.5)
    vp = None if case == "mla" else _bf(n_blocks * bs, Hkv, dv, scale=0.5)
    kp_arg = kp.view(n_blocks * bs, dqk) if case == "mla" else kp
    splits = 5
    for it in range(2):                            # two calls in a row reuse the same built-in scratch
        q = _bf(len(ctxs), H, dqk, scale=0.3)
        out = torch.full((len(ctxs), H, dvo), float("nan"), dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        reserved_before = torch.cuda.memory_reserved(dev)
        rc = _call(lib, q, kp, vp, bt, cl, w_uv, out, H, Hkv, dqk, dv, dvo, bs, splits, scale)
        assert rc == 0, (rc, lib.mmb_paged_attention_noalloc_error())
        torch.cuda.synchronize()
        if it == 1:     # the first call may make the driver load the module's kernels; the second must not move a byte
            assert torch.cuda.mem_get_info(dev)[0] >= free_before, "the entry point took device memory"
        assert torch.cuda.memory_reserved(dev) == reserved_before, "the entry point went through torch's allocator"
        o_reg = ops.paged_attention(q, kp_arg, vp, bt, cl, Hq=H, Hkv=Hkv, dqk=dqk, dv=dv, block_size=bs, scale=scale,
                                    splits=splits, w_uv=w_uv)
        with ops.force_reference():
            o_ref = ops.paged_attention(q, kp_arg, vp, bt, cl, Hq=H, Hkv=Hkv, dqk=dqk, dv=dv, block_size=bs, scale=scale,
                                        w_uv=w_uv)
        assert torch.isfinite(out.float()).all()
        # same kernels, same split count: the two entry points agree to the last bit
        assert torch.equal(out, o_reg.view_as(out)), (it, (out.float() - o_reg.float().view_as(out)).abs().max())
        torch.testing.assert_close(out.float(), o_ref.float().view_as(out), rtol=3e-2, atol=1e-2)


def test_noalloc_rejects_sizes_beyond_the_scratch():
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _lib()
    max_f, max_r = ctypes.c_longlong(0), ctypes.c_longlong(0)
    lib.mmb_paged_attention_noalloc_limits(ctypes.byref(max_f), ctypes.byref(max_r))
    assert max_f.value == 2 << 20 and max_r.value == 16 << 10
    # the size check comes before any launch or dereference: tiny placeholder tensors are enough
    t = torch.zeros(16, dtype=torch.int32, device=dev)
    rc = _call(lib, t, t, t, t.view(1, 16), torch.zeros(128, dtype=torch.int32, device=dev), None, t, 32, 8, 128, 128, 128, 16,
               16, 0.1)
    assert rc == -1, rc                            # 128 x 32 x 16 = 65536 rows > 16 Ki
    assert b"exceeds the scratch limit" in lib.mmb_paged_attention_noalloc_error()
    rc = _call(lib, t, t, t, t.view(1, 16), torch.zeros(40, dtype=torch.int32, device=dev), None, t, 20, 1, 576, 512, 512, 16,
               8, 0.1)
    assert rc == -1, rc                            # 40 x 20 x 8 x 512 floats > 2 Mi
    rc = _call(lib, t, t, t, t.view(1, 16), torch.zeros(1, dtype=torch.int32, device=dev), None, t, 4, 4, 64, 64, 32, 16, 1, 0.1)
    assert rc == -2, rc                            # dvo != dv without an up projection
    torch.cuda.synchronize()
