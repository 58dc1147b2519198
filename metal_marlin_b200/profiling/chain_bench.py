"""Cost of the persistent decode-chain kernel (``csrc/decode_chain.cu``) phase by phase: each phase alone, cumulative prefixes,
and the whole chain, on MoE layers of a layer-reduced GLM-4.7-Flash at batch ``B`` and context 4096.  Every variant is
captured ``reps`` times over four layers' weights (about 200 MB, more than L2 holds of one layer's reuse) in one CUDA graph
and timed with CUDA events; "empty" is the launch with no phase selected (cooperative launch + the barriers' fixed cost).

    python -m metal_marlin_b200.profiling.chain_bench [B]

The seven stand-alone kernels the chain replaces cost 46 us per layer in the same setting
(``python -m metal_marlin_b200.profiling.kernel_bench --chain 48``).
"""
import ctypes
import sys

import torch

from .. import ops
from ..models.config import get_preset
from ..models.mmfp4_causal_lm import MMFP4ForCausalLM
from ..models.transformer import BatchMeta
from ..ops.chain import DecodeChain, _Params


def main():
    dev = "cuda"
    cfg = get_preset("glm-4.7-flash")
    cfg.num_hidden_layers = 6
    lm = MMFP4ForCausalLM.from_config(cfg, device=dev, seed=0)
    m = lm.model
    B = int(sys.argv[1]) if len(sys.argv) > 1 else 1
    nb = 260
    kv = lm.new_cache(B * nb, 16)
    pos = torch.full((B,), 4096, dtype=torch.int32, device=dev)
    slots = torch.arange(B, dtype=torch.int64, device=dev) * nb * 16 + 4096
    bt = torch.arange(B * nb, dtype=torch.int32, device=dev).view(B, nb)
    ctx = torch.full((B,), 4097, dtype=torch.int32, device=dev)
    meta = BatchMeta(positions=pos, slots=slots, block_tables=bt, ctx_lens=ctx, decode=True, max_ctx=nb*16, splits=ops.default_splits(B,1,nb*16,mla_latent=True))
    ops.native_available()
    dc = DecodeChain(m)
    st = dc._build(B, kv, meta)
    for k in ("attn_o","delta_attn","delta_mlp","hmid","a","q"):
        st[k].normal_(0, 0.1)
    for h in st["h"]: h.normal_(0, 0.5)
    anchor = st["sync"]
    def variant(i, phases):
        raw = bytearray(st["descs"][i].numpy().tobytes())
        p = _Params.from_buffer(raw)
        p.phases = phases
        return torch.frombuffer(bytearray(bytes(p)), dtype=torch.uint8).clone()
    def timeit(descs, reps=20, iters=10):
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            for d in descs: ops.K.mmb200.decode_chain(d, anchor)
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=s):
                for _ in range(reps):
                    for d in descs: ops.K.mmb200.decode_chain(d, anchor)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g.replay(); torch.cuda.synchronize()
        e0.record()
        for _ in range(iters): g.replay()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1000 / (iters * reps * len(descs))
    names = {0:"empty",1:"A",2:"B",4:"C",8:"D",16:"E",32:"F",64:"G",3:"A+B",7:"A+B+C",15:"A..D",112:"E..G",127:"all"}
    # use layers 2..5 (MoE) descriptors in rotation so weights differ (no L2 reuse across reps beyond 4 layers ~200MB)
    for ph, nm in names.items():
        ds = [variant(i, ph) for i in (2,3,4,5)]
        t = timeit(ds)
        print(f"phases {nm:8s}: {t:7.2f} us per launch", flush=True)
    print("status", ops.check_status(dev))



if __name__ == "__main__":
    main()
