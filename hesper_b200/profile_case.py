"""Small fixed workloads for profiler captures: `python -m hesper_b200.profile_case <name>`.

Each case runs a handful of launches of one kernel on inputs larger than the L2 but well
under a few GB, so that a full-metric capture of one to three launches ends in a minute.
  q4k      ring of 12 Q4_K matrices K=2560 N=10240 (177 MB), 3 passes
  q80      ring of 8 Q8_0 matrices (223 MB), 3 passes
  i2s      ring of 40 ternary matrices K=2560 N=6912 (177 MB), 3 passes
  attn     decode attention B=16 L=4096, 8q/2kv heads, D=256 (268 MB of KV), 6 calls
  i2s_mma  64-token ternary product on the tensor cores, ring of 40 matrices K=2560 N=6912
           (177 MB), 2 passes
  lmhead64 64-token LM head on the tensor cores, one bf16 table V=128256 K=2560 (657 MB), 3 calls
  q4k_b32  32-token Q4_K product on the tensor cores (dequantise to f16 + 16-bit product),
           ring of 12 matrices K=2560 N=10240, 2 passes
  bitnet1 / bitnet64   BitNet-2B-shaped decode loop at batch 1 / 64: 2 prompt positions and
           3 new tokens, launched one by one (no graph) so that a launch list sees each kernel
  gemma1 / gemma32 / gemma256   Gemma-4-E4B-shaped Q4_K decode loop (one rank) at batch 1 / 32 /
           256: 3 tokens at position 8000, launched one by one
"""
from __future__ import annotations

import sys

import numpy as np
import torch

import hesper_b200 as hb
from hesper_b200 import formats


def main(name: str) -> None:
    ctx = hb.Context(0)
    rng = np.random.default_rng(0)
    if name in ("q4k", "q80"):
        fmt, R = (12, 12) if name == "q4k" else (8, 8)
        K, N = 2560, 10240
        base = torch.from_numpy(formats.random_kquant(rng, fmt, N, K)).cuda()
        rb = formats.kquant_row_bytes(fmt, K)
        layers = [hb.LinearLayer(ctx, torch.roll(base, r * rb), fmt, K, N) for r in range(R)]
        x = torch.randn(1, K, device="cuda")
        y = torch.empty(1, N, device="cuda")
        torch.cuda.synchronize()
        for _ in range(3):
            for l in layers:
                l.forward(x, out=y)
    elif name == "i2s":
        K, N, R = 2560, 6912, 40
        base = torch.from_numpy(formats.i2s_pack(formats.random_ternary(rng, N, K))).cuda()
        sc = torch.tensor([0.05], device="cuda")
        layers = [hb.BitLinear(ctx, torch.roll(base, r * 640), sc, K, N) for r in range(R)]
        x = torch.randn(1, K, device="cuda")
        y = torch.empty(1, N, device="cuda")
        torch.cuda.synchronize()
        for _ in range(3):
            for l in layers:
                l.forward(x, out=y)
    elif name == "q4k_b32":
        K, N, R, M = 2560, 10240, 12, 32
        base = torch.from_numpy(formats.random_kquant(rng, 12, N, K)).cuda()
        rb = formats.kquant_row_bytes(12, K)
        layers = [hb.LinearLayer(ctx, torch.roll(base, r * rb), 12, K, N) for r in range(R)]
        x = torch.randn(M, K, device="cuda")
        y = torch.empty(M, N, device="cuda")
        torch.cuda.synchronize()
        for _ in range(2):
            for l in layers:
                l.forward(x, out=y)
    elif name == "i2s_mma":
        K, N, R, M = 2560, 6912, 40, 64
        base = torch.from_numpy(formats.i2s_pack(formats.random_ternary(rng, N, K))).cuda()
        sc = torch.tensor([0.05], device="cuda")
        layers = [hb.BitLinear(ctx, torch.roll(base, r * 640), sc, K, N) for r in range(R)]
        x = torch.randn(M, K, device="cuda")
        y = torch.empty(M, N, device="cuda")
        torch.cuda.synchronize()
        for _ in range(2):
            for l in layers:
                l.forward(x, out=y)
    elif name == "lmhead64":
        from hesper_b200 import _lib
        lib = _lib.load()
        V, K, M = 128256, 2560, 64
        table = (torch.randn(V, K, device="cuda") * 0.02).to(torch.bfloat16)
        x = torch.randn(M, K, device="cuda")
        arg = torch.zeros(M, dtype=torch.int32, device="cuda")
        scr = torch.zeros(M, dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        for _ in range(3):
            rc = lib.hb200_lmhead_argmax(ctx.handle, table.data_ptr(), 0, V, K, x.data_ptr(), M,
                                         None, 0.0, None, arg.data_ptr(), scr.data_ptr(), None,
                                         None, 0, None)
            assert rc == 0
    elif name in ("bitnet1", "bitnet64"):
        from hesper_b200.models import BitNetModel, BitNetShape, random_bitnet_weights_device
        B = 1 if name == "bitnet1" else 64
        shape = BitNetShape.bitnet_2b(max_seq=2304)
        w = random_bitnet_weights_device(shape)
        m = BitNetModel(ctx, shape, w, batch=B, max_new_tokens=8)
        prompt = rng.integers(0, shape.vocab, (B, 2)).astype(np.int32)
        m.generate(prompt, 3, use_graph=False)
        m.close()
    elif name in ("gemma1", "gemma32", "gemma256"):
        from hesper_b200 import tp
        B = int(name[5:])
        S = tp.GemmaShape()
        plan = tp.plan(S, 0, 1)
        shard = tp.random_gemma_shard_device(S, plan, seed=7)
        m = tp.GemmaModel(ctx, S, shard, plan, None, batch=B, max_new_tokens=8)
        m.set_position(8000)
        m.generate(None, 3, use_graph=False)
        m.close()
    elif name == "attn":
        B, H, Hkv, D, L = 16, 8, 2, 256, 4096
        q = torch.randn(B, H, D, device="cuda").half()
        k = torch.randn(B, Hkv, L, D, device="cuda").half()
        v = torch.randn(B, Hkv, L, D, device="cuda").half()
        lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
        ws = hb.flash_attention_workspace(ctx, B, H, Hkv, D, L)
        torch.cuda.synchronize()
        for _ in range(6):
            hb.execute_flash_attention_v11(ctx, q, k, v, lens, num_heads=H, num_kv_heads=Hkv,
                                           head_dim=D, max_seq_len=L, scale=1 / 16, workspace=ws)
    else:
        raise SystemExit(f"unknown case {name}")
    torch.cuda.synchronize()
    ctx.check()
    print("ok")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "q4k")
