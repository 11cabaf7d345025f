"""Small fixed workloads for profiler captures: `python -m hesper_b200.profile_case <name>`.

Each case runs a handful of launches of one kernel on inputs larger than the L2 but well
under a few GB, so that a full-metric capture of one to three launches ends in a minute.
  q4k      ring of 12 Q4_K matrices K=2560 N=10240 (177 MB), 3 passes
  q80      ring of 8 Q8_0 matrices (223 MB), 3 passes
  i2s      ring of 40 ternary matrices K=2560 N=6912 (177 MB), 3 passes
  attn     decode attention B=16 L=4096, 8q/2kv heads, D=256 (268 MB of KV), 6 calls
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
