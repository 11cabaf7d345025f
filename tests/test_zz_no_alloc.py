"""GPU: the allocation-free decode-attention entry point (hb200_attn_decode_static).

Some hosts cannot give the library scratch memory when they call it -- they have pooled all
device memory themselves, or must not risk the device-wide stall of an allocation -- so this
entry point keeps its split-K partials in an array built into the library.  The test drives
it through the raw C ABI and checks it against the ordinary entry point and against the CPU
oracle, several calls in a row with different shapes, so every later call runs on top of the
earlier calls' leftovers in the shared array.  The shapes are chosen so that the partials
really go through that array (grids too large for the in-cluster merge, which keeps them in
shared memory), plus one shape of the in-cluster kind.  This file sorts last on purpose: a
run that stops at the first failure has then already executed every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2e-3  # the tolerance of the attention parity tests


def _splits(lib, ctx, B, H, Hkv, D, L):
    """Split count the library will use for this shape, from its workspace query."""
    nbytes = int(lib.hb200_attn_workspace_bytes(ctx.handle, B, H, Hkv, D, L))
    if nbytes <= 256:
        return 1
    return (nbytes - 256) // (B * Hkv * 8 * (D + 2) * 4)


def _call_pair(lib, ctx, oracle, B, H, Hkv, D, L, window, seed, check_oracle_rows):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, H, D, device="cuda", generator=g)
    k = torch.randn(B, Hkv, L, D, device="cuda", generator=g).half()
    v = torch.randn(B, Hkv, L, D, device="cuda", generator=g).half()
    lens = torch.randint(L // 2, L + 1, (B,), device="cuda", generator=g).to(torch.int32)
    scale = 1.0 / np.sqrt(D)
    p = lambda t: C.c_void_p(t.data_ptr())
    # reference result: the existing entry point with a caller-owned workspace
    nbytes = lib.hb200_attn_workspace_bytes(ctx.handle, B, H, Hkv, D, L)
    ws = torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device="cuda")
    ref = torch.empty(B, H, D, device="cuda")
    rc = lib.hb200_attn_decode(ctx.handle, p(q), 0, p(k), p(v), p(lens), B, H, Hkv, D, L, window,
                               C.c_float(scale), p(ws), C.c_size_t(ws.numel()), p(ref), None)
    assert rc == 0, lib.hb200_last_error()
    torch.cuda.synchronize()
    # the allocation-free entry point: inputs and output only.  Free device memory as the
    # driver reports it must not move across the call (torch's own counters would not see a
    # cudaMalloc made inside the library).
    out = torch.full((B, H, D), float("nan"), device="cuda")
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    rc = lib.hb200_attn_decode_static(ctx.handle, p(q), 0, p(k), p(v), p(lens), B, H, Hkv, D, L,
                                      window, C.c_float(scale), p(out), None)
    assert rc == 0, lib.hb200_last_error()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the allocation-free entry point changed free device memory"
    out, ref = out.cpu().numpy(), ref.cpu().numpy()
    assert np.isfinite(out).all()
    assert np.max(np.abs(out - ref)) <= TOL * np.max(np.abs(ref))
    # and against the CPU oracle on a few sequences (the f64 evaluation is slow)
    rows = check_oracle_rows
    want = oracle.attn_decode(q[rows].cpu().numpy(), k[rows].cpu().numpy(), v[rows].cpu().numpy(),
                              lens[rows].cpu().numpy(), H, Hkv, D, L, scale, window=window)
    assert np.max(np.abs(out[rows] - want)) <= TOL * np.max(np.abs(want))


def test_static_scratch_matches_workspace_entry_point_and_oracle(ctx, oracle):
    from hesper_b200 import _lib
    lib = _lib.load()
    sms = ctx.sm_count
    # 1: 32 (sequence, KV head) pairs x 10 splits -- too many CTAs for the in-cluster merge,
    #    so the partials travel through the built-in array
    B, H, Hkv, D, L = 16, 8, 2, 256, 4096
    ns = _splits(lib, ctx, B, H, Hkv, D, L)
    assert ns > 1 and B * Hkv * min(ns, 16) > 2 * sms
    _call_pair(lib, ctx, oracle, B, H, Hkv, D, L, 0, seed=1, check_oracle_rows=[0, 15])
    # 2: straight after, another shape of the same kind (80 pairs x 8 splits, D = 128, window)
    B, H, Hkv, D, L = 40, 8, 2, 128, 4096
    ns = _splits(lib, ctx, B, H, Hkv, D, L)
    assert ns > 1 and B * Hkv * min(ns, 16) > 2 * sms
    _call_pair(lib, ctx, oracle, B, H, Hkv, D, L, 3000, seed=2, check_oracle_rows=[1, 39])
    # 3: a small grid whose splits merge inside a cluster (the array is handed over, unused)
    _call_pair(lib, ctx, oracle, 4, 8, 2, 256, 6000, 0, seed=3, check_oracle_rows=[2])
    # 4: and the first shape again, now on top of everybody's leftovers
    _call_pair(lib, ctx, oracle, 16, 8, 2, 256, 4096, 0, seed=4, check_oracle_rows=[7])
    ctx.check()


def test_every_shape_fits_the_array(ctx):
    """The entry point refuses shapes whose split-K partials exceed its 8 MiB array.  With two
    waves of resident CTAs as the split target no supported shape does: check that over a
    sweep of shapes through the workspace query (no launch: a call that is expected to be
    refused must never be given buffers it could run on)."""
    from hesper_b200 import _lib
    lib = _lib.load()
    cap = 8 << 20
    worst = 0
    for D in (64, 128, 256):
        for G in (1, 4, 8):
            for Hkv in (1, 2, 5, 8, 16):
                for B in (1, 3, 16, 64, 256, 1024):
                    for max_seq in (128, 2304, 32768, 1 << 20):
                        n = int(lib.hb200_attn_workspace_bytes(ctx.handle, B, G * Hkv, Hkv, D, max_seq))
                        worst = max(worst, n)
    assert worst - 256 <= cap
