"""GPU: the allocation-free decode-attention entry point (hb200_attn_decode_static).

Some hosts cannot give the library scratch memory when they call it -- they have pooled all
device memory themselves, or must not risk the device-wide stall of an allocation -- so this
entry point keeps its split-K partials in an array built into the library.  The test drives
it through the raw C ABI and checks it against the ordinary entry point, twice in a row with
different shapes, so the second call runs on top of the first call's leftovers in the shared
array.  This file sorts last on purpose: a run that stops at the first failure has then
already executed every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2e-3  # the tolerance of the attention parity tests


def _call_pair(lib, ctx, B, H, Hkv, D, L, window, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, H, D, device="cuda", generator=g)
    k = torch.randn(B, Hkv, L, D, device="cuda", generator=g).half()
    v = torch.randn(B, Hkv, L, D, device="cuda", generator=g).half()
    lens = torch.randint(L // 2, L + 1, (B,), device="cuda", generator=g).to(torch.int32)
    scale = C.c_float(1.0 / np.sqrt(D))
    p = lambda t: C.c_void_p(t.data_ptr())
    # reference result: the existing entry point with a caller-owned workspace
    nbytes = lib.hb200_attn_workspace_bytes(ctx.handle, B, H, Hkv, D, L)
    ws = torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device="cuda")
    ref = torch.empty(B, H, D, device="cuda")
    rc = lib.hb200_attn_decode(ctx.handle, p(q), 0, p(k), p(v), p(lens), B, H, Hkv, D, L, window,
                               scale, p(ws), C.c_size_t(ws.numel()), p(ref), None)
    assert rc == 0, lib.hb200_last_error()
    # the allocation-free entry point: inputs and output only
    out = torch.full((B, H, D), float("nan"), device="cuda")
    rc = lib.hb200_attn_decode_static(ctx.handle, p(q), 0, p(k), p(v), p(lens), B, H, Hkv, D, L,
                                      window, scale, p(out), None)
    assert rc == 0, lib.hb200_last_error()
    torch.cuda.synchronize()
    return out.cpu().numpy(), ref.cpu().numpy()


def test_static_scratch_matches_workspace_entry_point_twice(ctx):
    from hesper_b200 import _lib
    lib = _lib.load()
    before = torch.cuda.memory_allocated()
    # first call: many splits, fills a large part of the shared array
    out, ref = _call_pair(lib, ctx, B=4, H=8, Hkv=2, D=256, L=6000, window=0, seed=1)
    assert np.isfinite(out).all()
    assert np.max(np.abs(out - ref)) <= TOL * np.max(np.abs(ref))
    # second call straight after: other shape, fewer partials, stale data all around them
    out2, ref2 = _call_pair(lib, ctx, B=3, H=20, Hkv=5, D=128, L=1500, window=700, seed=2)
    assert np.isfinite(out2).all()
    assert np.max(np.abs(out2 - ref2)) <= TOL * np.max(np.abs(ref2))
    ctx.check()
    assert torch.cuda.memory_allocated() <= before + (1 << 20)  # only the test's own tensors


def test_every_shape_fits_the_array(ctx):
    """The entry point refuses shapes whose split-K partials exceed its 8 MiB array.  With two
    waves of resident CTAs as the split target no supported shape does any more: check that
    over a sweep of shapes through the workspace query (no launch: a call that is expected to
    be refused must never be given buffers it could run on)."""
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
