"""GPU parity: causal prefill attention and the prefill RoPE + KV writer through the C ABI.
A prefill token is a decode query with its own visible length, so the oracle is the decode
oracle evaluated token by token (f64, bar 2e-3 as for decode attention); in EXACT mode the
result must be bit-identical to the oracle's mirror, and the prefill KV writer must leave
exactly the bytes that T single-token calls leave."""
import ctypes as C

import numpy as np
import pytest
import torch

from hesper_b200 import _lib, flash_attention_prefill

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _reference(oracle_fn, q, k16, v16, lens, T, H, Hkv, D, max_seq, scale, window):
    B = q.shape[0]
    out = np.empty((B, T, H, D), np.float32)
    for b in range(B):
        for t in range(T):
            vis = max(int(lens[b]) - (T - 1 - t), 0)
            out[b, t] = oracle_fn(q[b, t][None], k16[b:b + 1], v16[b:b + 1], [vis], H, Hkv, D,
                                  max_seq, scale, window)[0]
    return out


@pytest.mark.parametrize("H,Hkv,D,max_seq,T,lens,window", [
    (8, 2, 64, 96, 5, [5, 37], 0),          # first chunk of a prompt (len == T) and a later one
    (20, 5, 128, 300, 33, [33, 290], 0),    # BitNet head shape, chunk crosses split boundaries
    (8, 2, 256, 700, 16, [700, 16], 0),     # Gemma head shape
    (8, 2, 64, 400, 24, [400, 100], 64),    # sliding window on a linear cache
    (4, 4, 64, 64, 64, [64], 0),            # whole prompt at once, no GQA
])
def test_prefill_matches_tokenwise_oracle(ctx, oracle, H, Hkv, D, max_seq, T, lens, window):
    B = len(lens)
    rng = np.random.default_rng(H * D + T)
    q = rng.standard_normal((B, T, H, D)).astype(np.float32)
    k16 = rng.standard_normal((B, Hkv, max_seq, D)).astype(np.float16)
    v16 = rng.standard_normal((B, Hkv, max_seq, D)).astype(np.float16)
    scale = float(1.0 / np.sqrt(D))
    sl = np.asarray(lens, np.int32)
    ctx.set_attn_mode(ctx.ATTN_FAST)
    out = flash_attention_prefill(ctx, _dev(q), _dev(k16), _dev(v16), _dev(sl), num_heads=H,
                                  num_kv_heads=Hkv, head_dim=D, max_seq_len=max_seq, scale=scale,
                                  window=window).cpu().numpy()
    ctx.check()
    ref = _reference(oracle.attn_decode, q, k16, v16, sl, T, H, Hkv, D, max_seq, scale, window)
    s = np.abs(ref).max()
    assert np.abs(out - ref).max() / s <= TOL
    assert np.linalg.norm(out - ref) / np.linalg.norm(ref) <= TOL
    try:
        ctx.set_attn_mode(ctx.ATTN_EXACT)
        ex = flash_attention_prefill(ctx, _dev(q), _dev(k16), _dev(v16), _dev(sl), num_heads=H,
                                     num_kv_heads=Hkv, head_dim=D, max_seq_len=max_seq,
                                     scale=scale, window=window).cpu().numpy()
        ctx.check()
    finally:
        ctx.set_attn_mode(ctx.ATTN_FAST)
    ref_ex = _reference(oracle.attn_decode_exact, q, k16, v16, sl, T, H, Hkv, D, max_seq, scale,
                        window)
    assert np.array_equal(ex, ref_ex)


def test_prefill_kv_writer_equals_single_token_calls(ctx):
    lib = _lib.load()
    B, T, H, Hkv, D, slots, base = 2, 7, 8, 2, 64, 40, 500000.0
    rng = np.random.default_rng(3)
    q = rng.standard_normal((B, T, H, D)).astype(np.float32)
    k = rng.standard_normal((B, T, Hkv, D)).astype(np.float32)
    v = rng.standard_normal((B, T, Hkv, D)).astype(np.float32)
    pos0 = np.asarray([0, 21], np.int32)
    # chunk call
    dq, dk, dv, dp = _dev(q), _dev(k), _dev(v), _dev(pos0)  # keep the device copies alive
    kc = torch.zeros((B, Hkv, slots, D), dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    rc = lib.hb200_rope_kv_write_prefill(ctx.handle, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                         kc.data_ptr(), vc.data_ptr(), dp.data_ptr(), B, T, H,
                                         Hkv, D, slots, C.c_float(base), None)
    assert rc == 0, lib.hb200_last_error().decode()
    # token by token
    kc1 = torch.zeros_like(kc)
    vc1 = torch.zeros_like(kc)
    q1 = np.empty_like(q)
    for t in range(T):
        dqt, dkt, dvt, dpt = _dev(q[:, t]), _dev(k[:, t]), _dev(v[:, t]), _dev(pos0 + t)
        rc = lib.hb200_rope_kv_write(ctx.handle, dqt.data_ptr(), dkt.data_ptr(), dvt.data_ptr(),
                                     kc1.data_ptr(), vc1.data_ptr(), dpt.data_ptr(), B, H, Hkv, D,
                                     slots, 0, C.c_float(base), None)
        assert rc == 0
        torch.cuda.synchronize()
        q1[:, t] = dqt.cpu().numpy()
    ctx.check()
    assert torch.equal(kc, kc1) and torch.equal(vc, vc1)
    assert np.array_equal(dq.cpu().numpy(), q1)
