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
    (8, 1, 128, 260, 70, [260, 75], 0),     # 8 query heads per KV head, ragged last query tile
    (4, 2, 256, 300, 40, [300, 41], 100),   # head_dim 256 (32-position tiles) with a window
    (8, 2, 64, 128, 8, [128, 9], 0),        # the shortest chunk the tiled kernel takes
    (8, 2, 256, 4096, 128, [4096], 0),      # one sequence, long context: K/V range split 8 ways
    (20, 5, 128, 4096, 64, [3000], 0),      # the same at the BitNet head shape
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


@pytest.mark.parametrize("H,Hkv,D,slots,T,lens,window,q16", [
    (8, 2, 128, 80, 17, [200, 33], 64, False),   # ring wraps; second sequence has not wrapped yet
    (8, 2, 256, 767, 256, [8000, 700], 512, False),  # the Gemma engine's prompt pass
    (4, 2, 64, 40, 3, [90, 50], 38, True),       # short chunk: one decode query per token
    (4, 1, 64, 64, 33, [100, 64], 32, True),     # f16 queries
])
def test_ring_cache_prefill_matches_oracle(ctx, oracle, H, Hkv, D, slots, T, lens, window, q16):
    """hb200_attn_ring: the cache is a ring of `slots`, position p in slot p % slots, lengths
    beyond the ring; the oracle sees the same K/V on a linear cache with the window."""
    lib = _lib.load()
    B = len(lens)
    L = max(lens)
    rng = np.random.default_rng(D + T + slots)
    q = rng.standard_normal((B, T, H, D)).astype(np.float32)
    if q16:
        q = q.astype(np.float16).astype(np.float32)
    k_lin = rng.standard_normal((B, Hkv, L, D)).astype(np.float16)
    v_lin = rng.standard_normal((B, Hkv, L, D)).astype(np.float16)
    k_ring = np.zeros((B, Hkv, slots, D), np.float16)
    v_ring = np.zeros((B, Hkv, slots, D), np.float16)
    for b in range(B):  # what the ring holds after lens[b] positions: the last `slots` of them
        for pos in range(max(0, lens[b] - slots), lens[b]):
            k_ring[b, :, pos % slots] = k_lin[b, :, pos]
            v_ring[b, :, pos % slots] = v_lin[b, :, pos]
    scale = float(1.0 / np.sqrt(D))
    sl = np.asarray(lens, np.int32)
    dq = _dev(q.astype(np.float16) if q16 else q)
    dk, dv, dl = _dev(k_ring), _dev(v_ring), _dev(sl)
    nws = int(lib.hb200_attn_prefill_workspace_bytes(ctx.handle, B, T, H, Hkv, D, slots))
    ws = torch.empty(max(nws, 16), dtype=torch.uint8, device="cuda")
    out = torch.empty((B, T, H, D), dtype=torch.float32, device="cuda")
    rc = lib.hb200_attn_ring(ctx.handle, dq.data_ptr(), int(q16), dk.data_ptr(), dv.data_ptr(),
                             dl.data_ptr(), B, T, H, Hkv, D, slots, window, C.c_float(scale),
                             ws.data_ptr(), C.c_size_t(ws.numel()), out.data_ptr(), None)
    assert rc == 0, lib.hb200_last_error()
    ctx.check()
    ref = _reference(oracle.attn_decode, q, k_lin, v_lin, sl, T, H, Hkv, D, L, scale, window)
    out = out.cpu().numpy()
    assert np.abs(out - ref).max() / np.abs(ref).max() <= TOL
    assert np.linalg.norm(out - ref) / np.linalg.norm(ref) <= TOL


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
