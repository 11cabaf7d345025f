"""CPU: pins the attention part of the oracle and checks every oracle family against the
committed golden vectors (tests/golden/golden.json, made by tests/golden/make_golden.py from
an independent numpy restatement on the reference's own fixture inputs)."""
import json
import os

import numpy as np
import pytest

from refcases import FLASH_ATTN_CASES, LITERAL_ATTN

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "golden.json")))


def test_literal_fixture_matches_golden(oracle):
    # Tests/FlashAttentionTest.lean:24-49 -- 2 heads, 3 positions, head_dim 4, scale 1/sqrt(4)
    for h in range(2):
        out = oracle.attention_head(LITERAL_ATTN["q"][h], np.array(LITERAL_ATTN["k"][h]),
                                    np.array(LITERAL_ATTN["v"][h]), 0.5)
        assert np.allclose(out, GOLD["attention_literal"]["scale_inv_sqrt_d"][h], rtol=0, atol=1e-14)


def test_flash_equivalence_as_reference(oracle):
    # verifyFlashEquivalence (Hesper/WGSL/FlashAttention.lean:93-112): online == three-step, tol 1e-4
    q = LITERAL_ATTN["q"][0]
    k, v = np.array(LITERAL_ATTN["k"][0]), np.array(LITERAL_ATTN["v"][0])
    a = oracle.attention_head(q, k, v, 0.5)
    b = oracle.attention_head(q, k, v, 0.5, online=True)
    err = np.max(np.abs(a - b) / (np.abs(a) + np.abs(b)))
    assert err < 1e-4 and err < 1e-12
    assert np.allclose(a, GOLD["attention_literal"]["flash_equivalence_head0_scale_0.5"], atol=1e-14)


@pytest.mark.parametrize("H,Hkv,D,max_seq,L,seed,window", FLASH_ATTN_CASES)
def test_reference_lcg_cases(oracle, H, Hkv, D, max_seq, L, seed, window):
    """Inputs of Tests/CUDA/CUDAFlashAttnGoldenTest.lean (LCG arrays chained q -> k -> v).
    The batched f16-cache oracle must agree with the per-head online spec (the reference's
    cpuFlashAttn) on the f16-rounded cache within the reference's own 1e-3."""
    q, s1 = oracle.lcg_fill(seed, H * D)
    k, s2 = oracle.lcg_fill(s1, Hkv * max_seq * D)
    v, _ = oracle.lcg_fill(s2, Hkv * max_seq * D)
    k16 = k.reshape(1, Hkv, max_seq, D).astype(np.float16)
    v16 = v.reshape(1, Hkv, max_seq, D).astype(np.float16)
    scale = 1.0 / np.sqrt(D)
    out = oracle.attn_decode(q.reshape(1, H, D), k16, v16, [L], H, Hkv, D, max_seq, scale, window)
    start = max(0, L - window) if window else 0
    for h in range(H):
        kvh = h // (H // Hkv)
        ref = oracle.attention_head(q.reshape(H, D)[h].astype(np.float64),
                                    k16[0, kvh, start:L].astype(np.float64),
                                    v16[0, kvh, start:L].astype(np.float64), scale, online=True)
        assert np.max(np.abs(out[0, h] - ref)) < 1e-6
        # and against the un-rounded f32 cache the reference test uses: inside its 1e-3
        ref32 = oracle.attention_head(q.reshape(H, D)[h].astype(np.float64),
                                      k.reshape(Hkv, max_seq, D)[kvh, start:L].astype(np.float64),
                                      v.reshape(Hkv, max_seq, D)[kvh, start:L].astype(np.float64),
                                      scale)
        assert np.max(np.abs(out[0, h] - ref32)) < 1e-3


def test_f16_conversion_rne(oracle):
    rng = np.random.default_rng(0)
    xs = np.concatenate([rng.standard_normal(2000) * 10.0 ** rng.integers(-8, 5, 2000),
                         [0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 6.1e-5]])
    for x in xs.astype(np.float32):
        with np.errstate(over="ignore"):
            exp = np.float32(x).astype(np.float16).view(np.uint16)
        assert oracle.f32_to_f16(float(x)) == int(exp)
    for h in list(range(0, 0x7C00, 37)) + [0x0001, 0x03FF, 0x0400, 0x7BFF, 0x8001, 0xFBFF]:
        assert oracle.f16_to_f32(h) == float(np.array([h], np.uint16).view(np.float16)[0])


def test_empty_and_window_edges(oracle):
    H, Hkv, D, max_seq = 4, 2, 64, 32
    rng = np.random.default_rng(1)
    q = rng.standard_normal((2, H, D)).astype(np.float32)
    k = rng.standard_normal((2, Hkv, max_seq, D)).astype(np.float16)
    v = rng.standard_normal((2, Hkv, max_seq, D)).astype(np.float16)
    out = oracle.attn_decode(q, k, v, [0, 1], H, Hkv, D, max_seq, 0.125)
    assert not out[0].any()  # no cached position: zeros
    for h in range(H):  # one position: output is that V row
        assert np.allclose(out[1, h], v[1, h // 2, 0].astype(np.float32), atol=1e-7)
    # window >= len is the same as no window
    a = oracle.attn_decode(q, k, v, [20, 7], H, Hkv, D, max_seq, 0.125, window=0)
    b = oracle.attn_decode(q, k, v, [20, 7], H, Hkv, D, max_seq, 0.125, window=20)
    assert np.array_equal(a, b)


def test_golden_q4k_and_bitlinear(oracle):
    g = GOLD["q4k_reference_block"]
    blk = np.frombuffer(bytes.fromhex(g["bytes_hex"]), np.uint8)
    x = np.sin(0.1 * np.arange(256)).astype(np.float32)
    got = oracle.q4k_matvec(blk, 256, 1, x)[0, 0]
    assert abs(got - g["dot"]) <= 2e-6 * abs(g["dot"])
    assert np.allclose(oracle.q4k_dequant(blk)[0][:8], g["w_first8"], rtol=1e-6)
    b = GOLD["bitlinear_tiny"]
    t, xx, scale = oracle.gen_bitlinear_case(0xDEADBEEF, 128, 16, 1)
    assert list(t[0, :16]) == b["ternary_first16"]
    assert abs(scale - b["scale"]) < 1e-8
    packed = oracle.i2s_pack(t)
    assert np.allclose(oracle.bitlinear_spec(packed, scale, 128, 16, xx)[0], b["spec_f64"], rtol=1e-6)
    y, acc, d = oracle.bitlinear_forward(packed, scale, 128, 16, xx)
    assert list(acc[0]) == b["acc_int8_contract"]
    assert float(d[0]) == b["d"]
    a = GOLD["all_plus_one"]
    yk = oracle.bitlinear_spec(np.full(a["K"] // 4, a["byte"], np.uint8), 1.0, a["K"], 1,
                               np.ones((1, a["K"]), np.float32))
    assert yk[0, 0] == a["y"]


def test_exact_order_mirror_agrees_with_definition(oracle):
    """The f32 fixed-order attention (mirror of the library's EXACT mode) stays within 1e-5
    of the f64 definition, so using it for whole-model parity does not change what is tested."""
    rng = np.random.default_rng(5)
    B, H, Hkv, D, L = 2, 8, 2, 128, 400
    q = rng.standard_normal((B, H, D)).astype(np.float32)
    k = rng.standard_normal((B, Hkv, L, D)).astype(np.float16)
    v = rng.standard_normal((B, Hkv, L, D)).astype(np.float16)
    for window in (0, 100):
        a = oracle.attn_decode(q, k, v, [L, 37], H, Hkv, D, L, 0.09, window)
        b = oracle.attn_decode_exact(q, k, v, [L, 37], H, Hkv, D, L, 0.09, window)
        assert np.max(np.abs(a - b)) < 1e-5 * np.max(np.abs(a))
