"""CPU: pins the Q4_K / Q8_0 part of the oracle against an independent numpy
restatement of the block formats and against the one Q4_K block the reference's
own test builds (Tests/CUDA/CUDADP4ATest.lean:77-145,171-175)."""
import numpy as np
import pytest

from hesper_b200 import formats


def np_q4k_dequant(blocks: np.ndarray) -> np.ndarray:
    """Independent restatement of Hesper/Quantization/Q4_K_M.lean:13-52,120-144 in float64."""
    b = blocks.reshape(-1, 144)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float64)[:, 0]
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float64)[:, 0]
    s = b[:, 4:16].astype(np.int64)
    sc = np.empty((b.shape[0], 8), np.int64)
    m = np.empty((b.shape[0], 8), np.int64)
    for j in range(8):
        if j < 4:
            sc[:, j] = s[:, j] & 63
            m[:, j] = s[:, j + 4] & 63
        else:
            sc[:, j] = (s[:, j + 4] & 0xF) | ((s[:, j - 4] >> 6) << 4)
            m[:, j] = (s[:, j + 4] >> 4) | ((s[:, j] >> 6) << 4)
    qs = b[:, 16:].astype(np.int64).reshape(-1, 4, 32)
    out = np.empty((b.shape[0], 256), np.float64)
    for c in range(4):
        out[:, 64 * c:64 * c + 32] = d[:, None] * sc[:, 2 * c, None] * (qs[:, c] & 0xF) - dmin[:, None] * m[:, 2 * c, None]
        out[:, 64 * c + 32:64 * c + 64] = d[:, None] * sc[:, 2 * c + 1, None] * (qs[:, c] >> 4) - dmin[:, None] * m[:, 2 * c + 1, None]
    return out


def np_q80_dequant(blocks: np.ndarray) -> np.ndarray:
    b = blocks.reshape(-1, 34)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float64)[:, 0]
    q = b[:, 2:].copy().view(np.int8).astype(np.float64)
    return d[:, None] * q


def reference_q4k_block(seed: int = 42) -> np.ndarray:
    """The block genQ4KBlock builds in Tests/CUDA/CUDADP4ATest.lean:95-145."""
    words = np.empty(36, np.uint32)
    words[0] = 0x211F | (0x1D1F << 16)
    sc = list(range(10, 18))
    m = list(range(1, 9))
    words[1] = sc[0] | (sc[1] << 8) | (sc[2] << 16) | (sc[3] << 24)
    words[2] = m[0] | (m[1] << 8) | (m[2] << 16) | (m[3] << 24)
    w3 = 0
    for i in range(4):
        w3 |= ((sc[4 + i] & 0xF) | ((m[4 + i] & 0xF) << 4)) << (8 * i)
    words[3] = w3
    for i in range(32):
        s1 = ((seed + i) * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        words[4 + i] = s1 & 0xFFFFFFFF
    return words.view(np.uint8).copy()


def test_scale_min_unpack_matches_pack(oracle):
    rng = np.random.default_rng(0)
    sc = rng.integers(0, 64, (50, 8))
    m = rng.integers(0, 64, (50, 8))
    packed = formats.q4k_pack_scales(sc, m)
    import ctypes as C
    L = oracle.lib()
    for i in range(50):
        for j in range(8):
            a, b = C.c_int(), C.c_int()
            L.orc_q4k_scale_min(packed[i].ctypes.data_as(C.c_void_p), j, C.byref(a), C.byref(b))
            assert (a.value, b.value) == (sc[i, j], m[i, j])


def test_q4k_dequant_matches_numpy(oracle):
    rng = np.random.default_rng(1)
    blocks = formats.random_q4k(rng, 6, 512)
    got = oracle.q4k_dequant(blocks)
    exp = np_q4k_dequant(blocks)
    assert np.max(np.abs(got - exp)) < 2e-7 * np.max(np.abs(exp)) + 1e-9


def test_q4k_known_values():
    # hand-checkable block: d = 1, dmin = 0.5, sc_j = j + 1, m_j = j, q = element index % 16
    q = (np.arange(256) % 16)[None, :]
    blk = formats.q4k_build([1.0], [0.5], np.arange(1, 9)[None, :], np.arange(8)[None, :], q)
    w = np_q4k_dequant(blk)[0]
    for i in (0, 31, 32, 100, 255):
        j = i // 32
        assert w[i] == 1.0 * (j + 1) * (i % 16) - 0.5 * j


def test_reference_q4k_block_fixture(oracle):
    blk = reference_q4k_block(42)
    x = np.sin(0.1 * np.arange(256)).astype(np.float32)
    exp = float(np_q4k_dequant(blk)[0] @ x.astype(np.float64))
    got = oracle.q4k_matvec(blk, 256, 1, x)[0, 0]
    assert abs(got - exp) <= 1e-6 * max(1.0, abs(exp))
    # sc = 10..17 and m = 1..8 must come back out of the packed bytes
    w = oracle.q4k_dequant(blk)[0]
    d = np.float32(np.array([0x211F], np.uint16).view(np.float16)[0])
    dmin = np.float32(np.array([0x1D1F], np.uint16).view(np.float16)[0])
    q0 = blk[16] & 0xF
    assert w[0] == np.float32(d * np.float32(10)) * np.float32(q0) - np.float32(dmin * np.float32(1))


@pytest.mark.parametrize("fmt", [12, 8])
def test_matvec_matches_numpy(oracle, fmt):
    rng = np.random.default_rng(fmt)
    K, N, M = 512, 9, 3
    blocks = formats.random_kquant(rng, fmt, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    W = (np_q4k_dequant(blocks) if fmt == 12 else np_q80_dequant(blocks)).reshape(N, K)
    exp = x.astype(np.float64) @ W.T + res
    got = oracle.kquant_matvec(fmt, blocks, K, N, x, residual=res)
    assert np.max(np.abs(got - exp)) <= 2e-6 * np.max(np.abs(exp))


def test_gateup_gelu(oracle):
    rng = np.random.default_rng(3)
    K, N = 256, 5
    bg, bu = formats.random_q4k(rng, N, K), formats.random_q4k(rng, N, K)
    x = rng.standard_normal((1, K)).astype(np.float32)
    g = oracle.q4k_matvec(bg, K, N, x).astype(np.float64)
    u = oracle.q4k_matvec(bu, K, N, x).astype(np.float64)
    exp = 0.5 * g * (1 + np.tanh(np.sqrt(2 / np.pi) * (g + 0.044715 * g ** 3))) * u
    got = oracle.kquant_gateup_gelu(bg, bu, 12, K, N, x)
    assert np.allclose(got, exp, rtol=1e-6, atol=1e-7)
    # FusedFFNSpec: gelu(0) = 0, gelu(large) ~ identity
    assert oracle.gelu_tanh(0.0) == 0.0 and abs(oracle.gelu_tanh(10.0) - 10.0) < 1e-9


def test_q80_alignment_of_blocks():
    blk = formats.q80_build([0.5, 2.0], np.array([[1] * 32, [-3] * 32], np.int8))
    assert blk.shape == (2, 34)
    w = np_q80_dequant(blk)
    assert np.all(w[0] == 0.5) and np.all(w[1] == -6.0)
