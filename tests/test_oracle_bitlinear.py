"""CPU: pins the BitLinear part of the oracle against the reference's own
known-answer tests and test generators (no GPU, no CUDA library calls)."""
import numpy as np
import pytest

from hesper_b200 import formats
from refcases import BITLINEAR_CASES


def test_code_table(oracle):
    # Hesper/Layers/BitLinear.lean:25-32: -1/0/+1 <-> codes 00/01/10
    t = np.zeros((1, 128), np.int8)
    t[0, 0], t[0, 1], t[0, 2] = -1, 0, 1
    p = oracle.i2s_pack(t)
    assert (p[0] >> 6) & 3 == 0 and (p[1] >> 6) & 3 == 1 and (p[2] >> 6) & 3 == 2
    # element 32+j sits in bits 5:4 of byte j, 64+j in 3:2, 96+j in 1:0
    t[:] = 0
    t[0, 32], t[0, 64], t[0, 96] = 1, -1, 1
    p = oracle.i2s_pack(t)
    assert p[0] == (1 << 6) | (2 << 4) | (0 << 2) | 2


def test_all_plus_one_kat(oracle):
    # Tests/CUDA/CUDABitLinearTest.lean:57-71: weights 0xAA, x = 1, s = 1 -> y = K
    for K, N in [(128, 4), (2560, 3)]:
        packed = np.full(N * K // 4, 0xAA, np.uint8)
        y = oracle.bitlinear_spec(packed, 1.0, K, N, np.ones((1, K), np.float32))
        assert np.all(y == float(K))
        yq, acc, d = oracle.bitlinear_forward(packed, 1.0, K, N, np.ones((1, K), np.float32))
        assert np.all(acc == 127 * K)
        assert np.allclose(yq, K, rtol=1e-6)


def test_pack_roundtrip_and_numpy_agree(oracle):
    rng = np.random.default_rng(0)
    t = formats.random_ternary(rng, 24, 384)
    p_c = oracle.i2s_pack(t)
    p_np = formats.i2s_pack(t)
    assert np.array_equal(p_c, p_np)
    assert np.array_equal(formats.i2s_unpack(p_np, 384, 24), t)
    assert np.array_equal(oracle.i2s_decode_all(p_c[: 4 * 96], 384, 4), t[:4])


def test_xorshift_generator_first_values(oracle):
    # xorshift32 from seed 0xDEADBEEF, computed by hand: x^=x<<13; x^=x>>17; x^=x<<5
    def step(x):
        x ^= (x << 13) & 0xFFFFFFFF
        x ^= x >> 17
        x ^= (x << 5) & 0xFFFFFFFF
        return x
    s = 0xDEADBEEF
    exp = []
    for _ in range(5):
        s = step(s)
        exp.append(s % 3 - 1)
    t, x, scale = oracle.gen_bitlinear_case(0xDEADBEEF, 128, 16, 1)
    assert list(t.reshape(-1)[:5]) == exp
    assert 0.01 <= scale < 0.11
    assert np.all(np.abs(x) <= 1.0)


@pytest.mark.parametrize("name,K,N,M,seed", BITLINEAR_CASES, ids=[c[0] for c in BITLINEAR_CASES])
def test_int8_contract_within_reference_tolerance(oracle, name, K, N, M, seed):
    """The int8-activation contract stays inside the tolerance the reference's own
    equivalence harness accepts for a kernel (Tests/BitLinearEquivalence.lean:187-201:
    maxAbs/rms(spec) < 5e-2 and cosine > 0.999)."""
    t, x, scale = oracle.gen_bitlinear_case(seed, K, N, M)
    packed = oracle.i2s_pack(t)
    spec = oracle.bitlinear_spec(packed, scale, K, N, x)
    y, acc, d = oracle.bitlinear_forward(packed, scale, K, N, x)
    rms = np.sqrt(np.mean(spec ** 2))
    assert np.max(np.abs(y - spec)) / rms < 5e-2
    cos = np.sum(y * spec) / (np.linalg.norm(y) * np.linalg.norm(spec))
    assert cos > 0.999
    # exact integer identity: the spec run on the int8 activations with scale 1
    for m in range(min(M, 2)):
        q, dm = oracle.quant_act_i8(x[m])
        assert dm == d[m]
        spec_int = oracle.bitlinear_spec(packed, 1.0, K, N, q.astype(np.float32)[None, :])
        assert np.array_equal(spec_int[0].astype(np.int64), acc[m].astype(np.int64))
        # independent numpy restatement of the integer sum
        assert np.array_equal(t.astype(np.int32) @ q.astype(np.int32), acc[m])


def test_quantiser_rule(oracle):
    # Tests/CUDA/CUDAQuantizeTest.lean:70-73: x[i] = 0.1*i, K = 32 -> d = 3.1/127,
    # q[0] = 0, q[31] = 127 (print-only in the reference; asserted here)
    x = (0.1 * np.arange(32)).astype(np.float32)
    q, d = oracle.quant_act_i8(x)
    assert q[0] == 0 and q[31] == 127
    assert d == np.float32(x[31]) / np.float32(127.0)
    # ties round to even; zero vector gives zeros
    q0, d0 = oracle.quant_act_i8(np.zeros(128, np.float32))
    assert d0 == 0 and not q0.any()
    xt = np.array([127.0, 0.5, 1.5, 2.5, -0.5, -1.5], np.float32)  # d = 1
    qt, dt = oracle.quant_act_i8(xt)
    assert dt == 1.0 and list(qt) == [127, 0, 2, 2, 0, -2]


def test_rmsnorm_f32_contract_close_to_spec(oracle):
    rng = np.random.default_rng(1)
    x = rng.standard_normal(2560).astype(np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(2560)).astype(np.float32)
    a = oracle.rmsnorm_f64(x, g, 1e-5)
    b = oracle.rmsnorm_f32(x, g, 1e-5)
    assert np.max(np.abs(a - b)) < 1e-6 * np.max(np.abs(a)) * 4


def test_gateup_relu2(oracle):
    rng = np.random.default_rng(2)
    K, N = 256, 24
    tg, tu = formats.random_ternary(rng, N, K), formats.random_ternary(rng, N, K)
    x = rng.standard_normal((1, K)).astype(np.float32)
    y = oracle.bitlinear_gateup_relu2(formats.i2s_pack(tg), 0.05, formats.i2s_pack(tu), 0.03, K, N, x)
    g, _, _ = oracle.bitlinear_forward(formats.i2s_pack(tg), 0.05, K, N, x)
    u, _, _ = oracle.bitlinear_forward(formats.i2s_pack(tu), 0.03, K, N, x)
    assert np.array_equal(y, (np.maximum(g, 0) ** 2 * u).astype(np.float32))
