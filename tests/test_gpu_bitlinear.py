"""GPU parity: ternary x int8 BitLinear through the C ABI vs the CPU oracle.
Bar: bit-exact int32 accumulators and bit-exact f32 outputs."""
import numpy as np
import pytest
import torch

from hesper_b200 import BitLinear, formats
from refcases import BITLINEAR_CASES

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("name,K,N,M,seed", BITLINEAR_CASES, ids=[c[0] for c in BITLINEAR_CASES])
def test_reference_equivalence_cases(ctx, oracle, name, K, N, M, seed):
    t, x, scale = oracle.gen_bitlinear_case(seed, K, N, M)
    packed = oracle.i2s_pack(t)
    y_ref, acc_ref, d_ref = oracle.bitlinear_forward(packed, scale, K, N, x)
    layer = BitLinear.create_from_bytes(ctx, packed, scale, K, N)
    y, acc, d = layer.forward(_dev(x), return_acc=True)
    ctx.check()
    assert np.array_equal(acc.cpu().numpy(), acc_ref)
    assert np.array_equal(d.cpu().numpy(), d_ref)
    assert np.array_equal(y.cpu().numpy(), y_ref)
    # and inside the reference's own acceptance band against the f32 spec
    spec = oracle.bitlinear_spec(packed, scale, K, N, x)
    rms = np.sqrt(np.mean(spec ** 2))
    assert np.max(np.abs(y.cpu().numpy() - spec)) / rms < 5e-2


def test_all_plus_one_kat(ctx):
    # Tests/CUDA/CUDABitLinearTest.lean:57-71
    K, N = 128, 8
    layer = BitLinear.create_from_bytes(ctx, np.full(N * K // 4, 0xAA, np.uint8), 1.0, K, N)
    y, acc, d = layer.forward(torch.ones(1, K, device="cuda"), return_acc=True)
    assert torch.all(acc == 127 * K)
    assert torch.allclose(y, torch.full_like(y, float(K)), rtol=1e-6)


@pytest.mark.parametrize("K,N", [(2560, 6912), (6912, 2560), (2560, 2560), (2560, 640),
                                 (128, 1), (384, 7), (2048, 33), (4096, 1000), (8192, 257)])
def test_layer_shapes_bit_exact(ctx, oracle, K, N):
    rng = np.random.default_rng(K * 7 + N)
    packed = formats.i2s_pack(formats.random_ternary(rng, N, K))
    scale = float(rng.uniform(0.01, 0.1))
    x = rng.standard_normal((1, K)).astype(np.float32)
    y_ref, acc_ref, d_ref = oracle.bitlinear_forward(packed, scale, K, N, x)
    layer = BitLinear.create_from_bytes(ctx, packed, scale, K, N)
    y, acc, d = layer.forward(_dev(x), return_acc=True)
    ctx.check()
    assert np.array_equal(acc.cpu().numpy(), acc_ref)
    assert np.array_equal(y.cpu().numpy(), y_ref)


@pytest.mark.parametrize("M", [1, 3, 4, 5, 16, 64])
def test_residual_and_rmsnorm_prologue(ctx, oracle, M):
    K, N = 2560, 320
    rng = np.random.default_rng(100 + M)
    packed = formats.i2s_pack(formats.random_ternary(rng, N, K))
    scale = 0.037
    x = rng.standard_normal((M, K)).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    layer = BitLinear.create_from_bytes(ctx, packed, scale, K, N)
    # residual only
    y_ref, acc_ref, _ = oracle.bitlinear_forward(packed, scale, K, N, x, residual=res)
    y, acc, _ = layer.forward_with_residual(_dev(x), _dev(res), return_acc=True)
    assert np.array_equal(acc.cpu().numpy(), acc_ref)
    assert np.array_equal(y.cpu().numpy(), y_ref)
    # RMSNorm prologue + residual
    y_ref, acc_ref, d_ref = oracle.bitlinear_forward(packed, scale, K, N, x, gamma=gamma, eps=1e-5,
                                                     residual=res)
    y, acc, d = layer.forward_fused_rmsnorm_residual(_dev(x), _dev(gamma), _dev(res), eps=1e-5,
                                                     return_acc=True)
    ctx.check()
    assert np.array_equal(d.cpu().numpy(), d_ref)
    assert np.array_equal(acc.cpu().numpy(), acc_ref)
    assert np.array_equal(y.cpu().numpy(), y_ref)


@pytest.mark.parametrize("K,N,M", [(2560, 6912, 1), (256, 5, 1), (2560, 100, 3), (1024, 64, 8),
                                   (2560, 300, 32), (2560, 6912, 64), (6912, 130, 17),
                                   (2560, 6912, 128), (2560, 6912, 200), (1024, 700, 100)])
def test_gate_up_relu2(ctx, oracle, K, N, M):
    rng = np.random.default_rng(K + N + M)
    pg = formats.i2s_pack(formats.random_ternary(rng, N, K))
    pu = formats.i2s_pack(formats.random_ternary(rng, N, K))
    x = rng.standard_normal((M, K)).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    g = BitLinear.create_from_bytes(ctx, pg, 0.05, K, N)
    u = BitLinear.create_from_bytes(ctx, pu, 0.03, K, N)
    for gm in (None, gamma):
        y_ref = oracle.bitlinear_gateup_relu2(pg, 0.05, pu, 0.03, K, N, x, gamma=gm)
        y = BitLinear.forward_fused_gate_up_relu_sqr_mul(
            g, u, _dev(x), rms_gamma=None if gm is None else _dev(gm))
        ctx.check()
        assert np.array_equal(y.cpu().numpy(), y_ref)


def test_fused_qkv_multi(ctx, oracle):
    K = 2560
    rng = np.random.default_rng(5)
    shapes = [2560, 640, 640]
    packs = [formats.i2s_pack(formats.random_ternary(rng, n, K)) for n in shapes]
    scales = [0.02, 0.05, 0.08]
    x = rng.standard_normal((1, K)).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    layers = [BitLinear.create_from_bytes(ctx, p, s, K, n) for p, s, n in zip(packs, scales, shapes)]
    ys, accs = BitLinear.forward_multi(layers, _dev(x), rms_gamma=_dev(gamma), return_acc=True)
    ctx.check()
    for p, s, n, y, a in zip(packs, scales, shapes, ys, accs):
        y_ref, acc_ref, _ = oracle.bitlinear_forward(p, s, K, n, x, gamma=gamma)
        assert np.array_equal(a.cpu().numpy(), acc_ref)
        assert np.array_equal(y.cpu().numpy(), y_ref)


@pytest.mark.parametrize("K,N,M", [(2560, 6912, 64), (6912, 2560, 64), (2560, 2560, 33),
                                   (128, 1, 16), (1152, 129, 20), (8192, 257, 48),
                                   (2560, 640, 150), (2560, 6912, 128), (6912, 2560, 100),
                                   (2560, 2560, 65), (1152, 300, 256)])
def test_batched_tensor_core_path_bit_exact(ctx, oracle, K, N, M):
    """16 or more tokens run on tcgen05 (kind::i8, accumulators in tensor memory): the int32
    results must still be bit-exact, including ragged row tiles, partial K chunks and the
    split-K reduction that launches with few row tiles use.  Up to 64 tokens take the 64-wide
    kernel, 65 to 128 the 128-wide one, more go in passes of 128 (150 = 128 + 22)."""
    rng = np.random.default_rng(K + N + M)
    packed = formats.i2s_pack(formats.random_ternary(rng, N, K))
    x = rng.standard_normal((M, K)).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    layer = BitLinear.create_from_bytes(ctx, packed, 0.043, K, N)
    y_ref, acc_ref, d_ref = oracle.bitlinear_forward(packed, 0.043, K, N, x, gamma=gamma, residual=res)
    for _ in range(2):  # twice: the split-K arrival counters must be back at zero
        y, acc, d = layer.forward_fused_rmsnorm_residual(_dev(x), _dev(gamma), _dev(res),
                                                         return_acc=True)
        ctx.check()
        assert np.array_equal(d.cpu().numpy(), d_ref)
        assert np.array_equal(acc.cpu().numpy(), acc_ref)
        assert np.array_equal(y.cpu().numpy(), y_ref)


def test_zero_input_and_determinism(ctx, oracle):
    K, N = 2560, 6912
    rng = np.random.default_rng(9)
    packed = formats.i2s_pack(formats.random_ternary(rng, N, K))
    layer = BitLinear.create_from_bytes(ctx, packed, 0.05, K, N)
    y, acc, d = layer.forward(torch.zeros(1, K, device="cuda"), return_acc=True)
    assert not acc.any() and not y.any() and d.item() == 0.0
    x = _dev(rng.standard_normal((1, K)).astype(np.float32))
    a = layer.forward(x)
    b = layer.forward(x)
    assert torch.equal(a, b)


def test_linearity_property_full_size(ctx):
    """Size-independent check at the benchmark shape: acc(W, q) is linear in the
    weights' sign, so acc(W) + acc(-W) = 0 for the same activations."""
    K, N = 2560, 6912
    rng = np.random.default_rng(11)
    t = formats.random_ternary(rng, N, K)
    x = _dev(rng.standard_normal((1, K)).astype(np.float32))
    a = BitLinear.create_from_bytes(ctx, formats.i2s_pack(t), 1.0, K, N).forward(x, return_acc=True)[1]
    b = BitLinear.create_from_bytes(ctx, formats.i2s_pack(-t), 1.0, K, N).forward(x, return_acc=True)[1]
    assert not (a + b).any()


def test_bad_arguments_fail_loudly(ctx):
    from hesper_b200 import HesperB200Error
    layer = BitLinear.create_from_bytes(ctx, np.zeros(128 * 4 // 4, np.uint8), 1.0, 128, 4)
    with pytest.raises(HesperB200Error):
        layer.in_dim = 100  # not a multiple of 128
        layer.forward(torch.zeros(100, device="cuda"))


@pytest.mark.parametrize("K,H,Hkv,D,pos,ring", [(2560, 20, 5, 128, 37, 0), (256, 4, 2, 64, 5, 0),
                                                (2560, 8, 2, 256, 70, 1), (384, 4, 2, 64, 3, 0)])
def test_fused_qkv_rope_equals_the_two_launches(ctx, K, H, Hkv, D, pos, ring):
    """hb200_bitlinear_qkv_rope = hb200_bitlinear_forward_multi + hb200_rope_kv_write_angles, bit
    for bit: rotated q, and the f16 rows the caches receive at the token's slot (K = 384 is a
    shape the fused kernel does not cover: the entry point then makes the two launches itself)."""
    import ctypes as C
    from hesper_b200 import _lib
    from hesper_b200._lib import BitLinearSeg
    lib = _lib.load()
    rng = np.random.default_rng(K + H + D)
    slots = 64
    qd, kvd = H * D, Hkv * D
    ws = [torch.from_numpy(formats.i2s_pack(formats.random_ternary(rng, n, K))).cuda()
          for n in (qd, kvd, kvd)]
    sc = [torch.tensor([s], device="cuda") for s in (0.03, 0.05, 0.07)]
    x = torch.randn(1, K, device="cuda")
    gamma = (1 + 0.1 * torch.randn(K, device="cuda")).contiguous()
    dpos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    table = torch.empty(D, dtype=torch.float64, device="cuda")
    assert lib.hb200_rope_table(ctx.handle, dpos.data_ptr(), 1, 1, D, C.c_float(500000.0),
                                table.data_ptr(), None) == 0

    def run(fused):
        q = torch.zeros(1, qd, device="cuda")
        k = torch.zeros(1, kvd, device="cuda")
        v = torch.zeros(1, kvd, device="cuda")
        kc = torch.zeros(Hkv, slots, D, dtype=torch.float16, device="cuda")
        vc = torch.zeros(Hkv, slots, D, dtype=torch.float16, device="cuda")
        segs = (BitLinearSeg * 3)()
        for i, (w, s, y, n) in enumerate(zip(ws, sc, (q, k, v), (qd, kvd, kvd))):
            segs[i] = BitLinearSeg(w.data_ptr(), s.data_ptr(), None, y.data_ptr(), None, n)
        if fused:
            rc = lib.hb200_bitlinear_qkv_rope(ctx.handle, segs, K, x.data_ptr(), gamma.data_ptr(),
                                              C.c_float(1e-5), table.data_ptr(), dpos.data_ptr(),
                                              kc.data_ptr(), vc.data_ptr(), H, Hkv, D, slots, ring,
                                              None)
            assert rc == 0, lib.hb200_last_error()
        else:
            rc = lib.hb200_bitlinear_forward_multi(ctx.handle, segs, 3, K, x.data_ptr(), 1,
                                                   gamma.data_ptr(), C.c_float(1e-5), None, None)
            assert rc == 0, lib.hb200_last_error()
            rc = lib.hb200_rope_kv_write_angles(ctx.handle, q.data_ptr(), k.data_ptr(),
                                                v.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                                dpos.data_ptr(), table.data_ptr(), 1, H, Hkv, D,
                                                slots, ring, None)
            assert rc == 0, lib.hb200_last_error()
        torch.cuda.synchronize()
        return q, kc, vc

    q1, kc1, vc1 = run(True)
    q0, kc0, vc0 = run(False)
    ctx.check()
    assert torch.equal(q1, q0)
    assert torch.equal(kc1, kc0) and torch.equal(vc1, vc0)
    assert float(kc0[:, pos % slots if ring else pos].abs().sum()) > 0
