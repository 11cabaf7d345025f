"""GPU parity: LM head (16-bit table x f32 activations, fused final RMSNorm, greedy argmax)
through the C ABI vs an f64 reference, for the streaming path (M <= 8 per pass) and the
tensor-core path (16 <= M <= 64, activations split hi + lo so that f32 accuracy is kept).
Bar: logits within 2e-5 of max|logit| (f32 accumulation-order noise is ~1e-6; the bf16
hi + lo split drops 2^-17 of each activation), argmax equal to the reference's first maximum
whenever the reference's top-2 gap exceeds that bar."""
import ctypes as C

import numpy as np
import pytest
import torch

from hesper_b200 import _lib

pytestmark = pytest.mark.gpu

TOL = 2e-5


def _bf16_bits(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def _table(rng, V, K, dtype):
    w = (0.02 * rng.standard_normal((V, K))).astype(np.float32)
    if dtype == 0:
        bits = _bf16_bits(w)
        val = (bits.astype(np.uint32) << 16).view(np.float32)
    else:
        h = w.astype(np.float16)
        bits = h.view(np.uint16)
        val = h.astype(np.float32)
    return bits, val.astype(np.float64)


def _run(ctx, bits, dtype, x, gamma, eps, want_logits=True):
    lib = _lib.load()
    V, K = bits.shape
    M = x.shape[0]
    d_t = torch.from_numpy(bits.view(np.int16)).cuda()
    d_x = torch.from_numpy(x).cuda()
    d_g = torch.from_numpy(gamma).cuda() if gamma is not None else None
    d_logits = torch.full((M, V), float("nan"), device="cuda") if want_logits else None
    d_arg = torch.full((M,), -1, dtype=torch.int32, device="cuda")
    d_scr = torch.zeros(M, dtype=torch.int64, device="cuda")
    rc = lib.hb200_lmhead_argmax(ctx.handle, d_t.data_ptr(), dtype, V, K, d_x.data_ptr(), M,
                                 d_g.data_ptr() if d_g is not None else None, eps,
                                 d_logits.data_ptr() if want_logits else None, d_arg.data_ptr(),
                                 d_scr.data_ptr(), None, None, 0, None)
    assert rc == 0, lib.hb200_last_error().decode()
    torch.cuda.synchronize()
    ctx.check()
    assert int(d_scr.abs().sum()) == 0  # the keys are cleared for the next step
    return (d_logits.cpu().numpy() if want_logits else None), d_arg.cpu().numpy()


def _reference(val, x, gamma, eps):
    xn = x.astype(np.float64)
    if gamma is not None:
        # the kernels normalise in f32 from an f64 sum of squares
        ss = (x.astype(np.float64) ** 2).sum(axis=1, keepdims=True)
        rinv = (1.0 / np.sqrt(ss / x.shape[1] + eps)).astype(np.float32)
        xn = ((x * rinv).astype(np.float32) * gamma).astype(np.float32).astype(np.float64)
    return xn @ val.T


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("M", [1, 3, 8, 16, 17, 33, 64])
def test_logits_and_argmax(ctx, dtype, M):
    V, K = 5000, 2560  # V not a multiple of the 128-row tile
    rng = np.random.default_rng(100 * M + dtype)
    bits, val = _table(rng, V, K, dtype)
    x = rng.standard_normal((M, K)).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    ref = _reference(val, x, gamma, 1e-5)
    logits, arg = _run(ctx, bits, dtype, x, gamma, 1e-5)
    scale = np.abs(ref).max()
    assert np.abs(logits - ref).max() / scale <= TOL
    for m in range(M):
        top = np.sort(ref[m])[-2:]
        if top[1] - top[0] > TOL * scale:
            assert arg[m] == int(np.argmax(ref[m]))
        assert arg[m] == int(np.argmax(logits[m]))  # first maximum of what was computed


@pytest.mark.parametrize("M", [4, 32])
def test_no_norm_no_logits_small_k(ctx, M):
    V, K = 1000, 128
    rng = np.random.default_rng(M)
    bits, val = _table(rng, V, K, 0)
    x = rng.standard_normal((M, K)).astype(np.float32)
    ref = _reference(val, x, None, 0.0)
    _, arg = _run(ctx, bits, 0, x, None, 0.0, want_logits=False)
    scale = np.abs(ref).max()
    for m in range(M):
        top = np.sort(ref[m])[-2:]
        if top[1] - top[0] > TOL * scale:
            assert arg[m] == int(np.argmax(ref[m]))


def test_ties_pick_the_first_row(ctx):
    # identical rows in different tiles and different lanes: the smallest index must win
    V, K, M = 1024, 256, 20
    rng = np.random.default_rng(5)
    bits, val = _table(rng, V, K, 0)
    x = rng.standard_normal((M, K)).astype(np.float32)
    ref = _reference(val, x, None, 0.0)
    best = int(np.argmax(ref[0]))
    dup = [(best + 131) % V, (best + 700) % V]
    for d in dup:
        bits[d] = bits[best]
    first = min([best] + dup)
    _, arg = _run(ctx, bits, 0, x, None, 0.0, want_logits=False)
    assert arg[0] == first


def test_full_vocabulary_shape(ctx, oracle):
    # the BitNet-2B head: V = 128256, K = 2560, 64 tokens; reference = the f64 CPU restatement
    V, K, M = 128256, 2560, 64
    rng = np.random.default_rng(9)
    w = torch.randn(V, K, generator=torch.Generator().manual_seed(3)) * 0.02
    bits = w.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    x = rng.standard_normal((M, K)).astype(np.float32)
    logits, arg = _run(ctx, bits, 0, x, None, 0.0)
    for m in (0, 31, 63):
        ref = oracle.lmhead_bf16(bits, x[m]).astype(np.float64)
        scale = np.abs(ref).max()
        assert np.abs(logits[m] - ref).max() / scale <= TOL
        top = np.sort(ref)[-2:]
        if top[1] - top[0] > TOL * scale:
            assert arg[m] == int(np.argmax(ref))
