"""Generates tests/golden/golden.json.

The reference (a Lean 4 project) cannot be built or imported where this runs,
and its tests store inputs, not expected outputs (they compare a kernel with
the Lean CPU spec at run time).  The vectors here are therefore produced by a
small, independent numpy/float64 restatement of the same specs, written only
for this file -- it shares no code with oracle/hesper_oracle.c, so the C oracle
and the CUDA path are both checked against a second, separately written
derivation on the reference's own fixture inputs:

  * attention_literal : Tests/FlashAttentionTest.lean:24-49 inputs, three-step
    softmax attention (Hesper/Training/VerifiedBackward.lean:33-37,134-142),
    scale 1/sqrt(4) as in the test and 0.5 as in verifyFlashEquivalence
    (Hesper/WGSL/FlashAttention.lean:93-98)
  * q4k_reference_block : the Q4_K block of Tests/CUDA/CUDADP4ATest.lean:95-145
    (seed 42) dotted with x = sin(0.1 i)
  * bitlinear_tiny : Tests/BitLinearEquivalence.lean case "tiny-M1"
    (K=128, N=16, seed 0xDEADBEEF): f64 spec outputs and int8-contract accumulators
  * all_plus_one : Tests/CUDA/CUDABitLinearTest.lean:57-71

Run:  python tests/golden/make_golden.py
"""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

Q = [[1.0, 0.5, -0.3, 0.8], [-0.2, 0.7, 0.4, -0.6]]
K = [[[0.5, 1.0, 0.2, -0.5], [-0.3, 0.8, 1.0, 0.1], [0.7, -0.2, 0.5, 0.9]],
     [[0.3, 0.6, -0.4, 0.2], [0.8, -0.1, 0.7, -0.3], [-0.5, 0.4, 0.3, 0.6]]]
V = [[[1.0, 0.0, 0.5, -0.3], [0.2, 1.0, -0.5, 0.8], [-0.1, 0.5, 1.0, 0.2]],
     [[0.4, -0.2, 0.8, 0.1], [-0.3, 0.6, 0.2, 0.9], [0.7, 0.1, -0.4, 0.5]]]


def attention(q, k, v, scale):
    q, k, v = np.asarray(q, np.float64), np.asarray(k, np.float64), np.asarray(v, np.float64)
    s = scale * (k @ q)
    e = np.exp(s - s.max())
    return (e / e.sum()) @ v


def xorshift32(state):
    x = state
    x ^= (x << 13) & 0xFFFFFFFF
    x ^= x >> 17
    x ^= (x << 5) & 0xFFFFFFFF
    return x


def bitlinear_case(seed, Kdim, N, M):
    s = seed
    t = np.empty(N * Kdim, np.int64)
    for i in range(N * Kdim):
        s = xorshift32(s)
        t[i] = s % 3 - 1
    x = np.empty(M * Kdim, np.float64)
    for i in range(M * Kdim):
        s = xorshift32(s)
        x[i] = s / 4294967296.0 * 2.0 - 1.0
    s = xorshift32(s)
    scale = s / 4294967296.0 * 0.1 + 0.01
    return t.reshape(N, Kdim), x.reshape(M, Kdim), scale


def q4k_block(seed):
    words = np.zeros(36, np.uint64)
    words[0] = 0x211F | (0x1D1F << 16)
    sc, m = list(range(10, 18)), list(range(1, 9))
    words[1] = sc[0] | (sc[1] << 8) | (sc[2] << 16) | (sc[3] << 24)
    words[2] = m[0] | (m[1] << 8) | (m[2] << 16) | (m[3] << 24)
    w3 = 0
    for i in range(4):
        w3 |= ((sc[4 + i] & 0xF) | ((m[4 + i] & 0xF) << 4)) << (8 * i)
    words[3] = w3
    for i in range(32):
        words[4 + i] = (((seed + i) * 6364136223846793005 + 1442695040888963407) & (2 ** 64 - 1)) & 0xFFFFFFFF
    b = words.astype(np.uint32).view(np.uint8)
    # decode the 6-bit scales / mins back out of the 12 packed bytes (the fixture's
    # sc = 16, 17 do not fit its 4-bit packing, so the block really holds 0 and 1 there)
    pk = b[4:16].astype(np.int64)
    sc = [int(pk[j] & 63) if j < 4 else int((pk[j + 4] & 0xF) | ((pk[j - 4] >> 6) << 4)) for j in range(8)]
    m = [int(pk[j + 4] & 63) if j < 4 else int((pk[j + 4] >> 4) | ((pk[j] >> 6) << 4)) for j in range(8)]
    d = float(np.array([0x211F], np.uint16).view(np.float16)[0])
    dmin = float(np.array([0x1D1F], np.uint16).view(np.float16)[0])
    w = np.empty(256, np.float64)
    qs = b[16:].astype(np.int64)
    for c in range(4):
        for l in range(32):
            w[64 * c + l] = d * sc[2 * c] * (qs[32 * c + l] & 0xF) - dmin * m[2 * c]
            w[64 * c + 32 + l] = d * sc[2 * c + 1] * (qs[32 * c + l] >> 4) - dmin * m[2 * c + 1]
    return b, w


def main():
    out = {}
    out["attention_literal"] = {
        "scale_inv_sqrt_d": [attention(Q[h], K[h], V[h], 0.5).tolist() for h in range(2)],
        "flash_equivalence_head0_scale_0.5": attention(Q[0], K[0], V[0], 0.5).tolist(),
    }
    b, w = q4k_block(42)
    x = np.sin(0.1 * np.arange(256)).astype(np.float32).astype(np.float64)
    out["q4k_reference_block"] = {"bytes_hex": bytes(b).hex(), "dot": float(w @ x),
                                  "w_first8": w[:8].tolist()}
    t, xx, scale = bitlinear_case(0xDEADBEEF, 128, 16, 1)
    x32 = xx.astype(np.float32)
    amax = np.float32(np.max(np.abs(x32)))
    inv = np.float32(127.0) / amax
    q = np.rint(x32[0] * inv).astype(np.int64)
    out["bitlinear_tiny"] = {
        "scale": scale,
        "spec_f64": (scale * (t @ x32[0].astype(np.float64))).tolist(),
        "acc_int8_contract": (t @ q).tolist(),
        "d": float(amax / np.float32(127.0)),
        "ternary_first16": t[0, :16].tolist(),
    }
    out["all_plus_one"] = {"K": 128, "byte": 0xAA, "y": 128.0}
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote golden.json")


if __name__ == "__main__":
    main()
