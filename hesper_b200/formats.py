"""Host-side encoders for the on-disk weight formats the kernels consume verbatim.

These build byte images in exactly the layouts the reference uploads to the GPU:
  * i2_s ternary, 2 bits/weight, groups of 128 elements in 32 bytes
    (Hesper/Layers/BitLinearSpec.lean:17-29,120-143),
  * GGUF Q4_K super-blocks of 256 weights in 144 bytes
    (Hesper/Quantization/Q4_K_M.lean:13-52,120-144),
  * GGUF Q8_0 blocks of 32 weights in 34 bytes (Hesper/Layers/Linear.lean:6187-6223).
They are vectorised numpy (no per-element Python loops) so full-size layers can
be generated in seconds, and they are used for synthetic random-init weights:
no real checkpoint is needed to exercise the kernels.
"""
from __future__ import annotations

import numpy as np

GGML_TYPE_Q8_0 = 8
GGML_TYPE_Q4_K = 12
GGML_TYPE_I2_S = 36

Q4K_BLOCK_BYTES = 144
Q4K_BLOCK_ELEMS = 256
Q80_BLOCK_BYTES = 34
Q80_BLOCK_ELEMS = 32


def i2s_pack(ternary: np.ndarray) -> np.ndarray:
    """[N, K] values in {-1, 0, +1} -> N*K/4 packed bytes (codes 0/1/2).

    Byte j of a 32-byte group holds element j in bits 7:6, 32+j in bits 5:4,
    64+j in bits 3:2 and 96+j in bits 1:0.
    """
    t = np.asarray(ternary)
    N, K = t.shape
    if K % 128:
        raise ValueError("i2_s needs K to be a multiple of 128")
    c = (t.astype(np.int16) + 1).astype(np.uint8).reshape(N, K // 128, 4, 32)
    b = (c[:, :, 0] << 6) | (c[:, :, 1] << 4) | (c[:, :, 2] << 2) | c[:, :, 3]
    return np.ascontiguousarray(b.reshape(-1))


def i2s_unpack(packed: np.ndarray, K: int, N: int) -> np.ndarray:
    b = np.asarray(packed, dtype=np.uint8).reshape(N, K // 128, 1, 32)
    shifts = np.array([6, 4, 2, 0], dtype=np.uint8).reshape(1, 1, 4, 1)
    codes = (b >> shifts) & 3
    return (codes.astype(np.int8) - 1).reshape(N, K)


def random_ternary(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    """i.i.d. ternary with P(-1, 0, +1) = (1/4, 1/2, 1/4)."""
    u = rng.integers(0, 4, size=(N, K), dtype=np.uint8)
    return np.where(u == 0, -1, np.where(u == 3, 1, 0)).astype(np.int8)


def q4k_pack_scales(sc: np.ndarray, m: np.ndarray) -> np.ndarray:
    """8 six-bit scales and 8 six-bit mins per block -> the 12 packed bytes."""
    sc = sc.astype(np.uint8)
    m = m.astype(np.uint8)
    out = np.empty(sc.shape[:-1] + (12,), np.uint8)
    out[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = (m[..., 0:4] & 63) | ((m[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 0xF) | ((m[..., 4:8] & 0xF) << 4)
    return out


def q4k_build(d, dmin, sc, m, q) -> np.ndarray:
    """Assemble Q4_K blocks.

    d, dmin: float [nb]; sc, m: ints [nb, 8] in 0..63; q: ints [nb, 256] in 0..15
    in element order.  Returns uint8 [nb, 144].
    """
    nb = q.shape[0]
    blk = np.empty((nb, 144), np.uint8)
    blk[:, 0:2] = np.asarray(d, np.float16).reshape(nb, 1).view(np.uint8)
    blk[:, 2:4] = np.asarray(dmin, np.float16).reshape(nb, 1).view(np.uint8)
    blk[:, 4:16] = q4k_pack_scales(np.asarray(sc), np.asarray(m))
    qq = np.asarray(q, np.uint8).reshape(nb, 4, 2, 32)  # chunk, low/high, l
    blk[:, 16:] = (qq[:, :, 0, :] | (qq[:, :, 1, :] << 4)).reshape(nb, 128)
    return blk


def random_q4k(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    """Random Q4_K tensor [N, K] generated directly in block form:
    d ~ U(1e-3, 1e-2), dmin ~ U(0, 1e-2) (rounded to f16), scales and mins
    ~ U{0..63}, quants ~ U{0..15}.  Returns uint8 [N * K/256 * 144]."""
    if K % 256:
        raise ValueError("Q4_K needs K to be a multiple of 256")
    nb = N * (K // 256)
    blk = np.empty((nb, 144), np.uint8)
    blk[:, 0:2] = rng.uniform(1e-3, 1e-2, nb).astype(np.float16).reshape(nb, 1).view(np.uint8)
    blk[:, 2:4] = rng.uniform(0.0, 1e-2, nb).astype(np.float16).reshape(nb, 1).view(np.uint8)
    sc = rng.integers(0, 64, size=(nb, 8), dtype=np.uint8)
    m = rng.integers(0, 64, size=(nb, 8), dtype=np.uint8)
    blk[:, 4:16] = q4k_pack_scales(sc, m)
    blk[:, 16:] = rng.integers(0, 256, size=(nb, 128), dtype=np.uint8)
    return blk.reshape(-1)


def q80_build(d, q) -> np.ndarray:
    """d: float [nb]; q: int8 [nb, 32] -> uint8 [nb, 34]."""
    nb = q.shape[0]
    blk = np.empty((nb, 34), np.uint8)
    blk[:, 0:2] = np.asarray(d, np.float16).reshape(nb, 1).view(np.uint8)
    blk[:, 2:] = np.asarray(q, np.int8).view(np.uint8)
    return blk


def random_q80(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    """Random Q8_0 tensor: d ~ U(1e-3, 1e-2) as f16, quants ~ U{-127..127}."""
    if K % 32:
        raise ValueError("Q8_0 needs K to be a multiple of 32")
    nb = N * (K // 32)
    d = rng.uniform(1e-3, 1e-2, nb)
    q = rng.integers(-127, 128, size=(nb, 32), dtype=np.int8)
    return q80_build(d, q).reshape(-1)


def kquant_row_bytes(fmt: int, K: int) -> int:
    if fmt == GGML_TYPE_Q4_K:
        return K // 256 * 144
    if fmt == GGML_TYPE_Q8_0:
        return K // 32 * 34
    raise ValueError(f"unsupported k-quant format id {fmt}")


def random_kquant(rng, fmt: int, N: int, K: int) -> np.ndarray:
    return random_q4k(rng, N, K) if fmt == GGML_TYPE_Q4_K else random_q80(rng, N, K)
