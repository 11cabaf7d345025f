"""numpy-facing wrapper over the CPU oracle (oracle/hesper_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and
by the CPU-baseline legs of ``bench.py``.  The shipped package never imports it.

The C file restates the reference's Lean specs (citations are in the C source);
this module only marshals numpy arrays.  ``build()`` compiles the shared object
with the recipe in oracle/Makefile when it is missing.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libhesper_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "hesper_oracle.c")
    stale = (not os.path.exists(_SO)) or os.path.getmtime(_SO) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
        _lib.orc_quant_act_i8.restype = C.c_float
        _lib.orc_lcg_fill.restype = C.c_uint64
        _lib.orc_lcg_fill.argtypes = [C.c_uint64, C.c_long, C.c_void_p]
        _lib.orc_gelu_tanh.restype = C.c_double
        _lib.orc_gelu_tanh.argtypes = [C.c_double]
        _lib.orc_argmax.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


def num_threads() -> int:
    return lib().orc_num_threads()


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


# ---- f16 ------------------------------------------------------------------

def f16_to_f32(h: int) -> float:
    return float(lib().orc_f16_to_f32(int(h)))


def f32_to_f16(f: float) -> int:
    return int(lib().orc_f32_to_f16(C.c_float(f)))


# ---- generators of the reference's tests ------------------------------------

def gen_bitlinear_case(seed: int, K: int, N: int, M: int):
    """(ternary int8 [N,K], x f32 [M,K], scale) as Tests/BitLinearEquivalence.lean genCase."""
    t = np.empty((N, K), np.int8)
    x = np.empty((M, K), np.float32)
    s = C.c_float(0)
    lib().orc_gen_bitlinear_case(C.c_uint32(seed), K, N, M, _p(t), _p(x), C.byref(s))
    return t, x, float(s.value)


def lcg_fill(seed: int, n: int):
    out = np.empty(n, np.float32)
    st = lib().orc_lcg_fill(C.c_uint64(seed), C.c_long(n), _p(out))
    return out, int(st)


# ---- i2_s / BitLinear -------------------------------------------------------

def i2s_pack(ternary: np.ndarray) -> np.ndarray:
    t = _c(ternary, np.int8)
    N, K = t.shape
    out = np.empty(N * K // 4, np.uint8)
    lib().orc_i2s_pack(_p(t), K, N, _p(out))
    return out


def i2s_decode_all(packed: np.ndarray, K: int, N: int) -> np.ndarray:
    p = _c(packed, np.uint8)
    out = np.empty((N, K), np.int8)
    L = lib()
    for n in range(N):
        for k in range(K):
            out[n, k] = L.orc_i2s_decode(_p(p), C.c_long(p.size), C.c_long(n * K // 4), k)
    return out


def bitlinear_spec(packed, scale, K, N, x) -> np.ndarray:
    """BitLinearSpec.forward in double; x f32 [M,K] -> f64 [M,N]."""
    p = _c(packed, np.uint8)
    x = _c(x, np.float32).reshape(-1, K)
    M = x.shape[0]
    y = np.empty((M, N), np.float64)
    lib().orc_bitlinear_spec(_p(p), C.c_float(scale), K, N, M, _p(x), _p(y))
    return y


def quant_act_i8(x):
    x = _c(x, np.float32).reshape(-1)
    q = np.empty(x.size, np.int8)
    d = lib().orc_quant_act_i8(_p(x), x.size, _p(q))
    return q, np.float32(d)


def bitlinear_i8(packed, K, N, q) -> np.ndarray:
    p = _c(packed, np.uint8)
    q = _c(q, np.int8)
    acc = np.empty(N, np.int32)
    lib().orc_bitlinear_i8(_p(p), K, N, _p(q), _p(acc))
    return acc


def bitlinear_forward(packed, scale, K, N, x, gamma=None, eps=1e-5, residual=None):
    """The CUDA path's contract: returns (y f32 [M,N], acc int32 [M,N], d f32 [M])."""
    p = _c(packed, np.uint8)
    x = _c(x, np.float32).reshape(-1, K)
    M = x.shape[0]
    g = _c(gamma, np.float32)
    r = _c(residual, np.float32)
    y = np.empty((M, N), np.float32)
    acc = np.empty((M, N), np.int32)
    d = np.empty(M, np.float32)
    lib().orc_bitlinear_forward(_p(p), C.c_float(scale), K, N, M, _p(x), _p(g),
                                C.c_float(eps), _p(r), _p(acc), _p(d), _p(y))
    return y, acc, d


def bitlinear_gateup_relu2(pg, sg, pu, su, K, N, x, gamma=None, eps=1e-5):
    pg = _c(pg, np.uint8)
    pu = _c(pu, np.uint8)
    x = _c(x, np.float32).reshape(-1, K)
    M = x.shape[0]
    g = _c(gamma, np.float32)
    y = np.empty((M, N), np.float32)
    lib().orc_bitlinear_gateup_relu2(_p(pg), C.c_float(sg), _p(pu), C.c_float(su), K, N, M,
                                     _p(x), _p(g), C.c_float(eps), _p(y))
    return y


def rmsnorm_f64(x, gamma, eps):
    x = _c(x, np.float32)
    g = _c(gamma, np.float32)
    y = np.empty(x.size, np.float64)
    lib().orc_rmsnorm_f64(_p(x), _p(g), x.size, C.c_double(eps), _p(y))
    return y


def rmsnorm_f32(x, gamma, eps):
    x = _c(x, np.float32)
    g = _c(gamma, np.float32)
    y = np.empty(x.size, np.float32)
    lib().orc_rmsnorm_f32(_p(x), _p(g), x.size, C.c_float(eps), _p(y))
    return y


# ---- k-quants ---------------------------------------------------------------

def q4k_dequant(blocks: np.ndarray) -> np.ndarray:
    b = _c(blocks, np.uint8).reshape(-1, 144)
    out = np.empty((b.shape[0], 256), np.float32)
    L = lib()
    for i in range(b.shape[0]):
        L.orc_q4k_dequant_block(_p(b[i]), _p(out[i]))
    return out


def q4k_matvec(blocks, K, N, x, residual=None):
    b = _c(blocks, np.uint8)
    x = _c(x, np.float32).reshape(-1, K)
    M = x.shape[0]
    r = _c(residual, np.float32)
    y = np.empty((M, N), np.float32)
    lib().orc_q4k_matvec(_p(b), K, N, M, _p(x), _p(r), _p(y))
    return y


def q8_0_matvec(blocks, K, N, x, residual=None):
    b = _c(blocks, np.uint8)
    x = _c(x, np.float32).reshape(-1, K)
    M = x.shape[0]
    r = _c(residual, np.float32)
    y = np.empty((M, N), np.float32)
    lib().orc_q8_0_matvec(_p(b), K, N, M, _p(x), _p(r), _p(y))
    return y


def kquant_matvec(fmt, blocks, K, N, x, residual=None):
    return (q4k_matvec if fmt == 12 else q8_0_matvec)(blocks, K, N, x, residual)


def kquant_gateup_gelu(bg, bu, fmt, K, N, x):
    bg = _c(bg, np.uint8)
    bu = _c(bu, np.uint8)
    x = _c(x, np.float32).reshape(-1, K)
    M = x.shape[0]
    y = np.empty((M, N), np.float32)
    lib().orc_kquant_gateup_gelu(_p(bg), _p(bu), fmt, K, N, M, _p(x), _p(y))
    return y


# ---- attention ----------------------------------------------------------------

def attention_head(q, k, v, scale, online=False):
    q = _c(q, np.float64)
    k = _c(k, np.float64)
    v = _c(v, np.float64)
    L, D = k.shape
    out = np.empty(D, np.float64)
    fn = lib().orc_flash_attention_head if online else lib().orc_attention_head
    fn(_p(q), _p(k), _p(v), L, D, C.c_double(scale), _p(out))
    return out


def attn_decode(q, k_f16, v_f16, seqlens, H, Hkv, D, max_seq, scale, window=0):
    """q: f32 or f16 array [B,H,D]; k/v: float16 arrays [B,Hkv,max_seq,D]."""
    q_is_f16 = q.dtype == np.float16
    qq = np.ascontiguousarray(q)
    kk = np.ascontiguousarray(k_f16, dtype=np.float16).view(np.uint16)
    vv = np.ascontiguousarray(v_f16, dtype=np.float16).view(np.uint16)
    sl = _c(seqlens, np.int32)
    B = sl.size
    out = np.empty((B, H, D), np.float32)
    qptr = qq.view(np.uint16) if q_is_f16 else qq.astype(np.float32, copy=False)
    lib().orc_attn_decode(_p(qptr), int(q_is_f16), _p(kk), _p(vv), _p(sl), B, H, Hkv, D,
                          max_seq, window, C.c_float(scale), _p(out))
    return out


def attn_decode_exact(q, k_f16, v_f16, seqlens, H, Hkv, D, max_seq, scale, window=0):
    """Mirror of the library's EXACT attention mode (same f32 operations in the same order)."""
    q_is_f16 = q.dtype == np.float16
    qq = np.ascontiguousarray(q)
    kk = np.ascontiguousarray(k_f16, dtype=np.float16).view(np.uint16)
    vv = np.ascontiguousarray(v_f16, dtype=np.float16).view(np.uint16)
    sl = _c(seqlens, np.int32)
    B = sl.size
    out = np.empty((B, H, D), np.float32)
    qptr = qq.view(np.uint16) if q_is_f16 else qq.astype(np.float32, copy=False)
    scale_log2 = np.float32(scale) * np.float32(1.4426950408889634)
    lib().orc_attn_decode_exact(_p(qptr), int(q_is_f16), _p(kk), _p(vv), _p(sl), B, H, Hkv, D,
                                max_seq, window, C.c_float(scale_log2), _p(out))
    return out


# ---- glue -----------------------------------------------------------------------

def rope_neox(x, pos, base):
    x = np.array(x, dtype=np.float32, copy=True)
    lib().orc_rope_neox(_p(x), x.size, int(pos), C.c_double(base))
    return x


def argmax(x) -> int:
    x = _c(x, np.float32)
    return int(lib().orc_argmax(_p(x), C.c_long(x.size)))


def lmhead_bf16(table_u16, x):
    t = _c(table_u16, np.uint16)
    V, K = t.shape
    x = _c(x, np.float32)
    out = np.empty(V, np.float32)
    lib().orc_lmhead_bf16(_p(t), C.c_long(V), K, _p(x), _p(out))
    return out


def gelu_tanh(x: float) -> float:
    return float(lib().orc_gelu_tanh(C.c_double(x)))


# ---- whole-model BitNet decode ------------------------------------------------------------

class _OrcLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("attn_norm", "attn_sub_norm", "ffn_norm", "ffn_sub_norm",
                                          "wq", "wk", "wv", "wo", "wgate", "wup", "wdown")] + \
               [(n, C.c_float) for n in ("sq", "sk", "sv", "so", "sgate", "sup", "sdown")]


class BitNetOracle:
    """CPU model of one sequence (orc_bitnet_step); weights as produced by
    hesper_b200.models.random_bitnet_weights."""

    def __init__(self, shape, weights):
        L = lib()
        L.orc_bitnet_create.restype = C.c_void_p
        L.orc_bitnet_step.restype = C.c_int
        self.shape = shape
        self._keep = []
        arr = (_OrcLayer * shape.n_layers)()
        for i, W in enumerate(weights["layers"]):
            f = {}
            for n in ("attn_norm", "attn_sub_norm", "ffn_norm", "ffn_sub_norm"):
                a = _c(W[n], np.float32); self._keep.append(a); f[n] = a.ctypes.data
            for n in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown"):
                a = _c(W[n], np.uint8); self._keep.append(a); f[n] = a.ctypes.data
                f["s" + n[1:]] = float(W["s" + n[1:]])
            arr[i] = _OrcLayer(**f)
        self._arr = arr
        self._emb = _c(weights["embed"], np.uint16)
        self._fn = _c(weights["final_norm"], np.float32)
        self._h = C.c_void_p(L.orc_bitnet_create(
            shape.n_layers, shape.hidden, shape.n_heads, shape.n_kv_heads, shape.head_dim,
            shape.ffn, shape.vocab, shape.max_seq, C.c_double(shape.rope_base),
            C.c_float(shape.rms_eps), arr, _p(self._emb), _p(self._fn)))
        self.pos = 0

    def set_exact_attention(self, on: bool):
        lib().orc_bitnet_set_exact_attention(self._h, int(bool(on)))

    def step(self, token: int):
        """Feeds one token at the next position; returns (greedy token, logits f32 [vocab])."""
        logits = np.empty(self.shape.vocab, np.float32)
        tok = lib().orc_bitnet_step(self._h, int(token), self.pos, _p(logits))
        self.pos += 1
        return int(tok), logits

    def close(self):
        if self._h:
            lib().orc_bitnet_destroy(self._h)
            self._h = None


class _OrcGemmaLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("attn_norm", "post_attn_norm", "ffn_norm", "post_ffn_norm",
                                          "wq", "wk", "wv", "wo", "wgate", "wup", "wdown")]


class GemmaOracle:
    """Unsharded CPU model of one sequence (orc_gemma_step); weights as produced by
    hesper_b200.tp.random_gemma_weights."""

    def __init__(self, shape, weights):
        L = lib()
        L.orc_gemma_create.restype = C.c_void_p
        self.shape = shape
        self._keep = []
        arr = (_OrcGemmaLayer * shape.n_layers)()
        for i, W in enumerate(weights["layers"]):
            f = {}
            for n in ("attn_norm", "post_attn_norm", "ffn_norm", "post_ffn_norm"):
                a = _c(W[n], np.float32); self._keep.append(a); f[n] = a.ctypes.data
            for n in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown"):
                a = _c(W[n], np.uint8); self._keep.append(a); f[n] = a.ctypes.data
            arr[i] = _OrcGemmaLayer(**f)
        self._arr = arr
        self._emb = _c(weights["embed"], np.uint16)
        self._lm = _c(weights["lm_head"], np.uint8)
        self._fn = _c(weights["final_norm"], np.float32)
        self._h = C.c_void_p(L.orc_gemma_create(
            shape.n_layers, shape.hidden, shape.n_heads, shape.n_kv_heads, shape.head_dim,
            shape.ffn, shape.vocab, shape.max_seq, shape.window, shape.global_every,
            C.c_double(shape.rope_base), C.c_float(shape.rms_eps), C.c_float(shape.attn_scale),
            C.c_float(shape.embed_scale), arr, _p(self._emb), _p(self._lm), _p(self._fn)))
        self.pos = 0

    def step(self, token: int):
        logits = np.empty(self.shape.vocab, np.float32)
        tok = lib().orc_gemma_step(self._h, int(token), self.pos, _p(logits))
        self.pos += 1
        return int(tok), logits

    def close(self):
        if self._h:
            lib().orc_gemma_destroy(self._h)
            self._h = None
