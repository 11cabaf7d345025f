"""Host-side mirror of the reference's layer API for the hot path.

Names and argument meaning follow the Lean layers so that tests read like the
reference's own:
  * ``BitLinear``      -- Hesper/Layers/BitLinear.lean:1127-1453
  * ``LinearLayer``    -- Hesper/Layers/Linear.lean:5636-5669, 7115-7942
  * ``execute_flash_attention_v11`` -- Hesper/WGSL/FlashAttentionExperiments.lean:572
torch is used for device memory and streams only; every computation goes
through the C ABI (``include/hesper_b200.h``).  There is no CPU path: without
the CUDA library or a GPU these calls raise.
"""
from __future__ import annotations

import ctypes as C
import enum
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import BitLinearSeg, KQuantSeg, check


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream_handle(stream) -> C.c_void_p:
    if stream is None:
        stream = torch.cuda.current_stream()
    return C.c_void_p(stream.cuda_stream)


def _need(t: torch.Tensor, dtype, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must live on the GPU (there is no CPU fallback)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


class Context:
    """One per GPU: mirrors CUDAContext.init (Hesper/Backend/CUDA.lean:46)."""

    def __init__(self, device: int = 0, adopt_current: bool = False):
        """`adopt_current`: build the context inside the CUDA context that is current on this
        thread (a host that called cuCtxCreate itself, as native/cuda_bridge.cpp:78-82 does)
        instead of binding to `device`'s primary context."""
        self._lib = _lib.load()
        self.device = int(device)
        h = C.c_void_p()
        if adopt_current:
            check(self._lib.hb200_ctx_create_current(C.byref(h)))
        else:
            check(self._lib.hb200_ctx_create(self.device, C.byref(h)))
        self._h = h

    @property
    def handle(self) -> C.c_void_p:
        return self._h

    @property
    def sm_count(self) -> int:
        return self._lib.hb200_ctx_sm_count(self._h)

    ATTN_FAST, ATTN_PRECISE, ATTN_EXACT = 0, 1, 2

    def set_attn_mode(self, mode: int) -> None:
        """Decode-attention arithmetic: fast f16, hi+lo f16 split, or the bit-reproducible
        reference-order kernel (see the header)."""
        check(self._lib.hb200_ctx_set_attn_mode(self._h, int(mode)))

    def check(self, stream=None) -> int:
        """Synchronise and return the device status flags (raises on a device-side timeout)."""
        flags = C.c_uint32(0)
        check(self._lib.hb200_ctx_check(self._h, _stream_handle(stream), C.byref(flags)))
        return flags.value

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.hb200_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class BitLinear:
    """Ternary i2_s linear layer: packed bytes + one f32 scale on the device.

    ``create_from_bytes`` mirrors BitLinear.createFromBytes
    (Hesper/Layers/BitLinear.lean:1141-1217): the packed GGUF bytes are uploaded
    verbatim, the per-tensor scale goes to a separate 4-byte buffer.
    """

    def __init__(self, ctx: Context, packed: torch.Tensor, scale: torch.Tensor, in_dim: int,
                 out_dim: int):
        self.ctx = ctx
        self.packed = _need(packed, torch.uint8, "packed")
        self.scale = _need(scale, torch.float32, "scale")
        self.in_dim = int(in_dim)
        self.out_dim = int(out_dim)
        if packed.numel() != in_dim * out_dim // 4:
            raise ValueError("packed size does not match in_dim*out_dim/4")

    @classmethod
    def create_from_bytes(cls, ctx: Context, packed_bytes: np.ndarray, scale: float, in_dim: int,
                          out_dim: int) -> "BitLinear":
        dev = torch.device("cuda", ctx.device)
        p = torch.from_numpy(np.ascontiguousarray(packed_bytes, dtype=np.uint8)).to(dev)
        s = torch.tensor([scale], dtype=torch.float32, device=dev)
        return cls(ctx, p, s, in_dim, out_dim)

    def _x(self, x: torch.Tensor):
        x = _need(x, torch.float32, "input")
        if x.numel() % self.in_dim:
            raise ValueError("input size is not a multiple of in_dim")
        return x, x.numel() // self.in_dim

    def forward(self, x: torch.Tensor, *, residual: Optional[torch.Tensor] = None,
                rms_gamma: Optional[torch.Tensor] = None, eps: float = 1e-5,
                return_acc: bool = False, out: Optional[torch.Tensor] = None, stream=None):
        """BitLinear.forward (:1226); with ``residual`` forwardWithResidual (:1308); with
        ``rms_gamma`` as well forwardFusedRMSNormResidual (:1370).

        Returns y [M, out_dim] f32, or (y, acc int32 [M, out_dim], d f32 [M]) with return_acc.
        """
        x, M = self._x(x)
        y = out if out is not None else torch.empty((M, self.out_dim), dtype=torch.float32,
                                                    device=x.device)
        acc = d = None
        if return_acc:
            acc = torch.empty((M, self.out_dim), dtype=torch.int32, device=x.device)
            d = torch.empty((M,), dtype=torch.float32, device=x.device)
        if residual is not None:
            _need(residual, torch.float32, "residual")
        if rms_gamma is not None:
            _need(rms_gamma, torch.float32, "rms_gamma")
        check(self.ctx._lib.hb200_bitlinear_forward(
            self.ctx.handle, _ptr(self.packed), _ptr(self.scale), self.in_dim, self.out_dim,
            _ptr(x), M, _ptr(rms_gamma), C.c_float(eps), _ptr(residual), _ptr(acc), _ptr(d),
            _ptr(y), _stream_handle(stream)))
        return (y, acc, d) if return_acc else y

    def forward_with_residual(self, x, residual, **kw):
        return self.forward(x, residual=residual, **kw)

    def forward_fused_rmsnorm_residual(self, x, rms_gamma, residual, eps: float = 1e-5, **kw):
        return self.forward(x, residual=residual, rms_gamma=rms_gamma, eps=eps, **kw)

    @staticmethod
    def forward_fused_gate_up_relu_sqr_mul(gate: "BitLinear", up: "BitLinear", x: torch.Tensor, *,
                                           rms_gamma=None, eps: float = 1e-5, out=None,
                                           stream=None) -> torch.Tensor:
        """BitLinear.forwardFusedGateUpReluSqrMul (Hesper/Layers/BitLinear.lean:1419)."""
        if (gate.in_dim, gate.out_dim) != (up.in_dim, up.out_dim):
            raise ValueError("gate and up must have the same shape")
        x, M = gate._x(x)
        y = out if out is not None else torch.empty((M, gate.out_dim), dtype=torch.float32,
                                                    device=x.device)
        check(gate.ctx._lib.hb200_bitlinear_gateup_relu2(
            gate.ctx.handle, _ptr(gate.packed), _ptr(gate.scale), _ptr(up.packed), _ptr(up.scale),
            gate.in_dim, gate.out_dim, _ptr(x), M, _ptr(rms_gamma), C.c_float(eps), _ptr(y),
            _stream_handle(stream)))
        return y

    @staticmethod
    def forward_multi(layers: Sequence["BitLinear"], x: torch.Tensor, *, rms_gamma=None,
                      eps: float = 1e-5, residuals=None, return_acc: bool = False, stream=None):
        """Several BitLinear layers over the same input in one launch (fused q/k/v)."""
        l0 = layers[0]
        x, M = l0._x(x)
        segs = (BitLinearSeg * len(layers))()
        ys, accs = [], []
        for i, l in enumerate(layers):
            if l.in_dim != l0.in_dim:
                raise ValueError("all layers must share in_dim")
            y = torch.empty((M, l.out_dim), dtype=torch.float32, device=x.device)
            a = torch.empty((M, l.out_dim), dtype=torch.int32, device=x.device) if return_acc else None
            r = residuals[i] if residuals is not None else None
            ys.append(y)
            accs.append(a)
            segs[i] = BitLinearSeg(l.packed.data_ptr(), l.scale.data_ptr(),
                                   r.data_ptr() if r is not None else None, y.data_ptr(),
                                   a.data_ptr() if a is not None else None, l.out_dim)
        check(l0.ctx._lib.hb200_bitlinear_forward_multi(
            l0.ctx.handle, segs, len(layers), l0.in_dim, _ptr(x), M, _ptr(rms_gamma),
            C.c_float(eps), None, _stream_handle(stream)))
        return (ys, accs) if return_acc else ys


class QuantFormat(enum.IntEnum):
    """GGUF type ids (Hesper/GGUF/Types.lean:86-132; Hesper/Layers/Linear.lean:5639)."""
    Q8_0 = 8
    Q4_K = 12


class LinearLayer:
    """GGUF k-quant linear layer: raw blocks on the device, f32 activations.

    Mirrors Linear.LinearLayer (Hesper/Layers/Linear.lean:5636-5669).
    """

    def __init__(self, ctx: Context, blocks: torch.Tensor, fmt: QuantFormat, in_dim: int,
                 out_dim: int):
        self.ctx = ctx
        self.blocks = _need(blocks, torch.uint8, "blocks")
        self.fmt = QuantFormat(fmt)
        self.in_dim = int(in_dim)
        self.out_dim = int(out_dim)
        per = (in_dim // 256 * 144) if self.fmt == QuantFormat.Q4_K else (in_dim // 32 * 34)
        if blocks.numel() != per * out_dim:
            raise ValueError("block bytes do not match the shape")

    @classmethod
    def create_from_bytes(cls, ctx: Context, block_bytes: np.ndarray, fmt, in_dim: int,
                          out_dim: int) -> "LinearLayer":
        dev = torch.device("cuda", ctx.device)
        b = torch.from_numpy(np.ascontiguousarray(block_bytes, dtype=np.uint8).reshape(-1)).to(dev)
        return cls(ctx, b, QuantFormat(fmt), in_dim, out_dim)

    def _x(self, x):
        x = _need(x, torch.float32, "input")
        if x.numel() % self.in_dim:
            raise ValueError("input size is not a multiple of in_dim")
        return x, x.numel() // self.in_dim

    def forward(self, x: torch.Tensor, *, residual=None, rms_gamma=None, eps: float = 1e-6,
                out=None, stream=None) -> torch.Tensor:
        """LinearLayer.forward (:7115); with rms_gamma forwardFusedRMSNormLinear."""
        x, M = self._x(x)
        y = out if out is not None else torch.empty((M, self.out_dim), dtype=torch.float32,
                                                    device=x.device)
        check(self.ctx._lib.hb200_kquant_forward(
            self.ctx.handle, int(self.fmt), _ptr(self.blocks), self.in_dim, self.out_dim, _ptr(x),
            M, _ptr(rms_gamma), C.c_float(eps), _ptr(residual), _ptr(y), _stream_handle(stream)))
        return y

    @staticmethod
    def forward_fused_gate_up(gate: "LinearLayer", up: "LinearLayer", x, *, rms_gamma=None,
                              eps: float = 1e-6, out=None, stream=None, pre=None):
        """forwardFusedGateUp / forwardFusedNormGateUp (Hesper/Layers/Linear.lean:7295,7506).

        pre=(base, gamma): the layer input becomes x' = base + rmsnorm(x) * gamma first
        (a post-norm with its residual add); returns (y, x') in that case."""
        x, M = gate._x(x)
        y = out if out is not None else torch.empty((M, gate.out_dim), dtype=torch.float32,
                                                    device=x.device)
        if pre is not None:
            base, pg = pre
            xo = torch.empty_like(x)
            check(gate.ctx._lib.hb200_kquant_gateup_gelu_pre(
                gate.ctx.handle, int(gate.fmt), _ptr(gate.blocks), _ptr(up.blocks), gate.in_dim,
                gate.out_dim, _ptr(x), M, _ptr(base), _ptr(pg), _ptr(xo), _ptr(rms_gamma),
                C.c_float(eps), _ptr(y), _stream_handle(stream)))
            return y, xo
        check(gate.ctx._lib.hb200_kquant_gateup_gelu(
            gate.ctx.handle, int(gate.fmt), _ptr(gate.blocks), _ptr(up.blocks), gate.in_dim,
            gate.out_dim, _ptr(x), M, _ptr(rms_gamma), C.c_float(eps), _ptr(y),
            _stream_handle(stream)))
        return y

    @staticmethod
    def forward_multi(layers: Sequence["LinearLayer"], x, *, rms_gamma=None, eps: float = 1e-6,
                      residuals=None, stream=None, pre=None):
        """forwardFusedQKV / forwardFusedNormQKV / forwardFusedKV (:7413-7660).

        pre=(base, gamma): the layers' input becomes x' = base + rmsnorm(x) * gamma first;
        returns (ys, x') in that case."""
        l0 = layers[0]
        x, M = l0._x(x)
        segs = (KQuantSeg * len(layers))()
        ys = []
        for i, l in enumerate(layers):
            y = torch.empty((M, l.out_dim), dtype=torch.float32, device=x.device)
            r = residuals[i] if residuals is not None else None
            ys.append(y)
            segs[i] = KQuantSeg(l.blocks.data_ptr(), r.data_ptr() if r is not None else None,
                                y.data_ptr(), l.out_dim)
        if pre is not None:
            base, pg = pre
            xo = torch.empty_like(x)
            check(l0.ctx._lib.hb200_kquant_forward_multi_pre(
                l0.ctx.handle, int(l0.fmt), segs, len(layers), l0.in_dim, _ptr(x), M, _ptr(base),
                _ptr(pg), _ptr(xo), _ptr(rms_gamma), C.c_float(eps), _stream_handle(stream)))
            return ys, xo
        check(l0.ctx._lib.hb200_kquant_forward_multi(
            l0.ctx.handle, int(l0.fmt), segs, len(layers), l0.in_dim, _ptr(x), M, _ptr(rms_gamma),
            C.c_float(eps), _stream_handle(stream)))
        return ys


def flash_attention_workspace(ctx: Context, B: int, H: int, Hkv: int, D: int, max_seq: int,
                              device=None) -> torch.Tensor:
    n = ctx._lib.hb200_attn_workspace_bytes(ctx.handle, B, H, Hkv, D, max_seq)
    dev = device if device is not None else torch.device("cuda", ctx.device)
    return torch.empty((max(int(n), 16),), dtype=torch.uint8, device=dev)


def flash_attention_prefill(ctx: Context, q: torch.Tensor, k_cache: torch.Tensor,
                            v_cache: torch.Tensor, seqlens: torch.Tensor, *, num_heads: int,
                            num_kv_heads: int, head_dim: int, max_seq_len: int, scale: float,
                            window: int = 0, stream=None) -> torch.Tensor:
    """Causal prefill attention (the prefill kernels of Hesper/WGSL/FlashAttention.lean:495-715).

    q [B, T, H, D] f32 or f16: T new tokens per sequence whose K/V already sit at positions
    seqlens[b]-T .. seqlens[b]-1 of the f16 caches [B, Hkv, max_seq_len, D]; returns [B, T, H, D].
    """
    _need(q, q.dtype, "q")
    _need(k_cache, torch.float16, "k_cache")
    _need(v_cache, torch.float16, "v_cache")
    _need(seqlens, torch.int32, "seqlens")
    B, T = int(q.shape[0]), int(q.shape[1])
    n = ctx._lib.hb200_attn_prefill_workspace_bytes(ctx.handle, B, T, num_heads, num_kv_heads,
                                                    head_dim, max_seq_len)
    ws = torch.empty((max(int(n), 16),), dtype=torch.uint8, device=q.device)
    o = torch.empty((B, T, num_heads, head_dim), dtype=torch.float32, device=q.device)
    check(ctx._lib.hb200_attn_prefill(
        ctx.handle, _ptr(q), int(q.dtype == torch.float16), _ptr(k_cache), _ptr(v_cache),
        _ptr(seqlens), B, T, num_heads, num_kv_heads, head_dim, max_seq_len, int(window),
        C.c_float(scale), _ptr(ws), C.c_size_t(ws.numel()), _ptr(o), _stream_handle(stream)))
    return o


def execute_flash_attention_v11(ctx: Context, q: torch.Tensor, k_cache: torch.Tensor,
                                v_cache: torch.Tensor, seqlens: torch.Tensor, *, num_heads: int,
                                num_kv_heads: int, head_dim: int, max_seq_len: int, scale: float,
                                window: int = 0, workspace: Optional[torch.Tensor] = None,
                                out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """executeFlashAttentionV11 (Hesper/WGSL/FlashAttentionExperiments.lean:572), batched.

    q [B, H, D] f32 or f16; k_cache / v_cache [B, Hkv, max_seq_len, D] f16;
    seqlens [B] int32 (the reference's params[1] = cacheLen, one per sequence).
    """
    if q.dtype not in (torch.float32, torch.float16):
        raise TypeError("q must be f32 or f16")
    _need(q, q.dtype, "q")
    _need(k_cache, torch.float16, "k_cache")
    _need(v_cache, torch.float16, "v_cache")
    _need(seqlens, torch.int32, "seqlens")
    B = seqlens.numel()
    if workspace is None:
        workspace = flash_attention_workspace(ctx, B, num_heads, num_kv_heads, head_dim,
                                              max_seq_len, q.device)
    o = out if out is not None else torch.empty((B, num_heads, head_dim), dtype=torch.float32,
                                                device=q.device)
    check(ctx._lib.hb200_attn_decode(
        ctx.handle, _ptr(q), int(q.dtype == torch.float16), _ptr(k_cache), _ptr(v_cache),
        _ptr(seqlens), B, num_heads, num_kv_heads, head_dim, max_seq_len, int(window),
        C.c_float(scale), _ptr(workspace), C.c_size_t(workspace.numel()), _ptr(o),
        _stream_handle(stream)))
    return o
