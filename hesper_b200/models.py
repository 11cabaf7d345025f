"""Host-side mirror of Hesper.Models.BitNet (Hesper/Models/BitNet.lean:189-199,403,594)
over the C++ decode engine in the CUDA library.  Weights are uploaded verbatim; all
computation happens in the library."""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import List, Optional

import numpy as np
import torch

from . import _lib, formats
from ._lib import BitNetConfig, BitNetLayer, check
from .layers import Context, _stream_handle


@dataclasses.dataclass
class BitNetShape:
    n_layers: int = 30
    hidden: int = 2560
    n_heads: int = 20
    n_kv_heads: int = 5
    head_dim: int = 128
    ffn: int = 6912
    vocab: int = 128256
    max_seq: int = 2304
    rope_base: float = 500000.0
    rms_eps: float = 1e-5

    @classmethod
    def bitnet_2b(cls, max_seq: int = 2304) -> "BitNetShape":
        """Config.bitnet2B (Hesper/Models/BitNet.lean:189-199)."""
        return cls(max_seq=max_seq)


LAYER_TENSORS = [("wq", "hidden", "qdim"), ("wk", "hidden", "kvdim"), ("wv", "hidden", "kvdim"),
                 ("wo", "qdim", "hidden"), ("wgate", "hidden", "ffn"), ("wup", "hidden", "ffn"),
                 ("wdown", "ffn", "hidden")]


def random_bitnet_weights(shape: BitNetShape, seed: int = 0x1337C0DE, device=None):
    """Random-init weights in the on-disk formats: ternary i2_s linears (P = 1/4, 1/2, 1/4,
    scale ~ U(0.01, 0.1)), norm gains 1 + small jitter, bf16 embedding ~ N(0, 0.02).
    Returns a dict of numpy arrays (host) or, with `device`, generates large tensors there."""
    rng = np.random.default_rng(seed)
    dims = {"hidden": shape.hidden, "qdim": shape.n_heads * shape.head_dim,
            "kvdim": shape.n_kv_heads * shape.head_dim, "ffn": shape.ffn}
    layers = []
    for _ in range(shape.n_layers):
        L = {}
        for name, kin, nout in LAYER_TENSORS:
            K, N = dims[kin], dims[nout]
            L[name] = formats.i2s_pack(formats.random_ternary(rng, N, K))
            L["s" + name[1:]] = np.float32(rng.uniform(0.01, 0.1))
        L["attn_norm"] = (1.0 + 0.05 * rng.standard_normal(shape.hidden)).astype(np.float32)
        L["attn_sub_norm"] = (1.0 + 0.05 * rng.standard_normal(dims["qdim"])).astype(np.float32)
        L["ffn_norm"] = (1.0 + 0.05 * rng.standard_normal(shape.hidden)).astype(np.float32)
        L["ffn_sub_norm"] = (1.0 + 0.05 * rng.standard_normal(shape.ffn)).astype(np.float32)
        layers.append(L)
    emb = (0.02 * rng.standard_normal((shape.vocab, shape.hidden), dtype=np.float32))
    emb_bf16 = torch.from_numpy(emb).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    final_norm = (1.0 + 0.05 * rng.standard_normal(shape.hidden)).astype(np.float32)
    return {"layers": layers, "embed": emb_bf16, "final_norm": final_norm}


def random_bitnet_weights_device(shape: BitNetShape, seed: int = 0x1337C0DE, device="cuda"):
    """Same distributions as random_bitnet_weights, generated on the GPU (seconds instead of
    minutes at the 2B size).  Values differ from the host generator; use it where no CPU
    comparison is needed (benchmarks)."""
    g = torch.Generator(device=device).manual_seed(seed)
    dims = {"hidden": shape.hidden, "qdim": shape.n_heads * shape.head_dim,
            "kvdim": shape.n_kv_heads * shape.head_dim, "ffn": shape.ffn}

    def ternary_packed(N, K):
        u = torch.randint(0, 4, (N, K // 128, 4, 32), device=device, generator=g, dtype=torch.uint8)
        c = (u + 1) // 2  # codes 0,1,1,2 -> P(-1,0,+1) = 1/4,1/2,1/4
        b = (c[:, :, 0] << 6) | (c[:, :, 1] << 4) | (c[:, :, 2] << 2) | c[:, :, 3]
        return b.reshape(-1).contiguous()

    layers = []
    for _ in range(shape.n_layers):
        L = {}
        for name, kin, nout in LAYER_TENSORS:
            L[name] = ternary_packed(dims[nout], dims[kin])
            L["s" + name[1:]] = float(torch.empty(1).uniform_(0.01, 0.1).item())
        for nm, d in (("attn_norm", shape.hidden), ("attn_sub_norm", dims["qdim"]),
                      ("ffn_norm", shape.hidden), ("ffn_sub_norm", shape.ffn)):
            L[nm] = 1.0 + 0.05 * torch.randn(d, device=device, generator=g)
        layers.append(L)
    emb = (0.02 * torch.randn(shape.vocab, shape.hidden, device=device, generator=g)).to(torch.bfloat16)
    final_norm = 1.0 + 0.05 * torch.randn(shape.hidden, device=device, generator=g)
    return {"layers": layers, "embed": emb.view(torch.int16), "final_norm": final_norm}


class BitNetModel:
    """BitNet-b1.58-shaped model resident on one GPU."""

    def __init__(self, ctx: Context, shape: BitNetShape, weights: dict, batch: int = 1,
                 max_new_tokens: int = 128):
        self.ctx, self.shape, self.batch = ctx, shape, batch
        self.max_new_tokens = max_new_tokens
        dev = torch.device("cuda", ctx.device)
        self._keep: List[torch.Tensor] = []

        def up(a, dt=None):
            if isinstance(a, torch.Tensor):
                t = a.to(dev).contiguous()
            else:
                a = np.ascontiguousarray(a)
                t = torch.from_numpy(a if a.flags.writeable else a.copy()).to(dev)
            self._keep.append(t)
            return t

        arr = (BitNetLayer * shape.n_layers)()
        for i, L in enumerate(weights["layers"]):
            f = {}
            for name in ("attn_norm", "attn_sub_norm", "ffn_norm", "ffn_sub_norm"):
                f[name] = up(L[name]).data_ptr()
            for name, _, _ in LAYER_TENSORS:
                f[name] = up(L[name]).data_ptr()
                f["s" + name[1:]] = up(np.array([L["s" + name[1:]]], np.float32)).data_ptr()
            arr[i] = BitNetLayer(**f)
        emb = weights["embed"]
        self.embed = up(emb if isinstance(emb, torch.Tensor) else emb.view(np.int16))
        self.final_norm = up(weights["final_norm"])
        cfg = BitNetConfig(shape.n_layers, shape.hidden, shape.n_heads, shape.n_kv_heads,
                           shape.head_dim, shape.ffn, shape.vocab, shape.max_seq,
                           shape.rope_base, shape.rms_eps)
        h = C.c_void_p()
        check(ctx._lib.hb200_bitnet_create(ctx.handle, C.byref(cfg), arr, self.embed.data_ptr(),
                                           int(weights.get("embed_dtype", 0)),
                                           self.final_norm.data_ptr(), batch, max_new_tokens,
                                           C.byref(h)))
        self._h = h

    def reset(self):
        check(self.ctx._lib.hb200_bitnet_reset(self._h, None))

    def step(self, tokens: Optional[torch.Tensor] = None, want_logits: bool = False, stream=None):
        """forwardSingleToken for every sequence; returns (tokens [B] int32, logits or None)."""
        if tokens is not None and (tokens.dtype != torch.int32 or not tokens.is_cuda):
            raise TypeError("tokens must be an int32 CUDA tensor")
        check(self.ctx._lib.hb200_bitnet_step(self._h, None if tokens is None else tokens.data_ptr(),
                                              int(want_logits), _stream_handle(stream)))
        torch.cuda.synchronize()
        n = self.batch
        tp = self.ctx._lib.hb200_bitnet_tokens(self._h)
        toks = _from_ptr(tp, n, np.int32)
        logits = None
        if want_logits:
            logits = _from_ptr(self.ctx._lib.hb200_bitnet_logits(self._h), n * self.shape.vocab,
                               np.float32).reshape(n, self.shape.vocab)
        return toks, logits

    def generate(self, prompt: np.ndarray, n_new: int, use_graph: bool = True):
        """generate (Hesper/Models/BitNet.lean:594): returns (tokens [B, n_new], ms_prefill, ms_decode)."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int32).reshape(self.batch, -1)
        out = np.empty((self.batch, n_new), np.int32)
        a, b = C.c_float(0), C.c_float(0)
        check(self.ctx._lib.hb200_bitnet_generate(
            self._h, prompt.ctypes.data_as(C.c_void_p), prompt.shape[1], n_new, int(use_graph),
            out.ctypes.data_as(C.c_void_p), C.byref(a), C.byref(b), None))
        return out, a.value, b.value

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self.ctx._lib.hb200_bitnet_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _from_ptr(ptr: int, n: int, dtype) -> np.ndarray:
    """Copy n elements from a raw device pointer to the host (test / inspection helper)."""
    nbytes = n * np.dtype(dtype).itemsize
    # wrap the raw pointer as a torch tensor through the CUDA array interface
    class _Raw:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False),
                                    "version": 2}
    t = torch.as_tensor(_Raw(), device="cuda")
    return t.cpu().numpy().view(dtype).copy()
