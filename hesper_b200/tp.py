"""Tensor-parallel sharding of the Gemma-shaped model and the host side of the exchange.

The reference is single-GPU; this module is new.  Sharding rules (one process per GPU):
  * q/k/v, gate, up and the LM head are split by OUTPUT rows: a rank takes a contiguous range
    of query heads, the KV head(s) those heads attend to, and the same fraction of the FFN and
    vocabulary rows.  Rows are contiguous in the GGUF layout, so a shard is a byte slice.
  * o_proj and down_proj are split by INPUT columns on Q4_K super-block (256-weight)
    boundaries: for every output row the rank keeps the blocks of its input slice.  Each rank
    then produces a full-length partial vector; one f32 sum all-reduce makes the result.
  * KV heads are sharded while there are at least as many as ranks and replicated beyond
    (8 query / 2 KV heads at TP 4: ranks 0,1 hold KV head 0, ranks 2,3 KV head 1).
"""
from __future__ import annotations

import os

import ctypes as C
import dataclasses

import numpy as np
import torch

from . import formats
from ._lib import GemmaConfig, GemmaLayer, HesperB200Error, check
from .layers import Context, _stream_handle

Q4K = formats.Q4K_BLOCK_BYTES


@dataclasses.dataclass
class GemmaShape:
    """Gemma-4-E4B-shaped benchmark model (Hesper/Models/Gemma4/Config.lean:19-45, simplified:
    one head size, 5 sliding-window layers per global layer, plain Q4_K layers)."""
    n_layers: int = 42
    hidden: int = 2560
    n_heads: int = 8
    n_kv_heads: int = 2
    head_dim: int = 256
    ffn: int = 10240
    vocab: int = 262144
    max_seq: int = 8192
    window: int = 512
    global_every: int = 6
    rope_base: float = 1000000.0
    rms_eps: float = 1e-6
    attn_scale: float = 1.0 / 16.0
    embed_scale: float = 2560.0 ** 0.5


@dataclasses.dataclass
class ShardPlan:
    rank: int
    size: int
    q_heads: range       # global query heads of this rank
    kv_heads: range      # global KV heads this rank needs
    ffn_rows: range
    vocab_rows: range

    @property
    def local_q(self):
        return len(self.q_heads)

    @property
    def local_kv(self):
        return len(self.kv_heads)


def plan(shape: GemmaShape, rank: int, size: int) -> ShardPlan:
    if shape.n_heads % size or shape.ffn % (size * 256) or shape.vocab % size:
        raise ValueError("heads, FFN/256 and vocab must divide by the TP size")
    lq = shape.n_heads // size
    G = shape.n_heads // shape.n_kv_heads
    q = range(rank * lq, (rank + 1) * lq)
    kv = range(q.start // G, (q.stop - 1) // G + 1)
    if (lq * shape.head_dim) % 256:
        raise ValueError("a rank's attention width must be a multiple of 256")
    lf, lv = shape.ffn // size, shape.vocab // size
    return ShardPlan(rank, size, q, kv, range(rank * lf, (rank + 1) * lf),
                     range(rank * lv, (rank + 1) * lv))


def shard_rows(blocks: np.ndarray, K: int, rows: range) -> np.ndarray:
    """Rows [rows) of a Q4_K tensor [N][K]: a contiguous byte slice."""
    rb = K // 256 * Q4K
    return np.ascontiguousarray(blocks.reshape(-1)[rows.start * rb:rows.stop * rb])


def shard_cols(blocks: np.ndarray, N: int, K: int, cols: range) -> np.ndarray:
    """Input columns [cols) (multiples of 256) of a Q4_K tensor [N][K] as a tensor [N][len(cols)]."""
    if cols.start % 256 or cols.stop % 256:
        raise ValueError("column shards must fall on 256-weight super-block boundaries")
    b = blocks.reshape(N, K // 256, Q4K)
    return np.ascontiguousarray(b[:, cols.start // 256:cols.stop // 256, :]).reshape(-1)


def random_gemma_weights(shape: GemmaShape, seed: int = 0x1337C0DE):
    """Full (unsharded) random-init weights in GGUF Q4_K block form, numpy, with d in U(1e-3, 1e-2), dmin in U(0, 1e-2),
    uniform 6-bit scales / mins and 4-bit quants; bf16 embedding ~ N(0, 0.02)."""
    rng = np.random.default_rng(seed)
    qd, kvd = shape.n_heads * shape.head_dim, shape.n_kv_heads * shape.head_dim
    layers = []
    for _ in range(shape.n_layers):
        L = {"wq": formats.random_q4k(rng, qd, shape.hidden),
             "wk": formats.random_q4k(rng, kvd, shape.hidden),
             "wv": formats.random_q4k(rng, kvd, shape.hidden),
             "wo": formats.random_q4k(rng, shape.hidden, qd),
             "wgate": formats.random_q4k(rng, shape.ffn, shape.hidden),
             "wup": formats.random_q4k(rng, shape.ffn, shape.hidden),
             "wdown": formats.random_q4k(rng, shape.hidden, shape.ffn)}
        for n in ("attn_norm", "post_attn_norm", "ffn_norm", "post_ffn_norm"):
            L[n] = (1.0 + 0.05 * rng.standard_normal(shape.hidden)).astype(np.float32)
        layers.append(L)
    emb = 0.02 * rng.standard_normal((shape.vocab, shape.hidden), dtype=np.float32)
    emb = torch.from_numpy(emb).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    return {"layers": layers, "embed": emb,
            "lm_head": formats.random_q4k(rng, shape.vocab, shape.hidden),
            "final_norm": (1.0 + 0.05 * rng.standard_normal(shape.hidden)).astype(np.float32)}


def shard_weights(shape: GemmaShape, w: dict, p: ShardPlan) -> dict:
    D, Hd = shape.head_dim, shape.hidden
    qrows = range(p.q_heads.start * D, p.q_heads.stop * D)
    kvrows = range(p.kv_heads.start * D, p.kv_heads.stop * D)
    qd = shape.n_heads * D
    layers = []
    for L in w["layers"]:
        S = {n: L[n] for n in ("attn_norm", "post_attn_norm", "ffn_norm", "post_ffn_norm")}
        S["wq"] = shard_rows(L["wq"], Hd, qrows)
        S["wk"] = shard_rows(L["wk"], Hd, kvrows)
        S["wv"] = shard_rows(L["wv"], Hd, kvrows)
        S["wo"] = shard_cols(L["wo"], Hd, qd, qrows)
        S["wgate"] = shard_rows(L["wgate"], Hd, p.ffn_rows)
        S["wup"] = shard_rows(L["wup"], Hd, p.ffn_rows)
        S["wdown"] = shard_cols(L["wdown"], Hd, shape.ffn, p.ffn_rows)
        layers.append(S)
    return {"layers": layers, "embed": w["embed"], "final_norm": w["final_norm"],
            "lm_head": shard_rows(w["lm_head"], Hd, p.vocab_rows)}


def random_q4k_device(n_blocks: int, gen: torch.Generator, device="cuda") -> torch.Tensor:
    """Random Q4_K blocks generated on the GPU (benchmarks): d in U(1e-3, 1e-2), dmin in U(0, 1e-2) as
    f16, every other byte uniform (all bit patterns of scales and quants are valid)."""
    b = torch.randint(0, 256, (n_blocks, Q4K), dtype=torch.uint8, device=device, generator=gen)
    d = torch.empty(n_blocks, device=device).uniform_(1e-3, 1e-2, generator=gen).half()
    m = torch.empty(n_blocks, device=device).uniform_(0.0, 1e-2, generator=gen).half()
    b[:, 0:2] = d.view(torch.uint8).reshape(n_blocks, 2)
    b[:, 2:4] = m.view(torch.uint8).reshape(n_blocks, 2)
    return b.reshape(-1)


def random_gemma_shard_device(shape: GemmaShape, p: ShardPlan, seed: int = 7, device="cuda") -> dict:
    """This rank's shard of a random-init model, generated on its GPU.  Every tensor is drawn
    whole from its own seed (the same on every rank) and the rank keeps its slice, so the
    shards of any TP size are slices of ONE model and the tokens of different TP sizes can be
    compared.  One full tensor is alive at a time (the largest, the LM head, is 377 MB)."""
    D, Hd = shape.head_dim, shape.hidden
    qd, kvd = shape.n_heads * D, shape.n_kv_heads * D
    qrows = slice(p.q_heads.start * D, p.q_heads.stop * D)
    kvrows = slice(p.kv_heads.start * D, p.kv_heads.stop * D)
    frows = slice(p.ffn_rows.start, p.ffn_rows.stop)
    counter = [0]

    def gen():
        counter[0] += 1
        return torch.Generator(device=device).manual_seed(seed * 100003 + counter[0])

    def full(N, K):
        return random_q4k_device(N * (K // 256), gen(), device).view(N, K // 256, Q4K)

    def rows(N, K, sl):
        return full(N, K)[sl].contiguous().reshape(-1)

    def cols(N, K, sl):  # input columns, in super-blocks of 256
        return full(N, K)[:, sl.start // 256:sl.stop // 256].contiguous().reshape(-1)

    layers = []
    for _ in range(shape.n_layers):
        S = {n: 1.0 + 0.05 * torch.randn(Hd, device=device, generator=gen())
             for n in ("attn_norm", "post_attn_norm", "ffn_norm", "post_ffn_norm")}
        S["wq"] = rows(qd, Hd, qrows)
        S["wk"] = rows(kvd, Hd, kvrows)
        S["wv"] = rows(kvd, Hd, kvrows)
        S["wo"] = cols(Hd, qd, qrows)
        S["wgate"] = rows(shape.ffn, Hd, frows)
        S["wup"] = rows(shape.ffn, Hd, frows)
        S["wdown"] = cols(Hd, shape.ffn, frows)
        layers.append(S)
    emb = (0.02 * torch.randn(shape.vocab, Hd, device=device, generator=gen())).to(torch.bfloat16)
    final_norm = 1.0 + 0.05 * torch.randn(Hd, device=device, generator=gen())
    lm_head = rows(shape.vocab, Hd, slice(p.vocab_rows.start, p.vocab_rows.stop))
    return {"layers": layers, "embed": emb.view(torch.int16), "final_norm": final_norm,
            "lm_head": lm_head}


class TensorParallel:
    """NCCL communicator behind the C ABI.  `exchange_id` carries rank 0's 128-byte id to the
    other ranks through an already initialised torch.distributed group (any backend)."""

    def __init__(self, ctx: Context, rank: int, size: int, id_bytes: bytes):
        self.ctx, self.rank, self.size = ctx, rank, size
        h = C.c_void_p()
        buf = (C.c_ubyte * 128).from_buffer_copy(id_bytes)
        check(ctx._lib.hb200_tp_init(ctx.handle, rank, size, buf, C.byref(h)))
        self._h = h

    @staticmethod
    def make_id(ctx: Context) -> bytes:
        buf = (C.c_ubyte * 128)()
        check(ctx._lib.hb200_tp_unique_id(buf))
        return bytes(buf)

    @classmethod
    def from_torch_distributed(cls, ctx: Context) -> "TensorParallel":
        import torch.distributed as dist
        rank, size = dist.get_rank(), dist.get_world_size()
        box = [cls.make_id(ctx) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        tp = cls(ctx, rank, size, box[0])
        if size > 1 and size <= 8 and os.environ.get("HB200_TP_NO_PEER", "0") != "1":
            tp.attach_peers(dist)
        return tp

    def attach_peers(self, dist) -> bool:
        """Map every rank's exchange buffer (CUDA IPC) so that the small all-reduces of decode
        run as one push kernel per rank instead of an NCCL call.  All ranks attach or none:
        a rank that cannot export or open a handle makes every rank stay on NCCL."""
        lib = self.ctx._lib
        nb = int(lib.hb200_tp_peer_handle_bytes())
        mine = (C.c_ubyte * nb)()
        ok = lib.hb200_tp_peer_export(self._h, mine) == 0
        gathered = [None] * self.size
        dist.all_gather_object(gathered, bytes(mine) if ok else None)
        if any(g is None for g in gathered):
            return False
        blob = (C.c_ubyte * (nb * self.size)).from_buffer_copy(b"".join(gathered))
        ok = lib.hb200_tp_peer_attach(self._h, blob) == 0
        flags = [None] * self.size
        dist.all_gather_object(flags, bool(ok))
        if not all(flags):
            raise HesperB200Error(-1, "tp: some ranks attached the peer buffers and some did not")
        return True

    @property
    def peer_attached(self) -> bool:
        return bool(self.ctx._lib.hb200_tp_peer_attached(self._h))

    @property
    def handle(self):
        return self._h

    def allreduce_f32(self, t: torch.Tensor, stream=None):
        check(self.ctx._lib.hb200_tp_allreduce_f32(self._h, C.c_void_p(t.data_ptr()),
                                                   C.c_size_t(t.numel()), _stream_handle(stream)))

    def check(self):
        check(self.ctx._lib.hb200_tp_check(self._h))

    def set_timeout_ms(self, ms: int):
        """Bound of the exchange kernels' device-side waits (default one second)."""
        check(self.ctx._lib.hb200_tp_set_timeout_ms(self._h, int(ms)))

    def align(self, stream=None):
        """Host-side meeting point of the ranks before a run of bounded waits."""
        check(self.ctx._lib.hb200_tp_align(self._h, _stream_handle(stream)))

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self.ctx._lib.hb200_tp_destroy(self._h)
            self._h = C.c_void_p()


class GemmaModel:
    """This rank's part of a Gemma-shaped model resident on its GPU."""

    def __init__(self, ctx: Context, shape: GemmaShape, shard: dict, p: ShardPlan,
                 tp: "TensorParallel | None" = None, batch: int = 1, max_new_tokens: int = 128):
        self.ctx, self.shape, self.plan, self.batch, self.tp = ctx, shape, p, batch, tp
        dev = torch.device("cuda", ctx.device)
        self._keep = []

        def up(a):
            if isinstance(a, torch.Tensor):
                t = a.to(dev).contiguous()
            else:
                a = a.view(np.int16) if a.dtype == np.uint16 else a
                t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
            self._keep.append(t)
            return t.data_ptr()

        arr = (GemmaLayer * shape.n_layers)()
        names = ("attn_norm", "post_attn_norm", "ffn_norm", "post_ffn_norm", "wq", "wk", "wv", "wo",
                 "wgate", "wup", "wdown")
        for i, L in enumerate(shard["layers"]):
            arr[i] = GemmaLayer(**{n: up(L[n]) for n in names})
        cfg = GemmaConfig(shape.n_layers, shape.hidden, shape.head_dim, shape.vocab, shape.max_seq,
                          shape.window, shape.global_every, p.local_q, p.local_kv, len(p.ffn_rows),
                          len(p.vocab_rows), p.vocab_rows.start, shape.rope_base, shape.rms_eps,
                          shape.attn_scale, shape.embed_scale)
        h = C.c_void_p()
        check(ctx._lib.hb200_gemma_create(ctx.handle, tp.handle if tp else None, C.byref(cfg), arr,
                                          up(shard["embed"]), up(shard["lm_head"]),
                                          up(shard["final_norm"]), batch, max_new_tokens,
                                          C.byref(h)))
        self._h = h

    def set_position(self, pos: int):
        check(self.ctx._lib.hb200_gemma_set_position(self._h, int(pos), None))

    def generate(self, prompt, n_new: int, use_graph: bool = True):
        if prompt is None:
            pp, plen = None, 0
        else:
            prompt = np.ascontiguousarray(prompt, dtype=np.int32).reshape(self.batch, -1)
            pp, plen = prompt.ctypes.data_as(C.c_void_p), prompt.shape[1]
        out = np.empty((self.batch, n_new), np.int32)
        a, b = C.c_float(0), C.c_float(0)
        check(self.ctx._lib.hb200_gemma_generate(self._h, pp, plen, n_new, int(use_graph),
                                                 out.ctypes.data_as(C.c_void_p), C.byref(a),
                                                 C.byref(b), None))
        return out, a.value, b.value

    def step(self, tokens: "torch.Tensor | None" = None):
        """One decode step; returns (tokens [B], this rank's logits slice [B, local_vocab])."""
        from .models import _from_ptr
        check(self.ctx._lib.hb200_gemma_step(self._h, None if tokens is None else tokens.data_ptr(),
                                             None))
        torch.cuda.synchronize()
        n, lv = self.batch, len(self.plan.vocab_rows)
        toks = _from_ptr(self.ctx._lib.hb200_gemma_tokens(self._h), n, np.int32)
        logits = _from_ptr(self.ctx._lib.hb200_gemma_local_logits(self._h), n * lv, np.float32)
        return toks, logits.reshape(n, lv)

    @property
    def chunk(self) -> int:
        """Prompt positions per sequence one prefill pass takes."""
        return int(self.ctx._lib.hb200_gemma_chunk(self._h))

    def prefill(self, tokens: "torch.Tensor"):
        """One pass over T consecutive prompt positions per sequence (tokens int32 [B, T],
        T <= chunk); returns what step() returns, for each sequence's last position."""
        from .models import _from_ptr
        assert tokens.dtype == torch.int32 and tokens.is_cuda and tokens.is_contiguous()
        assert tokens.shape[0] == self.batch
        check(self.ctx._lib.hb200_gemma_prefill(self._h, tokens.data_ptr(), int(tokens.shape[1]),
                                                1, None))
        torch.cuda.synchronize()
        n, lv = self.batch, len(self.plan.vocab_rows)
        toks = _from_ptr(self.ctx._lib.hb200_gemma_tokens(self._h), n, np.int32)
        logits = _from_ptr(self.ctx._lib.hb200_gemma_local_logits(self._h), n * lv, np.float32)
        return toks, logits.reshape(n, lv)

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self.ctx._lib.hb200_gemma_destroy(self._h)
            self._h = C.c_void_p()
