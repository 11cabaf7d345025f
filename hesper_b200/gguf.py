"""Minimal GGUF (v3) reader/writer for the tensor types the kernels consume verbatim.

Mirrors what the reference's loader hands to its layers (Hesper/GGUF/Parser.lean:108-310,
Hesper/GGUF/Loader.lean:369-405,589-619, type ids Hesper/GGUF/Types.lean:86-132):
  * i2_s ternary tensors are stored under GGML type id 36; the blob is numel/4 packed bytes,
    then the f32 per-tensor scale at byte numel/4, then 28 bytes of padding;
  * Q4_K (12) and Q8_0 (8) tensors are raw block arrays; F32 (0), F16 (1), BF16 (30) are plain.
The payload bytes are returned as numpy views of the memory-mapped file, so they can be
uploaded to the GPU without any re-encoding.  `write_gguf` produces files in the same layout
(used by the tests; no real checkpoint is needed).
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Dict, List, Tuple

import numpy as np

GGUF_MAGIC = 0x46554747  # "GGUF" little-endian
GGUF_VERSION = 3
DEFAULT_ALIGNMENT = 32

T_F32, T_F16, T_Q8_0, T_Q4_K, T_BF16, T_I2_S = 0, 1, 8, 12, 30, 36

# (block elements, block bytes)
BLOCK = {T_F32: (1, 4), T_F16: (1, 2), T_BF16: (1, 2), T_Q8_0: (32, 34), T_Q4_K: (256, 144)}

_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q",
            11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9


@dataclass
class TensorInfo:
    name: str
    shape: Tuple[int, ...]   # GGUF order: innermost (K) first
    ggml_type: int
    offset: int              # relative to the data section

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    def nbytes(self) -> int:
        if self.ggml_type == T_I2_S:
            return self.numel // 4 + 32
        be, bb = BLOCK[self.ggml_type]
        return self.numel // be * bb


class GGUFFile:
    def __init__(self, path: str):
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.metadata: Dict[str, object] = {}
        self.tensors: Dict[str, TensorInfo] = {}
        self._parse()

    # -- parsing -----------------------------------------------------------------------
    def _rd(self, fmt: str, off: int):
        v = struct.unpack_from(fmt, self._mm, off)
        return v[0], off + struct.calcsize(fmt)

    def _rd_str(self, off: int):
        n, off = self._rd("<Q", off)
        return bytes(self._mm[off:off + n]).decode("utf-8", "replace"), off + n

    def _rd_value(self, vt: int, off: int):
        if vt in _SCALARS:
            return self._rd(_SCALARS[vt], off)
        if vt == _STRING:
            return self._rd_str(off)
        if vt == _ARRAY:
            et, off = self._rd("<I", off)
            n, off = self._rd("<Q", off)
            out = []
            for _ in range(n):
                v, off = self._rd_value(et, off)
                out.append(v)
            return out, off
        raise ValueError(f"unknown GGUF metadata value type {vt}")

    def _parse(self):
        magic, off = self._rd("<I", 0)
        if magic != GGUF_MAGIC:
            raise ValueError(f"Invalid GGUF magic: 0x{magic:x} (expected 0x{GGUF_MAGIC:x})")
        version, off = self._rd("<I", off)
        if version != GGUF_VERSION:
            raise ValueError(f"Unsupported GGUF version: {version} (expected {GGUF_VERSION})")
        n_tensors, off = self._rd("<Q", off)
        n_kv, off = self._rd("<Q", off)
        for _ in range(n_kv):
            key, off = self._rd_str(off)
            vt, off = self._rd("<I", off)
            self.metadata[key], off = self._rd_value(vt, off)
        infos: List[TensorInfo] = []
        for _ in range(n_tensors):
            name, off = self._rd_str(off)
            nd, off = self._rd("<I", off)
            shape = []
            for _ in range(nd):
                d, off = self._rd("<Q", off)
                shape.append(d)
            tt, off = self._rd("<I", off)
            toff, off = self._rd("<Q", off)
            infos.append(TensorInfo(name, tuple(shape), tt, toff))
        self.alignment = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        self.data_start = (off + self.alignment - 1) // self.alignment * self.alignment
        for t in infos:
            self.tensors[t.name] = t

    # -- tensor access -------------------------------------------------------------------
    def raw(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        if t.ggml_type != T_I2_S and t.ggml_type not in BLOCK:
            raise ValueError(f"Tensor '{name}' has unsupported type id {t.ggml_type}")
        start = self.data_start + t.offset
        return np.frombuffer(self._mm, dtype=np.uint8, count=t.nbytes(), offset=start)

    def get_i2s(self, name: str):
        """(packed bytes [numel/4], scale, numel): getI2_S_Tensor (Hesper/GGUF/Loader.lean:369-405)."""
        t = self.tensors[name]
        if t.ggml_type not in (36, 37, 38):
            raise ValueError(f"Tensor '{name}' is not i2_s format (type: {t.ggml_type})")
        blob = self.raw(name)
        packed = t.numel // 4
        scale = float(np.frombuffer(blob[packed:packed + 4].tobytes(), np.float32)[0])
        return blob[:packed], scale, t.numel

    def get_blocks(self, name: str, ggml_type: int) -> np.ndarray:
        """Raw Q4_K / Q8_0 blocks, row-major [N][K/block]."""
        t = self.tensors[name]
        if t.ggml_type != ggml_type:
            raise ValueError(f"Tensor '{name}' has type id {t.ggml_type}, wanted {ggml_type}")
        return self.raw(name)

    def get_f32(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        raw = self.raw(name)
        if t.ggml_type == T_F32:
            return raw.view(np.float32)
        if t.ggml_type == T_F16:
            return raw.view(np.float16).astype(np.float32)
        if t.ggml_type == T_BF16:
            return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
        raise ValueError(f"Tensor '{name}' is not a plain float tensor")

    def close(self):
        try:
            self._mm.close()
        except BufferError:
            pass  # tensor views still alive: the mapping goes away with the last of them
        self._f.close()


def write_gguf(path: str, metadata: Dict[str, object], tensors: List[Tuple[str, Tuple[int, ...], int, bytes]]):
    """Write a GGUF v3 file.  tensors: (name, shape innermost-first, type id, payload bytes);
    for type 36 the payload must already be packed bytes + f32 scale + 28 bytes of padding."""
    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    out = bytearray(struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(tensors), len(metadata)))
    for k, v in metadata.items():
        out += s(k)
        if isinstance(v, str):
            out += struct.pack("<I", _STRING) + s(v)
        elif isinstance(v, float):
            out += struct.pack("<If", 6, v)
        elif isinstance(v, int):
            out += struct.pack("<II", 4, v)
        else:
            raise TypeError(f"unsupported metadata value for {k}")
    off = 0
    offsets = []
    for _, _, _, payload in tensors:
        offsets.append(off)
        off = (off + len(payload) + DEFAULT_ALIGNMENT - 1) // DEFAULT_ALIGNMENT * DEFAULT_ALIGNMENT
    for (name, shape, tt, _), toff in zip(tensors, offsets):
        out += s(name) + struct.pack("<I", len(shape))
        for d in shape:
            out += struct.pack("<Q", d)
        out += struct.pack("<IQ", tt, toff)
    pad = (-len(out)) % DEFAULT_ALIGNMENT
    out += b"\0" * pad
    for (_, _, _, payload), toff in zip(tensors, offsets):
        out += payload
        out += b"\0" * ((-len(payload)) % DEFAULT_ALIGNMENT)
    with open(path, "wb") as f:
        f.write(out)


def i2s_payload(packed: np.ndarray, scale: float) -> bytes:
    """numel/4 packed bytes + f32 scale + 28 bytes of padding (the i2_s blob of a GGUF file)."""
    return bytes(np.asarray(packed, np.uint8)) + struct.pack("<f", scale) + b"\0" * 28


# ---- BitNet-shaped checkpoints -------------------------------------------------------------
#
# Tensor names and types as BitNetModel.fromGGUFObject reads them
# (Hesper/Models/BitNet.lean:788-941): token_embd.weight (F16, or BF16 here as well),
# blk.N.{attn_norm,attn_sub_norm,ffn_norm,ffn_sub_norm}.weight (F32),
# blk.N.{attn_q,attn_k,attn_v,attn_output,ffn_gate,ffn_up,ffn_down}.weight (i2_s),
# output_norm.weight (F32).  The reference takes its dimensions from a fixed configuration
# (extractConfig, :773-777); this loader reads the standard `<arch>.*` metadata keys
# (Hesper/GGUF/Reader.lean:186-202) and falls back to the tensor shapes.

_BITNET_LINEARS = (("wq", "attn_q"), ("wk", "attn_k"), ("wv", "attn_v"), ("wo", "attn_output"),
                   ("wgate", "ffn_gate"), ("wup", "ffn_up"), ("wdown", "ffn_down"))
_BITNET_NORMS = ("attn_norm", "attn_sub_norm", "ffn_norm", "ffn_sub_norm")


def save_bitnet_gguf(path: str, shape, weights: dict, arch: str = "bitnet-b1.58") -> None:
    """Write a weights dict in the layout of hesper_b200.models.random_bitnet_weights (host
    arrays) as a GGUF file; the embedding is stored as BF16 bits unless
    weights['embed_dtype'] == 1 (F16)."""
    dims = {"hidden": shape.hidden, "qdim": shape.n_heads * shape.head_dim,
            "kvdim": shape.n_kv_heads * shape.head_dim, "ffn": shape.ffn}
    io = {"wq": ("hidden", "qdim"), "wk": ("hidden", "kvdim"), "wv": ("hidden", "kvdim"),
          "wo": ("qdim", "hidden"), "wgate": ("hidden", "ffn"), "wup": ("hidden", "ffn"),
          "wdown": ("ffn", "hidden")}
    meta = {"general.architecture": arch, f"{arch}.block_count": int(shape.n_layers),
            f"{arch}.embedding_length": int(shape.hidden),
            f"{arch}.attention.head_count": int(shape.n_heads),
            f"{arch}.attention.head_count_kv": int(shape.n_kv_heads),
            f"{arch}.attention.key_length": int(shape.head_dim),
            f"{arch}.feed_forward_length": int(shape.ffn),
            f"{arch}.context_length": int(shape.max_seq),
            f"{arch}.vocab_size": int(shape.vocab),
            f"{arch}.rope.freq_base": float(shape.rope_base),
            f"{arch}.attention.layer_norm_rms_epsilon": float(shape.rms_eps)}
    emb = np.ascontiguousarray(weights["embed"]).view(np.uint16).reshape(shape.vocab, shape.hidden)
    emb_type = T_F16 if int(weights.get("embed_dtype", 0)) == 1 else T_BF16
    tensors = [("token_embd.weight", (shape.hidden, shape.vocab), emb_type, emb.tobytes())]
    for i, L in enumerate(weights["layers"]):
        for nm in _BITNET_NORMS:
            a = np.ascontiguousarray(L[nm], np.float32)
            tensors.append((f"blk.{i}.{nm}.weight", (a.size,), T_F32, a.tobytes()))
        for key, gname in _BITNET_LINEARS:
            K, N = dims[io[key][0]], dims[io[key][1]]
            tensors.append((f"blk.{i}.{gname}.weight", (K, N), T_I2_S,
                            i2s_payload(np.ascontiguousarray(L[key], np.uint8),
                                        float(L["s" + key[1:]]))))
    fn = np.ascontiguousarray(weights["final_norm"], np.float32)
    tensors.append(("output_norm.weight", (fn.size,), T_F32, fn.tobytes()))
    write_gguf(path, meta, tensors)


def load_bitnet_gguf(path: str, max_seq: int = 0):
    """(BitNetShape, weights dict) from a GGUF file: the payloads are views of the mapped
    file in exactly the bytes the kernels consume (packed i2_s + one f32 scale per tensor)."""
    from .models import BitNetShape
    g = GGUFFile(path)
    arch = g.metadata.get("general.architecture", "bitnet-b1.58")

    def md(key, default=None):
        return g.metadata.get(f"{arch}.{key}", default)

    emb_t = g.tensors["token_embd.weight"]
    hidden = int(md("embedding_length", emb_t.shape[0]))
    vocab = int(md("vocab_size", emb_t.shape[1]))
    n_layers = int(md("block_count", 0))
    if not n_layers:
        while f"blk.{n_layers}.attn_q.weight" in g.tensors:
            n_layers += 1
    n_heads = int(md("attention.head_count", 0))
    qdim = g.tensors["blk.0.attn_q.weight"].shape[1]
    kvdim = g.tensors["blk.0.attn_k.weight"].shape[1]
    head_dim = int(md("attention.key_length", qdim // n_heads if n_heads else 128))
    n_heads = n_heads or qdim // head_dim
    n_kv = int(md("attention.head_count_kv", kvdim // head_dim))
    ffn = int(md("feed_forward_length", g.tensors["blk.0.ffn_gate.weight"].shape[1]))
    ctx_len = int(md("context_length", 2304))
    shape = BitNetShape(n_layers=n_layers, hidden=hidden, n_heads=n_heads, n_kv_heads=n_kv,
                        head_dim=head_dim, ffn=ffn, vocab=vocab, max_seq=max_seq or ctx_len,
                        rope_base=float(md("rope.freq_base", 500000.0)),
                        rms_eps=float(md("attention.layer_norm_rms_epsilon", 1e-5)))
    if emb_t.ggml_type not in (T_F16, T_BF16):
        raise ValueError(f"token_embd.weight has type id {emb_t.ggml_type}; F16 or BF16 expected")
    layers = []
    for i in range(n_layers):
        L = {nm: g.get_f32(f"blk.{i}.{nm}.weight") for nm in _BITNET_NORMS}
        for key, gname in _BITNET_LINEARS:
            packed, scale, _ = g.get_i2s(f"blk.{i}.{gname}.weight")
            L[key] = packed
            L["s" + key[1:]] = np.float32(scale)
        layers.append(L)
    weights = {"layers": layers,
               "embed": g.raw("token_embd.weight").view(np.uint16).reshape(vocab, hidden),
               "embed_dtype": 1 if emb_t.ggml_type == T_F16 else 0,
               "final_norm": g.get_f32("output_norm.weight"), "_file": g}
    return shape, weights
