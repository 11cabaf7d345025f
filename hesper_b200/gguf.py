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
