"""ctypes binding of libhesper_b200.so -- the C ABI declared in include/hesper_b200.h.

There is no fallback: if the shared object is missing or a call fails, an
exception is raised.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libhesper_b200.so")

HB200_OK = 0
FMT_Q8_0 = 8
FMT_Q4_K = 12
FMT_I2_S = 36


class HesperB200Error(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"hesper_b200 error {code}: {msg}")
        self.code = code


class BitLinearSeg(C.Structure):
    _fields_ = [("d_packed", C.c_void_p), ("d_scale", C.c_void_p), ("d_residual", C.c_void_p),
                ("d_y", C.c_void_p), ("d_acc", C.c_void_p), ("N", C.c_int)]


class BitNetConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim",
                                       "ffn", "vocab", "max_seq")] + \
               [("rope_base", C.c_float), ("rms_eps", C.c_float)]


class BitNetLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "attn_norm", "attn_sub_norm", "ffn_norm", "ffn_sub_norm",
        "wq", "wk", "wv", "wo", "wgate", "wup", "wdown",
        "sq", "sk", "sv", "so", "sgate", "sup", "sdown")]


class GemmaConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_layers", "hidden", "head_dim", "vocab", "max_seq", "window",
                                       "global_every", "local_q_heads", "local_kv_heads",
                                       "local_ffn", "local_vocab", "vocab_offset")] + \
               [(n, C.c_float) for n in ("rope_base", "rms_eps", "attn_scale", "embed_scale")]


class GemmaLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("attn_norm", "post_attn_norm", "ffn_norm", "post_ffn_norm",
                                          "wq", "wk", "wv", "wo", "wgate", "wup", "wdown")]


class KQuantSeg(C.Structure):
    _fields_ = [("d_blocks", C.c_void_p), ("d_residual", C.c_void_p), ("d_y", C.c_void_p),
                ("N", C.c_int)]


_vp, _i, _f, _sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t

# name -> (restype, argtypes); the single source of truth for the Python side.
SIGNATURES = {
    "hb200_ctx_create": (_i, [_i, C.POINTER(_vp)]),
    "hb200_ctx_create_current": (_i, [C.POINTER(_vp)]),
    "hb200_ctx_destroy": (_i, [_vp]),
    "hb200_last_error": (C.c_char_p, []),
    "hb200_version": (_i, []),
    "hb200_ctx_sm_count": (_i, [_vp]),
    "hb200_ctx_check": (_i, [_vp, _vp, C.POINTER(C.c_uint32)]),
    "hb200_ctx_set_attn_mode": (_i, [_vp, _i]),
    "hb200_ctx_read_status": (_i, [_vp, _vp, C.POINTER(C.c_uint32)]),
    "hb200_bitlinear_forward": (_i, [_vp, _vp, _vp, _i, _i, _vp, _i, _vp, _f, _vp, _vp, _vp, _vp, _vp]),
    "hb200_bitlinear_forward_multi": (_i, [_vp, C.POINTER(BitLinearSeg), _i, _i, _vp, _i, _vp, _f, _vp, _vp]),
    "hb200_bitlinear_gateup_relu2": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _i, _vp, _f, _vp, _vp]),
    "hb200_kquant_forward": (_i, [_vp, _i, _vp, _i, _i, _vp, _i, _vp, _f, _vp, _vp, _vp]),
    "hb200_kquant_forward_multi": (_i, [_vp, _i, C.POINTER(KQuantSeg), _i, _i, _vp, _i, _vp, _f, _vp]),
    "hb200_kquant_gateup_gelu": (_i, [_vp, _i, _vp, _vp, _i, _i, _vp, _i, _vp, _f, _vp, _vp]),
    "hb200_kquant_forward_multi_pre": (_i, [_vp, _i, C.POINTER(KQuantSeg), _i, _i, _vp, _i, _vp, _vp,
                                            _vp, _vp, _f, _vp]),
    "hb200_kquant_gateup_gelu_pre": (_i, [_vp, _i, _vp, _vp, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _f,
                                          _vp, _vp]),
    "hb200_attn_workspace_bytes": (_sz, [_vp, _i, _i, _i, _i, _i]),
    "hb200_attn_decode_static": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _vp]),
    "hb200_embed_lookup": (_i, [_vp, _vp, _i, C.c_long, _i, _vp, _i, _f, _vp, _vp]),
    "hb200_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _f, _i, _i, _vp, _vp]),
    "hb200_rope_kv_write": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "hb200_argmax": (_i, [_vp, _vp, C.c_long, _i, _vp, _vp]),
    "hb200_rope_kv_write_angles": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "hb200_rope_table": (_i, [_vp, _vp, _i, _i, _i, _f, _vp, _vp]),
    "hb200_lmhead_scratch_bytes": (_sz, [_i]),
    "hb200_lmhead_argmax": (_i, [_vp, _vp, _i, C.c_long, _i, _vp, _i, _vp, _f, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "hb200_relu2_mul": (_i, [_vp, _vp, _vp, C.c_long, _vp, _vp]),
    "hb200_gelu_mul": (_i, [_vp, _vp, _vp, C.c_long, _vp, _vp]),
    "hb200_add_i32": (_i, [_vp, _vp, _i, _i, _vp]),
    "hb200_bitnet_create": (_i, [_vp, C.POINTER(BitNetConfig), C.POINTER(BitNetLayer), _vp, _i, _vp, _i, _i, C.POINTER(_vp)]),
    "hb200_bitnet_destroy": (_i, [_vp]),
    "hb200_bitnet_reset": (_i, [_vp, _vp]),
    "hb200_bitnet_step": (_i, [_vp, _vp, _i, _vp]),
    "hb200_bitnet_logits": (_vp, [_vp]),
    "hb200_bitnet_tokens": (_vp, [_vp]),
    "hb200_bitnet_generate": (_i, [_vp, _vp, _i, _i, _i, _vp, C.POINTER(_f), C.POINTER(_f), _vp]),
    "hb200_tp_unique_id": (_i, [_vp]),
    "hb200_tp_init": (_i, [_vp, _i, _i, _vp, C.POINTER(_vp)]),
    "hb200_tp_destroy": (_i, [_vp]),
    "hb200_tp_rank": (_i, [_vp]),
    "hb200_tp_size": (_i, [_vp]),
    "hb200_tp_allreduce_f32": (_i, [_vp, _vp, _sz, _vp]),
    "hb200_tp_allreduce_max_u64": (_i, [_vp, _vp, _sz, _vp]),
    "hb200_tp_check": (_i, [_vp]),
    "hb200_tp_set_timeout_ms": (_i, [_vp, _i]),
    "hb200_tp_align": (_i, [_vp, _vp]),
    "hb200_tp_allreduce_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _vp, _f, _i, _i, _vp, _vp]),
    "hb200_tp_peer_handle_bytes": (_sz, []),
    "hb200_tp_peer_export": (_i, [_vp, _vp]),
    "hb200_tp_peer_attach": (_i, [_vp, _vp]),
    "hb200_tp_peer_attached": (_i, [_vp]),
    "hb200_gemma_create": (_i, [_vp, _vp, C.POINTER(GemmaConfig), C.POINTER(GemmaLayer), _vp, _vp, _vp, _i, _i, C.POINTER(_vp)]),
    "hb200_gemma_destroy": (_i, [_vp]),
    "hb200_gemma_reset": (_i, [_vp, _vp]),
    "hb200_gemma_set_position": (_i, [_vp, _i, _vp]),
    "hb200_bitlinear_qkv_rope": (_i, [_vp, C.POINTER(BitLinearSeg), _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "hb200_gemma_step": (_i, [_vp, _vp, _vp]),
    "hb200_gemma_prefill": (_i, [_vp, _vp, _i, _i, _vp]),
    "hb200_gemma_chunk": (_i, [_vp]),
    "hb200_gemma_local_logits": (_vp, [_vp]),
    "hb200_gemma_tokens": (_vp, [_vp]),
    "hb200_gemma_generate": (_i, [_vp, _vp, _i, _i, _i, _vp, C.POINTER(_f), C.POINTER(_f), _vp]),
    "hb200_attn_decode": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp, _vp]),
    "hb200_attn_prefill_workspace_bytes": (_sz, [_vp, _i, _i, _i, _i, _i, _i]),
    "hb200_attn_prefill": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp, _vp]),
    "hb200_attn_ring": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp, _vp]),
    "hb200_rope_kv_write_prefill_angles": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "hb200_rope_kv_write_prefill": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared object and bind every declared symbol (raises if one is missing)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise HesperB200Error(-2, f"{LIB_PATH} is missing: run `python -m hesper_b200.build` "
                                      "(there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(code: int) -> None:
    if code != HB200_OK:
        raise HesperB200Error(code, load().hb200_last_error().decode("utf-8", "replace"))
