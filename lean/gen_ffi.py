#!/usr/bin/env python
"""Writes the Lean-side binding of include/hesper_b200.h:

  lean/lean_ffi.cpp     one `lean_hesper_b200_*` wrapper per exported C function, in the
                        conventions of the reference's native/cuda_bridge.cpp (no world token,
                        USize / UInt32 / Float scalars unboxed, borrowed Array USize / ByteArray
                        objects, errors as IO.userError strings, never throws or aborts)
  lean/HesperB200Extern.lean   the matching `@[extern]` declarations

Run `python lean/gen_ffi.py` after the header changes.  The plain wrappers are derived from the
declarations; the ones that take structs, host arrays or out-parameters are written out below.
"""
from __future__ import annotations

import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "..", "include", "hesper_b200.h")

# ---- declarations of the header ---------------------------------------------------------


def declarations():
    s = open(HEADER).read()
    s = re.sub(r"/\*.*?\*/", "", s, flags=re.S)
    pat = (r"\n((?:int|size_t|const char \*|const float \*|const int32_t \*)\s*\*?"
           r"(hb200_\w+)\s*\(([^;]*?)\));")
    out = []
    for full, name, args in re.findall(pat, s):
        ret = " ".join(full.split(name)[0].split())
        params = []
        args = " ".join(args.split())
        if args != "void":
            for a in args.split(","):
                a = a.strip()
                m = re.match(r"(.*?)(\w+)(\[\d+\])?$", a)
                ctype = (m.group(1).strip() + (" *" if m.group(3) else "")).strip()
                params.append((ctype, m.group(2)))
        out.append((ret, name, params))
    return out


# Lean type / C parameter type / cast expression for a scalar or pointer parameter
def scalar(ctype):
    if ctype == "int":
        return "UInt32", "uint32_t", "(int){}"
    if ctype in ("long", "size_t"):
        return "USize", "size_t", "(%s){}" % ctype
    if ctype == "float":
        return "Float", "double", "(float){}"
    if ctype == "hb200_stream":
        return "USize", "size_t", "(hb200_stream){}"
    if ctype.endswith("*"):
        return "USize", "size_t", "(%s){}" % ctype
    raise ValueError(ctype)


def lean_name(cname):
    parts = cname[len("hb200_"):].split("_")
    return parts[0] + "".join(p.capitalize() for p in parts[1:])


# ---- wrappers that are not a plain forward of scalars ---------------------------------------

SPECIAL_CPP = r'''
// ---- context -------------------------------------------------------------------------------

extern "C" lean_obj_res lean_hesper_b200_ctx_create(uint32_t device) {
  hb200_ctx* c = nullptr;
  const int rc = hb200_ctx_create((int)device, &c);
  if (rc != HB200_OK) return hb_fail();
  return lean_io_result_mk_ok(lean_box_usize((size_t)c));
}

// The context Hesper made itself (cuCtxCreate, native/cuda_bridge.cpp:78-82) is current on the
// thread: adopt it.
extern "C" lean_obj_res lean_hesper_b200_ctx_create_current() {
  hb200_ctx* c = nullptr;
  const int rc = hb200_ctx_create_current(&c);
  if (rc != HB200_OK) return hb_fail();
  return lean_io_result_mk_ok(lean_box_usize((size_t)c));
}

extern "C" lean_obj_res lean_hesper_b200_last_error() {
  return lean_io_result_mk_ok(lean_mk_string(hb200_last_error()));
}

// IO UInt32: the device status flags (0 = no bounded wait expired)
extern "C" lean_obj_res lean_hesper_b200_ctx_check(size_t ctx, size_t stream) {
  uint32_t flags = 0;
  const int rc = hb200_ctx_check((hb200_ctx*)ctx, (hb200_stream)stream, &flags);
  if (rc != HB200_OK && rc != HB200_ERR_TIMEOUT) return hb_fail();
  return lean_io_result_mk_ok(lean_box_uint32(flags));
}

// IO ByteArray: the 64 status words
extern "C" lean_obj_res lean_hesper_b200_ctx_read_status(size_t ctx, size_t stream) {
  lean_obj_res arr = lean_alloc_sarray(1, 256, 256);
  const int rc = hb200_ctx_read_status((hb200_ctx*)ctx, (hb200_stream)stream,
                                       (uint32_t*)lean_sarray_cptr(arr));
  if (rc != HB200_OK) {
    lean_dec_ref(arr);
    return hb_fail();
  }
  return lean_io_result_mk_ok(arr);
}

// ---- operators over several tensors: segments arrive as a flat Array USize ------------------

// segs: nseg x {packed, scale, residual, y, acc, N}
extern "C" lean_obj_res lean_hesper_b200_bitlinear_forward_multi(
    size_t ctx, b_lean_obj_arg segs, uint32_t K, size_t x, uint32_t M, size_t gamma, double eps,
    size_t act_scale, size_t stream) {
  const size_t n = lean_array_size(segs) / 6;
  if (n < 1 || n > 4 || lean_array_size(segs) != 6 * n) return hb_msg("bitlinearForwardMulti: 6 values per tensor, 1..4 tensors");
  hb200_bitlinear_seg s[4];
  for (size_t i = 0; i < n; ++i) {
    s[i].d_packed = (const void*)hb_usize(segs, 6 * i + 0);
    s[i].d_scale = (const float*)hb_usize(segs, 6 * i + 1);
    s[i].d_residual = (const float*)hb_usize(segs, 6 * i + 2);
    s[i].d_y = (float*)hb_usize(segs, 6 * i + 3);
    s[i].d_acc = (int32_t*)hb_usize(segs, 6 * i + 4);
    s[i].N = (int)hb_usize(segs, 6 * i + 5);
  }
  return hb_result(hb200_bitlinear_forward_multi((hb200_ctx*)ctx, s, (int)n, (int)K, (const float*)x,
                                                 (int)M, (const float*)gamma, (float)eps,
                                                 (float*)act_scale, (hb200_stream)stream));
}

// segs: nseg x {blocks, residual, y, N}
static int hb_kquant_segs(b_lean_obj_arg segs, hb200_kquant_seg* s) {
  const size_t n = lean_array_size(segs) / 4;
  if (n < 1 || n > 4 || lean_array_size(segs) != 4 * n) return -1;
  for (size_t i = 0; i < n; ++i) {
    s[i].d_blocks = (const void*)hb_usize(segs, 4 * i + 0);
    s[i].d_residual = (const float*)hb_usize(segs, 4 * i + 1);
    s[i].d_y = (float*)hb_usize(segs, 4 * i + 2);
    s[i].N = (int)hb_usize(segs, 4 * i + 3);
  }
  return (int)n;
}

extern "C" lean_obj_res lean_hesper_b200_kquant_forward_multi(
    size_t ctx, uint32_t fmt, b_lean_obj_arg segs, uint32_t K, size_t x, uint32_t M, size_t gamma,
    double eps, size_t stream) {
  hb200_kquant_seg s[4];
  const int n = hb_kquant_segs(segs, s);
  if (n < 0) return hb_msg("kquantForwardMulti: 4 values per tensor, 1..4 tensors");
  return hb_result(hb200_kquant_forward_multi((hb200_ctx*)ctx, (int)fmt, s, n, (int)K,
                                              (const float*)x, (int)M, (const float*)gamma,
                                              (float)eps, (hb200_stream)stream));
}

extern "C" lean_obj_res lean_hesper_b200_kquant_forward_multi_pre(
    size_t ctx, uint32_t fmt, b_lean_obj_arg segs, uint32_t K, size_t o, uint32_t M, size_t pre_base,
    size_t pre_gamma, size_t x_out, size_t gamma, double eps, size_t stream) {
  hb200_kquant_seg s[4];
  const int n = hb_kquant_segs(segs, s);
  if (n < 0) return hb_msg("kquantForwardMultiPre: 4 values per tensor, 1..4 tensors");
  return hb_result(hb200_kquant_forward_multi_pre(
      (hb200_ctx*)ctx, (int)fmt, s, n, (int)K, (const float*)o, (int)M, (const float*)pre_base,
      (const float*)pre_gamma, (float*)x_out, (const float*)gamma, (float)eps,
      (hb200_stream)stream));
}

// ---- decode loops: configuration as Array USize, layer tensors as a flat Array USize --------

// cfg: {n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, max_seq};
// layers: n_layers x 18 device pointers in the order of hb200_bitnet_layer
extern "C" lean_obj_res lean_hesper_b200_bitnet_create(
    size_t ctx, b_lean_obj_arg cfg, double rope_base, double rms_eps, b_lean_obj_arg layers,
    size_t embed, uint32_t embed_dtype, size_t final_norm, uint32_t batch, uint32_t max_new) {
  if (lean_array_size(cfg) != 8) return hb_msg("bitnetCreate: 8 configuration values");
  hb200_bitnet_config c;
  int* ci = &c.n_layers;
  for (int i = 0; i < 8; ++i) ci[i] = (int)hb_usize(cfg, i);
  c.rope_base = (float)rope_base;
  c.rms_eps = (float)rms_eps;
  const size_t per = sizeof(hb200_bitnet_layer) / sizeof(void*);
  if (c.n_layers < 1 || lean_array_size(layers) != per * (size_t)c.n_layers)
    return hb_msg("bitnetCreate: 18 pointers per layer");
  hb200_bitnet_layer* L = (hb200_bitnet_layer*)malloc(sizeof(hb200_bitnet_layer) * c.n_layers);
  if (!L) return hb_msg("bitnetCreate: out of host memory");
  const void** lp = (const void**)L;
  for (size_t i = 0; i < per * (size_t)c.n_layers; ++i) lp[i] = (const void*)hb_usize(layers, i);
  hb200_bitnet* m = nullptr;
  const int rc = hb200_bitnet_create((hb200_ctx*)ctx, &c, L, (const void*)embed, (int)embed_dtype,
                                     (const float*)final_norm, (int)batch, (int)max_new, &m);
  free(L);
  if (rc != HB200_OK) return hb_fail();
  return lean_io_result_mk_ok(lean_box_usize((size_t)m));
}

// cfg: the 12 integers of hb200_gemma_config; fl: rope_base, rms_eps, attn_scale, embed_scale
extern "C" lean_obj_res lean_hesper_b200_gemma_create(
    size_t ctx, size_t tp, b_lean_obj_arg cfg, double rope_base, double rms_eps, double attn_scale,
    double embed_scale, b_lean_obj_arg layers, size_t embed, size_t lm_head, size_t final_norm,
    uint32_t batch, uint32_t max_new) {
  if (lean_array_size(cfg) != 12) return hb_msg("gemmaCreate: 12 configuration values");
  hb200_gemma_config c;
  int* ci = &c.n_layers;
  for (int i = 0; i < 12; ++i) ci[i] = (int)hb_usize(cfg, i);
  c.rope_base = (float)rope_base;
  c.rms_eps = (float)rms_eps;
  c.attn_scale = (float)attn_scale;
  c.embed_scale = (float)embed_scale;
  const size_t per = sizeof(hb200_gemma_layer) / sizeof(void*);
  if (c.n_layers < 1 || lean_array_size(layers) != per * (size_t)c.n_layers)
    return hb_msg("gemmaCreate: 11 pointers per layer");
  hb200_gemma_layer* L = (hb200_gemma_layer*)malloc(sizeof(hb200_gemma_layer) * c.n_layers);
  if (!L) return hb_msg("gemmaCreate: out of host memory");
  const void** lp = (const void**)L;
  for (size_t i = 0; i < per * (size_t)c.n_layers; ++i) lp[i] = (const void*)hb_usize(layers, i);
  hb200_gemma* m = nullptr;
  const int rc = hb200_gemma_create((hb200_ctx*)ctx, (hb200_tp*)tp, &c, L, (const void*)embed,
                                    (const void*)lm_head, (const float*)final_norm, (int)batch,
                                    (int)max_new, &m);
  free(L);
  if (rc != HB200_OK) return hb_fail();
  return lean_io_result_mk_ok(lean_box_usize((size_t)m));
}

// prompt: ByteArray of batch x prompt_len little-endian int32 (empty: continue from the
// model's own tokens).  IO ByteArray: batch x n_new int32 tokens, then ms_prefill and ms_decode
// as two f32.
template <typename Model, typename Fn>
static lean_obj_res hb_generate(Model* m, Fn fn, b_lean_obj_arg prompt, uint32_t batch,
                                uint32_t prompt_len, uint32_t n_new, uint32_t use_graph,
                                size_t stream) {
  const size_t need = (size_t)batch * prompt_len * 4;
  if (lean_sarray_size(prompt) != need) return hb_msg("generate: prompt bytes != batch * prompt_len * 4");
  const size_t out_bytes = (size_t)batch * n_new * 4 + 8;
  lean_obj_res arr = lean_alloc_sarray(1, out_bytes, out_bytes);
  uint8_t* o = lean_sarray_cptr(arr);
  float ms[2] = {0.f, 0.f};
  const int rc = fn(m, need ? (const int32_t*)lean_sarray_cptr(prompt) : nullptr, (int)prompt_len,
                    (int)n_new, (int)use_graph, (int32_t*)o, &ms[0], &ms[1], (hb200_stream)stream);
  if (rc != HB200_OK) {
    lean_dec_ref(arr);
    return hb_fail();
  }
  memcpy(o + (size_t)batch * n_new * 4, ms, 8);
  return lean_io_result_mk_ok(arr);
}

extern "C" lean_obj_res lean_hesper_b200_bitnet_generate(size_t m, b_lean_obj_arg prompt,
                                                         uint32_t batch, uint32_t prompt_len,
                                                         uint32_t n_new, uint32_t use_graph,
                                                         size_t stream) {
  return hb_generate((hb200_bitnet*)m, hb200_bitnet_generate, prompt, batch, prompt_len, n_new,
                     use_graph, stream);
}

extern "C" lean_obj_res lean_hesper_b200_gemma_generate(size_t m, b_lean_obj_arg prompt,
                                                        uint32_t batch, uint32_t prompt_len,
                                                        uint32_t n_new, uint32_t use_graph,
                                                        size_t stream) {
  return hb_generate((hb200_gemma*)m, hb200_gemma_generate, prompt, batch, prompt_len, n_new,
                     use_graph, stream);
}

// ---- tensor parallelism: ids and handles as ByteArray ----------------------------------------

extern "C" lean_obj_res lean_hesper_b200_tp_unique_id() {
  lean_obj_res arr = lean_alloc_sarray(1, 128, 128);
  if (hb200_tp_unique_id(lean_sarray_cptr(arr)) != HB200_OK) {
    lean_dec_ref(arr);
    return hb_fail();
  }
  return lean_io_result_mk_ok(arr);
}

extern "C" lean_obj_res lean_hesper_b200_tp_init(size_t ctx, uint32_t rank, uint32_t nranks,
                                                 b_lean_obj_arg id) {
  if (lean_sarray_size(id) != 128) return hb_msg("tpInit: the id has 128 bytes");
  hb200_tp* tp = nullptr;
  const int rc = hb200_tp_init((hb200_ctx*)ctx, (int)rank, (int)nranks, lean_sarray_cptr(id), &tp);
  if (rc != HB200_OK) return hb_fail();
  return lean_io_result_mk_ok(lean_box_usize((size_t)tp));
}

extern "C" lean_obj_res lean_hesper_b200_tp_peer_export(size_t tp) {
  const size_t n = hb200_tp_peer_handle_bytes();
  lean_obj_res arr = lean_alloc_sarray(1, n, n);
  if (hb200_tp_peer_export((hb200_tp*)tp, lean_sarray_cptr(arr)) != HB200_OK) {
    lean_dec_ref(arr);
    return hb_fail();
  }
  return lean_io_result_mk_ok(arr);
}

extern "C" lean_obj_res lean_hesper_b200_tp_peer_attach(size_t tp, b_lean_obj_arg all_handles) {
  const size_t per = hb200_tp_peer_handle_bytes();
  const size_t n = (size_t)hb200_tp_size((hb200_tp*)tp);
  if (lean_sarray_size(all_handles) != per * n) return hb_msg("tpPeerAttach: one handle per rank, in rank order");
  return hb_result(hb200_tp_peer_attach((hb200_tp*)tp, lean_sarray_cptr(all_handles)));
}
'''

SPECIAL_LEAN = '''
@[extern "lean_hesper_b200_ctx_create"]
opaque ctxCreate (device : UInt32) : IO USize
/-- Adopts the CUDA context that is current on the thread (the one `CUDAContext.init` made). -/
@[extern "lean_hesper_b200_ctx_create_current"]
opaque ctxCreateCurrent : IO USize
@[extern "lean_hesper_b200_last_error"]
opaque lastError : IO String
@[extern "lean_hesper_b200_ctx_check"]
opaque ctxCheck (ctx stream : USize) : IO UInt32
@[extern "lean_hesper_b200_ctx_read_status"]
opaque ctxReadStatus (ctx stream : USize) : IO ByteArray
/-- `segs`: per tensor `packed, scale, residual, y, acc, N`. -/
@[extern "lean_hesper_b200_bitlinear_forward_multi"]
opaque bitlinearForwardMulti (ctx : USize) (segs : @& Array USize) (K : UInt32) (x : USize)
    (M : UInt32) (gamma : USize) (eps : Float) (actScale stream : USize) : IO Unit
/-- `segs`: per tensor `blocks, residual, y, N`. -/
@[extern "lean_hesper_b200_kquant_forward_multi"]
opaque kquantForwardMulti (ctx : USize) (fmt : UInt32) (segs : @& Array USize) (K : UInt32)
    (x : USize) (M : UInt32) (gamma : USize) (eps : Float) (stream : USize) : IO Unit
@[extern "lean_hesper_b200_kquant_forward_multi_pre"]
opaque kquantForwardMultiPre (ctx : USize) (fmt : UInt32) (segs : @& Array USize) (K : UInt32)
    (o : USize) (M : UInt32) (preBase preGamma xOut gamma : USize) (eps : Float)
    (stream : USize) : IO Unit
@[extern "lean_hesper_b200_bitnet_create"]
opaque bitnetCreate (ctx : USize) (cfg : @& Array USize) (ropeBase rmsEps : Float)
    (layers : @& Array USize) (embed : USize) (embedDtype : UInt32) (finalNorm : USize)
    (batch maxNew : UInt32) : IO USize
@[extern "lean_hesper_b200_gemma_create"]
opaque gemmaCreate (ctx tp : USize) (cfg : @& Array USize)
    (ropeBase rmsEps attnScale embedScale : Float) (layers : @& Array USize)
    (embed lmHead finalNorm : USize) (batch maxNew : UInt32) : IO USize
@[extern "lean_hesper_b200_bitnet_generate"]
opaque bitnetGenerate (m : USize) (prompt : @& ByteArray) (batch promptLen nNew useGraph : UInt32)
    (stream : USize) : IO ByteArray
@[extern "lean_hesper_b200_gemma_generate"]
opaque gemmaGenerate (m : USize) (prompt : @& ByteArray) (batch promptLen nNew useGraph : UInt32)
    (stream : USize) : IO ByteArray
@[extern "lean_hesper_b200_tp_unique_id"]
opaque tpUniqueId : IO ByteArray
@[extern "lean_hesper_b200_tp_init"]
opaque tpInit (ctx : USize) (rank nranks : UInt32) (id : @& ByteArray) : IO USize
@[extern "lean_hesper_b200_tp_peer_export"]
opaque tpPeerExport (tp : USize) : IO ByteArray
@[extern "lean_hesper_b200_tp_peer_attach"]
opaque tpPeerAttach (tp : USize) (allHandles : @& ByteArray) : IO Unit
'''

SPECIAL = {
    "hb200_ctx_create", "hb200_ctx_create_current", "hb200_last_error", "hb200_ctx_check",
    "hb200_ctx_read_status", "hb200_bitlinear_forward_multi", "hb200_kquant_forward_multi",
    "hb200_kquant_forward_multi_pre", "hb200_bitnet_create", "hb200_gemma_create",
    "hb200_bitnet_generate", "hb200_gemma_generate", "hb200_tp_unique_id", "hb200_tp_init",
    "hb200_tp_peer_export", "hb200_tp_peer_attach",
}

PRELUDE = r'''// lean_ffi.cpp -- Lean 4 FFI shim over the C ABI of include/hesper_b200.h.
//
// GENERATED by lean/gen_ffi.py: edit the generator, not this file.
//
// Sits beside Hesper's native/cuda_bridge.cpp and follows its conventions
// (native/cuda_bridge.cpp:3,18-30,374-444; Hesper/CUDA/FFI.lean:21-25,234-258):
//   * `extern "C" lean_obj_res lean_hesper_b200_<name>(args...)`, no world-token argument;
//   * USize (device pointers, streams, handles), UInt32 and Float scalars arrive unboxed;
//     `@&` Array USize / ByteArray arguments are borrowed objects;
//   * success = lean_io_result_mk_ok(...), failure = an IO.userError carrying
//     hb200_last_error(); nothing throws or aborts.
// Build: compiled into the Lake package with `-I<lean prefix>/include -I<this repo>/include` and
// linked with `-lhesper_b200` next to `-lcuda` (lakefile.lean:123-129, cudaExeArgs).
#include <lean/lean.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "hesper_b200.h"

static lean_obj_res hb_msg(const char* msg) {
  return lean_io_result_mk_error(lean_mk_io_user_error(lean_mk_string(msg)));
}
static lean_obj_res hb_fail() { return hb_msg(hb200_last_error()); }
static lean_obj_res hb_result(int rc) {
  if (rc == HB200_OK) return lean_io_result_mk_ok(lean_box(0));
  return hb_fail();
}
static size_t hb_usize(b_lean_obj_arg arr, size_t i) {
  return lean_unbox_usize(lean_array_get_core(arr, i));
}
'''


def main():
    decls = declarations()
    cpp = [PRELUDE, SPECIAL_CPP, "\n// ---- plain forwards ---------------------------------"
           "---------------------------------------\n"]
    lean = ["/-\n  GENERATED by lean/gen_ffi.py from include/hesper_b200.h: the `@[extern]` side of\n"
            "  lean/lean_ffi.cpp.  Device pointers, streams and handles are `USize`, as in\n"
            "  Hesper/CUDA/FFI.lean:21-25.\n-/\nnamespace Hesper.Backend.B200\n", SPECIAL_LEAN]
    for ret, name, params in decls:
        if name in SPECIAL:
            continue
        lname = lean_name(name)
        cargs, largs, call = [], [], []
        for ctype, pname in params:
            lt, ct, cast = scalar(ctype)
            cargs.append(f"{ct} {pname}")
            largs.append(f"({pname} : {lt})")
            call.append(cast.format(pname))
        callexpr = f"{name}({', '.join(call)})"
        if ret == "int" and name in ("hb200_version", "hb200_ctx_sm_count", "hb200_tp_rank",
                                     "hb200_tp_size", "hb200_tp_peer_attached"):
            body = f"  return lean_io_result_mk_ok(lean_box_uint32((uint32_t){callexpr}));"
            lret = "IO UInt32"
        elif ret == "int":
            body = f"  return hb_result({callexpr});"
            lret = "IO Unit"
        else:  # size_t and pointer getters
            body = f"  return lean_io_result_mk_ok(lean_box_usize((size_t){callexpr}));"
            lret = "IO USize"
        cpp.append(f'extern "C" lean_obj_res lean_{name.replace("hb200_", "hesper_b200_")}'
                   f'({", ".join(cargs)}) {{\n{body}\n}}\n')
        sig = " ".join(largs)
        lean.append(f'@[extern "lean_{name.replace("hb200_", "hesper_b200_")}"]\n'
                    f'opaque {lname} {sig + " " if sig else ""}: {lret}\n')
    lean.append("end Hesper.Backend.B200\n")
    open(os.path.join(HERE, "lean_ffi.cpp"), "w").write("\n".join(cpp))
    open(os.path.join(HERE, "HesperB200Extern.lean"), "w").write("\n".join(lean))


if __name__ == "__main__":
    main()
