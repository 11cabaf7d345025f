"""GPU: the library inside a CUDA context the HOST made with the driver API.

The reference creates its context with cuCtxCreate (native/cuda_bridge.cpp:78-82), allocates
with cuMemAlloc and passes raw CUdeviceptr / CUstream values across its FFI
(Hesper/CUDA/FFI.lean:21-25).  hb200_ctx_create_current adopts exactly such a context.  The
test plays the host through ctypes on libcuda: context, buffers and stream come from the
driver API, the three operator families run on those raw handles, results are read back with
cuMemcpyDtoH and compared with the CPU oracle.  A second test keeps two such contexts alive in
one process (kernel attributes are per context, not per process)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


class Driver:
    def __init__(self):
        try:
            self.cu = C.CDLL("libcuda.so.1")
        except OSError:
            pytest.skip("libcuda.so.1 not found")
        self.ok(self.cu.cuInit(0), "cuInit")

    def ok(self, rc, what):
        assert rc == 0, f"{what} failed with CUresult {rc}"

    def current(self):
        c = C.c_void_p()
        self.ok(self.cu.cuCtxGetCurrent(C.byref(c)), "cuCtxGetCurrent")
        return c

    def set_current(self, c):
        self.ok(self.cu.cuCtxSetCurrent(c), "cuCtxSetCurrent")

    def create(self, ordinal=0):
        dev = C.c_int()
        self.ok(self.cu.cuDeviceGet(C.byref(dev), ordinal), "cuDeviceGet")
        c = C.c_void_p()
        self.ok(self.cu.cuCtxCreate_v2(C.byref(c), 0, dev), "cuCtxCreate")
        return c

    def destroy(self, c):
        self.ok(self.cu.cuCtxDestroy_v2(c), "cuCtxDestroy")

    def upload(self, a):
        a = np.ascontiguousarray(a)
        p = C.c_uint64()
        self.ok(self.cu.cuMemAlloc_v2(C.byref(p), C.c_size_t(max(a.nbytes, 16))), "cuMemAlloc")
        self.ok(self.cu.cuMemcpyHtoD_v2(p, a.ctypes.data_as(C.c_void_p), C.c_size_t(a.nbytes)),
                "cuMemcpyHtoD")
        return p

    def empty(self, nbytes):
        p = C.c_uint64()
        self.ok(self.cu.cuMemAlloc_v2(C.byref(p), C.c_size_t(max(nbytes, 16))), "cuMemAlloc")
        return p

    def download(self, p, shape, dtype):
        out = np.empty(shape, dtype)
        self.ok(self.cu.cuMemcpyDtoH_v2(out.ctypes.data_as(C.c_void_p), p, C.c_size_t(out.nbytes)),
                "cuMemcpyDtoH")
        return out

    def stream(self):
        s = C.c_void_p()
        self.ok(self.cu.cuStreamCreate(C.byref(s), 1), "cuStreamCreate")  # non-blocking
        return s

    def sync(self, s):
        self.ok(self.cu.cuStreamSynchronize(s), "cuStreamSynchronize")


def _vp(p):
    return C.c_void_p(p.value)


def _run_three_ops(drv, lib, oracle, seed):
    """Ternary, Q4_K and attention on driver-API buffers in the context that is current."""
    from hesper_b200 import formats
    h = C.c_void_p()
    assert lib.hb200_ctx_create_current(C.byref(h)) == 0, lib.hb200_last_error()
    st = drv.stream()
    rng = np.random.default_rng(seed)
    # ternary i2_s x int8: bit-exact accumulators
    K, N = 2560, 640
    packed = formats.i2s_pack(formats.random_ternary(rng, N, K))
    x = rng.standard_normal((1, K)).astype(np.float32)
    y_ref, acc_ref, _ = oracle.bitlinear_forward(packed, 0.05, K, N, x)
    d_w, d_s, d_x = drv.upload(packed), drv.upload(np.float32([0.05])), drv.upload(x)
    d_acc, d_y = drv.empty(N * 4), drv.empty(N * 4)
    rc = lib.hb200_bitlinear_forward(h, _vp(d_w), _vp(d_s), K, N, _vp(d_x), 1, None, 0.0, None,
                                     _vp(d_acc), None, _vp(d_y), st)
    assert rc == 0, lib.hb200_last_error()
    drv.sync(st)
    assert np.array_equal(drv.download(d_acc, (1, N), np.int32), acc_ref)
    assert np.array_equal(drv.download(d_y, (1, N), np.float32), y_ref)
    # Q4_K: <= 1e-3 (a shape of the streaming kernel and one of the mma.sync kernel)
    for K, N in ((2560, 1000), (2560, 10240)):
        blocks = formats.random_q4k(rng, N, K)
        x = rng.standard_normal((1, K)).astype(np.float32)
        ref = oracle.q4k_matvec(blocks, K, N, x)
        d_b, d_x, d_y = drv.upload(blocks), drv.upload(x), drv.empty(N * 4)
        rc = lib.hb200_kquant_forward(h, 12, _vp(d_b), K, N, _vp(d_x), 1, None, 0.0, None,
                                      _vp(d_y), st)
        assert rc == 0, lib.hb200_last_error()
        drv.sync(st)
        y = drv.download(d_y, (1, N), np.float32)
        assert np.max(np.abs(y - ref)) <= 1e-3 * np.max(np.abs(ref))
    # decode attention: <= 2e-3
    B, H, Hkv, D, L = 2, 8, 2, 256, 700
    q = rng.standard_normal((B, H, D)).astype(np.float32)
    k = rng.standard_normal((B, Hkv, L, D)).astype(np.float16)
    v = rng.standard_normal((B, Hkv, L, D)).astype(np.float16)
    lens = np.array([L, L // 3], np.int32)
    ref = oracle.attn_decode(q, k, v, lens, H, Hkv, D, L, 1 / 16)
    nws = int(lib.hb200_attn_workspace_bytes(h, B, H, Hkv, D, L))
    d_q, d_k, d_v, d_l = drv.upload(q), drv.upload(k), drv.upload(v), drv.upload(lens)
    d_ws, d_o = drv.empty(nws), drv.empty(B * H * D * 4)
    rc = lib.hb200_attn_decode(h, _vp(d_q), 0, _vp(d_k), _vp(d_v), _vp(d_l), B, H, Hkv, D, L, 0,
                               C.c_float(1 / 16), _vp(d_ws), C.c_size_t(nws), _vp(d_o), st)
    assert rc == 0, lib.hb200_last_error()
    drv.sync(st)
    out = drv.download(d_o, (B, H, D), np.float32)
    assert np.max(np.abs(out - ref)) <= 2e-3 * np.max(np.abs(ref))
    flags = C.c_uint32(0)
    assert lib.hb200_ctx_check(h, st, C.byref(flags)) == 0 and flags.value == 0
    return h


def test_operators_inside_a_cuCtxCreate_context(oracle):
    from hesper_b200 import _lib
    lib = _lib.load()
    drv = Driver()
    before = drv.current()  # torch's primary context, if another test made one
    c = drv.create(0)       # pushed and current, like native/cuda_bridge.cpp:78-82
    try:
        h = _run_three_ops(drv, lib, oracle, seed=11)
        assert lib.hb200_ctx_destroy(h) == 0
    finally:
        drv.destroy(c)
        drv.set_current(before)


def test_two_driver_contexts_in_one_process(oracle):
    from hesper_b200 import _lib
    lib = _lib.load()
    drv = Driver()
    before = drv.current()
    c1 = drv.create(0)
    c2 = None
    try:
        h1 = _run_three_ops(drv, lib, oracle, seed=21)
        c2 = drv.create(0)  # a second context; c1 stays alive underneath
        h2 = _run_three_ops(drv, lib, oracle, seed=22)
        assert lib.hb200_ctx_destroy(h2) == 0
        drv.set_current(c1)
        assert lib.hb200_ctx_destroy(h1) == 0
    finally:
        if c2 is not None:
            drv.destroy(c2)
        drv.destroy(c1)
        drv.set_current(before)


def test_create_current_without_a_context_is_refused():
    """Checked in a child process so that no other test's context is current on the thread."""
    import subprocess
    import sys
    code = ("import ctypes as C, sys; sys.path.insert(0, %r)\n"
            "from hesper_b200 import _lib\n"
            "lib = _lib.load(); h = C.c_void_p()\n"
            "rc = lib.hb200_ctx_create_current(C.byref(h))\n"
            "print(rc, lib.hb200_last_error().decode())\n") % __import__("os").path.dirname(
                __import__("os").path.dirname(__import__("os").path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    assert r.stdout.startswith("-1 "), r.stdout
    assert "no CUDA context is current" in r.stdout
