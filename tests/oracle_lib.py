"""ctypes access to the test oracle (oracle/liboracle.so): numpy in, numpy out.

Test infrastructure only.  The shared object is built by `make -C oracle oracle`
(__graft_entry__.build() does it); it is rebuilt here if missing."""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SO = os.path.join(ROOT, "oracle", "liboracle.so")

ROW_MAJOR, COL_MAJOR, COL32, COL32_2R_4R4, COL4_4R2_8C = range(5)
TOKEN_UP, HIDDEN_UP = 4096.0, 8192.0
TOKEN_DOWN, HIDDEN_DOWN = 1.0 / 4096.0, 1.0 / 8192.0


def _load():
    if not os.path.exists(SO):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "oracle"], check=True)
    L = ctypes.CDLL(SO)
    vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_float
    L.orc_f32_to_f16.restype = ctypes.c_uint16
    L.orc_f32_to_f16.argtypes = [f32]
    L.orc_f64_to_f16.restype = ctypes.c_uint16
    L.orc_f64_to_f16.argtypes = [ctypes.c_double]
    L.orc_f16_to_f32.restype = f32
    L.orc_f16_to_f32.argtypes = [ctypes.c_uint16]
    L.orc_f16_add.restype = ctypes.c_uint16
    L.orc_f16_add.argtypes = [ctypes.c_uint16, ctypes.c_uint16]
    L.orc_layout_offset.restype = i64
    L.orc_layout_offset.argtypes = [i32, i64, i64, i64, i64]
    L.orc_set_threads.argtypes = [i32]
    L.orc_minmax_quantize_fp16.argtypes = [vp, i64, i64, f32, i32, vp, vp]
    L.orc_gemm_i8i8i32.argtypes = [vp, i64, vp, i64, i64, i64, i64, vp, i64]
    L.orc_gemm_i8i8i32.restype = None
    L.orc_gemm_i8i8i32_rows.argtypes = [vp, i64, vp, i64, i64, i64, i64, i64, vp, i64]
    L.orc_gemm_i8i8i32_rows.restype = None
    L.orc_minmax_dequantize_fp16.argtypes = [vp, vp, vp, vp, i64, i64, f32, f32, i32, vp]
    L.orc_skip_rmsnorm_minmax_quantize_fp16.argtypes = [vp, vp, vp, f32, i64, i64, f32, i32, vp, vp, vp]
    L.orc_activation_requantize.argtypes = [i32, vp, vp, vp, vp, vp, vp, i64, i64, f32, f32, f32, f32, vp, vp, vp]
    L.orc_dequantize_split3.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, f32, f32, vp, vp, vp]
    L.orc_w8a8_linear.argtypes = [vp, vp, vp, vp, i64, i64, i64, f32, f32, f32, f32, vp, vp, vp, vp, vp, vp]
    return L


L = _load()
L.orc_set_threads(os.cpu_count() or 1)


def set_threads(n):
    L.orc_set_threads(n)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a)
    assert a.dtype == dt, (a.dtype, dt)
    return a


def f16_bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


def quantize(x, up_scale=TOKEN_UP, layout=ROW_MAJOR):
    """x float16 [M, K] -> (q int8 flat-or-[M,K], scale float16 [M])."""
    x = _c(x, np.float16)
    M, K = x.shape
    q = np.zeros((M, K), dtype=np.int8)
    s = np.zeros((M,), dtype=np.float16)
    rc = L.orc_minmax_quantize_fp16(_p(x), M, K, up_scale, layout, _p(q), _p(s))
    return rc, q, s


def gemm(a, b):
    a, b = _c(a, np.int8), _c(b, np.int8)
    M, K = a.shape
    N = b.shape[0]
    c = np.empty((M, N), dtype=np.int32)
    L.orc_gemm_i8i8i32(_p(a), K, _p(b), K, M, N, K, _p(c), N)
    return c


def gemm_rows(a, b, m0, m1):
    a, b = _c(a, np.int8), _c(b, np.int8)
    K = a.shape[1]
    N = b.shape[0]
    c = np.empty((m1 - m0, N), dtype=np.int32)
    L.orc_gemm_i8i8i32_rows(_p(a), K, _p(b), K, m0, m1, N, K, _p(c), N)
    return c


def dequantize(acc, scale_m, scale_n, bias=None, down_m=TOKEN_DOWN, down_n=HIDDEN_DOWN, layout=ROW_MAJOR, shape=None):
    acc = _c(acc, np.int32)
    M, N = shape if shape is not None else acc.shape
    out = np.empty((M, N), dtype=np.float16)
    rc = L.orc_minmax_dequantize_fp16(_p(acc), _p(None if bias is None else _c(bias, np.float16)),
                                      _p(_c(scale_m, np.float16)), _p(_c(scale_n, np.float16)), M, N,
                                      down_m, down_n, layout, _p(out))
    return rc, out


def linear(x, w, scale_n, bias=None, requant=False, up_scale=TOKEN_UP, down_m=TOKEN_DOWN, down_n=HIDDEN_DOWN,
           requant_up=TOKEN_UP):
    """Whole path.  Returns dict(xq, sm, acc, y[, yq, ys])."""
    x, w = _c(x, np.float16), _c(w, np.int8)
    M, K = x.shape
    N = w.shape[0]
    r = dict(xq=np.empty((M, K), np.int8), sm=np.empty((M,), np.float16), acc=np.empty((M, N), np.int32),
             y=np.empty((M, N), np.float16))
    if requant:
        r["yq"] = np.empty((M, N), np.int8)
        r["ys"] = np.empty((M,), np.float16)
    rc = L.orc_w8a8_linear(_p(x), _p(w), _p(_c(scale_n, np.float16)), _p(None if bias is None else _c(bias, np.float16)),
                           M, N, K, up_scale, down_m, down_n, requant_up, _p(r["xq"]), _p(r["sm"]), _p(r["acc"]),
                           _p(r["y"]), _p(r.get("yq")), _p(r.get("ys")))
    assert rc == 0, rc
    return r


def skip_rmsnorm_quantize(x, weight, skip=None, eps=1e-5, up_scale=TOKEN_UP, layout=ROW_MAJOR):
    """Returns (rc, skip_out float16 [M,K], q int8 [M,K], scale float16 [M])."""
    x, weight = _c(x, np.float16), _c(weight, np.float16)
    M, K = x.shape
    z = np.empty((M, K), np.float16)
    q = np.zeros((M, K), np.int8)
    s = np.empty((M,), np.float16)
    rc = L.orc_skip_rmsnorm_minmax_quantize_fp16(_p(x), _p(weight), _p(None if skip is None else _c(skip, np.float16)), eps,
                                                 M, K, up_scale, layout, _p(z), _p(s), _p(q))
    return rc, z, q, s


def activation_requantize(kind, acc, scale_b, scale_c, gate=None, gate_scale_b=None, gate_scale_c=None, beta=1.0,
                          up_scale=TOKEN_UP, down_b=TOKEN_DOWN, down_c=HIDDEN_DOWN):
    """kind 0 SiLU, 1 gated SiLU, 2 SwiGLU (acc [M, 2 dim]).  Returns (workspace f16, q int8, scale f16)."""
    acc = _c(acc, np.int32)
    M = acc.shape[0]
    dim = acc.shape[1] // 2 if kind == 2 else acc.shape[1]
    ws = np.empty((M, dim), np.float16); q = np.empty((M, dim), np.int8); s = np.empty((M,), np.float16)
    rc = L.orc_activation_requantize(kind, _p(acc), _p(_c(scale_b, np.float16)), _p(_c(scale_c, np.float16)),
                                     _p(None if gate is None else _c(gate, np.int32)),
                                     _p(None if gate_scale_b is None else _c(gate_scale_b, np.float16)),
                                     _p(None if gate_scale_c is None else _c(gate_scale_c, np.float16)),
                                     M, dim, beta, up_scale, down_b, down_c, _p(ws), _p(q), _p(s))
    assert rc == 0
    return ws, q, s


def dequantize_split3(acc, scale_m, scale_n, splits, bias=None, down_m=TOKEN_DOWN, down_n=HIDDEN_DOWN):
    acc = _c(acc, np.int32)
    M, N = acc.shape
    outs = [np.zeros((M, d), np.float16) for d in splits]
    rc = L.orc_dequantize_split3(_p(acc), _p(None if bias is None else _c(bias, np.float16)), _p(_c(scale_m, np.float16)),
                                 _p(_c(scale_n, np.float16)), M, N, splits[0], splits[1], splits[2], down_m, down_n,
                                 _p(outs[0]), _p(outs[1]), _p(outs[2]))
    return rc, outs


def layout_offset(layout, rows, cols, r, c):
    return L.orc_layout_offset(layout, rows, cols, r, c)


def to_layout(mat, layout):
    """Row-major numpy matrix -> flat array in `layout` (rows/cols padded as the layout needs)."""
    rows, cols = mat.shape
    idx = np.empty((rows, cols), dtype=np.int64)
    for r in range(rows):
        for c in range(cols):
            idx[r, c] = L.orc_layout_offset(layout, rows, cols, r, c)
    flat = np.zeros((int(idx.max()) + 1,), dtype=mat.dtype)
    flat[idx.ravel()] = mat.ravel()
    return flat, idx


def ulp_diff_f16(a, b):
    """Distance in fp16 units-in-the-last-place between two float16 arrays (same shape)."""
    def key(v):
        u = f16_bits(v).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a) - key(b))
