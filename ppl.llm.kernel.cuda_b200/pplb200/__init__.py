"""Host-side Python binding of the sm_100a i8i8 (W8A8) linear library.

Thin ctypes layer over the C ABI declared in include/pplb200_i8i8.h; function names and
argument meaning mirror the reference's operator API
(include/ppl/kernel/llm/cuda/pmx/i8i8/{quantize,column_parallel_linear,row_parallel_linear}.h,
include/ppl/kernel/llm/cuda/cublas/gemm.h).  torch is used only for device memory and streams.

There is no CPU fallback: importing this module without the built shared library raises.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "..", "lib", "libpplb200_i8i8.so")

# ppl.common RetCode values used by this path
RC_SUCCESS, RC_UNSUPPORTED, RC_INVALID_VALUE, RC_DEVICE_RUNTIME_ERROR = 0, 2, 4, 10

# matrix_layout_t (common/matrix_layout.h:25-31)
MATRIX_LAYOUT_ROW_MAJOR, MATRIX_LAYOUT_COL_MAJOR, MATRIX_LAYOUT_COL32 = 0, 1, 2
MATRIX_LAYOUT_COL32_2R_4R4, MATRIX_LAYOUT_COL4_4R2_8C = 3, 4

EPI_RAW_I32, EPI_DEQUANT_F16, EPI_DEQUANT_F16_REQUANT_I8 = 0, 1, 2

# scale conventions (pmx/i8i8/quantize.h:26-30)
TOKEN_UP_SCALE, HIDDEN_UP_SCALE = 4096.0, 8192.0
TOKEN_DOWN_SCALE, HIDDEN_DOWN_SCALE = 1.0 / 4096.0, 1.0 / 8192.0

EXPORTS = [
    "pplb200_version", "pplb200_last_error",
    "pplb200_i8i8_minmax_quantize_fp16", "pplb200_i8i8_minmax_dequantize_fp16",
    "pplb200_i8i8_gemm_workspace_bytes", "pplb200_i8i8_gemm",
    "pplb200_i8i8_linear_workspace_bytes", "pplb200_i8i8_linear_fp16",
    "pplb200_i8i8_column_parallel_linear", "pplb200_i8i8_row_parallel_linear",
    "pplb200_nccl_get_unique_id", "pplb200_nccl_comm_init", "pplb200_nccl_comm_destroy",
    "pplb200_i8i8_gemm_status", "pplb200_layout_offset",
    "pplb200_i8i8_gemm_requant_static_scratch", "pplb200_i8i8_skip_rmsnorm_minmax_quantize_fp16",
    "pplb200_i8i8_minmax_dequantize_split3_fp16", "pplb200_i8i8_minmax_dequantize_silu_fp16",
    "pplb200_i8i8_minmax_requantize_silu_fp16", "pplb200_i8i8_minmax_requantize_swiglu_fp16",
    "pplb200_i8i8_gate_up_swiglu_workspace_bytes", "pplb200_i8i8_gate_up_swiglu_requant",
    "pplb200_i8i8_row_parallel_p2p_bytes", "pplb200_p2p_create", "pplb200_p2p_export", "pplb200_p2p_connect",
    "pplb200_p2p_connect_local", "pplb200_p2p_destroy", "pplb200_p2p_status", "pplb200_i8i8_row_parallel_linear_p2p",
    "pplb200_i8i8_minmax_quantize_fp16_p2p",
    "pplb200_probe_tensor_peak", "pplb200_probe_stream_read", "pplb200_i8i8_gemm_i32", "pplb200_debug_gemm_stall_counters", "pplb200_debug_gemm_tail_split", "pplb200_i8i8_relayout", "pplb200_i8i8_column_parallel_linear_p2p", "pplb200_i8i8_linear_host_workspace_bytes", "pplb200_i8i8_linear_fp16_host",
]
STATIC_SCRATCH_MAX_ROWS = 16384


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libpplb200_i8i8.so is not built (%s); run `python ppl.llm.kernel.cuda_b200/build.py`. "
            "There is no fallback path." % os.path.normpath(LIB_PATH))
    lib = ctypes.CDLL(os.path.normpath(LIB_PATH))
    vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_float
    lib.pplb200_version.restype = ctypes.c_char_p
    lib.pplb200_last_error.restype = ctypes.c_char_p
    lib.pplb200_i8i8_minmax_quantize_fp16.argtypes = [vp, vp, i64, i64, f32, i32, vp, vp]
    lib.pplb200_i8i8_skip_rmsnorm_minmax_quantize_fp16.argtypes = [vp, vp, vp, vp, f32, i64, i64, f32, i32, vp, vp, vp]
    lib.pplb200_i8i8_minmax_dequantize_split3_fp16.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, f32, f32, i32, vp, vp, vp]
    lib.pplb200_i8i8_minmax_dequantize_silu_fp16.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, f32, f32, vp]
    lib.pplb200_i8i8_minmax_requantize_silu_fp16.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, f32, f32, f32, vp, vp, vp]
    lib.pplb200_i8i8_minmax_requantize_swiglu_fp16.argtypes = [vp, vp, vp, vp, i64, i64, f32, i32, f32, f32, f32, vp, vp, vp]
    lib.pplb200_i8i8_gate_up_swiglu_workspace_bytes.argtypes = [i64, i64, i64]
    lib.pplb200_i8i8_gate_up_swiglu_workspace_bytes.restype = i64
    lib.pplb200_i8i8_gate_up_swiglu_requant.argtypes = [vp, vp, i64, vp, i64, i64, i64, vp, vp, f32, f32, f32, f32, vp, i64, vp, vp, vp]
    lib.pplb200_i8i8_minmax_dequantize_fp16.argtypes = [vp, vp, vp, vp, vp, i64, i64, f32, f32, i32, vp]
    lib.pplb200_i8i8_gemm_workspace_bytes.argtypes = [i64, i64, i64, i32]
    lib.pplb200_i8i8_gemm_workspace_bytes.restype = i64
    lib.pplb200_i8i8_gemm.argtypes = [vp, vp, i64, vp, i64, i64, i64, i64, i32, vp, vp, vp, f32, f32, f32,
                                      vp, i64, vp, i64, vp, vp]
    lib.pplb200_i8i8_gemm_requant_static_scratch.argtypes = [vp, vp, i64, vp, i64, i64, i64, i64, vp, vp, vp, f32, f32, f32,
                                                             vp, vp, vp]
    lib.pplb200_i8i8_linear_workspace_bytes.argtypes = [i64, i64, i64, i32]
    lib.pplb200_i8i8_linear_workspace_bytes.restype = i64
    lib.pplb200_i8i8_linear_fp16.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, f32, f32, f32, i32, f32,
                                             vp, i64, vp, vp, vp]
    lib.pplb200_i8i8_linear_host_workspace_bytes.argtypes = [i64, i64, i64, i32, i64]
    lib.pplb200_i8i8_linear_host_workspace_bytes.restype = i64
    lib.pplb200_i8i8_linear_fp16_host.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, f32, f32, f32, i32, f32, i64, vp, i64, vp, vp, vp]
    lib.pplb200_i8i8_column_parallel_linear.argtypes = [vp, vp, i64, vp, vp, vp, vp, f32, f32, i64, i64, i32,
                                                        i32, i32, vp, i32, vp, vp, vp, i64, vp]
    lib.pplb200_i8i8_row_parallel_linear.argtypes = [vp, vp, i64, i64, vp, vp, vp, vp, f32, f32, i64, i64, i32,
                                                     i32, i32, vp, i32, i32, vp, vp, i64, vp]
    lib.pplb200_i8i8_row_parallel_p2p_bytes.argtypes = [i64, i64, i32]
    lib.pplb200_i8i8_row_parallel_p2p_bytes.restype = i64
    lib.pplb200_p2p_create.argtypes = [i32, i32, i64, ctypes.POINTER(vp)]
    lib.pplb200_p2p_export.argtypes = [vp, vp]
    lib.pplb200_p2p_connect.argtypes = [vp, vp]
    lib.pplb200_p2p_connect_local.argtypes = [vp, ctypes.POINTER(vp)]
    lib.pplb200_p2p_destroy.argtypes = [vp]
    lib.pplb200_p2p_status.argtypes = [vp, i32]
    lib.pplb200_i8i8_row_parallel_linear_p2p.argtypes = [vp, vp, vp, i64, i64, vp, vp, vp, vp, f32, f32, i64, i64, i32, vp]
    lib.pplb200_i8i8_column_parallel_linear_p2p.argtypes = [vp, vp, vp, i64, vp, vp, vp, vp, f32, f32, i64, i64, i32, vp]
    lib.pplb200_i8i8_minmax_quantize_fp16_p2p.argtypes = [vp, vp, vp, i64, i64, f32, i32, vp, vp]
    lib.pplb200_i8i8_gemm_i32.argtypes = [vp, vp, i64, vp, i64, i64, i64, i64, i32, i32, vp, vp, i64]
    lib.pplb200_probe_tensor_peak.argtypes = [vp, i32, i32, i32, vp, i64, vp]
    lib.pplb200_i8i8_relayout.argtypes = [vp, vp, i32, vp, i32, i64, i64, i32]
    lib.pplb200_debug_gemm_stall_counters.argtypes = [vp]
    lib.pplb200_debug_gemm_stall_counters.restype = None
    lib.pplb200_debug_gemm_tail_split.argtypes = [i32]
    lib.pplb200_debug_gemm_tail_split.restype = None
    lib.pplb200_probe_stream_read.argtypes = [vp, vp, i64, vp]
    lib.pplb200_nccl_get_unique_id.argtypes = [vp]
    lib.pplb200_nccl_comm_init.argtypes = [vp, i32, i32, ctypes.POINTER(vp)]
    lib.pplb200_nccl_comm_destroy.argtypes = [vp]
    lib.pplb200_i8i8_gemm_status.argtypes = [i32]
    lib.pplb200_layout_offset.argtypes = [i32, i64, i64, i64, i64]
    lib.pplb200_layout_offset.restype = i64
    for name in EXPORTS:
        fn = getattr(lib, name)
        if not name.startswith("pplb200_debug_") and fn.restype is ctypes.c_int:
            fn.restype = i32
    return lib


lib = _load()


class PplError(RuntimeError):
    def __init__(self, rc):
        self.rc = rc
        super().__init__("pplb200 call failed: RetCode %d: %s" % (rc, last_error()))


def version():
    return lib.pplb200_version().decode()


def last_error():
    return lib.pplb200_last_error().decode()


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc):
    if rc != RC_SUCCESS:
        raise PplError(rc)


def minmax_quantize_fp16(x, up_scale=TOKEN_UP_SCALE, to_layout=MATRIX_LAYOUT_ROW_MAJOR, out=None, scale=None):
    """x fp16 [batch, dim] (cuda) -> (q int8 [batch, dim] in `to_layout`, scale fp16 [batch])."""
    import torch
    batch, dim = x.shape
    q = out if out is not None else torch.empty((batch, dim), dtype=torch.int8, device=x.device)
    s = scale if scale is not None else torch.empty((batch,), dtype=torch.float16, device=x.device)
    _check(lib.pplb200_i8i8_minmax_quantize_fp16(_stream(), _ptr(x), batch, dim, up_scale, to_layout, _ptr(q), _ptr(s)))
    return q, s


def skip_rmsnorm_minmax_quantize_fp16(x, weight, skip=None, eps=1e-5, up_scale=TOKEN_UP_SCALE,
                                      to_layout=MATRIX_LAYOUT_ROW_MAJOR):
    """x (+ skip) fp16 [batch, dim], weight fp16 [dim] -> (skip_out fp16, q int8, scale fp16 [batch])."""
    import torch
    batch, dim = x.shape
    skip_out = torch.empty_like(x)
    q = torch.empty((batch, dim), dtype=torch.int8, device=x.device)
    s = torch.empty((batch,), dtype=torch.float16, device=x.device)
    _check(lib.pplb200_i8i8_skip_rmsnorm_minmax_quantize_fp16(_stream(), _ptr(x), _ptr(weight), _ptr(skip), eps, batch, dim,
                                                              up_scale, to_layout, _ptr(skip_out), _ptr(s), _ptr(q)))
    return skip_out, q, s


def minmax_dequantize_split3_fp16(acc, scale_m, scale_n, splits, bias=None, down_m=TOKEN_DOWN_SCALE,
                                  down_n=HIDDEN_DOWN_SCALE, from_layout=MATRIX_LAYOUT_ROW_MAJOR, shape=None):
    import torch
    batch, dim = shape if shape is not None else acc.shape
    outs = [torch.empty((batch, d), dtype=torch.float16, device=acc.device) for d in splits]
    _check(lib.pplb200_i8i8_minmax_dequantize_split3_fp16(_stream(), _ptr(acc), _ptr(bias), _ptr(scale_m), _ptr(scale_n), batch, dim,
                                                          splits[0], splits[1], splits[2], down_m, down_n, from_layout,
                                                          _ptr(outs[0]), _ptr(outs[1]), _ptr(outs[2])))
    return outs


def minmax_silu_fp16(acc, scale_m, scale_n, gate=None, gate_scale_m=None, gate_scale_n=None, requant=True,
                     up_scale=TOKEN_UP_SCALE, down_m=TOKEN_DOWN_SCALE, down_n=HIDDEN_DOWN_SCALE,
                     layout=MATRIX_LAYOUT_ROW_MAJOR):
    """requant=True: (workspace fp16, q int8, scale fp16 [batch]); requant=False: fp16 output."""
    import torch
    batch, dim = acc.shape
    if not requant:
        out = torch.empty((batch, dim), dtype=torch.float16, device=acc.device)
        _check(lib.pplb200_i8i8_minmax_dequantize_silu_fp16(_stream(), _ptr(acc), _ptr(scale_m), _ptr(scale_n), _ptr(gate),
                                                            _ptr(gate_scale_m), _ptr(gate_scale_n), batch, dim, layout, down_m,
                                                            down_n, _ptr(out)))
        return out
    ws = torch.empty((batch, dim), dtype=torch.float16, device=acc.device)
    q = torch.empty((batch, dim), dtype=torch.int8, device=acc.device)
    s = torch.empty((batch,), dtype=torch.float16, device=acc.device)
    _check(lib.pplb200_i8i8_minmax_requantize_silu_fp16(_stream(), _ptr(acc), _ptr(scale_m), _ptr(scale_n), _ptr(gate),
                                                        _ptr(gate_scale_m), _ptr(gate_scale_n), batch, dim, layout, up_scale,
                                                        down_m, down_n, _ptr(ws), _ptr(q), _ptr(s)))
    return ws, q, s


def minmax_requantize_swiglu_fp16(acc, scale_m, scale_n, beta=1.0, up_scale=TOKEN_UP_SCALE, down_m=TOKEN_DOWN_SCALE,
                                  down_n=HIDDEN_DOWN_SCALE, layout=MATRIX_LAYOUT_ROW_MAJOR):
    """acc int32 [batch, 2 * dim] = [x | gate] -> (workspace fp16 [batch, dim], q int8, scale fp16 [batch])."""
    import torch
    batch, dim = acc.shape[0], acc.shape[1] // 2
    ws = torch.empty((batch, dim), dtype=torch.float16, device=acc.device)
    q = torch.empty((batch, dim), dtype=torch.int8, device=acc.device)
    s = torch.empty((batch,), dtype=torch.float16, device=acc.device)
    _check(lib.pplb200_i8i8_minmax_requantize_swiglu_fp16(_stream(), _ptr(acc), _ptr(scale_m), _ptr(scale_n), batch, dim, beta,
                                                          layout, up_scale, down_m, down_n, _ptr(ws), _ptr(q), _ptr(s)))
    return ws, q, s


def gate_up_swiglu_requant(xq, w, scale_m, scale_n, beta=1.0, up_scale=TOKEN_UP_SCALE, down_m=TOKEN_DOWN_SCALE,
                           down_n=HIDDEN_DOWN_SCALE, ws=None, out=None):
    """xq int8 [M,K], w int8 [2D,K] = [x | gate] rows -> (activated fp16 [M,D], q int8 [M,D], scale fp16 [M])."""
    import torch
    M, K = xq.shape
    D = w.shape[0] // 2
    need = lib.pplb200_i8i8_gate_up_swiglu_workspace_bytes(M, D, K)
    if ws is None:
        ws = torch.empty((need,), dtype=torch.uint8, device=xq.device)
    act, q, s = out if out is not None else (torch.empty((M, D), dtype=torch.float16, device=xq.device),
                                            torch.empty((M, D), dtype=torch.int8, device=xq.device),
                                            torch.empty((M,), dtype=torch.float16, device=xq.device))
    _check(lib.pplb200_i8i8_gate_up_swiglu_requant(_stream(), _ptr(xq), xq.stride(0), _ptr(w), M, D, K, _ptr(scale_m), _ptr(scale_n),
                                                   beta, up_scale, down_m, down_n, _ptr(ws), ws.numel(), _ptr(act), _ptr(q), _ptr(s)))
    return act, q, s


def minmax_dequantize_fp16(acc, scale_m, scale_n, bias=None, down_m=TOKEN_DOWN_SCALE, down_n=HIDDEN_DOWN_SCALE,
                           from_layout=MATRIX_LAYOUT_ROW_MAJOR, out=None, shape=None):
    import torch
    batch, dim = shape if shape is not None else acc.shape
    y = out if out is not None else torch.empty((batch, dim), dtype=torch.float16, device=acc.device)
    _check(lib.pplb200_i8i8_minmax_dequantize_fp16(_stream(), _ptr(acc), _ptr(bias), _ptr(scale_m), _ptr(scale_n),
                                                   batch, dim, down_m, down_n, from_layout, _ptr(y)))
    return y


def relayout(src, src_layout, dst_layout, rows, cols):
    """Flat int8 / int32 tensor holding a [rows, cols] matrix in `src_layout` -> new flat tensor in `dst_layout`."""
    import torch
    dst = torch.zeros_like(src)
    _check(lib.pplb200_i8i8_relayout(_stream(), _ptr(src), src_layout, _ptr(dst), dst_layout, rows, cols, src.element_size()))
    return dst


def gemm_workspace_bytes(M, N, K, mode):
    return lib.pplb200_i8i8_gemm_workspace_bytes(M, N, K, mode)


def gemm_i8i8(a, b, mode=EPI_RAW_I32, scale_m=None, scale_n=None, bias=None, down_m=TOKEN_DOWN_SCALE,
              down_n=HIDDEN_DOWN_SCALE, requant_up_scale=TOKEN_UP_SCALE, ws=None, out=None):
    """a int8 [M,K], b int8 [N,K] -> int32 [M,N] (mode 0) / fp16 [M,N] (mode 1) / (fp16, int8, fp16 scales) (mode 2)."""
    import torch
    M, K = a.shape
    N = b.shape[0]
    dt = torch.int32 if mode == EPI_RAW_I32 else torch.float16
    y = out if out is not None else torch.empty((M, N), dtype=dt, device=a.device)
    yq = ys = None
    need = gemm_workspace_bytes(M, N, K, mode)
    if need and ws is None:
        ws = torch.empty((need,), dtype=torch.uint8, device=a.device)
    if mode == EPI_DEQUANT_F16_REQUANT_I8:
        yq = torch.empty((M, N), dtype=torch.int8, device=a.device)
        ys = torch.empty((M,), dtype=torch.float16, device=a.device)
    _check(lib.pplb200_i8i8_gemm(_stream(), _ptr(a), a.stride(0), _ptr(b), b.stride(0), M, N, K, mode, _ptr(scale_m),
                                 _ptr(scale_n), _ptr(bias), down_m, down_n, requant_up_scale, _ptr(ws),
                                 0 if ws is None else ws.numel(), _ptr(y), y.stride(0), _ptr(yq), _ptr(ys)))
    return y if mode != EPI_DEQUANT_F16_REQUANT_I8 else (y, yq, ys)


def gemm_i8i8i32(a, b, alpha=1, beta=0, bias_i32=None, out=None):
    """C int32 [M,N] = alpha * (a int8 [M,K] @ b int8 [N,K]^T) + beta * C + bias_i32[n] (wrapping int32)."""
    import torch
    M, K = a.shape
    N = b.shape[0]
    c = out if out is not None else torch.zeros((M, N), dtype=torch.int32, device=a.device)
    _check(lib.pplb200_i8i8_gemm_i32(_stream(), _ptr(a), a.stride(0), _ptr(b), b.stride(0), M, N, K, alpha, beta,
                                     _ptr(bias_i32), _ptr(c), c.stride(0)))
    return c


def gemm_requant_static_scratch(a, b, scale_m, scale_n, bias=None, down_m=TOKEN_DOWN_SCALE, down_n=HIDDEN_DOWN_SCALE,
                                requant_up_scale=TOKEN_UP_SCALE, out=None, out_q=None, out_q_scale=None):
    """GEMM + dequant + per-token re-quantize through the entry point that needs no workspace (its
    scratch is a fixed array inside the library; M <= STATIC_SCRATCH_MAX_ROWS).  The output tensors
    are created here only when the caller does not pass them; the C call itself allocates nothing."""
    import torch
    M, K = a.shape
    N = b.shape[0]
    y = out if out is not None else torch.empty((M, N), dtype=torch.float16, device=a.device)
    yq = out_q if out_q is not None else torch.empty((M, N), dtype=torch.int8, device=a.device)
    ys = out_q_scale if out_q_scale is not None else torch.empty((M,), dtype=torch.float16, device=a.device)
    _check(lib.pplb200_i8i8_gemm_requant_static_scratch(_stream(), _ptr(a), a.stride(0), _ptr(b), b.stride(0), M, N, K,
                                                        _ptr(scale_m), _ptr(scale_n), _ptr(bias), down_m, down_n,
                                                        requant_up_scale, _ptr(y), _ptr(yq), _ptr(ys)))
    return y, yq, ys


def linear_workspace_bytes(M, N, K, mode):
    return lib.pplb200_i8i8_linear_workspace_bytes(M, N, K, mode)


class W8A8Linear:
    """Pre-allocated single-device W8A8 linear: y = dequant(quantize(x) @ W^T) (+bias) [-> re-quantize].

    Owns the outputs and workspace so that __call__ allocates nothing (the C ABI never does)."""

    def __init__(self, w, scale_n, bias=None, max_tokens=None, requant=False):
        import torch
        self.w, self.scale_n, self.bias = w, scale_n, bias
        self.N, self.K = w.shape
        self.max_tokens = max_tokens
        self.mode = EPI_DEQUANT_F16_REQUANT_I8 if requant else EPI_DEQUANT_F16
        dev = w.device
        self.ws = torch.empty((linear_workspace_bytes(max_tokens, self.N, self.K, self.mode),), dtype=torch.uint8, device=dev)
        self.y = torch.empty((max_tokens, self.N), dtype=torch.float16, device=dev)
        self.yq = torch.empty((max_tokens, self.N), dtype=torch.int8, device=dev) if requant else None
        self.ys = torch.empty((max_tokens,), dtype=torch.float16, device=dev) if requant else None

    def __call__(self, x):
        M = x.shape[0]
        assert M <= self.max_tokens and x.shape[1] == self.K
        _check(lib.pplb200_i8i8_linear_fp16(_stream(), _ptr(x), _ptr(self.w), _ptr(self.scale_n), _ptr(self.bias),
                                            M, self.N, self.K, TOKEN_UP_SCALE, TOKEN_DOWN_SCALE, HIDDEN_DOWN_SCALE,
                                            self.mode, TOKEN_UP_SCALE, _ptr(self.ws), self.ws.numel(),
                                            _ptr(self.y), _ptr(self.yq), _ptr(self.ys)))
        if self.yq is None:
            return self.y[:M]
        return self.y[:M], self.yq[:M], self.ys[:M]


class W8A8LinearHost:
    """The fused linear on HOST buffers (pinned tensors): activations are copied in, quantized, multiplied and the
    result copied out chunk by chunk on three streams (pplb200_i8i8_linear_fp16_host).  Owns the device staging."""

    def __init__(self, w, scale_n, bias=None, max_tokens=None, requant=False, chunk_rows=0):
        import torch
        self.w, self.scale_n, self.bias = w, scale_n, bias
        self.N, self.K = w.shape
        self.max_tokens, self.chunk_rows = max_tokens, chunk_rows
        self.mode = EPI_DEQUANT_F16_REQUANT_I8 if requant else EPI_DEQUANT_F16
        need = lib.pplb200_i8i8_linear_host_workspace_bytes(max_tokens, self.N, self.K, self.mode, chunk_rows)
        self.ws = torch.empty((need,), dtype=torch.uint8, device=w.device)

    def __call__(self, x_host, y_host, yq_host=None, ys_host=None):
        M = x_host.shape[0]
        assert M <= self.max_tokens and x_host.shape[1] == self.K and not x_host.is_cuda and not y_host.is_cuda
        _check(lib.pplb200_i8i8_linear_fp16_host(_stream(), _ptr(x_host), _ptr(self.w), _ptr(self.scale_n), _ptr(self.bias),
                                                 M, self.N, self.K, TOKEN_UP_SCALE, TOKEN_DOWN_SCALE, HIDDEN_DOWN_SCALE,
                                                 self.mode, TOKEN_UP_SCALE, self.chunk_rows, _ptr(self.ws), self.ws.numel(),
                                                 _ptr(y_host), _ptr(yq_host), _ptr(ys_host)))
        return y_host


def column_parallel_linear(xq, w, scale_m, scale_n, bias, in_features, out_features, rank=0, size=1, comm=None,
                           gather_output=True, gather_buffer=None, out=None, down_m=TOKEN_DOWN_SCALE,
                           down_n=HIDDEN_DOWN_SCALE, weight_layout=MATRIX_LAYOUT_ROW_MAJOR, ws=None, M=None):
    import torch
    M = xq.shape[0] if M is None else M
    Nw = out_features // size
    if out is None:
        if gather_output:
            out = torch.empty((M, out_features), dtype=torch.float16, device=xq.device)
        else:
            out = torch.empty((M, Nw), dtype=torch.int32, device=xq.device)
    _check(lib.pplb200_i8i8_column_parallel_linear(_stream(), _ptr(xq), M, _ptr(w), _ptr(bias), _ptr(scale_m),
                                                   _ptr(scale_n), down_m, down_n, in_features, out_features,
                                                   weight_layout, rank, size, comm, 1 if gather_output else 0,
                                                   _ptr(gather_buffer), None, _ptr(ws), 0 if ws is None else ws.numel(), _ptr(out)))
    return out


def row_parallel_linear(xq, w, scale_m, scale_n, bias, in_features, out_features, rank=0, size=1, comm=None,
                        input_is_parallel=True, reduce_mode=0, quant_buffer=None, out=None,
                        down_m=TOKEN_DOWN_SCALE, down_n=HIDDEN_DOWN_SCALE, weight_layout=MATRIX_LAYOUT_ROW_MAJOR, ws=None, M=None):
    import torch
    legacy = weight_layout != MATRIX_LAYOUT_ROW_MAJOR
    M = (xq.shape[0] if M is None else M)
    if out is None:
        out = torch.empty((M, out_features), dtype=torch.float16, device=xq.device)
    if quant_buffer is None and size > 1 and reduce_mode == 0:
        quant_buffer = torch.empty((M, out_features), dtype=torch.int32, device=xq.device)
    _check(lib.pplb200_i8i8_row_parallel_linear(_stream(), _ptr(xq), M, 0 if legacy else xq.stride(0), _ptr(w), _ptr(bias), _ptr(scale_m),
                                                _ptr(scale_n), down_m, down_n, in_features, out_features,
                                                weight_layout, rank, size, comm, 1 if input_is_parallel else 0,
                                                reduce_mode, _ptr(quant_buffer), _ptr(ws), 0 if ws is None else ws.numel(), _ptr(out)))
    return out


def gemm_status(reset=True):
    return lib.pplb200_i8i8_gemm_status(1 if reset else 0)


def nccl_unique_id():
    buf = ctypes.create_string_buffer(128)
    _check(lib.pplb200_nccl_get_unique_id(buf))
    return bytes(buf.raw)


def nccl_comm_init(uid, rank, size):
    comm = ctypes.c_void_p()
    buf = ctypes.create_string_buffer(uid, 128)
    _check(lib.pplb200_nccl_comm_init(buf, rank, size, ctypes.byref(comm)))
    return comm


def nccl_comm_destroy(comm):
    _check(lib.pplb200_nccl_comm_destroy(comm))


class P2PContext:
    """One rank's peer-mapped buffer for `row_parallel_linear_p2p` (cudaMalloc'd by the library on
    the current device).  Ranks in different processes exchange `handle()` bytes themselves and call
    `connect(all_handles)`; ranks driven by one process use `connect_local(contexts)`."""

    def __init__(self, rank, size, max_m, max_n):
        self.rank, self.size = rank, size
        self.bytes = lib.pplb200_i8i8_row_parallel_p2p_bytes(max_m, max_n, size)
        if self.bytes < 0:
            raise ValueError("bad extents for a peer buffer")
        self.ctx = ctypes.c_void_p()
        _check(lib.pplb200_p2p_create(rank, size, self.bytes, ctypes.byref(self.ctx)))

    def handle(self):
        buf = ctypes.create_string_buffer(64)
        _check(lib.pplb200_p2p_export(self.ctx, buf))
        return bytes(buf.raw)

    def connect(self, handles):
        assert len(handles) == self.size and all(len(h) == 64 for h in handles)
        blob = b"".join(handles)  # length given explicitly: create_string_buffer(bytes) would add a terminator
        _check(lib.pplb200_p2p_connect(self.ctx, ctypes.create_string_buffer(blob, len(blob))))

    def connect_local(self, contexts):
        arr = (ctypes.c_void_p * self.size)(*[c.ctx for c in contexts])
        _check(lib.pplb200_p2p_connect_local(self.ctx, arr))

    def status(self, reset=True):
        return lib.pplb200_p2p_status(self.ctx, 1 if reset else 0)

    def destroy(self):
        if self.ctx:
            lib.pplb200_p2p_destroy(self.ctx)
            self.ctx = ctypes.c_void_p()


def row_parallel_linear_p2p(p2p, xq, w, scale_m, scale_n, bias, in_features, out_features, out=None, phases=7,
                            down_m=TOKEN_DOWN_SCALE, down_n=HIDDEN_DOWN_SCALE):
    import torch
    M = xq.shape[0]
    if out is None:
        out = torch.empty((M, out_features), dtype=torch.float16, device=xq.device)
    _check(lib.pplb200_i8i8_row_parallel_linear_p2p(_stream(), p2p.ctx, _ptr(xq), M, xq.stride(0), _ptr(w), _ptr(bias),
                                                    _ptr(scale_m), _ptr(scale_n), down_m, down_n, in_features,
                                                    out_features, phases, _ptr(out)))
    return out


def column_parallel_linear_p2p(p2p, xq, w_shard, scale_m, scale_n_shard, bias_shard, in_features, out_features, out=None,
                               phases=3, down_m=TOKEN_DOWN_SCALE, down_n=HIDDEN_DOWN_SCALE):
    """Column-parallel linear whose gathered fp16 output [M, out_features] is assembled by the GEMM epilogues of all
    ranks over peer-mapped memory."""
    import torch
    M = xq.shape[0]
    if out is None:
        out = torch.empty((M, out_features), dtype=torch.float16, device=xq.device)
    _check(lib.pplb200_i8i8_column_parallel_linear_p2p(_stream(), p2p.ctx, _ptr(xq), M, _ptr(w_shard), _ptr(bias_shard),
                                                       _ptr(scale_m), _ptr(scale_n_shard), down_m, down_n, in_features,
                                                       out_features, phases, _ptr(out)))
    return out


def minmax_quantize_fp16_p2p(p2p, x_shard, up_scale=TOKEN_UP_SCALE, out=None, scale=None, phases=3):
    """Quantizes this rank's K shard [M, K / size] with the row scale of the whole row."""
    import torch
    M, Kw = x_shard.shape
    assert x_shard.is_contiguous()
    if out is None:
        out = torch.empty((M, Kw), dtype=torch.int8, device=x_shard.device)
    if scale is None:
        scale = torch.empty((M,), dtype=torch.float16, device=x_shard.device)
    _check(lib.pplb200_i8i8_minmax_quantize_fp16_p2p(_stream(), p2p.ctx, _ptr(x_shard), M, Kw, up_scale, phases,
                                                     _ptr(out), _ptr(scale)))
    return out, scale


def _probe_record(t):
    import struct
    cycles, nanos, status, copies = struct.unpack("<QQII", bytes(t.cpu().numpy().tobytes()))
    return cycles, nanos, status, copies


def _peak_case(pairs, mmas_per_cta, src, launches, commit_pattern=0):
    """(best single-launch TOP/s, SM MHz of that launch, TOP/s over `launches` back-to-back launches, its SM MHz,
    32 KiB copies CTA 0 made per launch)."""
    import torch
    rec = torch.zeros((24,), dtype=torch.uint8, device="cuda")
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    ctas = sms // 2 if pairs else sms
    ops = 2.0 * (256 if pairs else 128) * 256 * 32 * mmas_per_cta * ctas
    sp, sb = (None, 0) if src is None else (_ptr(src), src.numel())

    def launch():
        _check(lib.pplb200_probe_tensor_peak(_stream(), pairs, mmas_per_cta, commit_pattern, sp, sb, _ptr(rec)))

    launch()  # warm-up, module load
    best, mhz, copies = None, None, 0
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        launch()
        e1.record()
        torch.cuda.synchronize()
        cycles, nanos, status, cp = _probe_record(rec)
        if status:
            raise RuntimeError("tensor peak probe: a bounded wait gave up")
        ms = e0.elapsed_time(e1)
        if best is None or ms < best:
            best, mhz, copies = ms, cycles / max(nanos, 1) * 1e3, cp
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        launch()
    e1.record()
    torch.cuda.synchronize()
    cycles, nanos, _, _ = _probe_record(rec)
    sus = e0.elapsed_time(e1) / launches
    d = {"tops": round(ops / (best * 1e-3) / 1e12, 1), "launch_ms": round(best, 4), "sm_mhz": round(mhz, 1),
         "sustained_tops": round(ops / (sus * 1e-3) / 1e12, 1), "sustained_sm_mhz": round(cycles / max(nanos, 1) * 1e3, 1)}
    if src is not None:
        d["fill_gb_per_s_per_sm"] = round(copies * 32768 / (best * 1e-3) / 1e9, 1)
    return d


def tensor_peak_probe(mmas_per_cta=8192, sustained_launches=100, with_loads=True):
    """int8 tcgen05 issue-rate ceiling of the current device: all SMs issue kind::i8 MMAs on operands that stay
    in shared memory.  "tops" is the best single launch over the two MMA shapes; "sustained_tops" the rate over
    `sustained_launches` launches back to back (tens of milliseconds, long enough for the power limit to pull the
    clock down).  with_loads adds the same measurement while every SM also streams bulk copies from global memory
    into spare shared memory (what a GEMM main loop does to the shared-memory ports and to the power budget)."""
    import torch
    out = {"cta_group_1_m128_n256": _peak_case(0, mmas_per_cta, None, sustained_launches),
           "cta_group_2_m256_n256": _peak_case(1, mmas_per_cta, None, sustained_launches)}
    if with_loads:
        pool = torch.randint(0, 255, (24 << 20,), dtype=torch.uint8, device="cuda")  # stays in L2, as a GEMM's operands mostly do
        out["cta_group_2_m256_n256_with_loads"] = _peak_case(1, mmas_per_cta, pool, sustained_launches)
        del pool
    no_load = [out["cta_group_1_m128_n256"], out["cta_group_2_m256_n256"]]
    return dict(out, tops=max(c["tops"] for c in no_load), sustained_tops=max(c["sustained_tops"] for c in no_load),
                how="tcgen05.mma kind::i8, operands resident in shared memory, no loads; %d MMAs per CTA, all SMs; best of 5 "
                    "launches, SM clock read inside the kernel; sustained = %d launches back to back"
                    % (mmas_per_cta, sustained_launches))


def gemm_tail_split(enabled):
    """Diagnostics: switch the column split of the CTA-pair GEMM's last wave of tiles on / off (default on)."""
    lib.pplb200_debug_gemm_tail_split(int(enabled))  # 0 off, 1 (True) by the launcher's rule, 2 whenever possible


def gemm_stall_profile(fn):
    """Runs fn() (which launches the CTA-pair GEMM) with the kernel's wait counters switched on and returns
    their means over the CTAs as fractions of the thread's run time."""
    import torch
    buf = torch.zeros((296 * 8,), dtype=torch.int64, device="cuda")
    lib.pplb200_debug_gemm_stall_counters(_ptr(buf))
    try:
        fn()
        torch.cuda.synchronize()
    finally:
        lib.pplb200_debug_gemm_stall_counters(None)
    c = buf.view(296, 8).double().cpu().numpy()
    lead = c[c[:, 0] > 0]      # leader CTAs carry the MMA thread
    prod = c[c[:, 4] > 0]
    epi = c[c[:, 6] > 0]
    if len(lead) == 0:
        return None
    return {"mma_thread_cycles": float(lead[:, 0].mean()),
            "mma_waits_for_operands": float((lead[:, 1] / lead[:, 0]).mean()),
            "mma_waits_for_accumulator": float((lead[:, 2] / lead[:, 0]).mean()),
            "tma_thread_waits_for_slot": float((prod[:, 3] / prod[:, 4]).mean()),
            "epilogue_waits_for_accumulator": float((epi[:, 5] / epi[:, 6]).mean())}


def decode_phase_profile(fn):
    """Runs fn() (which launches the small-batch GEMM once) with the kernel's phase stamps switched on.  Returns, in
    microseconds of the device's global timer: the span of the launch (earliest CTA start to latest CTA end) and
    the mean over the CTAs of set-up, main loop, K-split exchange and epilogue."""
    import torch
    buf = torch.zeros((296 * 8,), dtype=torch.int64, device="cuda")
    lib.pplb200_debug_gemm_stall_counters(_ptr(buf))
    try:
        fn()
        torch.cuda.synchronize()
    finally:
        lib.pplb200_debug_gemm_stall_counters(None)
    c = buf.view(296, 8).cpu().numpy().astype("float64")
    c = c[c[:, 0] > 0]
    if len(c) == 0:
        return None
    us = lambda a: round(float(a) * 1e-3, 2)
    return {"ctas": int(len(c)), "span_us": us(c[:, 4].max() - c[:, 0].min()),
            "start_skew_us": us(c[:, 0].max() - c[:, 0].min()),
            "setup_us": us((c[:, 1] - c[:, 0]).mean()), "main_loop_us": us((c[:, 2] - c[:, 1]).mean()),
            "main_loop_max_us": us((c[:, 2] - c[:, 1]).max()),
            "exchange_us": us((c[:, 3] - c[:, 2]).mean()), "epilogue_us": us((c[:, 4] - c[:, 3]).mean())}


def stream_read_probe(sizes=(16 << 20, 48 << 20, 384 << 20), pool_bytes=1536 << 20, reps=12):
    """Single-launch read-only bulk-copy stream of `size` bytes, each launch on a different slice of a pool larger
    than L2 (so the bytes come from HBM).  Per size: the median device-side duration of the launch (earliest CTA
    start to latest CTA end, global timer) and the GB/s that gives."""
    import torch
    pool = torch.empty((pool_bytes,), dtype=torch.uint8, device="cuda")
    pool.fill_(1)
    rec = torch.zeros((24,), dtype=torch.uint8, device="cuda")
    out = {}
    for size in sizes:
        slots = max(1, pool_bytes // size)
        times = []
        for r in range(reps + 2):
            off = (r % slots) * size
            _check(lib.pplb200_probe_stream_read(_stream(), ctypes.c_void_p(pool.data_ptr() + off), size, _ptr(rec)))
            torch.cuda.synchronize()
            start, end, status, _ = _probe_record(rec)
            if status:
                raise RuntimeError("stream read probe: a bounded wait gave up")
            if r >= 2:
                times.append((end - start) * 1e-3)
        times.sort()
        med = times[len(times) // 2]
        out["%d MiB" % (size >> 20)] = {"us": round(med, 2), "gb_per_s": round(size / (med * 1e-6) / 1e9, 1)}
    return out
