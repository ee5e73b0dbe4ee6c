"""Consumers of the raw int32 GEMM output -- dequantize + split3, dequantize + SiLU [x gate]
[+ re-quantize], dequantize + SwiGLU + re-quantize -- through the C ABI.

Bars: against the reference's own kernels BIT-EXACT (same operations in the same order, including
the approximate __expf); against the CPU oracle (exact expf) a tolerance: fp16 values within 2 ulp,
row scales within 1 ulp, int8 within 1 and at most 0.5 % of them different.  split3 has no
transcendental: bit-exact against both."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libref_i8i8.so")


def _t(torch, a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _P(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


@pytest.fixture(scope="module")
def ref(cuda):
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref not built")
    lib = ctypes.CDLL(REF_SO)
    vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_float
    lib.ref_minmax_dequantize_split3_fp16.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, f32, f32, i32, vp, vp, vp]
    lib.ref_minmax_requantize_silu_fp16.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, f32, f32, f32, vp, vp, vp]
    lib.ref_minmax_requantize_swiglu_fp16.argtypes = [vp, vp, vp, vp, i64, i64, f32, i32, f32, f32, f32, vp, vp, vp]
    return lib


def _acc(rng, M, N):
    """int32 accumulators and scales sized so that the dequantized values are O(1) (SiLU's interesting range)."""
    acc = rng.integers(-(2 ** 20), 2 ** 20, (M, N), dtype=np.int32)
    sm = (rng.uniform(0.5, 3.0, M) * 4096 / 127).astype(np.float16)          # token scale * 4096
    sn = (rng.uniform(0.5, 2.0, N) * 8192 / 2 ** 18).astype(np.float16)      # channel scale * 8192
    return acc, sm, sn


def _close(oracle, ws, q, s, ws_o, q_o, s_o):
    assert oracle.ulp_diff_f16(ws, ws_o).max() <= 2
    assert oracle.ulp_diff_f16(s, s_o).max() <= 1
    d = np.abs(q.astype(np.int32) - q_o.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() <= 5e-3


@pytest.mark.parametrize("M,D", [(1, 16), (16, 11008), (128, 4096), (33, 1008), (5, 28672)])
@pytest.mark.parametrize("beta", [1.0, 1.702])
def test_swiglu_requantize(cuda, oracle, ref, M, D, beta):
    import pplb200
    rng = np.random.default_rng(M + D)
    acc, sm, sn = _acc(rng, M, 2 * D)
    ta, tsm, tsn = _t(cuda, acc), _t(cuda, sm), _t(cuda, sn)
    ws, q, s = pplb200.minmax_requantize_swiglu_fp16(ta, tsm, tsn, beta=beta)
    ws_r = cuda.empty((M, D), dtype=cuda.float16, device="cuda")
    q_r = cuda.empty((M, D), dtype=cuda.int8, device="cuda")
    s_r = cuda.empty((M,), dtype=cuda.float16, device="cuda")
    assert ref.ref_minmax_requantize_swiglu_fp16(None, _P(ta), _P(tsm), _P(tsn), M, D, beta, 0, 4096.0, 1 / 4096, 1 / 8192,
                                                 _P(ws_r), _P(q_r), _P(s_r)) == 0
    cuda.cuda.synchronize()
    assert cuda.equal(ws.view(cuda.int16), ws_r.view(cuda.int16)), "fp16 activated values vs reference kernel"
    assert cuda.equal(s.view(cuda.int16), s_r.view(cuda.int16)) and cuda.equal(q, q_r), "int8 / scales vs reference kernel"
    ws_o, q_o, s_o = oracle.activation_requantize(2, acc, sm, sn, beta=beta)
    _close(oracle, ws.cpu().numpy(), q.cpu().numpy(), s.cpu().numpy(), ws_o, q_o, s_o)


@pytest.mark.parametrize("M,D", [(16, 4096), (40, 11008), (3, 48)])
@pytest.mark.parametrize("gated", [False, True])
def test_silu_requantize(cuda, oracle, ref, M, D, gated):
    import pplb200
    rng = np.random.default_rng(M * 3 + D + int(gated))
    acc, sm, sn = _acc(rng, M, D)
    gate, gsm, gsn = _acc(rng, M, D) if gated else (None, None, None)
    ta, tsm, tsn, tg, tgsm, tgsn = (_t(cuda, v) for v in (acc, sm, sn, gate, gsm, gsn))
    ws, q, s = pplb200.minmax_silu_fp16(ta, tsm, tsn, tg, tgsm, tgsn)
    ws_r = cuda.empty((M, D), dtype=cuda.float16, device="cuda")
    q_r = cuda.empty((M, D), dtype=cuda.int8, device="cuda")
    s_r = cuda.empty((M,), dtype=cuda.float16, device="cuda")
    assert ref.ref_minmax_requantize_silu_fp16(None, _P(ta), _P(tsm), _P(tsn), _P(tg), _P(tgsm), _P(tgsn), M, D, 0, 4096.0,
                                               1 / 4096, 1 / 8192, _P(ws_r), _P(q_r), _P(s_r)) == 0
    cuda.cuda.synchronize()
    assert cuda.equal(ws.view(cuda.int16), ws_r.view(cuda.int16))
    assert cuda.equal(s.view(cuda.int16), s_r.view(cuda.int16)) and cuda.equal(q, q_r)
    ws_o, q_o, s_o = oracle.activation_requantize(1 if gated else 0, acc, sm, sn, gate, gsm, gsn)
    _close(oracle, ws.cpu().numpy(), q.cpu().numpy(), s.cpu().numpy(), ws_o, q_o, s_o)
    # dequantize + SiLU without re-quantize == the fp16 workspace of the re-quantizing call
    y = pplb200.minmax_silu_fp16(ta, tsm, tsn, tg, tgsm, tgsn, requant=False)
    assert cuda.equal(y.view(cuda.int16), ws.view(cuda.int16))


@pytest.mark.parametrize("layout", [2, 3])
def test_swiglu_col32_layouts(cuda, oracle, layout):
    import pplb200
    rng = np.random.default_rng(layout)
    M, D = 64, 128
    acc, sm, sn = _acc(rng, M, 2 * D)
    flat, _ = oracle.to_layout(acc, layout)
    ws, q, s = pplb200.minmax_requantize_swiglu_fp16(_t(cuda, acc), _t(cuda, sm), _t(cuda, sn))
    tf = _t(cuda, flat).view(M, 2 * D)  # same bytes, carried in a [M, 2D]-shaped tensor
    ws_l, q_l, s_l = pplb200.minmax_requantize_swiglu_fp16(tf, _t(cuda, sm), _t(cuda, sn), layout=layout)
    q_rm, idx = oracle.to_layout(q.cpu().numpy(), layout)
    assert np.array_equal(q_l.cpu().numpy().ravel()[: q_rm.size], q_rm)
    assert cuda.equal(s_l.view(cuda.int16), s.view(cuda.int16))


@pytest.mark.parametrize("M,splits", [(16, (4096, 1024, 1024)), (33, (512, 256, 128)), (128, (4096, 4096, 4096)), (5, (8, 4, 12))])
@pytest.mark.parametrize("with_bias", [False, True])
def test_dequantize_split3(cuda, oracle, ref, M, splits, with_bias):
    import pplb200
    rng = np.random.default_rng(M + sum(splits))
    N = sum(splits)
    acc, sm, sn = _acc(rng, M, N)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16) if with_bias else None
    ta, tsm, tsn, tb = _t(cuda, acc), _t(cuda, sm), _t(cuda, sn), _t(cuda, bias)
    outs = pplb200.minmax_dequantize_split3_fp16(ta, tsm, tsn, splits, tb)
    refs = [cuda.empty((M, d), dtype=cuda.float16, device="cuda") for d in splits]
    assert ref.ref_minmax_dequantize_split3_fp16(None, _P(ta), _P(tb), _P(tsm), _P(tsn), M, N, splits[0], splits[1], splits[2],
                                                 1 / 4096, 1 / 8192, 0, _P(refs[0]), _P(refs[1]), _P(refs[2])) == 0
    rc, outs_o = oracle.dequantize_split3(acc, sm, sn, splits, bias)
    assert rc == 0
    full = pplb200.minmax_dequantize_fp16(ta, tsm, tsn, tb)
    cuda.cuda.synchronize()
    col = 0
    for o, r, oo, d in zip(outs, refs, outs_o, splits):
        assert cuda.equal(o.view(cuda.int16), r.view(cuda.int16))
        assert np.array_equal(oracle.f16_bits(o.cpu().numpy()), oracle.f16_bits(oo))
        assert cuda.equal(o.view(cuda.int16), full[:, col:col + d].contiguous().view(cuda.int16))  # == slices of the plain dequantizer
        col += d


def test_activation_error_codes(cuda):
    import pplb200
    acc = cuda.zeros((4, 80), dtype=cuda.int32, device="cuda")
    s4 = cuda.ones((4,), dtype=cuda.float16, device="cuda")
    s80 = cuda.ones((80,), dtype=cuda.float16, device="cuda")
    with pytest.raises(pplb200.PplError) as e:
        pplb200.minmax_requantize_swiglu_fp16(acc, s4, s80)   # quant_dim 40 not a multiple of 16
    assert e.value.rc == pplb200.RC_INVALID_VALUE
    acc = cuda.zeros((4, 64), dtype=cuda.int32, device="cuda")
    s64 = cuda.ones((64,), dtype=cuda.float16, device="cuda")
    with pytest.raises(pplb200.PplError) as e:
        pplb200.minmax_silu_fp16(acc, s4, s64, layout=4)
    assert e.value.rc == pplb200.RC_UNSUPPORTED
    with pytest.raises(pplb200.PplError) as e:
        pplb200.minmax_dequantize_split3_fp16(acc, s4, s64, (30, 30, 4))
    assert e.value.rc == pplb200.RC_INVALID_VALUE


@pytest.mark.parametrize("M,D,K", [(2304, 1152, 272), (4096, 1280, 512), (64, 256, 128), (300, 208, 144)])  # fused (first two) and fallback
def test_fused_gate_up_swiglu_matches_two_step(cuda, oracle, M, D, K):
    """GEMM + SwiGLU + re-quantize in one pass == raw-int32 linear followed by the stand-alone SwiGLU kernel, bit for bit."""
    import pplb200
    rng = np.random.default_rng(M + D + K)
    xq = _t(cuda, rng.integers(-127, 128, (M, K), dtype=np.int8))
    w = _t(cuda, rng.integers(-127, 128, (2 * D, K), dtype=np.int8))
    sm = _t(cuda, (rng.uniform(0.5, 3.0, M) * 4096 / 127).astype(np.float16))
    sn = _t(cuda, (rng.uniform(0.5, 2.0, 2 * D) * 8192 * 127 / (1.5 * 5400 * np.sqrt(K))).astype(np.float16))
    acc = pplb200.column_parallel_linear(xq, w, None, None, None, K, 2 * D, gather_output=False)
    ws2, q2, s2 = pplb200.minmax_requantize_swiglu_fp16(acc, sm, sn, beta=1.3)
    act, q, s = pplb200.gate_up_swiglu_requant(xq, w, sm, sn, beta=1.3)
    cuda.cuda.synchronize()
    assert pplb200.gemm_status() == 0
    assert cuda.equal(act.view(cuda.int16), ws2.view(cuda.int16))
    assert cuda.equal(s.view(cuda.int16), s2.view(cuda.int16)) and cuda.equal(q, q2)
    assert float(act.float().abs().max()) > 0.01  # the scales put the values in SiLU's interesting range
