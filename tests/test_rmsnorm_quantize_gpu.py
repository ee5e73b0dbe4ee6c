"""Fused skip-add + RMSNorm + per-token quantize (the producer that feeds the W8A8 linear) through
the C ABI, against the oracle and against the reference's own kernel.

This op has floating-point reductions whose order the reference leaves to CUB and an approximate
rsqrtf, so the bar is a tolerance, stated here: skip_out bit-exact (it is one fp16 add); the fp16
row scale within 1 ulp; int8 values within 1, and at most 0.2 % of them different at all."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libref_i8i8.so")


def _t(torch, a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _inputs(rng, M, K, with_skip):
    x = (rng.standard_normal((M, K)) * np.exp(rng.uniform(-2, 2, (M, 1)))).astype(np.float16)
    skip = (rng.standard_normal((M, K)) * 0.5).astype(np.float16) if with_skip else None
    w = (1.0 + 0.2 * rng.standard_normal(K)).astype(np.float16)
    if M > 2:
        x[1, :] = 0
        if skip is not None:
            skip[1, :] = 0  # an all-zero row: scale floor via eps
    return x, skip, w


def _close(oracle, q_a, s_a, q_b, s_b):
    assert oracle.ulp_diff_f16(s_a, s_b).max() <= 1
    d = np.abs(q_a.astype(np.int32) - q_b.astype(np.int32))
    assert d.max() <= 1
    assert (d != 0).mean() <= 2e-3


@pytest.mark.parametrize("M,K", [(1, 16), (16, 4096), (128, 4096), (33, 5120), (7, 8192), (5, 1008), (3, 28672)])
@pytest.mark.parametrize("with_skip", [False, True])
def test_vs_oracle(cuda, oracle, M, K, with_skip):
    import pplb200
    rng = np.random.default_rng(M * 17 + K + int(with_skip))
    x, skip, w = _inputs(rng, M, K, with_skip)
    rc, z_o, q_o, s_o = oracle.skip_rmsnorm_quantize(x, w, skip, eps=1e-5)
    assert rc == 0
    z, q, s = pplb200.skip_rmsnorm_minmax_quantize_fp16(_t(cuda, x), _t(cuda, w), _t(cuda, skip), eps=1e-5)
    cuda.cuda.synchronize()
    assert np.array_equal(oracle.f16_bits(z.cpu().numpy()), oracle.f16_bits(z_o))
    _close(oracle, q.cpu().numpy(), s.cpu().numpy(), q_o, s_o)
    assert int(np.abs(q.cpu().numpy().astype(np.int32)).max()) <= 127


@pytest.mark.parametrize("M,K", [(16, 4096), (128, 4096), (40, 5120), (9, 1008)])  # specialised dims and the generic path
@pytest.mark.parametrize("with_skip", [False, True])
def test_vs_reference_kernel(cuda, oracle, M, K, with_skip):
    import pplb200
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref not built")
    ref = ctypes.CDLL(REF_SO)
    vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_float
    ref.ref_skip_rmsnorm_minmax_quantize_fp16.argtypes = [vp, vp, vp, vp, f32, i64, i64, f32, i32, vp, vp, vp]
    rng = np.random.default_rng(M + K * 3 + int(with_skip))
    x, skip, w = _inputs(rng, M, K, with_skip)
    tx, tw, ts = _t(cuda, x), _t(cuda, w), _t(cuda, skip)
    z_r = cuda.empty((M, K), dtype=cuda.float16, device="cuda")
    q_r = cuda.empty((M, K), dtype=cuda.int8, device="cuda")
    s_r = cuda.empty((M,), dtype=cuda.float16, device="cuda")
    P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    assert ref.ref_skip_rmsnorm_minmax_quantize_fp16(None, P(tx), P(tw), P(ts), 1e-5, M, K, 4096.0, 0, P(z_r), P(s_r), P(q_r)) == 0
    z, q, s = pplb200.skip_rmsnorm_minmax_quantize_fp16(tx, tw, ts, eps=1e-5)
    cuda.cuda.synchronize()
    assert cuda.equal(z.view(cuda.int16), z_r.view(cuda.int16))
    _close(oracle, q.cpu().numpy(), s.cpu().numpy(), q_r.cpu().numpy(), s_r.cpu().numpy())
    rc, z_o, q_o, s_o = oracle.skip_rmsnorm_quantize(x, w, skip, eps=1e-5)
    _close(oracle, q_r.cpu().numpy(), s_r.cpu().numpy(), q_o, s_o)  # pins the oracle to the reference kernel


@pytest.mark.parametrize("layout", [2, 3])
def test_col32_layouts(cuda, oracle, layout):
    import pplb200
    rng = np.random.default_rng(layout)
    x, skip, w = _inputs(rng, 64, 256, True)
    rc, z_o, q_o, s_o = oracle.skip_rmsnorm_quantize(x, w, skip, layout=layout)
    z, q, s = pplb200.skip_rmsnorm_minmax_quantize_fp16(_t(cuda, x), _t(cuda, w), _t(cuda, skip), to_layout=layout)
    _close(oracle, q.cpu().numpy(), s.cpu().numpy(), q_o, s_o)


def test_feeds_the_linear(cuda, oracle):
    """Producer output plugs straight into the int8 GEMM: same result as the oracle's GEMM on the same int8 rows."""
    import pplb200
    rng = np.random.default_rng(9)
    M, K, N = 48, 1024, 512
    x, skip, w = _inputs(rng, M, K, True)
    wt = rng.integers(-127, 128, (N, K), dtype=np.int8)
    z, q, s = pplb200.skip_rmsnorm_minmax_quantize_fp16(_t(cuda, x), _t(cuda, w), _t(cuda, skip))
    acc = pplb200.gemm_i8i8(q, _t(cuda, wt))
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm(q.cpu().numpy(), wt))


def test_error_codes(cuda):
    import pplb200
    x = cuda.zeros((4, 40), dtype=cuda.float16, device="cuda")
    w = cuda.ones((40,), dtype=cuda.float16, device="cuda")
    with pytest.raises(pplb200.PplError) as e:
        pplb200.skip_rmsnorm_minmax_quantize_fp16(x, w)
    assert e.value.rc == pplb200.RC_INVALID_VALUE
    x = cuda.zeros((4, 64), dtype=cuda.float16, device="cuda")
    w = cuda.ones((64,), dtype=cuda.float16, device="cuda")
    for bad in (1, 4, 7):
        with pytest.raises(pplb200.PplError) as e:
            pplb200.skip_rmsnorm_minmax_quantize_fp16(x, w, to_layout=bad)
        assert e.value.rc == pplb200.RC_UNSUPPORTED
