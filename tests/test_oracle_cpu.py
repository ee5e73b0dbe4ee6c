"""CPU tests of the oracle: pinned against (a) vectors produced by the reference's own kernels
(tests/golden/reference_i8i8.npz, made by tests/golden/make_golden.py on a GPU) and (b) an
independent numpy restatement of the same formulas."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_i8i8.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


# ---------------------------------------------------------------- golden vectors from the reference kernels

@pytest.mark.parametrize("kind", ["normal", "wide", "ties", "tiny"])
@pytest.mark.parametrize("layout", [0, 2])
def test_quantizer_matches_reference_kernel(oracle, golden, kind, layout):
    x = golden["quant_%s_x" % kind]
    rc, q, s = oracle.quantize(x, layout=layout)
    assert rc == 0
    assert np.array_equal(q, golden["quant_%s_l%d_q" % (kind, layout)])
    assert np.array_equal(bits(s), bits(golden["quant_%s_l%d_s" % (kind, layout)]))


@pytest.mark.parametrize("tag", ["nobias", "bias"])
def test_dequantizer_matches_reference_kernel(oracle, golden, tag):
    rc, y = oracle.dequantize(golden["deq_acc"], golden["deq_sm"], golden["deq_sn"],
                              golden["deq_bias"] if tag == "bias" else None)
    assert rc == 0
    assert np.array_equal(bits(y), bits(golden["deq_y_%s" % tag]))


def test_whole_path_matches_reference_operators(oracle, golden):
    r = oracle.linear(golden["lin_x"], golden["lin_w"], golden["lin_sn"], golden["lin_bias"], requant=True)
    assert np.array_equal(r["xq"], golden["lin_xq"])
    assert np.array_equal(bits(r["sm"]), bits(golden["lin_sm"]))
    assert np.array_equal(r["acc"], golden["lin_acc"])          # cuBLASLt int32 accumulators
    assert np.array_equal(bits(r["y"]), bits(golden["lin_y"]))
    assert np.array_equal(r["yq"], golden["lin_yq"])
    assert np.array_equal(bits(r["ys"]), bits(golden["lin_ys"]))


# ---------------------------------------------------------------- fp16 helpers vs numpy

def test_f16_conversions_exhaustive(oracle):
    L = oracle.L
    h = np.arange(65536, dtype=np.uint16)
    ref = h.view(np.float16).astype(np.float32)
    got = np.array([L.orc_f16_to_f32(int(i)) for i in h], dtype=np.float32)
    ok = (got.view(np.uint32) == ref.view(np.uint32)) | (np.isnan(got) & np.isnan(ref))
    assert ok.all()
    # every half converts back to itself (NaNs to a NaN)
    back = np.array([L.orc_f32_to_f16(float(v)) for v in ref], dtype=np.uint16)
    finite = ~np.isnan(ref)
    assert np.array_equal(back[finite], h[finite])


def test_f32_to_f16_rounding(oracle):
    L = oracle.L
    rng = np.random.default_rng(0)
    f = np.concatenate([
        rng.integers(0, 2 ** 32, 20000, dtype=np.uint64).astype(np.uint32).view(np.float32),
        (rng.standard_normal(20000) * np.exp(rng.uniform(-20, 12, 20000))).astype(np.float32),
        np.float32([65504, 65519.99, 65520, 65536, 5.96e-8, 2.98e-8, 2.9802322e-8, 2.9802326e-8, 6.1e-5, 6.097e-5, 0.0, -0.0]),
    ])
    with np.errstate(all="ignore"):
        want = f.astype(np.float16).view(np.uint16)
    for v, w in zip(f, want):
        if np.isnan(v):
            continue
        assert L.orc_f32_to_f16(float(v)) == w, v


def test_f16_add_single_rounding(oracle):
    L = oracle.L
    rng = np.random.default_rng(1)
    a = rng.integers(0, 65536, 30000).astype(np.uint16)
    b = rng.integers(0, 65536, 30000).astype(np.uint16)
    with np.errstate(all="ignore"):
        want = (a.view(np.float16).astype(np.float64) + b.view(np.float16).astype(np.float64)).astype(np.float16)
    for x, y, w in zip(a, b, want):
        if np.isnan(w):
            continue
        assert L.orc_f16_add(int(x), int(y)) == w.view(np.uint16)


# ---------------------------------------------------------------- numpy restatement

def np_quantize(x):
    xf = x.astype(np.float32)
    amax = np.abs(xf).max(axis=1)
    scale = np.maximum((amax / np.float32(127)).astype(np.float32), np.float32(1e-7))
    q = np.rint((xf / scale[:, None]).astype(np.float32)).astype(np.int32).astype(np.int8)
    return q, (scale * np.float32(4096)).astype(np.float16)


def np_dequantize(acc, sm, sn, bias):
    bs = (sm.astype(np.float32) * np.float32(1 / 4096)).astype(np.float32)
    t = (acc.astype(np.float32) * sn.astype(np.float32)[None, :]).astype(np.float32)
    t = (t * np.float32(1 / 8192)).astype(np.float32)
    t = (t * bs[:, None]).astype(np.float32)
    y = t.astype(np.float16)
    if bias is not None:
        y = (y.astype(np.float64) + bias.astype(np.float64)[None, :]).astype(np.float16)
    return y


@pytest.mark.parametrize("M,K", [(1, 16), (9, 64), (16, 4096), (3, 28672)])
def test_quantizer_vs_numpy(oracle, M, K):
    rng = np.random.default_rng(M + K)
    x = (rng.standard_normal((M, K)) * np.exp(rng.uniform(-6, 5, (M, 1)))).astype(np.float16)
    if M > 1:
        x[0] = 0
    rc, q, s = oracle.quantize(x)
    qn, sn = np_quantize(x)
    assert rc == 0 and np.array_equal(q, qn) and np.array_equal(bits(s), bits(sn))
    assert np.abs(q.astype(np.int32)).max() <= 127


def test_dequantizer_vs_numpy(oracle):
    rng = np.random.default_rng(3)
    M, N = 17, 200
    acc = rng.integers(-(2 ** 28), 2 ** 28, (M, N), dtype=np.int32)
    sm = (rng.uniform(0.001, 2.0, M) * 4096 / 127).astype(np.float16)
    sn = (rng.uniform(0.0005, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16)
    for b in (None, bias):
        rc, y = oracle.dequantize(acc, sm, sn, b)
        assert rc == 0 and np.array_equal(bits(y), bits(np_dequantize(acc, sm, sn, b)))


def test_gemm_vs_numpy(oracle):
    rng = np.random.default_rng(4)
    a = rng.integers(-128, 128, (19, 272), dtype=np.int8)
    b = rng.integers(-128, 128, (40, 272), dtype=np.int8)
    want = a.astype(np.int32) @ b.astype(np.int32).T
    assert np.array_equal(oracle.gemm(a, b), want)
    assert np.array_equal(oracle.gemm_rows(a, b, 5, 9), want[5:9])


def test_error_codes(oracle):
    x = np.zeros((4, 32), np.float16)
    assert oracle.quantize(x, layout=1)[0] == 2 and oracle.quantize(x, layout=4)[0] == 2 and oracle.quantize(x, layout=9)[0] == 2
    acc = np.zeros((4, 6), np.int32)
    s = np.ones(8, np.float16)
    assert oracle.dequantize(acc, s, s)[0] == 4
    assert oracle.dequantize(np.zeros((4, 8), np.int32), s, s, layout=9)[0] == 2
    rc, q, sc = oracle.quantize(np.zeros((0, 32), np.float16))
    assert rc == 0 and q.shape == (0, 32)


def test_requantize_is_quantizer_of_fp16_output(oracle):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((12, 128)).astype(np.float16)
    w = rng.integers(-127, 128, (48, 128), dtype=np.int8)
    sn = (rng.uniform(0.001, 0.01, 48) * 8192).astype(np.float16)
    bias = (rng.standard_normal(48) * 0.02).astype(np.float16)
    r = oracle.linear(x, w, sn, bias, requant=True)
    rc, q, s = oracle.quantize(r["y"])
    assert np.array_equal(q, r["yq"]) and np.array_equal(bits(s), bits(r["ys"]))
    assert np.array_equal(r["acc"], r["xq"].astype(np.int32) @ w.astype(np.int32).T)


def test_row_parallel_partials_sum_exactly(oracle):
    """Splitting K and summing int32 partials equals the unsharded accumulators: the property the
    exact row-parallel reduction rests on."""
    rng = np.random.default_rng(6)
    a = rng.integers(-127, 128, (8, 512), dtype=np.int8)
    b = rng.integers(-127, 128, (24, 512), dtype=np.int8)
    full = oracle.gemm(a, b)
    for size in (2, 4, 8):
        kw = 512 // size
        parts = sum(oracle.gemm(np.ascontiguousarray(a[:, r * kw:(r + 1) * kw]), np.ascontiguousarray(b[:, r * kw:(r + 1) * kw]))
                    for r in range(size))
        assert np.array_equal(parts, full)


@pytest.mark.parametrize("layout", [0, 1, 2, 3, 4])
def test_layout_offsets_are_bijections(oracle, layout):
    rows, cols = 64, 96
    _, idx = oracle.to_layout(np.zeros((rows, cols), np.int8), layout)
    flat = idx.ravel()
    assert len(np.unique(flat)) == rows * cols and flat.min() == 0 and flat.max() == rows * cols - 1


def test_skip_rmsnorm_quantize_vs_numpy(oracle):
    rng = np.random.default_rng(8)
    M, K = 9, 320
    x = rng.standard_normal((M, K)).astype(np.float16)
    skip = (rng.standard_normal((M, K)) * 0.5).astype(np.float16)
    w = (1.0 + 0.2 * rng.standard_normal(K)).astype(np.float16)
    rc, z, q, s = oracle.skip_rmsnorm_quantize(x, w, skip, eps=1e-5)
    assert rc == 0
    zn = (x.astype(np.float64) + skip.astype(np.float64)).astype(np.float16)
    assert np.array_equal(bits(z), bits(zn))
    zf, wf = zn.astype(np.float32), w.astype(np.float32)
    mean = ((zf.astype(np.float64) ** 2).sum(axis=1)).astype(np.float32) * np.float32(1.0 / K)
    r = (1.0 / np.sqrt((mean + np.float32(1e-5)).astype(np.float64))).astype(np.float32)
    amax = np.maximum(np.float32(1e-5), np.abs(zf * wf).max(axis=1))
    scale = np.maximum((amax * r) / np.float32(127), np.float32(1e-7)).astype(np.float32)
    v = ((zf * wf) * r[:, None]).astype(np.float32) * (np.float32(1) / scale)[:, None]
    qn = np.clip(np.sign(v) * np.floor(np.abs(v) + np.float32(0.5)), -127, 127).astype(np.int8)
    assert np.array_equal(q, qn)
    assert np.array_equal(bits(s), bits((scale * np.float32(4096)).astype(np.float16)))
    assert oracle.skip_rmsnorm_quantize(x, w, skip, layout=1)[0] == 2


def test_activation_consumers_vs_numpy(oracle):
    rng = np.random.default_rng(12)
    M, D = 6, 96
    acc = rng.integers(-(2 ** 20), 2 ** 20, (M, 2 * D), dtype=np.int32)
    sm = (rng.uniform(0.5, 3.0, M) * 4096 / 127).astype(np.float16)
    sn = (rng.uniform(0.5, 2.0, 2 * D) * 8192 / 2 ** 18).astype(np.float16)
    ws, q, s = oracle.activation_requantize(2, acc, sm, sn, beta=1.0)
    bs = (sm.astype(np.float32) * np.float32(1 / 4096))[:, None]
    def dq(a, sc):
        t = (a.astype(np.float32) * sc.astype(np.float32)[None, :]).astype(np.float32)
        return ((t * np.float32(1 / 8192)).astype(np.float32) * bs).astype(np.float32)
    x, g = dq(acc[:, :D], sn[:D]), dq(acc[:, D:], sn[D:])
    res = ((x / (np.float32(1) + np.exp(-x).astype(np.float32))).astype(np.float32) * g).astype(np.float32)
    assert np.abs(ws.astype(np.float32) - res).max() <= np.abs(res).max() * 2e-3
    scale = np.maximum(np.abs(res).max(axis=1) / np.float32(127), np.float32(1e-7))
    assert np.abs(s.astype(np.float32) - scale * 4096).max() <= (scale * 4096).max() * 2e-3
    assert np.abs(q.astype(np.int32)).max() == 127
    rc, outs = oracle.dequantize_split3(acc[:, :96].copy(), sm, sn[:96], (32, 48, 16))
    rc2, full = oracle.dequantize(acc[:, :96].copy(), sm, sn[:96])
    assert rc == 0 and np.array_equal(np.concatenate(outs, axis=1).view(np.uint16), full.view(np.uint16))
