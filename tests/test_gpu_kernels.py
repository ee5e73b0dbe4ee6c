"""GPU parity tests of the individual kernels, called through the C ABI, against the oracle.

Bar: int8 / int32 / fp16-scale outputs bit-exact; fp16 outputs at most 1 ulp from the oracle
(0 expected, because the epilogue keeps the reference's operation order)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _t(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _rand_x(rng, M, K, kind):
    if kind == "normal":
        x = rng.standard_normal((M, K)).astype(np.float32)
    elif kind == "tiny":  # exercises the 1e-7 scale floor and fp16 subnormals
        x = rng.standard_normal((M, K)).astype(np.float32) * 1e-6
    elif kind == "wide":
        x = rng.standard_normal((M, K)).astype(np.float32) * np.exp(rng.uniform(-8, 6, (M, 1))).astype(np.float32)
    elif kind == "ties":  # many values exactly on .5 quantization boundaries: row max 127 -> scale 1
        x = (rng.integers(-254, 255, (M, K)) / 2.0).astype(np.float32)
        x[:, 0] = 127.0
    else:
        raise ValueError(kind)
    x = x.astype(np.float16)
    if M > 2:
        x[1, :] = 0  # an all-zero row
    return x


@pytest.mark.parametrize("M,K", [(1, 16), (3, 48), (16, 4096), (128, 4096), (7, 1024), (5, 28672), (33, 8192),
                                 (2, 32768), (2, 32768 + 4096), (300, 512)])
@pytest.mark.parametrize("kind", ["normal", "tiny", "wide", "ties"])
def test_quantize_rowmajor(cuda, oracle, M, K, kind):
    import pplb200
    rng = np.random.default_rng(M * 131 + K)
    x = _rand_x(rng, M, K, kind)
    rc, q_ref, s_ref = oracle.quantize(x)
    assert rc == 0
    q, s = pplb200.minmax_quantize_fp16(_t(cuda, x))
    cuda.cuda.synchronize()
    assert np.array_equal(oracle.f16_bits(s.cpu().numpy()), oracle.f16_bits(s_ref))
    assert np.array_equal(q.cpu().numpy(), q_ref)


@pytest.mark.parametrize("M,K", [(600, 512), (1200, 4096), (700, 8192), (640, 28672), (2000, 48), (593, 51200)])
@pytest.mark.parametrize("kind", ["normal", "ties", "wide"])
def test_quantize_large_batch(cuda, oracle, M, K, kind):
    """Several rows per SM, including row lengths at the edge of the register-resident kernel."""
    import pplb200
    rng = np.random.default_rng(M + K)
    x = _rand_x(rng, M, K, kind)
    rc, q_ref, s_ref = oracle.quantize(x)
    q, s = pplb200.minmax_quantize_fp16(_t(cuda, x))
    cuda.cuda.synchronize()
    assert np.array_equal(oracle.f16_bits(s.cpu().numpy()), oracle.f16_bits(s_ref))
    assert np.array_equal(q.cpu().numpy(), q_ref)


def test_quantize_large_batch_col32(cuda, oracle):
    import pplb200
    rng = np.random.default_rng(11)
    x = _rand_x(rng, 640, 256, "normal")
    for layout in (2, 3):
        q_ref = oracle.quantize(x, layout=layout)[1]
        q, _ = pplb200.minmax_quantize_fp16(_t(cuda, x), to_layout=layout)
        assert np.array_equal(q.cpu().numpy(), q_ref)


@pytest.mark.parametrize("layout", [2, 3])
def test_quantize_col32_layouts(cuda, oracle, layout):
    import pplb200
    rng = np.random.default_rng(7)
    M, K = 64, 256
    x = _rand_x(rng, M, K, "normal")
    rc, q_ref, s_ref = oracle.quantize(x, layout=layout)
    assert rc == 0
    q, s = pplb200.minmax_quantize_fp16(_t(cuda, x), to_layout=layout)
    assert np.array_equal(q.cpu().numpy(), q_ref)
    assert np.array_equal(oracle.f16_bits(s.cpu().numpy()), oracle.f16_bits(s_ref))


def test_quantize_error_codes(cuda):
    import pplb200
    x = cuda.zeros((4, 40), dtype=cuda.float16, device="cuda")
    with pytest.raises(pplb200.PplError) as e:
        pplb200.minmax_quantize_fp16(x)  # K % 16 != 0
    assert e.value.rc == pplb200.RC_INVALID_VALUE
    x = cuda.zeros((4, 64), dtype=cuda.float16, device="cuda")
    for bad_layout in (1, 4, 9):  # COL_MAJOR, COL4_4R2_8C, unknown
        with pytest.raises(pplb200.PplError) as e:
            pplb200.minmax_quantize_fp16(x, to_layout=bad_layout)
        assert e.value.rc == pplb200.RC_UNSUPPORTED
    q, s = pplb200.minmax_quantize_fp16(cuda.zeros((0, 64), dtype=cuda.float16, device="cuda"))  # empty batch
    assert q.shape == (0, 64)


@pytest.mark.parametrize("M,N", [(1, 4), (16, 4096), (33, 1000), (128, 12288), (5, 36)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_dequantize_rowmajor(cuda, oracle, M, N, with_bias):
    import pplb200
    rng = np.random.default_rng(M * 7 + N)
    acc = rng.integers(-(2 ** 27), 2 ** 27, (M, N), dtype=np.int32)
    acc[0, :4] = [0, 1, -1, 2 ** 28 + 3]
    sm = (rng.uniform(0.001, 2.0, M) * 4096 / 127).astype(np.float16)
    sn = (rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16) if with_bias else None
    rc, y_ref = oracle.dequantize(acc, sm, sn, bias)
    assert rc == 0
    y = pplb200.minmax_dequantize_fp16(_t(cuda, acc), _t(cuda, sm), _t(cuda, sn), None if bias is None else _t(cuda, bias))
    assert np.array_equal(oracle.f16_bits(y.cpu().numpy()), oracle.f16_bits(y_ref))


@pytest.mark.parametrize("layout", [1, 2, 3, 4])
def test_dequantize_layouts(cuda, oracle, layout):
    import pplb200
    rng = np.random.default_rng(layout)
    M, N = 64, 128
    acc = rng.integers(-(2 ** 20), 2 ** 20, (M, N), dtype=np.int32)
    flat, _ = oracle.to_layout(acc, layout)
    sm = (rng.uniform(0.01, 2.0, M) * 4096 / 127).astype(np.float16)
    sn = (rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16)
    rc, y_ref = oracle.dequantize(flat, sm, sn, bias, layout=layout, shape=(M, N))
    assert rc == 0
    rc, y_rm = oracle.dequantize(acc, sm, sn, bias)
    assert np.array_equal(oracle.f16_bits(y_ref), oracle.f16_bits(y_rm))  # layouts only permute storage
    y = pplb200.minmax_dequantize_fp16(_t(cuda, flat), _t(cuda, sm), _t(cuda, sn), _t(cuda, bias), from_layout=layout, shape=(M, N))
    assert np.array_equal(oracle.f16_bits(y.cpu().numpy()), oracle.f16_bits(y_ref))


def test_dequantize_error_codes(cuda):
    import pplb200
    acc = cuda.zeros((4, 6), dtype=cuda.int32, device="cuda")
    s = cuda.ones((8,), dtype=cuda.float16, device="cuda")
    with pytest.raises(pplb200.PplError) as e:
        pplb200.minmax_dequantize_fp16(acc, s, s)  # N % 4 != 0
    assert e.value.rc == pplb200.RC_INVALID_VALUE
    acc = cuda.zeros((4, 8), dtype=cuda.int32, device="cuda")
    with pytest.raises(pplb200.PplError) as e:
        pplb200.minmax_dequantize_fp16(acc, s, s, from_layout=7)
    assert e.value.rc == pplb200.RC_UNSUPPORTED


GEMM_SHAPES = [(1, 8, 16), (16, 32, 128), (128, 256, 128), (128, 256, 512), (130, 264, 144), (257, 520, 1040),
               (16, 4096, 4096), (128, 12288, 4096), (300, 1000, 2048), (512, 4096, 1024), (1024, 2048, 3584),
               (2300, 2120, 272), (2048, 2560, 144), (4096, 2752, 512)]  # the last three: 256 x 256 tiles on CTA pairs


def _exact_gemm(torch, a, b):
    # fp64 products/sums of int8 data are exact far beyond these K
    return (a.double() @ b.double().T).to(torch.int32)


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_raw_i32(cuda, oracle, M, N, K):
    import pplb200
    rng = np.random.default_rng(M + 3 * N + 5 * K)
    a = rng.integers(-127, 128, (M, K), dtype=np.int8)
    b = rng.integers(-127, 128, (N, K), dtype=np.int8)
    ta, tb = _t(cuda, a), _t(cuda, b)
    c = pplb200.gemm_i8i8(ta, tb)
    cuda.cuda.synchronize()
    assert pplb200.gemm_status() == 0
    assert cuda.equal(c, _exact_gemm(cuda, ta, tb))
    rows = sorted(set([0, M - 1, M // 2]))
    for r in rows:  # and against the scalar oracle on a few rows
        assert np.array_equal(c[r].cpu().numpy(), oracle.gemm_rows(a, b, r, r + 1)[0])


DECODE_SHAPES = [(128, 6272, 2048), (100, 12288, 4096), (64, 8192, 1024), (72, 3200, 512), (128, 12288, 1024), (40, 4096, 4096)]


@pytest.mark.parametrize("M,N,K", DECODE_SHAPES + [(16, 4096, 4096), (128, 19072, 1024), (8, 1024, 256), (1, 2048, 8192)])
def test_decode_gemm_all_modes(cuda, oracle, M, N, K):
    """Small-batch kernel across its variants: one or two weight-row tiles per CTA, K split over clusters of
    different sizes, an odd number of weight-row tiles, token counts that are not multiples of 8."""
    import pplb200
    rng = np.random.default_rng(M + N + K)
    x = rng.standard_normal((M, K)).astype(np.float16)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sn = (rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16)
    ref = oracle.linear(x, w, sn, bias, requant=True)
    txq, tw, tsm, tsn, tb = _t(cuda, ref["xq"]), _t(cuda, w), _t(cuda, ref["sm"]), _t(cuda, sn), _t(cuda, bias)
    acc = pplb200.gemm_i8i8(txq, tw)
    y = pplb200.gemm_i8i8(txq, tw, mode=pplb200.EPI_DEQUANT_F16, scale_m=tsm, scale_n=tsn, bias=tb)
    y2, yq, ys = pplb200.gemm_i8i8(txq, tw, mode=pplb200.EPI_DEQUANT_F16_REQUANT_I8, scale_m=tsm, scale_n=tsn, bias=tb)
    cuda.cuda.synchronize()
    assert pplb200.gemm_status() == 0
    assert np.array_equal(acc.cpu().numpy(), ref["acc"])
    assert np.array_equal(oracle.f16_bits(y.cpu().numpy()), oracle.f16_bits(ref["y"]))
    assert np.array_equal(oracle.f16_bits(y2.cpu().numpy()), oracle.f16_bits(ref["y"]))
    assert np.array_equal(yq.cpu().numpy(), ref["yq"])
    assert np.array_equal(oracle.f16_bits(ys.cpu().numpy()), oracle.f16_bits(ref["ys"]))


def test_gemm_extreme_values(cuda):
    """All-(-128) x all-(-128): the largest products; also +127 x -128 (the reference's own test data includes -128)."""
    import pplb200
    M, N, K = 128, 64, 4096
    a = cuda.full((M, K), -128, dtype=cuda.int8, device="cuda")
    b = cuda.full((N, K), -128, dtype=cuda.int8, device="cuda")
    b[1::2] = 127
    c = pplb200.gemm_i8i8(a, b)
    assert cuda.equal(c, _exact_gemm(cuda, a, b))


def test_gemm_strided_operands(cuda):
    """lda / ldb larger than K: the K-shard views used by the row-parallel linear."""
    import pplb200
    rng = np.random.default_rng(3)
    M, N, K = 96, 136, 512
    a_full = _t(cuda, rng.integers(-127, 128, (M, 2 * K), dtype=np.int8))
    b_full = _t(cuda, rng.integers(-127, 128, (N, 2 * K), dtype=np.int8))
    a, b = a_full[:, K:], b_full[:, K:]
    c = pplb200.gemm_i8i8(a, b)
    assert cuda.equal(c, _exact_gemm(cuda, a, b))


@pytest.mark.parametrize("M,N,K", [(16, 4096, 4096), (130, 264, 144), (128, 12288, 4096), (257, 528, 1040),
                                   (2300, 2120, 272)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_gemm_dequant_epilogue(cuda, oracle, M, N, K, with_bias):
    import pplb200
    rng = np.random.default_rng(M + N + K + int(with_bias))
    x = rng.standard_normal((M, K)).astype(np.float16)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sn = (rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16) if with_bias else None
    ref = oracle.linear(x, w, sn, bias)
    y = pplb200.gemm_i8i8(_t(cuda, ref["xq"]), _t(cuda, w), mode=pplb200.EPI_DEQUANT_F16, scale_m=_t(cuda, ref["sm"]),
                          scale_n=_t(cuda, sn), bias=None if bias is None else _t(cuda, bias))
    cuda.cuda.synchronize()
    assert pplb200.gemm_status() == 0
    d = oracle.ulp_diff_f16(y.cpu().numpy(), ref["y"])
    assert d.max() == 0, "max ulp %d" % d.max()


@pytest.mark.parametrize("M,N,K", [(16, 4096, 4096), (128, 12288, 4096), (70, 272, 256), (2300, 2128, 272)])
def test_gemm_requant_epilogue(cuda, oracle, M, N, K):
    import pplb200
    rng = np.random.default_rng(M + N + K)
    x = rng.standard_normal((M, K)).astype(np.float16)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sn = (rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16)
    ref = oracle.linear(x, w, sn, bias, requant=True)
    y, yq, ys = pplb200.gemm_i8i8(_t(cuda, ref["xq"]), _t(cuda, w), mode=pplb200.EPI_DEQUANT_F16_REQUANT_I8,
                                  scale_m=_t(cuda, ref["sm"]), scale_n=_t(cuda, sn), bias=_t(cuda, bias))
    cuda.cuda.synchronize()
    assert pplb200.gemm_status() == 0
    assert np.array_equal(oracle.f16_bits(y.cpu().numpy()), oracle.f16_bits(ref["y"]))
    assert np.array_equal(oracle.f16_bits(ys.cpu().numpy()), oracle.f16_bits(ref["ys"]))
    assert np.array_equal(yq.cpu().numpy(), ref["yq"])


@pytest.mark.parametrize("M,N,K", [(2560, 2048, 4096), (2500, 2032, 4096), (4000, 1296, 7936), (4864, 1024, 4096),
                                   (2560, 7680, 3072), (2560, 2048, 3200)])
def test_gemm_tiles_shared_between_pairs(cuda, oracle, M, N, K):
    """Tile counts that are not a multiple of the 74 CTA pairs (80, 96, 76 and 300 tiles): the K blocks of the last
    waves are dealt out evenly, so tiles at the border of two pairs' shares are computed in two K segments that meet
    in the workspace.  All three epilogues must equal the oracle, with the sharing switched off and on, call after
    call on the same workspace."""
    import pplb200
    rng = np.random.default_rng(M + N + K)
    a = rng.integers(-127, 128, (M, K), dtype=np.int8)
    b = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sm = rng.uniform(0.2, 1.0, M).astype(np.float16)
    sn = (rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16)
    ta, tb, tsm, tsn, tbias = _t(cuda, a), _t(cuda, b), _t(cuda, sm), _t(cuda, sn), _t(cuda, bias)
    exact = _exact_gemm(cuda, ta, tb)
    acc_np = exact.cpu().numpy()
    rc, y_ref = oracle.dequantize(acc_np, sm, sn, bias)
    assert rc == 0
    rc, yq_ref, ys_ref = oracle.quantize(y_ref)
    assert rc == 0
    for r in (0, M - 1):
        assert np.array_equal(acc_np[r], oracle.gemm_rows(a, b, r, r + 1)[0])
    ws = cuda.empty((pplb200.gemm_workspace_bytes(M, N, K, pplb200.EPI_DEQUANT_F16_REQUANT_I8),), dtype=cuda.uint8, device="cuda")
    ws.fill_(0x5a)  # the workspace need not be initialised
    try:
        for split in (False, True, True):
            pplb200.gemm_tail_split(split)
            acc = pplb200.gemm_i8i8(ta, tb, ws=ws)
            y = pplb200.gemm_i8i8(ta, tb, mode=pplb200.EPI_DEQUANT_F16, scale_m=tsm, scale_n=tsn, bias=tbias, ws=ws)
            y2, yq, ys = pplb200.gemm_i8i8(ta, tb, mode=pplb200.EPI_DEQUANT_F16_REQUANT_I8, scale_m=tsm, scale_n=tsn, bias=tbias, ws=ws)
            cuda.cuda.synchronize()
            assert pplb200.gemm_status() == 0
            assert cuda.equal(acc, exact)
            assert np.array_equal(oracle.f16_bits(y.cpu().numpy()), oracle.f16_bits(y_ref))
            assert np.array_equal(oracle.f16_bits(y2.cpu().numpy()), oracle.f16_bits(y_ref))
            assert np.array_equal(yq.cpu().numpy(), yq_ref)
            assert np.array_equal(oracle.f16_bits(ys.cpu().numpy()), oracle.f16_bits(ys_ref))
    finally:
        pplb200.gemm_tail_split(True)


@pytest.mark.parametrize("M,N,K", [(4400, 1280, 8192), (2560, 2048, 16384), (5000, 1032, 8192), (4608, 4352, 8192)])
def test_gemm_tile_groups_ragged(cuda, M, N, K):
    """Large-batch GEMM with more m-tiles than one L2 group holds (groups of 16 at K = 8192, of 9 at K = 16384), the last
    group ragged (18 = 16 + 2, 10 = 9 + 1, 20 = 16 + 4 m-tiles), together with sliced leftover tiles and a ragged last
    column tile."""
    import pplb200
    torch = cuda
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda", generator=g)
    b = torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda", generator=g)
    exact = _exact_gemm(torch, a, b)
    for _ in range(2):
        c = pplb200.gemm_i8i8(a, b)
        torch.cuda.synchronize()
        assert pplb200.gemm_status() == 0
        assert torch.equal(c, exact)


def test_gemm_random_shapes(cuda):
    """Seeded sweep over shapes of the large-batch kernels (CTA pairs and single CTAs, every tile width, sliced and whole
    leftover tiles): raw int32 result against the exact product."""
    import pplb200
    torch = cuda
    rng = np.random.default_rng(20240611)
    g = torch.Generator(device="cuda").manual_seed(7)
    for _ in range(24):
        M = int(rng.integers(129, 5200))
        N = int(rng.integers(1, 700)) * 8
        K = int(rng.integers(1, 320)) * 16
        a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda", generator=g)
        b = torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda", generator=g)
        c = pplb200.gemm_i8i8(a, b)
        torch.cuda.synchronize()
        assert pplb200.gemm_status() == 0, (M, N, K)
        assert torch.equal(c, _exact_gemm(torch, a, b)), (M, N, K)


def test_gemm_error_codes(cuda):
    import pplb200
    a = cuda.zeros((8, 40), dtype=cuda.int8, device="cuda")
    b = cuda.zeros((8, 40), dtype=cuda.int8, device="cuda")
    with pytest.raises(pplb200.PplError) as e:
        pplb200.gemm_i8i8(a, b)  # K % 16
    assert e.value.rc == pplb200.RC_INVALID_VALUE
    a = cuda.zeros((8, 64), dtype=cuda.int8, device="cuda")
    b = cuda.zeros((12, 64), dtype=cuda.int8, device="cuda")
    with pytest.raises(pplb200.PplError) as e:
        pplb200.gemm_i8i8(a, b)  # N % 8
    assert e.value.rc == pplb200.RC_INVALID_VALUE
    b = cuda.zeros((16, 64), dtype=cuda.int8, device="cuda")
    with pytest.raises(pplb200.PplError) as e:
        pplb200.gemm_i8i8(a, b, mode=5)
    assert e.value.rc == pplb200.RC_UNSUPPORTED
    c = pplb200.gemm_i8i8(cuda.zeros((0, 64), dtype=cuda.int8, device="cuda"), b)  # empty M
    assert c.shape == (0, 16)


@pytest.mark.parametrize("M,N,K", [(300, 264, 256), (2300, 2120, 272), (130, 1000, 144)])
def test_gemm_strided_output_is_clipped(cuda, oracle, M, N, K):
    """Output rows longer than N (ldc > N) and ragged tile edges: the staged epilogue stores must write
    columns [0, N) of rows [0, M) and nothing else (sentinel columns and a sentinel row stay untouched)."""
    import pplb200
    rng = np.random.default_rng(M + N + K)
    x = rng.standard_normal((M, K)).astype(np.float16)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sn = (rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)
    ref = oracle.linear(x, w, sn, None)
    ldc = N + 72
    txq, tw = _t(cuda, ref["xq"]), _t(cuda, w)
    raw = cuda.full((M + 1, ldc), 0x5a5a5a5a, dtype=cuda.int32, device="cuda")
    pplb200.gemm_i8i8(txq, tw, out=raw[:M, :N])
    y = cuda.full((M + 1, ldc), 1.5, dtype=cuda.float16, device="cuda")
    pplb200.gemm_i8i8(txq, tw, mode=pplb200.EPI_DEQUANT_F16, scale_m=_t(cuda, ref["sm"]), scale_n=_t(cuda, sn), out=y[:M, :N])
    cuda.cuda.synchronize()
    assert pplb200.gemm_status() == 0
    assert np.array_equal(raw[:M, :N].cpu().numpy(), ref["acc"])
    assert bool((raw[:, N:] == 0x5a5a5a5a).all()) and bool((raw[M] == 0x5a5a5a5a).all())
    assert np.array_equal(oracle.f16_bits(y[:M, :N].cpu().numpy()), oracle.f16_bits(ref["y"]))
    assert bool((y[:, N:] == 1.5).all()) and bool((y[M] == 1.5).all())


@pytest.mark.parametrize("M,N,K", [(16, 256, 128), (100, 1032, 256), (300, 1000, 256), (2300, 2120, 272)])
@pytest.mark.parametrize("alpha,beta,with_bias", [(1, 0, True), (3, 0, False), (1, 1, False), (-2, 5, True)])
def test_gemm_i32_alpha_beta_bias(cuda, M, N, K, alpha, beta, with_bias):
    """The full contract of the reference's gemm_i8i8i32 (src/ppl/kernel/llm/cuda/cublas/gemm.cu:187-188,239-243):
    C = alpha * (A x B^T) + beta * C + bias[n], wrapping int32."""
    import pplb200
    rng = np.random.default_rng(M + N + K + alpha * 7 + beta)
    a = _t(cuda, rng.integers(-127, 128, (M, K), dtype=np.int8))
    b = _t(cuda, rng.integers(-127, 128, (N, K), dtype=np.int8))
    c0 = _t(cuda, rng.integers(-(2 ** 30), 2 ** 30, (M, N), dtype=np.int32))
    bias = _t(cuda, rng.integers(-(2 ** 20), 2 ** 20, (N,), dtype=np.int32)) if with_bias else None
    c = c0.clone()
    pplb200.gemm_i8i8i32(a, b, alpha=alpha, beta=beta, bias_i32=bias, out=c)
    cuda.cuda.synchronize()
    assert pplb200.gemm_status() == 0
    want = alpha * _exact_gemm(cuda, a, b).to(cuda.int64) + beta * c0.to(cuda.int64)
    if with_bias:
        want = want + bias.to(cuda.int64)[None, :]
    want = ((want + 2 ** 31) % (2 ** 32) - 2 ** 31).to(cuda.int32)
    assert cuda.equal(c, want)
