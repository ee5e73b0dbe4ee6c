"""Whole-path parity on the five benchmark configurations, through the C ABI.

c0 / c1 are checked in full against the oracle.  c2..c4 run at full size on the GPU and are
checked (a) bit-exactly against the oracle on a seeded sample of token rows -- first and last
rows included -- and (b) through size-independent properties: the quantized activations and the
int32 accumulators reproduce an exact fp64 GEMM on the GPU, and splitting K and summing the int32
partials reproduces the unsharded result bit for bit."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _t(torch, a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _inputs(name):
    import w8a8_workloads as wl
    return wl.CONFIGS[name], wl.make_activations(name), wl.make_weights(name), wl.make_column_scales(name), wl.make_bias(name)


@pytest.mark.parametrize("name", ["c0", "c1"])
def test_decode_configs_full(cuda, oracle, name):
    import pplb200
    cfg, x, w, sn, bias = _inputs(name)
    ref = oracle.linear(x, w, sn, bias, requant=cfg["requant"])
    lin = pplb200.W8A8Linear(_t(cuda, w), _t(cuda, sn), _t(cuda, bias), max_tokens=cfg["M"], requant=cfg["requant"])
    out = lin(_t(cuda, x))
    cuda.cuda.synchronize()
    assert pplb200.gemm_status() == 0
    y = out[0] if cfg["requant"] else out
    assert oracle.ulp_diff_f16(y.cpu().numpy(), ref["y"]).max() == 0
    if cfg["requant"]:
        assert np.array_equal(out[1].cpu().numpy(), ref["yq"])
        assert np.array_equal(oracle.f16_bits(out[2].cpu().numpy()), oracle.f16_bits(ref["ys"]))


@pytest.mark.parametrize("name", ["c2", "c3", "c4"])
def test_prefill_configs_sampled(cuda, oracle, name):
    import pplb200
    cfg, x, w, sn, bias = _inputs(name)
    M, K, N = cfg["M"], cfg["K"], cfg["N"]
    tx, tw, tsn, tb = _t(cuda, x), _t(cuda, w), _t(cuda, sn), _t(cuda, bias)
    lin = pplb200.W8A8Linear(tw, tsn, tb, max_tokens=M)
    y = lin(tx)
    cuda.cuda.synchronize()
    assert pplb200.gemm_status() == 0
    rng = np.random.default_rng(M + N)
    rows = np.unique(np.concatenate([[0, 1, M // 2, M - 2, M - 1], rng.integers(0, M, 27)]))
    ref = oracle.linear(x[rows], w, sn, bias)
    got = y[cuda.from_numpy(rows).cuda()].cpu().numpy()
    assert oracle.ulp_diff_f16(got, ref["y"]).max() == 0, name

    # full-size properties
    xq, sm = pplb200.minmax_quantize_fp16(tx)
    assert int(xq.abs().max()) <= 127
    assert np.array_equal(xq[cuda.from_numpy(rows).cuda()].cpu().numpy(), ref["xq"])
    acc = pplb200.gemm_i8i8(xq, tw)
    # exact check of a row block of the accumulators against an fp64 GEMM on the GPU
    blk = slice(0, min(M, 512))
    exact = (xq[blk].double() @ tw.double().T).to(cuda.int32)
    assert cuda.equal(acc[blk], exact)
    del exact
    # K split in 4 with strided operands, int32 partial sums == unsharded accumulators (linearity)
    parts = cuda.zeros_like(acc)
    kq = K // 4
    for r in range(4):
        parts += pplb200.gemm_i8i8(xq[:, r * kq:(r + 1) * kq], tw[:, r * kq:(r + 1) * kq])
    assert cuda.equal(parts, acc)
    # the standalone dequantizer applied to the accumulators reproduces the fused epilogue
    y2 = pplb200.minmax_dequantize_fp16(acc, sm, tsn, tb)
    assert cuda.equal(y2.view(cuda.int16), y.view(cuda.int16))


def test_column_parallel_shards_concatenate(cuda, oracle):
    """N split over 8 'ranks' run one after the other on one GPU: shard outputs == slices of the full output,
    including a shard width (2752) that is not a multiple of the tile width."""
    import pplb200
    import w8a8_workloads as wl
    cfg, x, w, sn, bias = _inputs("c2")
    M, K, N = 256, cfg["K"], cfg["N"]
    x = x[:M]
    tx, tw, tsn = _t(cuda, x), _t(cuda, w), _t(cuda, sn)
    xq, sm = pplb200.minmax_quantize_fp16(tx)
    full = pplb200.column_parallel_linear(xq, tw, sm, tsn, None, K, N)
    for size in (2, 8):
        for rank in range(size):
            n0, n1 = wl.shard_rows(N, size, rank)
            # size=1 call on the shard == what rank `rank` of `size` computes without gathering
            part = pplb200.column_parallel_linear(xq, tw[n0:n1].contiguous(), sm, tsn[n0:n1].contiguous(), None, K, n1 - n0)
            assert cuda.equal(part.view(cuda.int16), full[:, n0:n1].contiguous().view(cuda.int16))
            raw = pplb200.column_parallel_linear(xq, tw[n0:n1].contiguous(), None, None, None, K, n1 - n0, gather_output=False)
            assert raw.dtype == cuda.int32 and raw.shape == (M, n1 - n0)
    ref = oracle.linear(x[:8], w, sn, None)
    assert oracle.ulp_diff_f16(full[:8].cpu().numpy(), ref["y"]).max() == 0


def test_row_parallel_single_gpu_emulation(cuda, oracle):
    """The exact row-parallel reduction emulated on one GPU: per-shard int32 partials summed, then one
    dequant epilogue == the unsharded fused linear, bit for bit (what the NCCL path computes)."""
    import pplb200
    cfg, x, w, sn, bias = _inputs("c3")
    M, K, N = 128, cfg["K"], cfg["N"]
    x = x[:M]
    tx, tw, tsn, tb = _t(cuda, x), _t(cuda, w), _t(cuda, sn), _t(cuda, bias)
    xq, sm = pplb200.minmax_quantize_fp16(tx)
    full = pplb200.row_parallel_linear(xq, tw, sm, tsn, tb, K, N)  # size 1: fused epilogue
    for size in (2, 4, 8):
        kw = K // size
        acc = cuda.zeros((M, N), dtype=cuda.int32, device="cuda")
        for r in range(size):
            acc += pplb200.gemm_i8i8(xq[:, r * kw:(r + 1) * kw], tw[:, r * kw:(r + 1) * kw])
        y = pplb200.minmax_dequantize_fp16(acc, sm, tsn, tb)
        assert cuda.equal(y.view(cuda.int16), full.view(cuda.int16)), size
    ref = oracle.linear(x[:4], w, sn, bias)
    assert oracle.ulp_diff_f16(full[:4].cpu().numpy(), ref["y"]).max() == 0


def test_linear_error_codes(cuda):
    import pplb200
    w = cuda.zeros((64, 64), dtype=cuda.int8, device="cuda")
    s = cuda.ones((64,), dtype=cuda.float16, device="cuda")
    x = cuda.zeros((4, 64), dtype=cuda.int8, device="cuda")
    for layout in (pplb200.MATRIX_LAYOUT_COL4_4R2_8C, pplb200.MATRIX_LAYOUT_COL32_2R_4R4, pplb200.MATRIX_LAYOUT_COL_MAJOR):
        with pytest.raises(pplb200.PplError) as e:
            pplb200.column_parallel_linear(x, w, s, s, None, 64, 64, weight_layout=layout)
        assert e.value.rc == pplb200.RC_UNSUPPORTED
    with pytest.raises(pplb200.PplError) as e:
        pplb200.row_parallel_linear(x, w, s, s, None, 64, 64, input_is_parallel=False)
    assert e.value.rc == pplb200.RC_UNSUPPORTED


@pytest.mark.parametrize("M,K,N,chunk,requant", [(300, 512, 264, 128, False), (2500, 1024, 1032, 1024, False),
                                                 (96, 512, 272, 0, True), (1100, 256, 512, 256, True),
                                                 (2200, 512, 528, 1024, True)])  # the last: short first chunks + re-quantize
def test_linear_on_host_buffers_matches_device_path(cuda, oracle, M, K, N, chunk, requant):
    """pplb200_i8i8_linear_fp16_host: pinned host activations in, pinned host results out, chunks of the batch
    overlapped on three streams.  Bit-identical to the device-buffer linear (chunking is exact: every step works
    row by row), called twice in a row on the same staging buffers with different inputs."""
    import pplb200
    rng = np.random.default_rng(M + K + N)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sn = (rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16)
    tw, tsn, tb = _t(cuda, w), _t(cuda, sn), _t(cuda, bias)
    host = pplb200.W8A8LinearHost(tw, tsn, tb, max_tokens=M, requant=requant, chunk_rows=chunk)
    dev = pplb200.W8A8Linear(tw, tsn, tb, max_tokens=M, requant=requant)
    y_host = cuda.empty((M, N), dtype=cuda.float16).pin_memory()
    yq_host = cuda.empty((M, N), dtype=cuda.int8).pin_memory() if requant else None
    ys_host = cuda.empty((M,), dtype=cuda.float16).pin_memory() if requant else None
    for it in range(2):
        x = cuda.from_numpy(rng.standard_normal((M, K)).astype(np.float16)).pin_memory()
        host(x, y_host, yq_host, ys_host)
        want = dev(x.cuda())
        cuda.cuda.synchronize()
        if requant:
            assert cuda.equal(y_host.view(cuda.int16), want[0].cpu().view(cuda.int16))
            assert cuda.equal(yq_host, want[1].cpu()) and cuda.equal(ys_host.view(cuda.int16), want[2].cpu().view(cuda.int16))
        else:
            assert cuda.equal(y_host.view(cuda.int16), want.cpu().view(cuda.int16)), it
    ref = oracle.linear(x.numpy()[:8], w, sn, bias)
    assert np.array_equal(oracle.f16_bits(y_host[:8].numpy()), oracle.f16_bits(ref["y"]))
    assert pplb200.gemm_status() == 0
