"""Operands in the Turing / Ampere tensor-core storage orders (COL32 activations, COL32_2R_4R4 / COL4_4R2_8C weights),
which the reference routes to gemm_i8i8i32_col32 (src/ppl/kernel/llm/cuda/pmx/i8i8/column_parallel_linear.cu:66-75,120-131;
index maps include/ppl/kernel/llm/cuda/common/matrix_layout.h:66-142): the re-layout kernel against the oracle's index
maps, and the linears on such operands against the same linears on row-major operands and against the oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROW_MAJOR, COL32, COL32_2R_4R4, COL4_4R2_8C = 0, 2, 3, 4


def _t(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("layout", [COL32, COL32_2R_4R4, COL4_4R2_8C])
@pytest.mark.parametrize("dtype", [np.int8, np.int32])
@pytest.mark.parametrize("rows,cols", [(64, 128), (96, 256), (32, 32)])
def test_relayout_matches_the_index_maps(cuda, oracle, layout, dtype, rows, cols):
    import pplb200
    rng = np.random.default_rng(rows + cols + layout)
    info = np.iinfo(dtype)
    mat = rng.integers(info.min, info.max, (rows, cols), dtype=dtype)
    flat, _ = oracle.to_layout(mat, layout)
    assert flat.size == rows * cols
    got = pplb200.relayout(_t(cuda, mat.ravel()), ROW_MAJOR, layout, rows, cols)   # row-major -> tiled
    assert np.array_equal(got.cpu().numpy(), flat)
    back = pplb200.relayout(_t(cuda, flat), layout, ROW_MAJOR, rows, cols)         # tiled -> row-major
    assert np.array_equal(back.cpu().numpy().reshape(rows, cols), mat)
    other = COL32 if layout != COL32 else COL32_2R_4R4                             # tiled -> tiled
    flat2, _ = oracle.to_layout(mat, other)
    assert np.array_equal(pplb200.relayout(_t(cuda, flat), layout, other, rows, cols).cpu().numpy(), flat2)


def test_relayout_error_codes(cuda):
    import pplb200
    a = cuda.zeros((64 * 64,), dtype=cuda.int8, device="cuda")
    for args in ((1, ROW_MAJOR, 64, 64), (COL32, ROW_MAJOR, 64, 48), (COL32_2R_4R4, ROW_MAJOR, 40, 64), (COL4_4R2_8C, ROW_MAJOR, 12, 64)):
        with pytest.raises(pplb200.PplError):
            pplb200.relayout(a, args[0], args[1], args[2], args[3])


@pytest.mark.parametrize("weight_layout", [COL32_2R_4R4, COL4_4R2_8C])
@pytest.mark.parametrize("M,K,N", [(16, 256, 512), (300, 512, 1056)])
def test_linears_on_legacy_operand_orders(cuda, oracle, weight_layout, M, K, N):
    import pplb200
    rng = np.random.default_rng(M + K + N + weight_layout)
    x = rng.standard_normal((M, K)).astype(np.float16)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sn = (rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16)
    ref = oracle.linear(x, w, sn, bias)
    # what a caller built for the Ampere path holds: COL32 quantized activations, weights in the tensor-core order
    xq_col32, sm = pplb200.minmax_quantize_fp16(_t(cuda, x), to_layout=COL32)
    assert np.array_equal(xq_col32.cpu().numpy().ravel(), oracle.to_layout(ref["xq"], COL32)[0])
    w_legacy = _t(cuda, oracle.to_layout(w, weight_layout)[0])
    tsn, tb = _t(cuda, sn), _t(cuda, bias)
    ws = cuda.empty((M * K + N * K + M * N * 4 + 1024,), dtype=cuda.uint8, device="cuda")

    y = pplb200.column_parallel_linear(xq_col32, w_legacy, sm, tsn, tb, K, N, weight_layout=weight_layout, ws=ws, M=M)
    assert np.array_equal(oracle.f16_bits(y.cpu().numpy()), oracle.f16_bits(ref["y"]))
    raw = pplb200.column_parallel_linear(xq_col32, w_legacy, None, None, None, K, N, gather_output=False,
                                         weight_layout=weight_layout, ws=ws, M=M)
    assert np.array_equal(raw.cpu().numpy().ravel(), oracle.to_layout(ref["acc"], COL32)[0])   # COL32, as the reference leaves it
    y2 = pplb200.row_parallel_linear(xq_col32, w_legacy, sm, tsn, tb, K, N, weight_layout=weight_layout, ws=ws, M=M)
    assert np.array_equal(oracle.f16_bits(y2.cpu().numpy()), oracle.f16_bits(ref["y"]))
    cuda.cuda.synchronize()
    assert pplb200.gemm_status() == 0
    # without room to re-lay the operands out the call refuses and says how much it needs
    with pytest.raises(pplb200.PplError) as e:
        pplb200.column_parallel_linear(xq_col32, w_legacy, sm, tsn, tb, K, N, weight_layout=weight_layout, M=M)
    assert e.value.rc == pplb200.RC_UNSUPPORTED and "bytes" in str(e.value)

    # load-time conversion: the same weights turned row-major once, then the ordinary path
    w_rm = pplb200.relayout(w_legacy, weight_layout, ROW_MAJOR, N, K).view(N, K)
    assert np.array_equal(w_rm.cpu().numpy(), w)
