"""The workspace-free GEMM + re-quantize entry point (scratch in a fixed array inside the library,
for callers that cannot allocate device memory when they need the op) against the regular entry
point that takes a caller workspace.  Named so that pytest collects it last.

Two calls in a row on the same device share the built-in scratch: the second call uses inputs with
much smaller row maxima, so a scratch that was not cleared between calls would show up as wrong
re-quantization scales."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _t(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _case(cuda, rng, M, N, K, x_scale):
    import pplb200
    x = (rng.standard_normal((M, K)) * x_scale).astype(np.float16)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sn = (rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02 * x_scale).astype(np.float16)
    tx, tw, tsn, tb = _t(cuda, x), _t(cuda, w), _t(cuda, sn), _t(cuda, bias)
    xq, sm = pplb200.minmax_quantize_fp16(tx)
    want = pplb200.gemm_i8i8(xq, tw, mode=pplb200.EPI_DEQUANT_F16_REQUANT_I8, scale_m=sm, scale_n=tsn, bias=tb)
    got = pplb200.gemm_requant_static_scratch(xq, tw, sm, tsn, tb)
    cuda.cuda.synchronize()
    return want, got


@pytest.mark.parametrize("M,N,K", [(128, 1024, 512), (600, 2048, 256)])
def test_static_scratch_entry_matches_workspace_entry_twice(cuda, M, N, K):
    import pplb200
    rng = np.random.default_rng(M + N)
    for x_scale in (8.0, 0.05):  # second call: row maxima ~160x smaller than what the first call left behind
        want, got = _case(cuda, rng, M, N, K, x_scale)
        assert pplb200.gemm_status() == 0
        assert cuda.equal(got[0].view(cuda.int16), want[0].view(cuda.int16)), "fp16 output"
        assert cuda.equal(got[1], want[1]), "re-quantized int8 output"
        assert cuda.equal(got[2].view(cuda.int16), want[2].view(cuda.int16)), "re-quantization scales"
        assert int(got[1].abs().max()) == 127  # every row's maximum maps to +-127: the scales are the rows' own


def test_static_scratch_entry_rejects_too_many_rows(cuda):
    import pplb200
    M = pplb200.STATIC_SCRATCH_MAX_ROWS + 1
    a = cuda.zeros((M, 64), dtype=cuda.int8, device="cuda")
    b = cuda.zeros((64, 64), dtype=cuda.int8, device="cuda")
    s_m = cuda.ones((M,), dtype=cuda.float16, device="cuda")
    s_n = cuda.ones((64,), dtype=cuda.float16, device="cuda")
    with pytest.raises(pplb200.PplError) as e:
        pplb200.gemm_requant_static_scratch(a, b, s_m, s_n)
    assert e.value.rc == pplb200.RC_INVALID_VALUE
    assert "scratch" in pplb200.last_error()
