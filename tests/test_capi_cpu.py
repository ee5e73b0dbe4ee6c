"""GPU-less checks of the product's boundary: the shared library loads, exports every symbol the
C header declares, its host-only helpers agree with the oracle, and the reference-compatible C++
headers compile against the stand-in ppl.common headers."""
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "pplb200_i8i8.h")


def declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(pplb200_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    import pplb200
    names = declared_symbols()
    assert len(names) >= 32
    for n in names:
        assert hasattr(pplb200.lib, n), "missing export: " + n
    assert set(names) == set(pplb200.EXPORTS)
    assert "sm_100a" in pplb200.version()


def test_no_torch_types_in_c_header():
    src = open(HEADER).read()
    assert "torch" not in src.lower() and "at::" not in src and "#include <cuda" not in src


def test_c_header_is_plain_c99(tmp_path):
    """The boundary is a C ABI: the header compiles as strict C99 and a C program links against the library."""
    src = tmp_path / "c_caller.c"
    src.write_text('#include "pplb200_i8i8.h"\n#include <string.h>\n'
                   'int main(void) {\n'
                   '    if (strstr(pplb200_version(), "sm_100a") == 0) return 1;\n'
                   '    if (pplb200_layout_offset(0, 4, 8, 1, 2) != 10) return 2;\n'
                   '    if (pplb200_i8i8_row_parallel_p2p_bytes(-1, 8, 2) != -1) return 3;\n'
                   '    return 0;\n}\n')
    exe = tmp_path / "c_caller"
    lib_dir = os.path.join(ROOT, "ppl.llm.kernel.cuda_b200", "lib")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I" + os.path.join(ROOT, "include"),
                    str(src), "-o", str(exe), "-L" + lib_dir, "-lpplb200_i8i8", "-Wl,-rpath," + lib_dir], check=True)
    assert subprocess.run([str(exe)]).returncode == 0


@pytest.mark.parametrize("layout", [0, 1, 2, 3, 4])
def test_layout_offsets_match_oracle(oracle, layout):
    import pplb200
    rows, cols = 64, 96
    for r in range(rows):
        for c in range(0, cols, 5):
            assert pplb200.lib.pplb200_layout_offset(layout, rows, cols, r, c) == oracle.layout_offset(layout, rows, cols, r, c)
    assert pplb200.lib.pplb200_layout_offset(9, rows, cols, 0, 0) == -1


def test_workspace_sizes():
    import pplb200
    assert pplb200.gemm_workspace_bytes(128, 12288, 4096, pplb200.EPI_RAW_I32) == 0
    assert pplb200.gemm_workspace_bytes(128, 12288, 4096, pplb200.EPI_DEQUANT_F16) == 0
    assert pplb200.gemm_workspace_bytes(128, 12288, 4096, pplb200.EPI_DEQUANT_F16_REQUANT_I8) >= 128 * 4
    need = pplb200.linear_workspace_bytes(128, 12288, 4096, pplb200.EPI_DEQUANT_F16_REQUANT_I8)
    assert need >= 128 * 4096 + 128 * 2 + 128 * 4 and need % 256 == 0
    # peer buffer of the row-parallel linear: flags + row-maximum slots + int32 partials [M, N] + fp16 rows [M / size, N]
    b = pplb200.lib.pplb200_i8i8_row_parallel_p2p_bytes(2048, 8192, 8)
    assert b >= 2048 * 8192 * 4 + 256 * 8192 * 2 and b % 256 == 0
    assert pplb200.lib.pplb200_i8i8_row_parallel_p2p_bytes(2048, 8192, 9) == -1   # more ranks than one NVLink domain holds
    assert pplb200.lib.pplb200_i8i8_row_parallel_p2p_bytes(2048, 8192, 0) == -1


def test_reference_compatible_headers_compile(tmp_path):
    """A translation unit written against the reference's operator API (same namespaces, names and
    argument lists as its own call sites) compiles unchanged against include/."""
    src = tmp_path / "caller.cpp"
    src.write_text(r'''
#include "ppl/kernel/llm/cuda/pmx/i8i8/quantize.h"
#include "ppl/kernel/llm/cuda/pmx/i8i8/column_parallel_linear.h"
#include "ppl/kernel/llm/cuda/pmx/i8i8/row_parallel_linear.h"
#include "ppl/kernel/llm/cuda/cublas/gemm.h"
namespace k = ppl::kernel::llm::cuda;
ppl::common::RetCode run(cudaStream_t s, cublasLtHandle_t lt, k::cublas::AlgoCache* cache, ppl::common::NcclParam* nccl,
                         const void* x, void* xq, void* sm, const void* w, const void* sn, const void* bias,
                         void* qbuf, void* ws, void* y) {
    ppl::common::TensorShape in(ppl::common::DATATYPE_INT8, {2, 8, 4096}), wt(ppl::common::DATATYPE_INT8, {4096, 4096});
    ppl::common::TensorShape b(ppl::common::DATATYPE_FLOAT16, {4096}), out(ppl::common::DATATYPE_FLOAT16, {2, 8, 4096});
    auto rc = k::pmx::i8i8::minmax_quantize_fp16(s, x, 16, 4096, k::pmx::i8i8::token_up_scale, k::MATRIX_LAYOUT_ROW_MAJOR, xq, sm);
    if (rc != ppl::common::RC_SUCCESS) return rc;
    rc = k::pmx::i8i8::column_parallel_linear(s, lt, nullptr, &in, xq, &wt, w, &b, bias, sm, sn,
        k::pmx::i8i8::token_down_scale, k::pmx::i8i8::hidden_down_scale, 4096, 4096, k::MATRIX_LAYOUT_ROW_MAJOR,
        nccl, true, nullptr, qbuf, 0, ws, cache, &out, y);
    if (rc != ppl::common::RC_SUCCESS) return rc;
    rc = k::pmx::i8i8::row_parallel_linear(s, lt, nullptr, &in, xq, &wt, w, &b, bias, sm, sn,
        k::pmx::i8i8::token_down_scale, k::pmx::i8i8::hidden_down_scale, 4096, 4096, k::MATRIX_LAYOUT_ROW_MAJOR,
        nccl, true, nullptr, qbuf, 0, ws, cache, &out, y);
    if (rc != ppl::common::RC_SUCCESS) return rc;
    rc = k::cublas::gemm_i8i8i32(s, lt, nullptr, false, 4096, ppl::common::DATATYPE_INT8, xq, true, 4096,
        ppl::common::DATATYPE_INT8, w, nullptr, 16, 4096, 4096, 1, 0, 0, ws, cache, 4096, ppl::common::DATATYPE_INT32, qbuf);
    if (rc != ppl::common::RC_SUCCESS) return rc;
    rc = k::pmx::i8i8::minmax_dequantize_fp16(s, qbuf, bias, sm, sn, 16, 4096, k::pmx::i8i8::token_down_scale,
        k::pmx::i8i8::hidden_down_scale, k::MATRIX_LAYOUT_ROW_MAJOR, y);
    if (rc != ppl::common::RC_SUCCESS) return rc;
    // the producers / consumers around the linear, same argument lists as the reference header
    rc = k::pmx::i8i8::skip_rmsnorm_minmax_quantize_fp16(s, x, w, nullptr, 1e-5f, 16, 4096, k::pmx::i8i8::token_up_scale,
        k::MATRIX_LAYOUT_ROW_MAJOR, y, sm, xq);
    if (rc != ppl::common::RC_SUCCESS) return rc;
    rc = k::pmx::i8i8::minmax_dequantize_split3_fp16(s, qbuf, bias, sm, sn, 16, 4096, 2048, 1024, 1024,
        k::pmx::i8i8::token_down_scale, k::pmx::i8i8::hidden_down_scale, k::MATRIX_LAYOUT_ROW_MAJOR, y, y, y);
    if (rc != ppl::common::RC_SUCCESS) return rc;
    rc = k::pmx::i8i8::minmax_requantize_silu_fp16(s, qbuf, sm, sn, nullptr, nullptr, nullptr, 16, 4096,
        k::MATRIX_LAYOUT_ROW_MAJOR, k::pmx::i8i8::token_up_scale, k::pmx::i8i8::token_down_scale,
        k::pmx::i8i8::hidden_down_scale, y, xq, sm);
    if (rc != ppl::common::RC_SUCCESS) return rc;
    rc = k::pmx::i8i8::minmax_dequantize_silu_fp16(s, qbuf, sm, sn, nullptr, nullptr, nullptr, 16, 4096,
        k::MATRIX_LAYOUT_ROW_MAJOR, k::pmx::i8i8::token_down_scale, k::pmx::i8i8::hidden_down_scale, y);
    if (rc != ppl::common::RC_SUCCESS) return rc;
    rc = k::pmx::i8i8::minmax_requantize_swiglu_fp16(s, qbuf, sm, sn, 16, 2048, 1.0f, k::MATRIX_LAYOUT_ROW_MAJOR,
        k::pmx::i8i8::token_up_scale, k::pmx::i8i8::token_down_scale, k::pmx::i8i8::hidden_down_scale, y, xq, sm);
    if (rc != ppl::common::RC_SUCCESS) return rc;
    // additions without a reference counterpart: the peer-memory forms of the row-parallel pair
    void* p2p = nullptr;
    rc = k::pmx::i8i8::minmax_quantize_fp16_sharded(s, p2p, &in, x, k::pmx::i8i8::token_up_scale, xq, sm);
    if (rc != ppl::common::RC_SUCCESS) return rc;
    return k::pmx::i8i8::row_parallel_linear(s, p2p, &in, xq, &b, bias, sm, sn, k::pmx::i8i8::token_down_scale,
        k::pmx::i8i8::hidden_down_scale, 4096, 4096, w, y);
}
int main() {
    k::MatrixLayoutHelper<k::MATRIX_LAYOUT_COL32> h;
    h.Init(4, 64);
    return h.GetOffset(1, 33) == 4 * 32 + 32 + 1 ? 0 : 1;
}
''')
    exe = tmp_path / "caller"
    cmd = ["g++", "-std=c++17", "-Wall", "-Werror", "-I" + os.path.join(ROOT, "include"),
           "-I" + os.path.join(ROOT, "include", "compat"), "-I/usr/local/cuda/include", str(src), "-o", str(exe),
           "-L" + os.path.join(ROOT, "ppl.llm.kernel.cuda_b200", "lib"), "-lpplb200_i8i8",
           "-Wl,-rpath," + os.path.join(ROOT, "ppl.llm.kernel.cuda_b200", "lib")]
    subprocess.run(cmd, check=True)
    assert subprocess.run([str(exe)]).returncode == 0


def test_workload_generators_are_deterministic_and_shaped():
    import w8a8_workloads as wl
    assert [wl.algorithmic_bytes(n) for n in ("c0", "c1", "c2", "c3", "c4")] == \
        [17055744, 56148224, 304131072, 385908736, 838918144]
    x1, x2 = wl.make_activations("c2", 40), wl.make_activations("c2", 300)
    assert x1.dtype == np.float16 and x1.shape == (40, 4096) and np.array_equal(x1, x2[:40])
    ch = wl.outlier_channels("c2")
    assert len(ch) == 40 and len(np.unique(ch)) == 40
    col_rms = np.sqrt((x2.astype(np.float32) ** 2).mean(axis=0))
    assert col_rms[ch].min() > 20 and np.delete(col_rms, ch).max() < 2
    x4 = wl.make_activations("c4", 64).astype(np.float32)
    assert np.abs(x4).max() <= 200 and np.abs(x4).max() > 20      # heavy tails, clipped
    w = wl.make_weights("c0")
    assert w.dtype == np.int8 and w.min() == -127 and w.max() == 127
    s = wl.make_column_scales("c3").astype(np.float32) / 8192
    assert 0.0005 * 0.999 <= s.min() and s.max() <= 0.005 * 1.001
    assert wl.make_bias("c2") is None and wl.make_bias("c0").shape == (4096,)
    assert wl.shard_rows(22016, 8, 7) == (19264, 22016)
    with pytest.raises(AssertionError):
        wl.shard_rows(10, 4, 0)


REFERENCE_DIR = os.environ.get("PPL_LLM_KERNEL_CUDA_REFERENCE", "/root/reference")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE_DIR, "include")), reason="reference tree not present")
def test_shadow_headers_coexist_with_the_references_other_operators(tmp_path):
    """With this repository's include directory placed BEFORE the reference's, translation units of the
    reference's other linears (fp16 column / row parallel linear, MoE linears, i4f16, f8f8 headers) still compile:
    the shadowing cublas/gemm.h and cublas/gemm_algo.h keep every declaration those headers and their callers
    use (fp16 gemm, AlgoCache with its real key / hash types, find_best_algo, MatmulDesc ...)."""
    src = tmp_path / "mixed.cpp"
    src.write_text(r'''
#include "ppl/kernel/llm/cuda/pmx/i8i8/column_parallel_linear.h"   // this repository's
#include "ppl/kernel/llm/cuda/pmx/i8i8/row_parallel_linear.h"      // this repository's
#include "ppl/kernel/llm/cuda/pmx/column_parallel_linear.h"        // the reference's (fp16)
#include "ppl/kernel/llm/cuda/pmx/row_parallel_linear.h"           // the reference's (fp16)
#include "ppl/kernel/llm/cuda/pmx/moe_column_parallel_linear.h"    // the reference's
#include "ppl/kernel/llm/cuda/cublas/gemm.h"
#include <type_traits>
namespace c = ppl::kernel::llm::cuda::cublas;
static_assert(std::is_same<c::AlgoCache::key_type, c::AlgoCacheIndex>::value, "AlgoCache key type");
static_assert(std::is_same<c::AlgoCache::hasher, c::AlgoCacheIndexHash>::value, "AlgoCache hash type");
int main() {
    c::AlgoCache cache;
    c::AlgoCacheIndex idx{};
    idx.matmul_desc.transa = CUBLAS_OP_T;
    cache.emplace(idx, cublasLtMatmulAlgo_t{});
    // the fp16 GEMM and the algorithm search stay declared (their definitions live in the reference's library)
    auto gemm_ptr = &c::gemm;
    auto find_ptr = &c::find_best_algo;
    (void)gemm_ptr; (void)find_ptr;
    return cache.count(idx) == 1 ? 0 : 1;
}
''')
    obj = tmp_path / "mixed.o"
    cmd = ["g++", "-std=c++17", "-Wall", "-c", "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(REFERENCE_DIR, "include"),
           "-I" + os.path.join(ROOT, "include", "compat"), "-I/usr/local/cuda/include", str(src), "-o", str(obj)]
    subprocess.run(cmd, check=True)
