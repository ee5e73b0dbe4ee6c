"""The drop-in surface itself, executed: a C++ translation unit written against
ppl::kernel::llm::cuda::pmx::i8i8::* and ppl::kernel::llm::cuda::cublas::gemm_i8i8i32 exactly as the
reference's caller writes them (TensorShape, NcclParam, cublasLt handle, AlgoCache) is compiled against
include/, linked with the shared library, run on the GPU, and its outputs are compared bit for bit with
the oracle."""
import os
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CALLER = r'''
#include "ppl/kernel/llm/cuda/pmx/i8i8/quantize.h"
#include "ppl/kernel/llm/cuda/pmx/i8i8/column_parallel_linear.h"
#include "ppl/kernel/llm/cuda/pmx/i8i8/row_parallel_linear.h"
#include "ppl/kernel/llm/cuda/cublas/gemm.h"
#include <cuda_runtime.h>
#include <cublasLt.h>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>
namespace k = ppl::kernel::llm::cuda;
using ppl::common::TensorShape;

static std::vector<char> slurp(const std::string& path) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) { fprintf(stderr, "cannot open %s\n", path.c_str()); exit(2); }
    fseek(f, 0, SEEK_END); long n = ftell(f); fseek(f, 0, SEEK_SET);
    std::vector<char> v(n);
    if (fread(v.data(), 1, n, f) != (size_t)n) exit(2);
    fclose(f);
    return v;
}
static void* to_dev(const std::vector<char>& v) {
    void* p = nullptr;
    if (cudaMalloc(&p, v.size() ? v.size() : 16) != cudaSuccess) exit(3);
    cudaMemcpy(p, v.data(), v.size(), cudaMemcpyHostToDevice);
    return p;
}
static void dump(const std::string& path, const void* dev, size_t bytes) {
    std::vector<char> v(bytes);
    cudaMemcpy(v.data(), dev, bytes, cudaMemcpyDeviceToHost);
    FILE* f = fopen(path.c_str(), "wb");
    fwrite(v.data(), 1, bytes, f);
    fclose(f);
}
#define CHECK(call) do { auto rc_ = (call); if (rc_ != ppl::common::RC_SUCCESS) { fprintf(stderr, "%s -> %d\n", #call, (int)rc_); return 10 + (int)rc_; } } while (0)

int main(int argc, char** argv) {
    const std::string dir = argv[1];
    const int64_t M = atoll(argv[2]), K = atoll(argv[3]), N = atoll(argv[4]);
    void* x = to_dev(slurp(dir + "/x.bin"));      // fp16 [2, M/2, K]
    void* w = to_dev(slurp(dir + "/w.bin"));      // int8 [N, K]
    void* sn = to_dev(slurp(dir + "/sn.bin"));    // fp16 [N]
    void* bias = to_dev(slurp(dir + "/bias.bin")); // fp16 [N]
    void* bias32 = to_dev(slurp(dir + "/bias32.bin")); // int32 [N]
    void *xq, *sm, *acc, *y, *y_row, *y_deq, *acc_affine, *ws;
    cudaMalloc(&xq, M * K); cudaMalloc(&sm, M * 2); cudaMalloc(&acc, M * N * 4); cudaMalloc(&y, M * N * 2);
    cudaMalloc(&y_row, M * N * 2); cudaMalloc(&y_deq, M * N * 2); cudaMalloc(&acc_affine, M * N * 4); cudaMalloc(&ws, 1 << 20);
    cudaStream_t s;
    cudaStreamCreate(&s);
    cublasLtHandle_t lt = nullptr;   // accepted and ignored by the i8i8 operators
    k::cublas::AlgoCache cache;
    ppl::common::NcclParam nccl;     // one rank
    TensorShape in_shape(ppl::common::DATATYPE_INT8, {2, M / 2, K}), w_shape(ppl::common::DATATYPE_INT8, {N, K});
    TensorShape b_shape(ppl::common::DATATYPE_FLOAT16, {N}), out_shape(ppl::common::DATATYPE_FLOAT16, {2, M / 2, N});

    CHECK(k::pmx::i8i8::minmax_quantize_fp16(s, x, M, K, k::pmx::i8i8::token_up_scale, k::MATRIX_LAYOUT_ROW_MAJOR, xq, sm));
    // gather_output = true on one rank: dequantized fp16 output
    CHECK(k::pmx::i8i8::column_parallel_linear(s, lt, nullptr, &in_shape, xq, &w_shape, w, &b_shape, bias, sm, sn,
        k::pmx::i8i8::token_down_scale, k::pmx::i8i8::hidden_down_scale, K, N, k::MATRIX_LAYOUT_ROW_MAJOR, &nccl, true,
        nullptr, acc, 1 << 20, ws, &cache, &out_shape, y));
    // gather_output = false: raw int32 accumulators (the reference's quirk)
    CHECK(k::pmx::i8i8::column_parallel_linear(s, lt, nullptr, &in_shape, xq, &w_shape, w, &b_shape, bias, sm, sn,
        k::pmx::i8i8::token_down_scale, k::pmx::i8i8::hidden_down_scale, K, N, k::MATRIX_LAYOUT_ROW_MAJOR, &nccl, false,
        nullptr, nullptr, 1 << 20, ws, &cache, &out_shape, acc));
    CHECK(k::pmx::i8i8::row_parallel_linear(s, lt, nullptr, &in_shape, xq, &w_shape, w, &b_shape, bias, sm, sn,
        k::pmx::i8i8::token_down_scale, k::pmx::i8i8::hidden_down_scale, K, N, k::MATRIX_LAYOUT_ROW_MAJOR, &nccl, true,
        nullptr, acc_affine, 1 << 20, ws, &cache, &out_shape, y_row));
    CHECK(k::pmx::i8i8::minmax_dequantize_fp16(s, acc, bias, sm, sn, M, N, k::pmx::i8i8::token_down_scale,
        k::pmx::i8i8::hidden_down_scale, k::MATRIX_LAYOUT_ROW_MAJOR, y_deq));
    // the GEMM wrapper with its int32 scaling and bias: C = 2 * A B^T + 1 * C + bias32, C preset to the raw product
    cudaMemcpyAsync(acc_affine, acc, M * N * 4, cudaMemcpyDeviceToDevice, s);
    CHECK(k::cublas::gemm_i8i8i32(s, lt, nullptr, false, K, ppl::common::DATATYPE_INT8, xq, true, K, ppl::common::DATATYPE_INT8,
        w, bias32, M, N, K, 2, 1, 1 << 20, ws, &cache, N, ppl::common::DATATYPE_INT32, acc_affine));
    // argument checks answer like the reference's
    if (k::cublas::gemm_i8i8i32(s, lt, nullptr, true, K, ppl::common::DATATYPE_INT8, xq, true, K, ppl::common::DATATYPE_INT8,
        w, nullptr, M, N, K, 1, 0, 0, ws, &cache, N, ppl::common::DATATYPE_INT32, acc_affine) != ppl::common::RC_UNSUPPORTED) return 4;
    if (k::pmx::i8i8::row_parallel_linear(s, lt, nullptr, &in_shape, xq, &w_shape, w, &b_shape, bias, sm, sn,
        k::pmx::i8i8::token_down_scale, k::pmx::i8i8::hidden_down_scale, K, N, k::MATRIX_LAYOUT_ROW_MAJOR, &nccl, false,
        nullptr, acc_affine, 0, ws, &cache, &out_shape, y_row) != ppl::common::RC_UNSUPPORTED) return 5;
    if (cudaStreamSynchronize(s) != cudaSuccess) return 6;
    dump(dir + "/xq.out", xq, M * K); dump(dir + "/sm.out", sm, M * 2); dump(dir + "/acc.out", acc, M * N * 4);
    dump(dir + "/y.out", y, M * N * 2); dump(dir + "/y_row.out", y_row, M * N * 2); dump(dir + "/y_deq.out", y_deq, M * N * 2);
    dump(dir + "/acc_affine.out", acc_affine, M * N * 4);
    return 0;
}
'''


@pytest.mark.parametrize("M,K,N", [(16, 512, 264), (384, 1024, 1160)])
def test_cxx_caller_runs_and_matches_the_oracle(cuda, oracle, tmp_path, M, K, N):
    src = tmp_path / "caller.cpp"
    src.write_text(CALLER)
    exe = tmp_path / "caller"
    libdir = os.path.join(ROOT, "ppl.llm.kernel.cuda_b200", "lib")
    subprocess.run(["g++", "-std=c++17", "-O1", "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(ROOT, "include", "compat"),
                    "-I/usr/local/cuda/include", str(src), "-o", str(exe), "-L" + libdir, "-lpplb200_i8i8",
                    "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath," + libdir, "-Wl,-rpath,/usr/local/cuda/lib64"], check=True)
    rng = np.random.default_rng(M + K + N)
    x = rng.standard_normal((M, K)).astype(np.float16)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sn = (rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16)
    bias32 = rng.integers(-1000, 1000, N, dtype=np.int32)
    for name, arr in (("x", x), ("w", w), ("sn", sn), ("bias", bias), ("bias32", bias32)):
        arr.tofile(tmp_path / (name + ".bin"))
    r = subprocess.run([str(exe), str(tmp_path), str(M), str(K), str(N)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    ref = oracle.linear(x, w, sn, bias)
    got = lambda name, dt, shape: np.fromfile(tmp_path / (name + ".out"), dtype=dt).reshape(shape)
    assert np.array_equal(got("xq", np.int8, (M, K)), ref["xq"])
    assert np.array_equal(got("sm", np.uint16, (M,)), oracle.f16_bits(ref["sm"]))
    assert np.array_equal(got("acc", np.int32, (M, N)), ref["acc"])
    for name in ("y", "y_row", "y_deq"):
        assert np.array_equal(got(name, np.uint16, (M, N)), oracle.f16_bits(ref["y"])), name
    want = (3 * ref["acc"].astype(np.int64) + bias32[None, :]).astype(np.int32)
    assert np.array_equal(got("acc_affine", np.int32, (M, N)), want)
