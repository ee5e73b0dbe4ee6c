"""Generates tests/golden/reference_i8i8.npz: small input/output vectors produced by the
REFERENCE's own kernels (oracle/_ref/libref_i8i8.so, compiled unmodified from the reference tree)
running on a CUDA GPU.  The fixture pins the CPU oracle in the GPU-less test run.

    python tests/golden/make_golden.py [output.npz]

Needs a GPU and oracle/_ref (built by `make -C oracle ref` where the reference tree exists)."""
import ctypes
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_i8i8.npz")
    ref = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_i8i8.so"))
    vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_float
    ref.ref_minmax_quantize_fp16.argtypes = [vp, vp, i64, i64, f32, i32, vp, vp]
    ref.ref_minmax_dequantize_fp16.argtypes = [vp, vp, vp, vp, vp, i64, i64, f32, f32, i32, vp]
    ref.ref_column_parallel_linear.argtypes = [vp, vp, vp, vp, vp, vp, f32, f32, i64, i64, i64, i32, vp, vp, i64, vp]
    P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    T = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    rng = np.random.default_rng(20240607)
    d = {}

    # quantizer cases: (name, x)
    M, K = 24, 256
    xs = {
        "normal": rng.standard_normal((M, K)),
        "wide": rng.standard_normal((M, K)) * np.exp(rng.uniform(-8, 6, (M, 1))),
        "ties": np.concatenate([np.full((M, 1), 127.0), rng.integers(-254, 255, (M, K - 1)) / 2.0], axis=1),
        "tiny": rng.standard_normal((M, K)) * 1e-6,
    }
    for name, x in xs.items():
        x = x.astype(np.float16)
        x[3, :] = 0
        for layout in (0, 2):
            tx = T(x)
            q = torch.zeros((M, K), dtype=torch.int8, device="cuda")
            s = torch.zeros((M,), dtype=torch.float16, device="cuda")
            assert ref.ref_minmax_quantize_fp16(None, P(tx), M, K, 4096.0, layout, P(q), P(s)) == 0
            torch.cuda.synchronize()
            d["quant_%s_x" % name] = x
            d["quant_%s_l%d_q" % (name, layout)] = q.cpu().numpy()
            d["quant_%s_l%d_s" % (name, layout)] = s.cpu().numpy()

    # dequantizer cases
    M, N = 20, 96
    acc = rng.integers(-(2 ** 28), 2 ** 28, (M, N), dtype=np.int32)
    acc[0, :6] = [0, 1, -1, 2 ** 28 + 3, -(2 ** 27) - 1, 16777217]
    sm = (rng.uniform(0.001, 2.0, M) * 4096 / 127).astype(np.float16)
    sn = (rng.uniform(0.0005, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16)
    d.update(deq_acc=acc, deq_sm=sm, deq_sn=sn, deq_bias=bias)
    t_acc, t_sm, t_sn, t_bias = T(acc), T(sm), T(sn), T(bias)  # named: must outlive the asynchronous launches
    for tag, b in (("nobias", None), ("bias", t_bias)):
        y = torch.zeros((M, N), dtype=torch.float16, device="cuda")
        assert ref.ref_minmax_dequantize_fp16(None, P(t_acc), P(b), P(t_sm), P(t_sn), M, N,
                                              1 / 4096, 1 / 8192, 0, P(y)) == 0
        torch.cuda.synchronize()
        d["deq_y_%s" % tag] = y.cpu().numpy()

    # whole path through the reference's operators (cuBLASLt int8 GEMM inside)
    M, K, N = 64, 1024, 256  # M a power of 4: the reference tunes cuBLASLt on a rounded-down shape
    x = rng.standard_normal((M, K)).astype(np.float16)
    x[:, rng.choice(K, 5, replace=False)] *= 50
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sn = (rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16)
    tx, tw, tsn, tb = T(x), T(w), T(sn), T(bias)
    xq = torch.zeros((M, K), dtype=torch.int8, device="cuda")
    sm = torch.zeros((M,), dtype=torch.float16, device="cuda")
    acc = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    y = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    yq = torch.zeros((M, N), dtype=torch.int8, device="cuda")
    ys = torch.zeros((M,), dtype=torch.float16, device="cuda")
    ws = torch.zeros((32 << 20,), dtype=torch.uint8, device="cuda")
    assert ref.ref_minmax_quantize_fp16(None, P(tx), M, K, 4096.0, 0, P(xq), P(sm)) == 0
    rc = ref.ref_column_parallel_linear(None, P(xq), P(tw), P(tb), P(sm), P(tsn), 1 / 4096, 1 / 8192, M, N, K, 1, P(acc),
                                        P(ws), ws.numel(), P(y))
    assert rc == 0, "reference column_parallel_linear returned %d" % rc
    assert ref.ref_minmax_quantize_fp16(None, P(y), M, N, 4096.0, 0, P(yq), P(ys)) == 0
    torch.cuda.synchronize()
    d.update(lin_x=x, lin_w=w, lin_sn=sn, lin_bias=bias, lin_xq=xq.cpu().numpy(), lin_sm=sm.cpu().numpy(),
             lin_acc=acc.cpu().numpy(), lin_y=y.cpu().numpy(), lin_yq=yq.cpu().numpy(), lin_ys=ys.cpu().numpy())
    d["meta"] = np.array(["reference kernels (compute_80 PTX JIT + cuBLASLt) on %s, CUDA %s"
                          % (torch.cuda.get_device_name(0), torch.version.cuda)])
    np.savez_compressed(out, **d)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
