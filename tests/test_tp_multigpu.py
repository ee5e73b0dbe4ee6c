"""Tensor-parallel linears on real GPUs (one process per GPU, NCCL over NVLink), through the C ABI.

Needs >= 2 CUDA devices; skipped otherwise.  Checks, bit for bit, that
  * the row-parallel linear with the exact int32 reduction equals the unsharded fused linear,
  * the row-parallel linear over peer-mapped memory (inter-process handles, no collective library on
    the data path) equals it too, call after call on the same buffers,
  * the column-parallel linear with gather_output equals the unsharded fused linear,
and that the reference-order fp16 reduction stays within a few ulp of the exact result."""
import os
import sys
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, tmp):
    sys.path.insert(0, os.path.join(ROOT, "ppl.llm.kernel.cuda_b200"))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    torch.cuda.set_device(rank)
    import pplb200
    import w8a8_workloads as wl

    uid_path = os.path.join(tmp, "uid")
    if rank == 0:
        with open(uid_path + ".tmp", "wb") as f:
            f.write(pplb200.nccl_unique_id())
        os.rename(uid_path + ".tmp", uid_path)
    t0 = time.time()
    while not os.path.exists(uid_path):
        if time.time() - t0 > 60:
            raise RuntimeError("rank %d: no NCCL id from rank 0" % rank)
        time.sleep(0.05)
    comm = pplb200.nccl_comm_init(open(uid_path, "rb").read(), rank, world)

    def file_barrier(tag):
        open(os.path.join(tmp, "%s.%d" % (tag, rank)), "w").close()
        t1 = time.time()
        while not all(os.path.exists(os.path.join(tmp, "%s.%d" % (tag, r))) for r in range(world)):
            if time.time() - t1 > 120:
                raise RuntimeError("rank %d: barrier %s timed out" % (rank, tag))
            time.sleep(0.02)

    p2p = pplb200.P2PContext(rank, world, 2048, 8192)
    with open(os.path.join(tmp, "p2p%d.tmp" % rank), "wb") as f:
        f.write(p2p.handle())
    os.rename(os.path.join(tmp, "p2p%d.tmp" % rank), os.path.join(tmp, "p2p%d" % rank))
    t0 = time.time()
    while not all(os.path.exists(os.path.join(tmp, "p2p%d" % r)) for r in range(world)):
        if time.time() - t0 > 120:
            raise RuntimeError("rank %d: peer handles missing" % rank)
        time.sleep(0.02)
    p2p.connect([open(os.path.join(tmp, "p2p%d" % r), "rb").read() for r in range(world)])

    # a second context for the column-parallel gather (it keeps the gathered matrix where the row-parallel
    # operator keeps its partial sums, so the two operators get separate contexts)
    p2p_col = pplb200.P2PContext(rank, world, 2048, 8192)
    with open(os.path.join(tmp, "p2pc%d.tmp" % rank), "wb") as f:
        f.write(p2p_col.handle())
    os.rename(os.path.join(tmp, "p2pc%d.tmp" % rank), os.path.join(tmp, "p2pc%d" % rank))
    t0 = time.time()
    while not all(os.path.exists(os.path.join(tmp, "p2pc%d" % r)) for r in range(world)):
        if time.time() - t0 > 120:
            raise RuntimeError("rank %d: peer handles missing" % rank)
        time.sleep(0.02)
    p2p_col.connect([open(os.path.join(tmp, "p2pc%d" % r), "rb").read() for r in range(world)])

    # the reference's own row_parallel_linear, when its library was built (same NCCL instance: the communicator is shared)
    ref = None
    ref_so = os.path.join(ROOT, "oracle", "_ref", "libref_i8i8.so")
    if os.path.exists(ref_so):
        import ctypes
        ref = ctypes.CDLL(ref_so)
        vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_float
        ref.ref_row_parallel_linear.argtypes = [vp, vp, vp, vp, vp, vp, f32, f32, i64, i64, i64, i32, i32, vp, vp, vp, i64, vp]

    rng = np.random.default_rng(123)  # same inputs on every rank
    results = {}
    # (2048, 2048, 8192) is large enough for the peer-memory path's two-chunk schedule (second stream); the last shape
    # gives 80 output tiles on 74 CTA pairs with a K shard long enough (on 2 GPUs) for the leftover tiles to be sliced
    for (M, K, N) in [(64, 1024, 512), (300, 2048, 1536), (1024, 1024, 768), (33, 512, 256), (2048, 2048, 8192), (2560, 8192, 2048)]:
        x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float16)).cuda()
        w = torch.from_numpy(rng.integers(-127, 128, (N, K), dtype=np.int8)).cuda()
        sn = torch.from_numpy((rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)).cuda()
        bias = torch.from_numpy((rng.standard_normal(N) * 0.02).astype(np.float16)).cuda()
        xq, sm = pplb200.minmax_quantize_fp16(x)
        full = pplb200.row_parallel_linear(xq, w, sm, sn, bias, K, N)  # size 1: unsharded fused linear

        k0, k1 = wl.shard_rows(K, world, rank)
        y_row = pplb200.row_parallel_linear(xq[:, k0:k1], w[:, k0:k1].contiguous(), sm, sn, bias, K, N,
                                            rank=rank, size=world, comm=comm)
        y_ref_order = pplb200.row_parallel_linear(xq[:, k0:k1], w[:, k0:k1].contiguous(), sm, sn, bias, K, N,
                                                  rank=rank, size=world, comm=comm, reduce_mode=1)
        if K % (16 * world) == 0:  # sharded quantizer: every rank passes only its K shard
            ok_q = True
            for rnd in range(3):  # new activations every round, the row maximum moving from shard to shard
                x_r = x.clone()
                x_r[:, (rnd * 37) % K::world] *= 3.0 + rnd
                xq_r, sm_r = pplb200.minmax_quantize_fp16(x_r)
                q_p2p, s_p2p = pplb200.minmax_quantize_fp16_p2p(p2p, x_r[:, k0:k1].contiguous())
                ok_q = ok_q and bool(torch.equal(q_p2p, xq_r[:, k0:k1])) and bool(torch.equal(s_p2p.view(torch.int16), sm_r.view(torch.int16)))
            results["%dx%d sharded quantizer exact" % (M, K)] = ok_q
        if M % world == 0:
            w_shard = w[:, k0:k1].contiguous()
            ok_p2p = True
            for _ in range(3):  # the same peer buffers, three calls in a row
                y_p2p = pplb200.row_parallel_linear_p2p(p2p, xq[:, k0:k1], w_shard, sm, sn, bias, K, N)
                ok_p2p = ok_p2p and bool(torch.equal(y_p2p.view(torch.int16), full.view(torch.int16)))
                if M * N >= (4 << 20):  # the opt-in two-chunk schedule (second stream), mixed with the default one
                    y_p2p = pplb200.row_parallel_linear_p2p(p2p, xq[:, k0:k1], w_shard, sm, sn, bias, K, N, phases=7 + 8)
                    ok_p2p = ok_p2p and bool(torch.equal(y_p2p.view(torch.int16), full.view(torch.int16)))
            results["%dx%dx%d row p2p exact" % (M, K, N)] = ok_p2p
        # An unchanged caller of the reference: every rank quantizes ITS OWN K shard, so the row scales differ from
        # rank to rank, bias is passed on every rank (applied on rank 0 only), reduction order of the reference.
        xq_s, sm_s = pplb200.minmax_quantize_fp16(x[:, k0:k1].contiguous())
        w_s = w[:, k0:k1].contiguous()
        y_own = pplb200.row_parallel_linear(xq_s, w_s, sm_s, sn, bias, K, N, rank=rank, size=world, comm=comm, reduce_mode=1)
        if ref is not None:
            acc_ref = torch.empty((M, N), dtype=torch.int32, device="cuda")
            y_ref = torch.empty((M, N), dtype=torch.float16, device="cuda")
            ws_ref = torch.empty((32 << 20,), dtype=torch.uint8, device="cuda")
            P = lambda t: ctypes.c_void_p(t.data_ptr())
            rc = ref.ref_row_parallel_linear(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), P(xq_s), P(w_s), P(bias),
                                             P(sm_s), P(sn), 1.0 / 4096, 1.0 / 8192, M, N, K, rank, world, comm, P(acc_ref),
                                             P(ws_ref), ws_ref.numel(), P(y_ref))
            torch.cuda.synchronize()
            # M = 33 / 300 trip the reference's own cuBLASLt tuning quirk (non power-of-four M): compare where it ran
            if rc == 0:
                tol = 4e-3 * y_ref.float().abs().max().item() + 1e-3
                results["%dx%dx%d per-rank scales: reference order equals the reference" % (M, K, N)] = \
                    bool((y_own.float() - y_ref.float()).abs().max().item() <= tol)
        results["%dx%dx%d per-rank scales differ between ranks" % (M, K, N)] = not bool(torch.equal(sm_s.view(torch.int16), sm.view(torch.int16)))
        n0, n1 = wl.shard_rows(N, world, rank)
        ok_colp = True
        for _ in range(2):  # peer-memory gather, twice on the same context
            y_colp = pplb200.column_parallel_linear_p2p(p2p_col, xq, w[n0:n1].contiguous(), sm, sn[n0:n1].contiguous(),
                                                        bias[n0:n1].contiguous(), K, N)
            ok_colp = ok_colp and bool(torch.equal(y_colp.view(torch.int16), full.view(torch.int16)))
        results["%dx%dx%d col gather over peer memory exact" % (M, K, N)] = ok_colp
        gather = torch.empty((world, M, n1 - n0), dtype=torch.float16, device="cuda")
        y_col = pplb200.column_parallel_linear(xq, w[n0:n1].contiguous(), sm, sn[n0:n1].contiguous(),
                                               bias[n0:n1].contiguous(), K, N, rank=rank, size=world, comm=comm,
                                               gather_output=True, gather_buffer=gather)
        torch.cuda.synchronize()
        key = "%dx%dx%d" % (M, K, N)
        results[key + " row exact"] = bool(torch.equal(y_row.view(torch.int16), full.view(torch.int16)))
        results[key + " col gather"] = bool(torch.equal(y_col.view(torch.int16), full.view(torch.int16)))
        err = (y_ref_order.float() - full.float()).abs().max().item()
        scale = full.float().abs().max().item()
        results[key + " fp16-order close"] = bool(err <= 4e-3 * scale + 1e-3)
    ok = pplb200.gemm_status() == 0 and p2p.status() == 0 and p2p_col.status() == 0
    torch.cuda.synchronize()
    file_barrier("p2p_done")  # no rank unmaps its buffer while a peer may still read it
    p2p.destroy()
    p2p_col.destroy()
    pplb200.nccl_comm_destroy(comm)
    with open(os.path.join(tmp, "rank%d" % rank), "w") as f:
        f.write(repr((ok, results)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_linears_match_unsharded(cuda, tmp_path, world):
    if cuda.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        ok, results = eval(open(os.path.join(str(tmp_path), "rank%d" % r)).read())
        assert ok, "GEMM status word set on rank %d" % r
        bad = [k for k, v in results.items() if not v]
        assert not bad, "rank %d: %s" % (r, bad)
