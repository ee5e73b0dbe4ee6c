"""Host-side logic of the tensor-parallel paths with two CPU ranks over gloo: shard planning and
the exactness argument of the row-parallel reduction (int32 all-reduce of partials, then ONE
dequant epilogue == unsharded result), with the oracle as the compute on each rank."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    sys.path.insert(0, os.path.join(ROOT, "ppl.llm.kernel.cuda_b200"))
    import torch
    import torch.distributed as dist
    import oracle_lib as orc
    from pplb200 import workloads as wl
    orc.set_threads(1)
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    rng = np.random.default_rng(11)  # same stream on every rank: replicated inputs
    M, K, N = 12, 256, 64
    x = rng.standard_normal((M, K)).astype(np.float16)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sn = (rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float16)
    full = orc.linear(x, w, sn, bias)

    # row parallel: full-row scales, K shard, int32 all-reduce, one dequant epilogue with the bias
    k0, k1 = wl.shard_rows(K, world, rank)
    _, xq, sm = orc.quantize(x)
    part = orc.gemm(np.ascontiguousarray(xq[:, k0:k1]), np.ascontiguousarray(w[:, k0:k1]))
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    _, y_row = orc.dequantize(t.numpy(), sm, sn, bias)
    ok_row = np.array_equal(y_row.view(np.uint16), full["y"].view(np.uint16)) and np.array_equal(t.numpy(), full["acc"])

    # column parallel: N shard, no communication; gather only to check
    n0, n1 = wl.shard_rows(N, world, rank)
    shard = orc.linear(x, np.ascontiguousarray(w[n0:n1]), np.ascontiguousarray(sn[n0:n1]), np.ascontiguousarray(bias[n0:n1]))
    gathered = [torch.empty((M, (n1 - n0) * 2), dtype=torch.uint8) for _ in range(world)]  # fp16 as bytes
    dist.all_gather(gathered, torch.from_numpy(shard["y"].view(np.uint8).copy()))
    y_col = torch.stack(gathered, 0).permute(1, 0, 2).reshape(M, N * 2).contiguous().numpy()  # [w, M, N/w] -> [M, N]
    ok_col = np.array_equal(y_col.view(np.uint16), full["y"].view(np.uint16))

    with open(os.path.join(out_dir, "rank%d" % rank), "w") as f:
        f.write("%d %d" % (ok_row, ok_col))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_rank_sharding_is_exact(tmp_path, world):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(os.path.join(str(tmp_path), "rank%d" % r)).read() == "1 1"
