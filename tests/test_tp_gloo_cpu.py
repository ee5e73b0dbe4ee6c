"""Host-side logic of the tensor-parallel paths with two CPU ranks over gloo: shard planning and
the exactness argument of the row-parallel reduction (int32 all-reduce of partials, then ONE
dequant epilogue == unsharded result), with the oracle as the compute on each rank.  The schedule of
the peer-memory path is modelled too: quantize the K shard with the row maximum taken over all
shards, send each owner its row slice of the int32 partial, owner sums and dequantizes, rows are
gathered back."""
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
    import w8a8_workloads as wl
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

    # the peer-memory schedule.  (1) sharded quantizer: shard maxima exchanged, scale from the global maximum
    xs = np.ascontiguousarray(x[:, k0:k1])
    shard_max = np.abs(xs.astype(np.float32)).max(axis=1)
    maxima = [torch.empty(M, dtype=torch.float32) for _ in range(world)]
    dist.all_gather(maxima, torch.from_numpy(shard_max.copy()))
    row_max = torch.stack(maxima, 0).max(dim=0).values.numpy()
    scale = np.maximum(row_max / np.float32(127.0), np.float32(1e-7)).astype(np.float32)
    q_shard = np.rint(xs.astype(np.float32) / scale[:, None]).astype(np.int8)   # IEEE division, round half to even
    sm_shard = (scale * np.float32(4096.0)).astype(np.float16)
    ok_q = np.array_equal(q_shard, xq[:, k0:k1]) and np.array_equal(sm_shard.view(np.uint16), sm.view(np.uint16))
    # (2) every rank sends owner o the rows [o Ms, (o + 1) Ms) of its partial; (3) the owner sums the slices in
    # int32 and runs the epilogue once; (4) finished fp16 rows are gathered on every rank
    Ms = M // world
    part2 = orc.gemm(q_shard, np.ascontiguousarray(w[:, k0:k1]))
    send = [torch.from_numpy(part2[o * Ms:(o + 1) * Ms].copy()) for o in range(world)]
    recv = [torch.empty((Ms, N), dtype=torch.int32) for _ in range(world)]
    for o in range(world):  # gloo has no all_to_all: one gather per owner
        dist.gather(send[o], recv if rank == o else None, dst=o)
    mine = torch.stack(recv, 0).sum(dim=0, dtype=torch.int32).numpy()
    _, y_mine = orc.dequantize(mine, sm_shard[rank * Ms:(rank + 1) * Ms], sn, bias)
    rows = [torch.empty((Ms, N * 2), dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(rows, torch.from_numpy(np.ascontiguousarray(y_mine).view(np.uint8).copy()))
    y_p2p = torch.cat(rows, 0).numpy()
    ok_p2p = ok_q and np.array_equal(y_p2p.view(np.uint16).reshape(M, N), full["y"].view(np.uint16))

    # column parallel: N shard, no communication; gather only to check
    n0, n1 = wl.shard_rows(N, world, rank)
    shard = orc.linear(x, np.ascontiguousarray(w[n0:n1]), np.ascontiguousarray(sn[n0:n1]), np.ascontiguousarray(bias[n0:n1]))
    gathered = [torch.empty((M, (n1 - n0) * 2), dtype=torch.uint8) for _ in range(world)]  # fp16 as bytes
    dist.all_gather(gathered, torch.from_numpy(shard["y"].view(np.uint8).copy()))
    y_col = torch.stack(gathered, 0).permute(1, 0, 2).reshape(M, N * 2).contiguous().numpy()  # [w, M, N/w] -> [M, N]
    ok_col = np.array_equal(y_col.view(np.uint16), full["y"].view(np.uint16))

    with open(os.path.join(out_dir, "rank%d" % rank), "w") as f:
        f.write("%d %d %d" % (ok_row, ok_col, ok_p2p))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_rank_sharding_is_exact(tmp_path, world):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(os.path.join(str(tmp_path), "rank%d" % r)).read() == "1 1 1"
