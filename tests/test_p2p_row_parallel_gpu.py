"""Row-parallel linear over peer-mapped buffers, all ranks driven by ONE process on ONE device.

The ranks' contexts are connected with `connect_local` and the three phases are enqueued rank after
rank on one stream (all produce, then all reduce, then all gather), so every flag a kernel waits
for has already been written by an earlier launch: nothing ever spins on a kernel that is not
running.  The real one-process-per-GPU form (inter-process handles, NVLink) is covered by
tests/test_tp_multigpu.py.

Bar: bit-identical to the unsharded fused linear."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(torch, pplb200, wl, world, M, K, N, with_bias, rounds=1, seed=0):
    rng = np.random.default_rng(seed)
    ctxs = [pplb200.P2PContext(r, world, M, N) for r in range(world)]
    try:
        for c in ctxs:
            c.connect_local(ctxs)
        for it in range(rounds):
            x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float16)).cuda()
            w = torch.from_numpy(rng.integers(-127, 128, (N, K), dtype=np.int8)).cuda()
            sn = torch.from_numpy((rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)).cuda()
            bias = torch.from_numpy((rng.standard_normal(N) * 0.02).astype(np.float16)).cuda() if with_bias else None
            xq, sm = pplb200.minmax_quantize_fp16(x)
            full = pplb200.row_parallel_linear(xq, w, sm, sn, bias, K, N)
            shards = []
            for r in range(world):
                k0, k1 = wl.shard_rows(K, world, r)
                shards.append((xq[:, k0:k1], w[:, k0:k1].contiguous()))  # activation shard stays a strided view
            outs = [torch.zeros((M, N), dtype=torch.float16, device="cuda") for _ in range(world)]
            for phase in (1, 2, 4):
                for r in range(world):
                    pplb200.row_parallel_linear_p2p(ctxs[r], shards[r][0], shards[r][1], sm, sn, bias, K, N,
                                                    out=outs[r], phases=phase)
            torch.cuda.synchronize()
            for r in range(world):
                assert ctxs[r].status() == 0
                assert torch.equal(outs[r].view(torch.int16), full.view(torch.int16)), \
                    "rank %d of %d differs (round %d, M=%d K=%d N=%d)" % (r, world, it, M, K, N)
        assert pplb200.gemm_status() == 0
    finally:
        for c in ctxs:
            c.destroy()


@pytest.mark.parametrize("world,M,K,N,with_bias", [
    (2, 512, 1024, 512, True),      # whole 256 x 256 tiles
    (2, 64, 512, 264, False),       # one ragged tile, rows of both owners inside it
    (4, 1000, 2048, 1544, True),    # ragged in M and N; owner boundaries (250 rows) inside tiles
    (8, 2048, 1024, 1024, True),    # one tile row per owner
    (8, 40, 1024, 72, True),        # 5 rows per owner
    (3, 390, 768, 520, False),      # odd number of ranks
    (1, 300, 512, 256, True),       # a single rank: no exchange
    (2, 2560, 8192, 2048, True),    # 80 tiles on 74 CTA pairs: tiles shared between pairs as K segments
])
def test_p2p_row_parallel_matches_unsharded(cuda, pplb200, world, M, K, N, with_bias):
    import w8a8_workloads as wl
    _case(cuda, pplb200, wl, world, M, K, N, with_bias)


def test_p2p_buffers_are_reusable_across_calls(cuda, pplb200):
    import w8a8_workloads as wl
    _case(cuda, pplb200, wl, 4, 768, 1024, 768, True, rounds=4, seed=7)


def test_p2p_argument_checks(cuda, pplb200):
    torch = cuda
    ctx = pplb200.P2PContext(0, 2, 64, 64)
    try:
        xq = torch.zeros((64, 128), dtype=torch.int8, device="cuda")
        w = torch.zeros((64, 128), dtype=torch.int8, device="cuda")
        s = torch.ones(64, dtype=torch.float16, device="cuda")
        with pytest.raises(pplb200.PplError) as e:  # not connected yet
            pplb200.row_parallel_linear_p2p(ctx, xq, w, s, s, None, 256, 64)
        assert e.value.rc == pplb200.RC_INVALID_VALUE
        other = pplb200.P2PContext(1, 2, 64, 64)
        try:
            ctx.connect_local([ctx, other])
            with pytest.raises(pplb200.PplError) as e:  # buffer sized for 64 x 64
                pplb200.row_parallel_linear_p2p(ctx, torch.zeros((128, 128), dtype=torch.int8, device="cuda"), w,
                                                torch.ones(128, dtype=torch.float16, device="cuda"), s, None, 256, 64)
            assert e.value.rc == pplb200.RC_INVALID_VALUE
            with pytest.raises(pplb200.PplError) as e:  # M not divisible by the number of ranks
                pplb200.row_parallel_linear_p2p(ctx, xq[:63], w, s[:63], s, None, 256, 64)
            assert e.value.rc == pplb200.RC_UNSUPPORTED
        finally:
            other.destroy()
    finally:
        ctx.destroy()


def test_p2p_wait_gives_up_and_reports(cuda, pplb200):
    """A rank whose peer never produces: the bounded wait runs out (about two seconds), the status
    word says which phase was missing, later calls do not wait, and the device stays usable."""
    torch = cuda
    a, b = pplb200.P2PContext(0, 2, 64, 64), pplb200.P2PContext(1, 2, 64, 64)
    try:
        a.connect_local([a, b])
        b.connect_local([a, b])
        xq = torch.zeros((64, 128), dtype=torch.int8, device="cuda")
        w = torch.zeros((64, 128), dtype=torch.int8, device="cuda")
        s = torch.ones(64, dtype=torch.float16, device="cuda")
        pplb200.row_parallel_linear_p2p(a, xq, w, s, s, None, 256, 64, phases=1)  # rank 1 never produces
        pplb200.row_parallel_linear_p2p(a, xq, w, s, s, None, 256, 64, phases=2)
        torch.cuda.synchronize()
        assert a.status(reset=False) == 1
        pplb200.row_parallel_linear_p2p(a, xq, w, s, s, None, 256, 64, phases=6)  # returns without waiting again
        torch.cuda.synchronize()
        assert a.status() & 1
        assert a.status() == 0
        y = pplb200.minmax_quantize_fp16(torch.ones((4, 64), dtype=torch.float16, device="cuda"))[0]
        assert int(y.abs().max()) == 127
    finally:
        a.destroy()
        b.destroy()


@pytest.mark.parametrize("world,M,K", [
    (2, 64, 1024),       # 512-element shards: one unit per thread, partial block
    (4, 300, 8192),      # 2048-element shards
    (8, 2048, 28672),    # the row-parallel workload's shape: 3584-element shards, more rows than resident CTAs
    (2, 16, 65536),      # 32768-element shards: eight units per thread
    (3, 50, 3 * 400 * 16),
    (1, 40, 512),
])
def test_sharded_quantizer_matches_unsharded(cuda, pplb200, world, M, K):
    """Shard maxima are published for every rank first (phase 1), then every rank runs the whole
    operation (phase 3), so no kernel waits for one that has not run.  int8 and scales bit-exact."""
    torch = cuda
    import w8a8_workloads as wl
    rng = np.random.default_rng(M + K + world)
    x = rng.standard_normal((M, K)).astype(np.float16)
    x[:, rng.integers(0, K, 8)] *= 30.0   # the row maximum usually sits in one shard only
    if M > 3:
        x[3] = 0.0                         # an all-zero row: scale clamps to 1e-7
    x = torch.from_numpy(x).cuda()
    q_full, s_full = pplb200.minmax_quantize_fp16(x)
    ctxs = [pplb200.P2PContext(r, world, M, 64) for r in range(world)]
    try:
        for c in ctxs:
            c.connect_local(ctxs)
        for rounds in range(3):  # both slot banks, and a bank's reuse
            shards, outs = [], []
            for r in range(world):
                k0, k1 = wl.shard_rows(K, world, r)
                shards.append(x[:, k0:k1].contiguous())
            for r in range(world):
                pplb200.minmax_quantize_fp16_p2p(ctxs[r], shards[r], phases=1)
            for r in range(world):
                outs.append(pplb200.minmax_quantize_fp16_p2p(ctxs[r], shards[r]))
            torch.cuda.synchronize()
            for r in range(world):
                k0, k1 = wl.shard_rows(K, world, r)
                assert ctxs[r].status() == 0
                assert torch.equal(outs[r][1].view(torch.int16), s_full.view(torch.int16)), "scales, rank %d" % r
                assert torch.equal(outs[r][0], q_full[:, k0:k1]), "int8, rank %d" % r
    finally:
        for c in ctxs:
            c.destroy()


@pytest.mark.parametrize("world,M,K,N,with_bias", [
    (2, 512, 1024, 1024, True),     # whole tiles
    (4, 300, 512, 1056, False),     # ragged rows, 264-column blocks (ragged 64-column slabs)
    (8, 2048, 1024, 2048, True),    # one 256-column tile per rank
    (8, 40, 512, 192, True),        # small batch: 24-column blocks
    (3, 390, 768, 1560, False),     # odd number of ranks
    (1, 130, 512, 264, True),       # a single rank
    (2, 2560, 4096, 4096, True),    # 80 tiles per rank on 74 CTA pairs: tiles shared between pairs as K segments
])
def test_p2p_column_parallel_gather_matches_unsharded(cuda, pplb200, world, M, K, N, with_bias):
    """Column-parallel linear with gather_output: every rank's GEMM epilogue stores its fp16 block into every
    rank's [M, N] area (all ranks on one device here: produce for every rank, then finish for every rank), twice
    in a row on the same contexts with different inputs.  Bar: bit-identical to the unsharded fused linear, on
    every rank."""
    torch = cuda
    rng = np.random.default_rng(world * 1000 + M)
    ctxs = [pplb200.P2PContext(r, world, M, N) for r in range(world)]
    try:
        for c in ctxs:
            c.connect_local(ctxs)
        for it in range(2):
            x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float16)).cuda()
            w = torch.from_numpy(rng.integers(-127, 128, (N, K), dtype=np.int8)).cuda()
            sn = torch.from_numpy((rng.uniform(0.001, 0.01, N) * 8192).astype(np.float16)).cuda()
            bias = torch.from_numpy((rng.standard_normal(N) * 0.02).astype(np.float16)).cuda() if with_bias else None
            xq, sm = pplb200.minmax_quantize_fp16(x)
            full = pplb200.column_parallel_linear(xq, w, sm, sn, bias, K, N)
            nw = N // world
            outs = [torch.zeros((M, N), dtype=torch.float16, device="cuda") for _ in range(world)]
            for phase in (1, 2):
                for r in range(world):
                    pplb200.column_parallel_linear_p2p(ctxs[r], xq, w[r * nw:(r + 1) * nw], sm, sn[r * nw:(r + 1) * nw],
                                                       None if bias is None else bias[r * nw:(r + 1) * nw], K, N,
                                                       out=outs[r], phases=phase)
            torch.cuda.synchronize()
            for r in range(world):
                assert ctxs[r].status() == 0
                assert torch.equal(outs[r].view(torch.int16), full.view(torch.int16)), "rank %d of %d, round %d" % (r, world, it)
        assert pplb200.gemm_status() == 0
    finally:
        for c in ctxs:
            c.destroy()
