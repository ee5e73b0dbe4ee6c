"""Seeded synthetic inputs for the five W8A8 linear configurations that the benchmark and the
parity tests run.  They stand in for LLM activations / weights: shapes are those of Llama-class
7B / 70B projection layers; the value distributions are stated per configuration.

Everything is generated with numpy's PCG64 (stable across numpy versions) from
seed = 0xB2000000 + configuration index, one child stream per tensor.

Scale convention (pmx/i8i8/quantize.h:26-30 of the reference): the fp16 per-channel scale vector
holds s_n * 8192 and the dequantizer multiplies by 1/8192; per-token scales hold scale * 4096.
"""
import numpy as np

HIDDEN_UP = 8192.0

# name -> M, K, N, bias?, fused re-quantize?, activation kind, sigma, column-scale range, sharding
CONFIGS = {
    "c0": dict(index=0, M=16, K=4096, N=4096, bias=True, requant=False, x="normal", sigma=1.0,
               sn=(0.001, 0.01), shard=None, bound="hbm",
               desc="decode linear M16 K4096 N4096 +bias"),
    "c1": dict(index=1, M=128, K=4096, N=12288, bias=True, requant=True, x="normal", sigma=1.0,
               sn=(0.001, 0.01), shard=None, bound="hbm",
               desc="batched-decode fused QKV M128 K4096 N12288 +bias +re-quantize"),
    "c2": dict(index=2, M=4096, K=4096, N=22016, bias=False, requant=False, x="outlier", sigma=1.0,
               sn=(0.001, 0.01), shard="column", bound="tensor",
               desc="prefill gate+up M4096 K4096 N22016, 1% outlier channels x50"),
    "c3": dict(index=3, M=2048, K=28672, N=8192, bias=True, requant=False, x="normal", sigma=0.5,
               sn=(0.0005, 0.005), shard="row", bound="tensor",
               desc="70B down projection M2048 K28672 N8192 +bias, row-parallel"),
    "c4": dict(index=4, M=8192, K=8192, N=28672, bias=False, requant=False, x="student_t3", sigma=1.0,
               sn=(0.001, 0.01), shard="column", bound="tensor",
               desc="prefill MLP up M8192 K8192 N28672, Student-t(3) clipped +-200, column-parallel"),
}


def seed_of(name):
    return 0xB2000000 + CONFIGS[name]["index"]


def _streams(name):
    ss = np.random.SeedSequence(seed_of(name))
    return [np.random.Generator(np.random.PCG64(s)) for s in ss.spawn(5)]


def outlier_channels(name):
    """floor(0.01 * K) distinct seeded channel indices (ascending) for the 'outlier' activation kind."""
    cfg = CONFIGS[name]
    rng = _streams(name)[4]
    return np.sort(rng.choice(cfg["K"], size=cfg["K"] // 100, replace=False))


def make_activations(name, rows=None):
    """fp16 [M, K] (or the first `rows` rows; row r is the same whatever `rows` is)."""
    cfg = CONFIGS[name]
    M = cfg["M"] if rows is None else min(rows, cfg["M"])
    K = cfg["K"]
    rng = _streams(name)[0]
    out = np.empty((M, K), dtype=np.float16)
    block = 256
    for r0 in range(0, M, block):
        r1 = min(M, r0 + block)
        # always draw a full block so that row contents do not depend on `rows`
        z = rng.standard_normal((block, K), dtype=np.float32)
        if cfg["x"] == "student_t3":
            d = rng.standard_normal((3, block, K), dtype=np.float32)
            z = z / np.sqrt((d * d).sum(axis=0) / 3.0)
        z = z * np.float32(cfg["sigma"])
        if cfg["x"] == "outlier":
            z[:, outlier_channels(name)] *= np.float32(50.0)
        if cfg["x"] == "student_t3":
            np.clip(z, -200.0, 200.0, out=z)
        out[r0:r1] = z[: r1 - r0].astype(np.float16)
    return out


def make_weights(name, n_rows=None):
    """int8 [N, K], uniform integers on [-127, 127]."""
    cfg = CONFIGS[name]
    rng = _streams(name)[1]
    w = rng.integers(-127, 128, size=(cfg["N"], cfg["K"]), dtype=np.int8)
    return w if n_rows is None else w[:n_rows]


def make_column_scales(name):
    """fp16 [N] holding s_n * 8192 with s_n uniform on the configuration's range."""
    cfg = CONFIGS[name]
    rng = _streams(name)[2]
    lo, hi = cfg["sn"]
    s = rng.uniform(lo, hi, size=cfg["N"]).astype(np.float32)
    return (s * np.float32(HIDDEN_UP)).astype(np.float16)


def make_bias(name):
    cfg = CONFIGS[name]
    if not cfg["bias"]:
        return None
    rng = _streams(name)[3]
    return (rng.standard_normal(cfg["N"]).astype(np.float32) * np.float32(0.02)).astype(np.float16)


def algorithmic_ops(name):
    c = CONFIGS[name]
    return 2 * c["M"] * c["N"] * c["K"]


def algorithmic_bytes(name):
    """Compulsory HBM traffic of the fused op: X fp16 + W int8 + scale_N fp16 + bias fp16 + Y fp16
    (+ Yq int8 + Yq scales fp16 when the re-quantize is fused)."""
    c = CONFIGS[name]
    M, K, N = c["M"], c["K"], c["N"]
    b = 2 * M * K + N * K + 2 * N + 2 * M * N
    if c["bias"]:
        b += 2 * N
    if c["requant"]:
        b += M * N + 2 * M
    return b


def shard_rows(total, size, rank):
    """[begin, end) of an even split of `total` units over `size` ranks."""
    assert total % size == 0, "uneven shard"
    per = total // size
    return rank * per, (rank + 1) * per
