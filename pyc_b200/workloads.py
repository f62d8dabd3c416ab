"""Seeded synthetic inputs for the benchmark configurations.

No public dataset is involved: every tensor is drawn from a counter-based
generator (splitmix64 over the element index) so that any slice of any tensor
can be regenerated anywhere without state.  Seed convention: one 64-bit seed per
tensor = 0x5EED0000 + 16 * config + tensor_index.
"""
import numpy as np

_MASK = np.uint64(0xFFFFFFFFFFFFFFFF)


def tensor_seed(config, tensor_index):
    return 0x5EED0000 + 16 * int(config) + int(tensor_index)


def _splitmix64(idx, seed):
    with np.errstate(over="ignore"):
        z = (idx.astype(np.uint64) + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15) + np.uint64(seed)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def uniform01(n, seed, offset=0):
    """n doubles in [0,1), elements offset..offset+n of the stream `seed`."""
    idx = np.arange(offset, offset + n, dtype=np.uint64)
    return (_splitmix64(idx, seed) >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def uniform(shape, seed, lo=-1.0, hi=1.0):
    n = int(np.prod(shape))
    return (lo + (hi - lo) * uniform01(n, seed)).astype(np.float32).reshape(shape)


def normal(shape, seed, std=1.0):
    """Box-Muller on two decorrelated streams of the same seed."""
    n = int(np.prod(shape))
    u1 = uniform01(n, seed)
    u2 = uniform01(n, seed ^ 0xA5A5A5A5A5A5A5A5)
    r = np.sqrt(-2.0 * np.log(1.0 - u1))
    return (std * r * np.cos(2.0 * np.pi * u2)).astype(np.float32).reshape(shape)


def to_bf16_bits(x):
    """fp32 -> bf16 storage bits, round to nearest even (the rounding PyC's bench applies,
    benchmark/benchmarks/gpu/workloads/pyc_compiler_next_bench.c:248-256)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


# The five benchmark configurations (shapes and distributions only).
CONFIGS = {
    1: dict(name="mlp_f32_512", M=512, K=512, N=512, dtype="f32", bias="row", act="relu", dist=("uniform", -1.0, 1.0)),
    2: dict(name="gemm_bf16_8192_bias_gelu", M=8192, K=8192, N=8192, dtype="bf16", bias="row", act="gelu", dist=("normal", 0.02)),
    3: dict(name="attention_bf16_causal", batch=8, heads=32, seq=2048, d=128, dtype="bf16"),
    4: dict(name="conv2d_bf16_nhwc", cases=[dict(N=64, H=56, W=56, C=64, K=64), dict(N=256, H=14, W=14, C=256, K=256)], R=3, S=3),
    5: dict(name="ffn_fp8w_bf16", tokens=8192, hidden=4096, inner=16384),
}


def gemm_inputs(config, M, K, N, dist, bias=True):
    """fp32 arrays (A[M,K], B[K,N], bias[N]) for a GEMM-shaped config."""
    def draw(shape, idx):
        if dist[0] == "uniform":
            return uniform(shape, tensor_seed(config, idx), dist[1], dist[2])
        return normal(shape, tensor_seed(config, idx), dist[1])
    a, b = draw((M, K), 0), draw((K, N), 1)
    return (a, b, draw((N,), 2)) if bias else (a, b)
