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


def _normal_span(lo, hi, seed, std):
    u1 = uniform01(hi - lo, seed, lo)
    u2 = uniform01(hi - lo, seed ^ 0xA5A5A5A5A5A5A5A5, lo)
    r = np.sqrt(-2.0 * np.log(1.0 - u1))
    return (std * r * np.cos(2.0 * np.pi * u2)).astype(np.float32)


def normal(shape, seed, std=1.0):
    """Box-Muller on two decorrelated streams of the same seed.  Element i depends only on (seed, i), so large tensors
    are drawn in spans on a few threads (numpy releases the GIL) with the same values as one pass."""
    n = int(np.prod(shape))
    span = 1 << 21
    if n <= span:
        return _normal_span(0, n, seed, std).reshape(shape)
    from concurrent.futures import ThreadPoolExecutor
    import os
    out = np.empty(n, np.float32)

    def fill(lo):
        out[lo:min(n, lo + span)] = _normal_span(lo, min(n, lo + span), seed, std)

    with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as ex:
        list(ex.map(fill, range(0, n, span)))
    return out.reshape(shape)


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


# ---- fp8 e4m3 (OCP "fn" variant: no infinities, max finite 448) on the host -------------------------------------
def _e4m3_table():
    codes = np.arange(256, dtype=np.uint32)
    s, e, m = codes >> 7, (codes >> 3) & 0xF, codes & 7
    val = np.where(e == 0, m.astype(np.float64) * 2.0 ** -9, (8 + m).astype(np.float64) * 2.0 ** (e.astype(np.float64) - 10))
    val = np.where((e == 15) & (m == 7), np.nan, val)
    return np.where(s == 1, -val, val).astype(np.float32)


E4M3_VALUES = _e4m3_table()          # decode table, index = code
_E4M3_POS = E4M3_VALUES[:127].astype(np.float64)   # codes 0x00..0x7E ascending, 0 .. 448


def e4m3_encode(x):
    """fp32 -> e4m3 codes, round to nearest even, saturating at +-448 (integer arithmetic on the fp32 bit pattern)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    ax = np.minimum(np.abs(x), np.float32(448.0))
    u = ax.view(np.uint32)
    r = u + (np.uint32(0x7FFFF) + ((u >> np.uint32(20)) & np.uint32(1)))          # round the mantissa to 3 bits, ties to even
    normal = (((r >> np.uint32(23)) - np.uint32(120)) << np.uint32(3)) | ((r >> np.uint32(20)) & np.uint32(7))
    sub = np.rint(ax * np.float32(512.0)).astype(np.uint32)                        # below 2^-6: multiples of 2^-9 (8 -> code 0x08 = 2^-6)
    code = np.where(ax < np.float32(2.0 ** -6), sub, normal).astype(np.uint8)
    return code | (np.signbit(x).astype(np.uint8) << np.uint8(7))


def e4m3_decode(codes):
    return E4M3_VALUES[np.ascontiguousarray(codes, dtype=np.uint8)]


def quantize_weight_per_channel(w):
    """w [K,N] fp32 -> (e4m3 codes [K,N], scale [N] fp32) with scale = amax over the input dimension / 448."""
    amax = np.abs(w).max(axis=0)
    scale = np.where(amax > 0, amax / 448.0, 1.0).astype(np.float32)
    return e4m3_encode(w / scale[None, :]), scale


def ffn_inputs(tokens, hidden, inner, config=5):
    """Config 5 tensors: x ~ N(0,1) bf16 bits; W1 [H,I], W2 [I,H] ~ N(0,1)/sqrt(fan_in), fp8 codes + per-output-channel scales."""
    x = to_bf16_bits(normal((tokens, hidden), tensor_seed(config, 0)))
    w1, s1 = quantize_weight_per_channel(normal((hidden, inner), tensor_seed(config, 1), hidden ** -0.5))
    w2, s2 = quantize_weight_per_channel(normal((inner, hidden), tensor_seed(config, 2), inner ** -0.5))
    return x, w1, s1, w2, s2
