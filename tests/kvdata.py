"""Seeded synthetic K / V / Q rows with the value distribution of the benchmark configurations:
N(0,1) x per-channel scale U(0.5, 2), 1 % of the channels x 20; queries N(0,1). Rows are post-norm, post-RoPE fp16."""
import numpy as np

NH, NKV, HD = 24, 4, 256


def channel_scales(seed, layer, side):
    rng = np.random.default_rng([seed, layer, side, 7])
    ch = rng.uniform(0.5, 2.0, size=(NKV, HD)).astype(np.float32)
    out = rng.random((NKV, HD)) < 0.01
    return np.where(out, ch * 20.0, ch).astype(np.float32)


def kv_rows(seed, layer, pos0, n):
    """(K, V) fp16 [n][4][256] for positions pos0 .. pos0 + n - 1; blocks of 1024 positions are generated independently so
    any range gives the same rows"""
    out = []
    for side in range(2):
        ch = channel_scales(seed, layer, side)
        parts = []
        b0 = pos0 // 1024
        b1 = (pos0 + n + 1023) // 1024
        for b in range(b0, max(b1, b0 + 1)):
            rng = np.random.default_rng([seed, layer, side, 11, b])
            parts.append(rng.standard_normal((1024, NKV, HD), dtype=np.float32))
        x = np.concatenate(parts, axis=0)[pos0 - b0 * 1024: pos0 - b0 * 1024 + n]
        out.append((x * ch[None]).astype(np.float16))
    return out[0], out[1]


def q_rows(seed, layer, n, T):
    rng = np.random.default_rng([seed, layer, 13, n])
    return rng.standard_normal((T, NH, HD), dtype=np.float32).astype(np.float16)


def edge_rows():
    """fp32 rows [k][256] that hit the quantizer's corner cases: zero blocks, +- ties, clamp, rounding boundaries, range ends."""
    rows = []
    z = np.zeros(HD, dtype=np.float32)
    rows.append(z.copy())
    r = z.copy(); r[0] = -0.0; rows.append(r)
    r = z.copy(); r[3] = 1.0; r[7] = -1.0; rows.append(r)                      # tie of |x|: the positive value wins
    r = z.copy(); r[3] = -1.0; r[7] = 1.0; r[40] = -2.0; r[41] = 2.0; rows.append(r)
    r = z.copy(); r[0:32] = np.linspace(-1, 1, 32, dtype=np.float32); rows.append(r)  # v = -sv clamps at 2^b - 1
    r = np.full(HD, 65504.0, dtype=np.float32); r[1::2] = -65504.0; rows.append(r)     # fp16 range ends
    r = np.full(HD, 6e-8, dtype=np.float32); r[5] = -5.96e-8; rows.append(r)           # scale underflows in fp16
    r = z.copy(); r[0] = 16.0
    for i in range(1, 32):
        r[i] = (i - 15.5) * 1.0   # values exactly on index boundaries of a 5-bit grid with d = -1
    rows.append(r)
    r = z.copy(); r[64] = 127.0
    for i in range(1, 32):
        r[64 + i] = i + 0.5       # q8 ties: round to even
    rows.append(r)
    rng = np.random.default_rng(5)
    for _ in range(7):
        rows.append((rng.standard_normal(HD) * rng.uniform(0.01, 50)).astype(np.float16).astype(np.float32))
    return np.stack(rows).astype(np.float32)


def unit_multiset():
    """256 values on the 1/16 grid, shaped like N(0,1) quantiles, whose squares sum to exactly 256 (mean square exactly 1).
    Every partial sum of their squares is exact in fp32, so an RMS-norm of a row made of them sees exactly 1.0 in any
    summation order: the rows of the attention fixtures pass the reference kernels' norm prologue unchanged."""
    from statistics import NormalDist
    nd = NormalDist()
    a = np.array([round(16 * nd.inv_cdf((i + 0.5) / 256)) for i in range(256)], dtype=np.int64)
    target = 256 * 256
    # move single values by one grid step, largest magnitudes first, until the sum of squares is hit
    order = np.argsort(-np.abs(a))
    for _ in range(10000):
        s = int((a * a).sum())
        if s == target:
            break
        moved = False
        for i in order:
            step = 1 if s < target else -1
            b = abs(int(a[i])) + step
            delta = b * b - int(a[i]) ** 2
            if b >= 1 and ((s < target and s + delta <= target) or (s > target and s + delta >= target)):
                a[i] = b if a[i] >= 0 else -b
                moved = True
                break
        if not moved:  # the remaining gap is smaller than any single step of a large value: use the small ones
            order = np.argsort(np.abs(a))
    assert int((a * a).sum()) == target and np.abs(a).max() < 128
    return (a / 16.0).astype(np.float32)


def unit_rows(seed, tag, shape_prefix):
    """fp16 rows [*shape_prefix][256]: each a random signed permutation of unit_multiset()"""
    base = unit_multiset()
    rng = np.random.default_rng([seed, tag, 17])
    n = int(np.prod(shape_prefix))
    out = np.empty((n, HD), dtype=np.float32)
    for i in range(n):
        out[i] = base[rng.permutation(HD)] * rng.choice(np.array([-1.0, 1.0], dtype=np.float32), size=HD)
    return out.reshape(*shape_prefix, HD).astype(np.float16)
