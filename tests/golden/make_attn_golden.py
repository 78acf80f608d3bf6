#!/usr/bin/env python
"""Generates tests/golden/attn_golden.npz on a GPU box: what the REFERENCE's own decode-attention kernels
(oracle/_ref/libref_attn_witness.so, built by oracle/build_ref.py from the reference source) compute on caches this repository's
oracle quantized from seeded rows. Per case the reference kernels give the split partials (m, l, O) of every (kv head, chunk)
item and the K / V rows they stored for the T new positions. The script checks, while it runs, that the stored rows equal the
oracle's bytes (so both sides attend over identical caches) and prints how far the oracle's partials and merged output are from
the reference's; tests/test_golden.py then pins the oracle against the stored vectors on any machine.

    python tests/golden/make_attn_golden.py [out.npz]

The new tokens' query and key rows are signed permutations of one multiset whose mean square is exactly 1 (kvdata.unit_rows), the
RoPE table the kernels read is the identity and the norm weights are one constant w with rsqrtf(1 + eps) * w == 1.0f, so the
kernels' norm / RoPE prologue (qwen38_mk.cu:2848-2891) hands the rows on unchanged.
"""
import ctypes as C
import hashlib
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path[:0] = [os.path.join(ROOT, "tests"), os.path.join(ROOT, "oracle")]
import kv_oracle as ko  # noqa: E402
import kvdata  # noqa: E402

NKV, NH, HD = 4, 24, 256
ITEMS = NKV * 21

# name, MK_KV spec, window, cached positions n, query tokens T, seed
CASES = [
    ("config0_q8_T1", "", 0, 4096, 1, 0),
    ("config1_F6_T8", "K*=5r,V*=6", 2048, 38000, 8, 1),
    ("config1_F_T8", "K*=5r,V*=5", 2048, 38000, 8, 1),
    ("config2_F6_T8", "K*=5r,V*=6", 2048, 101600, 8, 2),
    ("ring_only_F6_T2", "K*=5r,V*=6", 2048, 2500, 2, 5),
    ("presetD_T5", "K*=6,V*=5", 2048, 5003, 5, 6),
    ("q4_rotV_T3", "K*=4,V*=4r", 2048, 7001, 3, 7),
    ("k7_v8_T4", "K*=7,V*=8", 2048, 4000, 4, 8),
]


def witness():
    L = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_attn_witness.so"))
    vp, ip, fl = C.c_void_p, C.c_int, C.c_float
    L.ref_rsqrt.argtypes = [vp, vp, ip]
    L.ref_attn.argtypes = [ip, ip, ip, ip, ip, ip, ip, ip, vp, vp, vp, vp, vp, vp, vp, fl, fl, vp, vp, vp, vp, vp, vp, ip, vp]
    return L


def norm_weight(L):
    """the constant norm weight w with fl(rsqrtf(fl(1 + 1e-6)) * w) == 1.0f"""
    x = np.array([np.float32(1.0) + np.float32(1e-6)], dtype=np.float32)
    y = np.zeros(1, dtype=np.float32)
    assert L.ref_rsqrt(x.ctypes.data, y.ctypes.data, 1) == 0
    rs = y[0]
    u = np.float32(2.0 ** -23)
    for k in range(0, 16):
        w = np.float32(1.0) + np.float32(k) * u
        if np.float32(rs * w) == np.float32(1.0):
            return float(w), float(rs)
    raise SystemExit("no norm weight makes rsqrtf(1 + eps) * w == 1 (rs = %r)" % rs)


def ptr_array(arrs):
    a = (C.c_void_p * len(arrs))()
    for i, x in enumerate(arrs):
        a[i] = x.ctypes.data if x is not None else None
    return a


def cache_digest(orc):
    h = hashlib.sha256()
    for w in range(2):
        for kind in range(4):
            b = orc.buffer(0, w, kind)
            if b is not None:
                h.update(b.tobytes())
    return h.hexdigest()


def fill(orc, seed, n):
    for a in range(0, n, 8192):
        m = min(8192, n - a)
        K, V = kvdata.kv_rows(seed, 0, a, m)
        orc.append(0, a, K, V)


def new_rows(seed, n, T):
    Kn = kvdata.unit_rows(seed, 1, (T, NKV))
    Q = kvdata.unit_rows(seed, 2, (T, NH))
    _, Vn = kvdata.kv_rows(seed, 0, n, T)
    return Kn, Vn, Q


def run_case(L, w_norm, name, spec, win, n, T, seed, reps):
    t0 = time.time()
    orc = ko.Cache(1, n + T + 64, spec, win)
    fill(orc, seed, n)
    Kn, Vn, Q = new_rows(seed, n, T)
    kb, vb = orc.bits(0, 0), orc.bits(1, 0)
    kvb, rot = ko.parse_spec(spec, 1)
    kr, vr = int(rot[0, 0]), int(rot[1, 0])
    digest = cache_digest(orc)  # the cache before the new rows
    bufs = [[orc.buffer(0, w, k) for w in range(2)] for k in range(4)]
    rb = [32 * kb, 32 * vb]
    apart = np.zeros((ITEMS, 48, HD), dtype=np.float32)
    aml = np.zeros((ITEMS, 48, 2), dtype=np.float32)
    rows_val = [np.zeros((NKV, T, rb[w]), dtype=np.uint8) for w in range(2)]
    rows_sc = [np.zeros((NKV, T, 8), dtype=np.uint16) for w in range(2)]
    rows_rval = [np.zeros((NKV, T, HD), dtype=np.uint8) for w in range(2)]
    rows_rsc = [np.zeros((NKV, T, 8), dtype=np.uint16) for w in range(2)]
    us = C.c_float(0)
    q32, k32, v32 = (np.ascontiguousarray(x.astype(np.float32)) for x in (Q, Kn, Vn))
    rc = L.ref_attn(kb, vb, kr, vr, win if spec else 0, orc.ctxp, n, T, ptr_array(bufs[0]), ptr_array(bufs[1]), ptr_array(bufs[2]),
                    ptr_array(bufs[3]), q32.ctypes.data, k32.ctypes.data, v32.ctypes.data, w_norm, w_norm, apart.ctypes.data,
                    aml.ctypes.data, ptr_array(rows_val), ptr_array(rows_sc), ptr_array(rows_rval), ptr_array(rows_rsc), reps,
                    C.byref(us))
    assert rc == 0, "ref_attn failed: %d" % rc
    # the oracle appends the same rows: its bytes must equal what the reference kernels stored
    orc.append(0, n, Kn, Vn)
    rcr = orc.rc
    for w in range(2):
        for g in range(NKV):
            for t in range(T):
                a, sa = orc.row(0, w, g, n + t)
                assert np.array_equal(a, rows_val[w][g, t]) and np.array_equal(sa, rows_sc[w][g, t]), ("main row", name, w, g, t)
                if orc.has_ring(w, 0):
                    a, sa = orc.row(0, w, g, (n + t) % rcr, ring=True)
                    assert np.array_equal(a, rows_rval[w][g, t]) and np.array_equal(sa, rows_rsc[w][g, t]), ("ring row", name, w, g, t)
    O, m, l, Op, nch = orc.attend_parts(0, n, Q, threads=os.cpu_count() or 8)
    R = 6 * T
    items = NKV * nch
    rm, rl, rO = aml[:items, :R, 0].copy(), aml[:items, :R, 1].copy(), apart[:items, :R].copy()
    fin = np.isfinite(rm)
    assert np.array_equal(fin, np.isfinite(m)), "an item is empty on one side only"
    dm = float(np.abs(rm[fin] - m[fin]).max())
    dl = float((np.abs(rl - l) / np.maximum(np.abs(rl), 1e-30))[fin].max())
    dO = float(np.abs(rO - Op).max())
    ref_O = ko.merge_parts(T, rm, rl, rO, rot_v=bool(vr))
    dout = float(np.abs(ref_O - O).max())
    print("%-18s n %6d T %d chunks %2d: rows bit-equal; |dm| %.3g  rel dl %.3g  |dO partial| %.3g  |d merged| %.3g  ref kernel %.1f us  (%.1f s)"
          % (name, n, T, nch, dm, dl, dO, dout, us.value, time.time() - t0), flush=True)
    d = {"meta": np.array([n, T, seed, win if spec else 0, nch, kb, vb, kr, vr], dtype=np.int64), "spec": np.array(spec),
         "cache_sha256": np.array(digest), "Kn": Kn, "Vn": Vn, "Q": Q, "ref_m": rm, "ref_l": rl,
         "ref_Osub": np.ascontiguousarray(rO[:, :, ::16]), "ref_merged": ref_O, "ref_kernel_us": np.float32(us.value)}
    for w in range(2):
        d["rows_val%d" % w] = rows_val[w]
        d["rows_sc%d" % w] = rows_sc[w]
        if orc.has_ring(w, 0):
            d["rows_rval%d" % w] = rows_rval[w]
            d["rows_rsc%d" % w] = rows_rsc[w]
    orc.close()
    return {name + "/" + k: v for k, v in d.items()}


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "attn_golden.npz")
    L = witness()
    w_norm, rs = norm_weight(L)
    print("rsqrtf(1 + 1e-6) = %.9g, norm weight %.9g" % (rs, w_norm), flush=True)
    d = {"names": np.array([c[0] for c in CASES]), "norm_weight": np.float32(w_norm)}
    only = os.environ.get("ATTN_GOLDEN_ONLY", "")
    for name, spec, win, n, T, seed in CASES:
        if only and name not in only.split(","):
            continue
        d.update(run_case(L, w_norm, name, spec, win, n, T, seed, reps=20))
    np.savez_compressed(out, **d)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
