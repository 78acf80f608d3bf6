"""CPU check of the oracle against the committed golden vectors: bytes produced by the reference's own device functions on a
B200 (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

import kv_oracle as ko

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kv_quant_golden.npz")


def same_half(a, b):
    """fp16 bit patterns equal, up to the sign of a zero product and the payload of a NaN (an overflowed scale times 0)"""
    nan = lambda x: (x & 0x7fff) > 0x7c00
    return (a == b) | (((a & 0x7fff) == 0) & ((b & 0x7fff) == 0)) | (nan(a) & nan(b))


@pytest.mark.skipif(not os.path.exists(GOLD), reason="golden vectors not generated yet")
def test_oracle_matches_reference_golden_vectors():
    g = np.load(GOLD)
    rows = g["rows"]
    for bits in (4, 5, 6, 7, 8):
        for rot in (0, 1):
            q, sc, f16 = g["q_%d_%d" % (bits, rot)], g["sc_%d_%d" % (bits, rot)], g["f16_%d_%d" % (bits, rot)]
            for i in range(rows.shape[0]):
                v = ko.fwht256(rows[i]) if rot else rows[i]
                oq, osc = ko.quant_row(v, bits)
                assert np.array_equal(oq, q[i]) and np.array_equal(osc, sc[i]), (bits, rot, i)
                of = ko.dequant_row(oq, osc, bits, f16=True).astype(np.float16).view(np.uint16)
                assert same_half(of, f16[i]).all(), (bits, rot, i)


# ---- attention: the reference's own decode-attention kernels on caches the oracle quantized (tests/golden/make_attn_golden.py) ----
ATTN_GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attn_golden.npz")
TOL = 2e-3  # the path's contract: attention output within 2e-3 max-abs of the reference's


def _attn_cases():
    if not os.path.exists(ATTN_GOLD):
        return []
    return [str(n) for n in np.load(ATTN_GOLD)["names"]]


def load_attn_case(name):
    g = np.load(ATTN_GOLD)
    return {k.split("/", 1)[1]: g[k] for k in g.files if k.startswith(name + "/")}


def build_case_cache(c):
    """the oracle cache the fixture was generated on: seeded rows [0, n), checked by digest, then the case's T new rows"""
    import hashlib
    import kvdata
    n, T, seed, win = (int(x) for x in c["meta"][:4])
    spec = str(c["spec"])
    orc = ko.Cache(1, n + T + 64, spec, win)
    for a in range(0, n, 8192):
        m = min(8192, n - a)
        K, V = kvdata.kv_rows(seed, 0, a, m)
        orc.append(0, a, K, V)
    h = hashlib.sha256()
    for w in range(2):
        for kind in range(4):
            b = orc.buffer(0, w, kind)
            if b is not None:
                h.update(b.tobytes())
    assert h.hexdigest() == str(c["cache_sha256"]), "the seeded rows differ from the ones the fixture was generated with"
    orc.append(0, n, c["Kn"], c["Vn"])
    return orc, n, T


@pytest.mark.parametrize("name", _attn_cases())
def test_oracle_attention_matches_reference_kernels(name):
    """Pins the oracle's softmax / P rounding / merge: per (kv head, chunk) item its (m, l, O) against the partials the reference's
    kernels left in apart / aml on the same cache bytes, and the merged output against the merge of the reference's partials."""
    c = load_attn_case(name)
    orc, n, T = build_case_cache(c)
    rc = orc.rc
    for w in range(2):  # the rows the reference kernels stored for the new positions are the oracle's bytes
        for g in range(4):
            for t in range(T):
                a, sa = orc.row(0, w, g, n + t)
                assert np.array_equal(a, c["rows_val%d" % w][g, t]) and np.array_equal(sa, c["rows_sc%d" % w][g, t]), (w, g, t)
                if orc.has_ring(w, 0):
                    a, sa = orc.row(0, w, g, (n + t) % rc, ring=True)
                    assert np.array_equal(a, c["rows_rval%d" % w][g, t]) and np.array_equal(sa, c["rows_rsc%d" % w][g, t]), (w, g, t)
    O, m, l, Op, nch = orc.attend_parts(0, n, c["Q"])
    assert nch == int(c["meta"][4])
    rm, rl, rO = c["ref_m"], c["ref_l"], c["ref_Osub"]
    fin = np.isfinite(rm)
    assert np.array_equal(fin, np.isfinite(m))
    assert np.abs(rm[fin] - m[fin]).max() <= 1e-4           # running maxima: fp32 score sums in a different order
    assert (np.abs(rl - l)[fin] / rl[fin]).max() <= 1e-4    # row sums
    # un-normalised partial outputs (every 16th dim is stored). Per item, after division by the item's own row sum: a single P value
    # that rounds to the other fp16 neighbour moves a short chunk's normalised output by up to a few 1e-3 in a x 20 channel, so this
    # bound only catches gross errors; the contract is the next one: the item's difference weighed as the merge weighs it
    # (w_c = exp(m_c - M) over sum_c w_c l_c), i.e. in units of the final output, must stay within the tolerance.
    d = np.abs(rO / np.where(fin, rl, 1)[..., None] - Op[:, :, ::16] / np.where(fin, l, 1)[..., None])
    assert d[fin].max() <= 1e-2, d[fin].max()
    R = m.shape[1]
    mm = np.where(fin, rm, -np.inf).reshape(4, nch, R)
    w = np.exp(mm - mm.max(axis=1, keepdims=True))
    den = (w * rl.reshape(4, nch, R)).sum(axis=1, keepdims=True)
    contrib = np.abs(rO - Op[:, :, ::16]).reshape(4, nch, R, -1) * (w / den)[..., None]
    assert contrib.max() <= TOL / 2, contrib.max()
    assert np.abs(O - c["ref_merged"]).max() <= 1e-3, np.abs(O - c["ref_merged"]).max()
