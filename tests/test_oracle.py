"""CPU tests of the parity oracle itself: conversions, quantizer identities, window / partition facts, attention properties."""
import numpy as np
import pytest

import kv_oracle as ko
import kvdata


def test_fp16_conversions_match_numpy():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(20000) * 10.0 ** rng.integers(-9, 6, 20000)).astype(np.float32)
    x = np.concatenate([x, np.array([0, -0.0, 65504, 65519.9, 65520, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-08, 6.1e-5, 6.0975552e-05,
                                     np.inf, -np.inf], dtype=np.float32)])
    L = ko.lib()
    mine = np.array([L.orc_f2h(float(v)) for v in x], dtype=np.uint16)
    with np.errstate(over="ignore"):
        ref = x.astype(np.float16).view(np.uint16)
    assert (mine == ref).all()
    allh = np.arange(65536, dtype=np.uint16)
    back = np.array([L.orc_h2f(int(h)) for h in allh], dtype=np.float32)
    refb = allh.view(np.float16).astype(np.float32)
    assert ((back.view(np.uint32) == refb.view(np.uint32)) | (np.isnan(back) & np.isnan(refb))).all()


def test_fwht_is_orthonormal_and_self_inverse():
    rng = np.random.default_rng(1)
    v = rng.standard_normal(256).astype(np.float32)
    H = np.array([[(-1) ** bin(i & j).count("1") for j in range(256)] for i in range(256)], dtype=np.float64) / 16
    assert np.abs(ko.fwht256(v) - H @ v).max() < 2e-6
    assert np.abs(ko.fwht256(ko.fwht256(v)) - v).max() < 2e-6


def _unpack(q, bits):
    """independent numpy decoder of the row layout (kv_store_qn's comment, qwen38_mk.cu:2071-2074)"""
    if bits == 8:
        return q.view(np.int8).astype(np.int32)
    hb = bits - 4
    n = np.zeros(256, dtype=np.int32)
    for lane in range(32):
        w = q[4 * lane:4 * lane + 4]
        hi = 0
        for j in range(hb):
            hi |= int(q[128 + lane * hb + j]) << (8 * j)
        for k in range(8):
            nib = (int(w[k]) & 15) if k < 4 else (int(w[k - 4]) >> 4)
            n[8 * lane + k] = nib | (((hi >> (hb * k)) & ((1 << hb) - 1)) << 4)
    return n - (1 << (bits - 1))


@pytest.mark.parametrize("bits", [4, 5, 6, 7, 8])
def test_quantizer_identities(bits):
    rows = kvdata.edge_rows()
    h = 1 << (bits - 1)
    for v in rows:
        q, sc = ko.quant_row(v, bits)
        ints = _unpack(q, bits)
        d = sc.view(np.float16).astype(np.float32)
        deq = ko.dequant_row(q, sc, bits)
        assert np.array_equal(deq, (d.repeat(32) * ints).astype(np.float32))
        for b in range(8):
            blk = v[32 * b:32 * b + 32]
            if bits == 8:
                am = np.abs(blk).max()
                assert sc[b] == np.float16(np.float32(am) / np.float32(127.0)).view(np.uint16)
                if am == 0:
                    assert (ints[32 * b:32 * b + 32] == 0).all() and sc[b] == 0
                else:
                    assert np.abs(ints[32 * b:32 * b + 32]).max() == 127
            else:
                am = np.abs(blk).max()
                if am == 0:  # sv stays +0: d = +0 / -h = -0 (bits 0x8000), every index is the midpoint
                    assert sc[b] == 0x8000 and (ints[32 * b:32 * b + 32] == 0).all()
                    continue
                cand = blk[np.abs(blk) == am]
                sv = cand.max()  # ties of |x| go to the larger x
                dd = np.float32(sv) / np.float32(-h)
                with np.errstate(over="ignore"):
                    assert sc[b] == np.float16(dd).view(np.uint16)
                i_sv = int(np.where(blk == sv)[0][0])
                assert ints[32 * b + i_sv] == -h  # v = sv -> n = 0
                neg = np.where(blk == -sv)[0]
                if len(neg) and sv != 0:
                    assert ints[32 * b + int(neg[0])] == h - 1  # v = -sv clamps to 2^b - 1


def test_q4_equals_qn_rule_and_fma_boundary():
    # index = trunc(fma(v, 1/d, h + 0.5)): a value on a rounding boundary moves with the fused rounding
    v = np.zeros(256, dtype=np.float32)
    v[0] = 3.0  # sv = 3, 5 bits: d = -3/16, id = 1/d (inexact)
    v[1] = np.float32(-3.0 / 16 * 7.5)
    q, sc = ko.quant_row(v, 5)
    ints = _unpack(q, 5)
    idv = np.float32(1.0) / (np.float32(3.0) / np.float32(-16.0))
    exact = float(np.float64(v[1]) * np.float64(idv) + 16.5)  # one rounding, as the fused multiply-add
    assert ints[1] + 16 == min(31, int(np.float32(exact)))


def test_q8_requantize_is_idempotent():
    # ring refill of an 8-bit side re-stores the same row (loader.cu:1487-1490)
    rng = np.random.default_rng(3)
    for _ in range(50):
        v = (rng.standard_normal(256) * rng.uniform(0.1, 30)).astype(np.float16).astype(np.float32)
        q, sc = ko.quant_row(v, 8)
        q2, sc2 = ko.quant_row(ko.dequant_row(q, sc, 8), 8)
        assert np.array_equal(q, q2) and np.array_equal(sc, sc2)


def test_window_and_partition_facts():
    assert ko.kv_rc(2048) == 3232
    assert ko.kv_ws(38008, 2048) == 35200
    assert ko.kv_ws(101608, 2048) == 98560
    assert ko.kv_ws(3200, 2048) == 0 and ko.kv_ws(3201, 2048) == 640
    assert ko.kv_ws(5000, 0) == 0
    assert ko.attn_dims(38008) == (20, 1920)
    assert ko.attn_dims(101608) == (20, 5088)
    assert ko.attn_dims(262152) == (20, 13120)
    assert ko.attn_dims(4097) == (19, 224)
    assert ko.attn_dims(1) == (1, 32)
    assert ko.att_cap_T(638, 8) == 2 and ko.att_cap_T(640, 8) == 8 and ko.att_cap_T(0, 8) == 8 and ko.att_cap_T(639, 8) == 1
    for L in range(1, 30000, 37):
        nch, cs = ko.attn_dims(L)
        assert nch <= 20 and cs % 32 == 0 and nch * cs >= L


def test_parse_spec_grammar():
    kvb, rot = ko.parse_spec("K*=5r,V*=6", 16)
    assert (kvb[0] == 5).all() and (kvb[1] == 6).all() and (rot[0] == 1).all() and (rot[1] == 0).all()
    kvb, rot = ko.parse_spec("V*=6r,K15=4r,*3=7", 16)
    assert kvb[0, 15] == 4 and rot[0, 15] == 1 and kvb[1, 0] == 6 and kvb[0, 3] == 7 and kvb[1, 3] == 7 and rot[1, 3] == 0
    kvb, rot = ko.parse_spec("", 4)
    assert (kvb == 8).all() and (rot == 0).all()
    for bad in ("K*=9", "X1=4", "K16=4", "K=3", "K*=4x", "=4"):
        with pytest.raises(ValueError):
            ko.parse_spec(bad, 16)


def _filled(spec, win, L, seed=1, layers=1, win_all=False):
    c = ko.Cache(layers, L + 64, spec, win, win_all)
    for l in range(layers):
        K, V = kvdata.kv_rows(seed, l, 0, L)
        c.append(l, 0, K, V)
    return c


def test_ring_rows_and_dual_write():
    L = 3500
    c = _filled("K*=5r,V*=6", 2048, L)
    assert c.rc == 3232 and c.has_ring(0, 0) and c.has_ring(1, 0)
    K, V = kvdata.kv_rows(1, 0, 0, L)
    for p in (0, 267, 268, 3231, 3232, 3499):
        for g in (0, 3):
            v = K[p, g].astype(np.float32)
            rv = ko.fwht256(v)
            q5, s5 = ko.quant_row(rv, 5)
            q8, s8 = ko.quant_row(rv, 8)
            mq, ms = c.row(0, 0, g, p)
            assert np.array_equal(mq, q5) and np.array_equal(ms, s5)
            if p >= L - 3232:  # still in the ring
                rq, rs = c.row(0, 0, g, p % 3232, ring=True)
                assert np.array_equal(rq, q8) and np.array_equal(rs, s8)
            q6, s6 = ko.quant_row(V[p, g].astype(np.float32), 6)
            mq, ms = c.row(0, 1, g, p)
            assert np.array_equal(mq, q6) and np.array_equal(ms, s6)


def test_attention_matches_float64_softmax():
    # the oracle against plain float64 attention over the same dequantised operands
    L, T = 700, 3
    c = _filled("K*=5r,V*=6", 2048, L)
    n = L - T
    Q = kvdata.q_rows(1, 0, n, T)
    O = c.attend(0, n, Q)
    Kd = np.zeros((4, L, 256)); Vd = np.zeros((4, L, 256))
    for g in range(4):
        for p in range(L):
            q, s = c.row(0, 0, g, p % 3232, ring=True)
            Kd[g, p] = ko.dequant_row(q, s, 8, f16=True)
            q, s = c.row(0, 1, g, p % 3232, ring=True)
            Vd[g, p] = ko.dequant_row(q, s, 8, f16=True)
    for t in range(T):
        for h in (0, 7, 23):
            qv = ko.fwht256(Q[t, h].astype(np.float32))
            qv = (qv * np.float32(0.0625)).astype(np.float16).astype(np.float64)
            s = Kd[h // 6, :n + t + 1] @ qv
            p = np.exp(s - s.max())
            y = (p[:, None] * Vd[h // 6, :n + t + 1]).sum(0) / p.sum()
            assert np.abs(O[t, h] - y).max() < 2e-3 * max(1.0, np.abs(y).max() / 8)


def test_t_invariance_bitwise():
    # row t of a T-row call equals the 1-row call at n + t (dattn_bench.cu:1123-1161): the partition depends on L's bucket only
    for spec, win, L in (("", 0, 1500), ("K*=5r,V*=6", 2048, 4000)):
        c = _filled(spec, win, L)
        T = 5
        n = L - T
        Q = kvdata.q_rows(2, 0, n, T)
        O = c.attend(0, n, Q)
        for t in range(T):
            O1 = c.attend(0, n + t, Q[t:t + 1])
            assert np.array_equal(O1[0], O[t])


def test_window_all_is_identity():
    # MK_KV_WIN_ALL: rings for the q8 sides too must leave the output byte-identical (loader.cu:1487-1490)
    L, T = 3900, 4
    a = _filled("K*=8,V*=8", 0, L)
    b = _filled("K*=8,V*=8", 2048, L, win_all=True)
    assert b.has_ring(0, 0) and not a.has_ring(0, 0)
    Q = kvdata.q_rows(3, 0, L - T, T)
    assert np.array_equal(a.attend(0, L - T, Q), b.attend(0, L - T, Q))
    # and a refill re-stores the same q8 rows
    before = [b.row(0, w, g, r, ring=True) for w in range(2) for g in range(4) for r in (0, 100, 667)]
    b.refill(0, L)
    after = [b.row(0, w, g, r, ring=True) for w in range(2) for g in range(4) for r in (0, 100, 667)]
    for x, y in zip(before, after):
        assert np.array_equal(x[0], y[0]) and np.array_equal(x[1], y[1])


def test_ring_rewind_range_and_lossy_refill():
    L = 7000
    c = _filled("K*=5r,V*=6", 2048, L)
    P = 5000
    done = c.ring_rewind(P)
    assert done == min(P, L - 3232) - max(0, P - 3232) and c.kv_top == P
    # a refilled ring row is the q8 of the low-bit row, not of the original values
    p = 3000
    K, _ = kvdata.kv_rows(1, 0, p, 1)
    q5, s5 = c.row(0, 0, 1, p)
    rq, rs = c.row(0, 0, 1, p % 3232, ring=True)
    eq, es = ko.quant_row(ko.dequant_row(q5, s5, 5), 8)
    assert np.array_equal(rq, eq) and np.array_equal(rs, es)
    # rows the continuation did not overwrite keep their original q8
    p = 4500
    K, _ = kvdata.kv_rows(1, 0, p, 1)
    rq, rs = c.row(0, 0, 2, p % 3232, ring=True)
    oq, os_ = ko.quant_row(ko.fwht256(K[0, 2].astype(np.float32)), 8)
    assert np.array_equal(rq, oq) and np.array_equal(rs, os_)


def test_digest_and_snapshot_order():
    L = 100
    c = _filled("K*=5r,V*=6", 2048, L, layers=2)
    d = c.digest(L)
    assert d[0] == 0x4d4b444701 and d[1] == L and d[3] == 3232 and d[4] == 0 and d[5] == 2 and d[6] == 4
    assert len(d) == 8 + 2 * 2 * 4 * L * 2
    snap = c.snapshot(0, L)
    per_tok = 2 * 4 * ((160 + 16) + (192 + 16))
    assert len(snap) == per_tok * L + 2 * 2 * 4 * 3232 * 272
    # first item: layer 0, K, head 0 values rows 0..L-1, then its scales
    q, s = c.row(0, 0, 0, 5)
    assert np.array_equal(snap[5 * 160:6 * 160], q)
    assert np.array_equal(snap[L * 160 + 5 * 16:L * 160 + 6 * 16].view(np.uint16), s)
    # a changed row changes exactly its digest word
    K, V = kvdata.kv_rows(9, 0, 0, 1)
    c.append(0, 7, K, V)
    d2 = c.digest(L)
    diff = np.nonzero(d != d2)[0]
    assert len(diff) == 2 * 4 * 2  # 8 main rows + 8 ring rows of layer 0 at position 7
