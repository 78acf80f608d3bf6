"""GPU tests at the full sizes of the benchmark configurations: the headline decode attention (101,600 positions, 8 queries)
against the oracle, and the conversation-cache round trip (snapshot 100,000 positions x 16 layers to pinned host memory,
restore the first 11,700, re-append 2,000, decode) through size-independent properties."""
import time

import numpy as np
import pytest

import kv_oracle as ko
import kvdata
from gpu_util import attend_both, fill_both

pytestmark = pytest.mark.gpu


def test_config2_101600_eight_queries_one_layer(mk, torch_cuda):
    """the benchmark's shape, one of its 16 layers: K5r / V6, window 2048, 101,608 positions, T = 8; max-abs <= 2e-3"""
    torch = torch_cuda
    spec, win, L, T = "K*=5r,V*=6", 2048, 101608, 8
    eng = mk.Engine(1, L + 16, spec, win)
    orc = ko.Cache(1, L + 16, spec, win)
    fill_both(torch, eng, orc, 0, 0, L, seed=2, chunk=8192)
    n = L - T
    Q = kvdata.q_rows(2, 0, n, T)
    O, Oref = attend_both(torch, eng, orc, 0, n, Q)
    assert np.isfinite(O).all()
    err = float(np.abs(O - Oref).max())
    assert err <= 2e-3, err
    # row t of the 8-row call equals the 1-row call at n + t (the reference's T-invariance check, dattn_bench.cu:1123-1161)
    for t in (0, 7):
        O1, _ = attend_both(torch, eng, orc, 0, n + t, Q[t:t + 1])
        assert np.abs(O1[0] - O[t]).max() <= 1e-4
    eng.close()


def test_config4_snapshot_restore_prefix_full_size(mk, torch_cuda):
    """100,000 positions x 16 layers (2.46 GB of rows + the rings) parked in pinned host memory; the first 11,700 positions
    restored into the emptied sequence; 2,000 rows appended; 8 tokens decoded. A second engine that appended the same rows and
    truncated to 11,700 (ring refill from the main rows, as after the restore) must hold the same bytes and give the same
    attention output bit for bit."""
    torch = torch_cuda
    spec, win, NL, L, P, A, T = "K*=5r,V*=6", 2048, 16, 100000, 11700, 2000, 8
    cap = L + 64
    a = mk.Engine(NL, cap, spec, win, spill=True)
    b = mk.Engine(NL, cap, spec, win, spill=True)
    g = torch.Generator(device="cuda")
    ch = [[(torch.rand((4, 256), generator=g.manual_seed(4000 + 2 * l + s), device="cuda") * 1.5 + 0.5) for s in range(2)] for l in range(NL)]
    for l in range(NL):
        g.manual_seed(40 + l)
        for p0 in range(0, L, 20000):
            m = min(20000, L - p0)
            K = (torch.randn((m, 4, 256), generator=g, device="cuda") * ch[l][0]).half()
            V = (torch.randn((m, 4, 256), generator=g, device="cuda") * ch[l][1]).half()
            a.append(l, p0, K, V)
            b.append(l, p0, K, V)
    a.commit(L)
    b.commit(L)
    a.store_budget(4 << 30)
    need = a.park_need()
    assert need >= L * NL * 4 * (176 + 208)  # every main row with its scales (rings on top)
    t0 = time.perf_counter()
    pid = a.park()
    t_park = time.perf_counter() - t0
    assert pid and a.park_bytes(pid) == need
    a.reset()
    assert a.position() == 0
    t0 = time.perf_counter()
    a.restore_prefix(pid, P, wait=True)
    t_restore = time.perf_counter() - t0
    info = a.store_info()
    restored = P * NL * 4 * (176 + 208)
    print("\nconfig 4: parked %.2f GB in %.2f s (first use of the pinned chunks included); restored %.1f MB of rows in %.1f ms = %.1f GB/s "
          "(engine's own clock: %d bytes in %d us)" % (need / 1e9, t_park, restored / 1e6, 1e3 * t_restore, restored / t_restore / 1e9,
                                                      info["last_bytes"], info["last_us"]))
    assert a.position() == P
    b.truncate(P)
    Kn = [(torch.randn((A, 4, 256), generator=g.manual_seed(900 + l), device="cuda") * ch[l][0]).half() for l in range(NL)]
    Vn = [(torch.randn((A, 4, 256), generator=g.manual_seed(950 + l), device="cuda") * ch[l][1]).half() for l in range(NL)]
    for l in range(NL):
        a.append(l, P, Kn[l], Vn[l])
        b.append(l, P, Kn[l], Vn[l])
    n = P + A - T
    a.commit(n)
    b.commit(n)
    Q = torch.randn((T, 24, 256), generator=g.manual_seed(77), device="cuda").half()
    Oa = torch.empty((T, 24, 256), dtype=torch.float32, device="cuda")
    Ob = torch.empty_like(Oa)
    ws = ko.kv_ws(n + T, win)
    rc = a.ring_rows()
    for l in (0, 7, 15):
        a.attend(l, n, Q, Oa)
        b.attend(l, n, Q, Ob)
        a.sync(); b.sync()
        assert torch.isfinite(Oa).all() and torch.equal(Oa, Ob)
        for side in range(2):
            for p in (0, 1, 4099, ws - 1, P - 1):  # main rows: restored from the host copy
                ra, sa = a.read_row(l, side, 1, p)
                rb, sb = b.read_row(l, side, 1, p)
                assert np.array_equal(ra, rb) and np.array_equal(sa, sb), (l, side, p)
            for p in (ws, P - 1, P, n + T - 1):  # ring rows: refilled below P, appended from P on
                ra, sa = a.read_row(l, side, 2, p % rc, ring=True)
                rb, sb = b.read_row(l, side, 2, p % rc, ring=True)
                assert np.array_equal(ra, rb) and np.array_equal(sa, sb), (l, side, p)
    assert a.park_drop(pid)
    a.close(); b.close()
