"""GPU tests at the full sizes of the benchmark configurations: the headline decode attention (101,600 positions, 8 queries)
against the oracle, and the conversation-cache round trip (snapshot 100,000 positions x 16 layers to pinned host memory,
restore the first 11,700, re-append 2,000, decode) through size-independent properties."""
import time

import numpy as np
import pytest

import kv_oracle as ko
import kvdata
from gpu_util import assert_rows_equal, attend_both, check_flips, fill_both

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


def test_config2_streaming_64_steps(mk, torch_cuda):
    """Config 2's stream on 2 of its layers: from 101,600 positions, 64 decode steps of up to 8 query tokens (capped where the rows
    would cross a multiple of 640), 1 .. T of them accepted per step (seeded), rows evicted from the q8_0 window spilled into the
    5/6-bit tier as the window start jumps. The oracle mirrors every append; the attention output is checked against it on the first
    step, on the steps right before and after the context crosses a multiple of 640 (the window start moves, tiles change from ring
    to tier) and on the last step; the bytes of evicted, window and newest rows are checked at the end."""
    torch = torch_cuda
    spec, win, NL, L0, STEPS = "K*=5r,V*=6", 2048, 2, 101600, 64
    cap = L0 + STEPS * 8 + 64
    eng = mk.Engine(NL, cap, spec, win, spill=True)
    orc = ko.Cache(NL, cap, spec, win)
    for l in range(NL):
        fill_both(torch, eng, orc, l, 0, L0, seed=2, chunk=8192)
    eng.commit(L0)
    rng = np.random.default_rng(2)
    n, checked, crossings = L0, [], 0
    O = torch.empty((NL, 8, 24, 256), dtype=torch.float32, device="cuda")
    plan, m = [], L0
    for s in range(STEPS):  # the stream first, so that the steps around a crossing are known
        T = mk.cap_T(m, 8)
        a = int(rng.integers(1, T + 1))
        plan.append((m, T, a))
        m += a
    cross = [i for i in range(1, STEPS) if plan[i][0] // 640 != plan[i - 1][0] // 640 or (plan[i][0] + plan[i][1] - 1) // 640 != (plan[i - 1][0] + plan[i - 1][1] - 1) // 640]
    want = {0, STEPS - 1} | {i for c in cross for i in (c - 1, c, c + 1) if 0 <= i < STEPS}
    for s, (n, T, a) in enumerate(plan):
        K = np.stack([kvdata.kv_rows(300 + s, l, n, T)[0] for l in range(NL)])
        V = np.stack([kvdata.kv_rows(300 + s, l, n, T)[1] for l in range(NL)])
        Q = np.stack([kvdata.q_rows(300 + s, l, n, T) for l in range(NL)])
        for l in range(NL):
            orc.append(l, n, K[l], V[l])
        eng.step_layers(n, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda(), torch.from_numpy(Q).cuda(), O[:, :T])
        eng.sync()
        if s in want:
            got = O[:, :T].cpu().numpy()
            for l in range(NL):
                err = float(np.abs(got[l] - orc.attend(l, n, Q[l])).max())
                assert np.isfinite(got[l]).all() and err <= 2e-3, (s, l, n, T, err)
            checked.append((s, n, T))
        eng.commit(n + a)
    assert len(cross) >= 1 and len(checked) >= 5, (cross, checked)
    n_end = plan[-1][0] + plan[-1][1]
    ws = ko.kv_ws(n_end, win)
    assert_rows_equal(eng, orc, 0, [0, 5000, L0 - 3000, ws - 640, ws - 1], ring_positions=[ws, L0, n_end - 1])
    assert_rows_equal(eng, orc, 1, [ws - 1], ring_positions=[n_end - 1])
    eng.close()


def test_config3_32_slots_log_uniform(mk, torch_cuda):
    """Config 3 at its stated size on one layer: 32 sequences with lengths log-uniform in [2,000, 100,000] (seed 3), 1 .. 8 query
    tokens each, one batched step; every slot's output against the oracle under the plain bar (an output beyond it must be shown to
    be a rounding flip of P by check_flips, at most two per slot and only for slots short enough to analyse), its new rows' bytes too."""
    torch = torch_cuda
    spec, win, NS = "K*=5r,V*=6", 2048, 32
    rng = np.random.default_rng(3)
    lens = np.exp(rng.uniform(np.log(2000), np.log(100000), size=NS)).astype(np.int64)
    Ts = [int(mk.cap_T(int(n), int(t))) for n, t in zip(lens, rng.integers(1, 9, size=NS))]
    cap = int(lens.max()) + 64
    eng = mk.Engine(1, 64, spec, win)
    eng.slots_open(NS, cap)
    eng.reserve_batch(NS)
    orcs = []
    for s in range(NS):
        orc = ko.Cache(1, int(lens[s]) + 64, spec, win)
        fill_both(torch, eng, orc, 0, 0, int(lens[s]), seed=700 + s, seq=s, chunk=8192)
        orcs.append(orc)
    Ks, Vs, Qs = [], [], []
    for s in range(NS):
        K, V = kvdata.kv_rows(800 + s, 0, int(lens[s]), Ts[s])
        orcs[s].append(0, int(lens[s]), K, V)
        Ks.append(K); Vs.append(V); Qs.append(kvdata.q_rows(800 + s, 0, int(lens[s]), Ts[s]))
    K = torch.from_numpy(np.concatenate(Ks)).cuda(); V = torch.from_numpy(np.concatenate(Vs)).cuda()
    Q = torch.from_numpy(np.concatenate(Qs)).cuda()
    O = torch.zeros((sum(Ts), 24, 256), dtype=torch.float32, device="cuda")
    eng.step_batch(list(range(NS)), 0, [int(x) for x in lens], Ts, K, V, Q, O)
    eng.sync()
    O = O.cpu().numpy()
    r, worst = 0, 0.0
    for s in range(NS):
        Oref = orcs[s].attend(0, int(lens[s]), Qs[s])
        worst = max(worst, check_flips(O[r:r + Ts[s]], Oref, orcs[s], 0, int(lens[s]), Qs[s], ("slot", s, int(lens[s]), Ts[s]), max_bad=2))
        assert_rows_equal(eng, orcs[s], 0, [int(lens[s]) + Ts[s] - 1], ring_positions=[int(lens[s])], seq=s)
        r += Ts[s]
    print("\nconfig 3: %d positions in 32 slots, %d tokens, worst max-abs error %.3g" % (int(lens.sum()), sum(Ts), worst))
    eng.close()


def test_config4_snapshot_restore_prefix_full_size(mk, torch_cuda):
    """100,000 positions x 16 layers (2.46 GB of rows + the rings) parked in pinned host memory; the first 11,700 positions
    restored into the emptied sequence; 2,000 rows appended; 8 tokens decoded. Layer 7 of the engine holds the same seeded rows as a
    one-layer oracle that takes the reference's route (rewind to 11,700 with the window rings refilled from the low-bit rows,
    ck_pool.cu:285-296; append; attend): restored rows, refilled ring rows, re-appended rows and the attention output of that layer
    must be the oracle's."""
    torch = torch_cuda
    spec, win, NL, L, P, A, T, LAYER = "K*=5r,V*=6", 2048, 16, 100000, 11700, 2000, 8, 7
    cap = L + 64
    a = mk.Engine(NL, cap, spec, win, spill=True)
    orc = ko.Cache(1, cap, spec, win)
    g = torch.Generator(device="cuda")
    for l in range(NL):
        if l == LAYER:
            for p0 in range(0, L, 8192):
                m = min(8192, L - p0)
                K, V = kvdata.kv_rows(4, LAYER, p0, m)
                orc.append(0, p0, K, V)
                a.append(l, p0, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
            continue
        g.manual_seed(40 + l)
        for p0 in range(0, L, 20000):
            m = min(20000, L - p0)
            a.append(l, p0, (torch.randn((m, 4, 256), generator=g, device="cuda") * 1.3).half(), (torch.randn((m, 4, 256), generator=g, device="cuda") * 1.3).half())
    a.commit(L)
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
    assert orc.ring_rewind(P) > 0  # the reference's rewind: ring rows of the kept prefix rebuilt from the main rows
    Kn, Vn = kvdata.kv_rows(44, LAYER, P, A)
    orc.append(0, P, Kn, Vn)
    for l in range(NL):
        if l == LAYER:
            a.append(l, P, torch.from_numpy(Kn).cuda(), torch.from_numpy(Vn).cuda())
        else:
            x = (torch.randn((A, 4, 256), generator=g.manual_seed(900 + l), device="cuda") * 1.3).half()
            a.append(l, P, x, x)
    n = P + A - T
    a.commit(n)
    Q = kvdata.q_rows(44, LAYER, n, T)
    Oa = torch.empty((T, 24, 256), dtype=torch.float32, device="cuda")
    a.attend(LAYER, n, torch.from_numpy(Q).cuda(), Oa)
    a.sync()
    err = float(np.abs(Oa.cpu().numpy() - orc.attend(0, n, Q)).max())
    assert err <= 2e-3, err
    ws = ko.kv_ws(n + T, win)
    rc = a.ring_rows()
    for side in range(2):
        for gh in range(4):
            for p in (0, 1, 4099, ws - 1, P - 1):  # main rows: restored from the host copy
                ra, sa = a.read_row(LAYER, side, gh, p)
                rb, sb = orc.row(0, side, gh, p)
                assert np.array_equal(ra, rb) and np.array_equal(sa, sb), ("main", side, gh, p)
            for p in (ws, P - 2048, P - 1, P, n + T - 1):  # ring rows: refilled below P, appended from P on
                ra, sa = a.read_row(LAYER, side, gh, p % rc, ring=True)
                rb, sb = orc.row(0, side, gh, p % rc, ring=True)
                assert np.array_equal(ra, rb) and np.array_equal(sa, sb), ("ring", side, gh, p)
    for l in (0, 15):  # the other layers: finite output
        a.attend(l, n, torch.from_numpy(Q).cuda(), Oa)
        a.sync()
        assert torch.isfinite(Oa).all()
    assert a.park_drop(pid)
    a.close()
