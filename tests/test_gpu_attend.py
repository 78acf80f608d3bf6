"""GPU parity: decode attention through the C ABI against the oracle, max-abs <= 2e-3 (the bar the path's contract states)."""
import numpy as np
import pytest

import kv_oracle as ko
import kvdata
from gpu_util import attend_both, check_flips, fill_both

pytestmark = pytest.mark.gpu
TOL = 2e-3


def check(O, Oref, tag):
    """the contract's bar: max-abs <= 2e-3 over every output (used on the benchmark configurations)"""
    assert np.isfinite(O).all(), tag
    err = np.abs(O - Oref).max()
    assert err <= TOL, (tag, float(err))
    return err


@pytest.mark.parametrize("spec,win,L", [("", 0, 66), ("", 0, 640), ("", 0, 4097), ("K*=5r,V*=6", 2048, 97), ("K*=5r,V*=6", 2048, 3201),
                                        ("K*=5r,V*=5", 2048, 7013), ("K*=6,V*=5", 2048, 5555), ("K*=4,V*=4r", 1024, 4000),
                                        ("K*=7r,V*=8", 2048, 4500), ("K*=8,V*=8", 0, 1281)])
def test_attention_matches_oracle(mk, torch_cuda, spec, win, L):
    torch = torch_cuda
    eng = mk.Engine(1, L + 16, spec, win)
    orc = ko.Cache(1, L + 16, spec, win)
    fill_both(torch, eng, orc, 0, 0, L, seed=L)
    vscale = kvdata.channel_scales(L, 0, 1)
    for T in (1, 2, 3, 5, 6, 8):
        n = L - T
        if T > L or mk.cap_T(n, T) < T:  # (a call's rows never cross a multiple of 640: test_calls_crossing_a_partition_are_rejected)
            continue
        Q = kvdata.q_rows(L, 0, n, T)
        O, Oref = attend_both(torch, eng, orc, 0, n, Q)
        check_flips(O, Oref, orc, 0, n, Q, (spec, L, T))
    eng.close()


def test_calls_crossing_a_partition_are_rejected(mk, torch_cuda):
    """rows n + 1 .. n + T of one call must not cross a multiple of 640 (mk_shared.cuh:288-291): the entry points refuse, the engine
    stays usable"""
    torch = torch_cuda
    eng = mk.Engine(1, 1400, "K*=5r,V*=6", 2048)
    fill_both(torch, eng, None, 0, 0, 1285, seed=3)
    Q = torch.zeros((8, 24, 256), dtype=torch.float16, device="cuda")
    O = torch.zeros((8, 24, 256), dtype=torch.float32, device="cuda")
    for call in (eng.attend, eng.attend_static):
        with pytest.raises(mk.EngineError, match="cross a multiple of 640"):
            call(0, 1277, Q, O)  # rows 1277 .. 1284 straddle 1280
    assert mk.cap_T(1277, 8) == 3
    eng.attend(0, 1277, Q[:3], O[:3])
    eng.attend(0, 1272, Q, O)  # 1272 + 8 = 1280: allowed
    eng.sync()
    eng.close()


def test_config0_q8_4096_append_one(mk, torch_cuda):
    """4,096 cached positions, q8_0 only, append 1, one query token, seed 0"""
    torch = torch_cuda
    eng = mk.Engine(1, 4200, "", 0)
    orc = ko.Cache(1, 4200, "", 0)
    fill_both(torch, eng, orc, 0, 0, 4096, seed=0)
    K, V = kvdata.kv_rows(0, 0, 4096, 1)
    Q = kvdata.q_rows(0, 0, 4096, 1)
    orc.append(0, 4096, K, V)
    O = torch.empty((1, 24, 256), dtype=torch.float32, device="cuda")
    eng.step(0, 4096, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda(), torch.from_numpy(Q).cuda(), O)
    eng.sync()
    check(O.cpu().numpy(), orc.attend(0, 4096, Q), "config0")
    a, sa = eng.read_row(0, 0, 1, 4096)
    b, sb = orc.row(0, 0, 1, 4096)
    assert np.array_equal(a, b) and np.array_equal(sa, sb)
    eng.close()


@pytest.mark.parametrize("spec", ["K*=5r,V*=6", "K*=5r,V*=5"])
def test_config1_presetF_38000_eight_queries(mk, torch_cuda, spec):
    """38,000 positions, window 2048, 8 query tokens (1 + 7 drafts), causal among them, seed 1"""
    torch = torch_cuda
    L, T = 38008, 8
    eng = mk.Engine(1, L + 16, spec, 2048)
    orc = ko.Cache(1, L + 16, spec, 2048)
    fill_both(torch, eng, orc, 0, 0, L, seed=1)
    n = L - T
    Q = kvdata.q_rows(1, 0, n, T)
    O, Oref = attend_both(torch, eng, orc, 0, n, Q)
    check(O, Oref, ("config1", spec))
    eng.close()


def test_t_invariance_and_causality(mk, torch_cuda):
    """row t of a T-row call equals the 1-row call at n + t (the reference's own check, dattn_bench.cu:1123-1161): here to
    the attention tolerance, and a draft token must not see later drafts"""
    torch = torch_cuda
    spec, win, L, T = "K*=5r,V*=6", 2048, 4808, 8
    eng = mk.Engine(1, L + 16, spec, win)
    orc = ko.Cache(1, L + 16, spec, win)
    fill_both(torch, eng, orc, 0, 0, L, seed=5)
    n = L - T
    Q = kvdata.q_rows(5, 0, n, T)
    O, Oref = attend_both(torch, eng, orc, 0, n, Q)
    check(O, Oref, "T8")
    for t in (0, 3, 7):
        O1, _ = attend_both(torch, eng, orc, 0, n + t, Q[t:t + 1])
        assert np.abs(O1[0] - O[t]).max() <= 1e-4
    # rewriting the later drafts' rows must not change row 0
    K, V = kvdata.kv_rows(99, 0, n + 1, T - 1)
    eng.append(0, n + 1, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
    O2, _ = attend_both(torch, eng, orc, 0, n, Q)
    assert np.array_equal(O2[0], O[0]) and not np.array_equal(O2[7], O[7])
    eng.close()


def test_slots_batch_matches_single(mk, torch_cuda):
    """several sequences in one pass (lanes): each job's output equals the same sequence run alone, bit for bit; the KV
    bytes of a slot do not depend on the batch it ran in"""
    torch = torch_cuda
    spec, win = "K*=5r,V*=6", 2048
    lens = [66, 700, 3300, 5100]
    Ts = [1, 8, 3, 6]
    eng = mk.Engine(1, 64, spec, win)
    eng.slots_open(len(lens), 5200)
    eng.reserve_batch(len(lens))
    orcs = []
    for s, L in enumerate(lens):
        orc = ko.Cache(1, 5200, spec, win)
        fill_both(torch, eng, orc, 0, 0, L, seed=60 + s, seq=s)
        orcs.append(orc)
    Ks, Vs, Qs = [], [], []
    for s, (L, T) in enumerate(zip(lens, Ts)):
        K, V = kvdata.kv_rows(80 + s, 0, L, T)
        orcs[s].append(0, L, K, V)
        Ks.append(K); Vs.append(V); Qs.append(kvdata.q_rows(80 + s, 0, L, T))
    K = torch.from_numpy(np.concatenate(Ks)).cuda(); V = torch.from_numpy(np.concatenate(Vs)).cuda()
    Q = torch.from_numpy(np.concatenate(Qs)).cuda()
    O = torch.zeros((sum(Ts), 24, 256), dtype=torch.float32, device="cuda")
    eng.step_batch(list(range(len(lens))), 0, lens, Ts, K, V, Q, O)
    eng.sync()
    O = O.cpu().numpy()
    r = 0
    for s, (L, T) in enumerate(zip(lens, Ts)):
        Oref = orcs[s].attend(0, L, Qs[s])
        check_flips(O[r:r + T], Oref, orcs[s], 0, L, Qs[s], ("slot", s))
        O1 = torch.zeros((T, 24, 256), dtype=torch.float32, device="cuda")
        eng.attend(0, L, torch.from_numpy(Qs[s]).cuda(), O1, seq=s)
        eng.sync()
        check_flips(O1.cpu().numpy(), Oref, orcs[s], 0, L, Qs[s], ("single", s))
        for p in (L, L + T - 1):
            a, sa = eng.read_row(0, 0, 3, p, seq=s)
            b, sb = orcs[s].row(0, 0, 3, p)
            assert np.array_equal(a, b) and np.array_equal(sa, sb)
        r += T
    eng.close()
