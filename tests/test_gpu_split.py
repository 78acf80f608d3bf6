"""GPU parity of the position-split sequence: G engines on one GPU, each owning a range of positions (the ranks of a
multi-GPU run emulated one after another), their partials merged by mk_kv_combine; against the oracle and against the plain
single-engine result."""
import numpy as np
import pytest

import kv_oracle as ko
import kvdata

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("spec,win,L,G", [("K*=5r,V*=6", 2048, 9000, 2), ("K*=5r,V*=6", 2048, 20008, 4), ("", 0, 3000, 3),
                                          ("K*=6,V*=5r", 1024, 6000, 2)])
def test_split_sequence_matches_oracle(mk, torch_cuda, spec, win, L, G):
    torch = torch_cuda
    T = 8
    cap = L + 64
    orc = ko.Cache(1, cap, spec, win)
    seqs = [mk.parallel.SplitSequence(mk.Engine, 1, cap, spec, win, r, G) for r in range(G)]
    for a in range(0, L, 2048):
        m = min(2048, L - a)
        K, V = kvdata.kv_rows(L, 0, a, m)
        orc.append(0, a, K, V)
        Kd, Vd = torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda()
        for s in seqs:
            s.append(0, a, Kd, Vd)
    n = L - T
    Q = kvdata.q_rows(L, 0, n, T)
    Qd = torch.from_numpy(Q).cuda()
    # the ranks' partials, gathered by hand (one process): parts [G][4][48][256]
    parts = torch.zeros((G, 4, 48, 256), dtype=torch.float32, device="cuda")
    mls = torch.zeros((G, 4, 48, 2), dtype=torch.float32, device="cuda")
    for r, s in enumerate(seqs):
        hi = min(s.hi, L)
        s.eng.attend_partial(0, n, Qd, s.lo, hi if hi > s.lo else s.lo, parts[r], mls[r])
        s.eng.sync()
    O = torch.empty((T, 24, 256), dtype=torch.float32, device="cuda")
    seqs[0].eng.combine(0, T, G, parts, mls, O)
    seqs[0].eng.sync()
    O = O.cpu().numpy()
    Oref = orc.attend(0, n, Q)
    assert np.isfinite(O).all()
    assert np.abs(O - Oref).max() <= 2e-3
    # the host-side numpy merge agrees with the kernel's
    kvb, rot = ko.parse_spec(spec, 1)
    O2 = mk.parallel.combine_partials_np(parts.cpu().numpy(), mls.cpu().numpy(), T, rot_v=bool(rot[1, 0]))
    assert np.abs(O2 - O).max() <= 1e-3
    # rows land only on their owner, bytes as the oracle's
    for r, s in enumerate(seqs):
        for p in (s.lo, min(s.hi, L) - 1):
            if s.lo <= p < min(s.hi, L):
                a, sa = s.eng.read_row(0, 0, 2, p)
                b, sb = orc.row(0, 0, 2, p)
                assert np.array_equal(a, b) and np.array_equal(sa, sb)
    for s in seqs:
        s.close()
