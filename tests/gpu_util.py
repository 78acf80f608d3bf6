"""Helpers shared by the GPU parity tests: feed identical rows to the engine (through the C ABI) and to the oracle."""
import numpy as np

import kv_oracle as ko
import kvdata


def fill_both(torch, eng, orc, layer, pos0, n, seed, seq=-1, chunk=4096):
    for a in range(pos0, pos0 + n, chunk):
        m = min(chunk, pos0 + n - a)
        K, V = kvdata.kv_rows(seed, layer, a, m)
        if orc is not None:
            orc.append(layer, a, K, V)
        eng.append(layer, a, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda(), seq=seq)


def assert_rows_equal(eng, orc, layer, positions, ring_positions=(), seq=-1, main=True):
    rc = eng.ring_rows()
    for w in range(2):
        for g in range(4):
            if main:
                for p in positions:
                    a, sa = eng.read_row(layer, w, g, p, seq=seq)
                    b, sb = orc.row(layer, w, g, p)
                    assert np.array_equal(a, b) and np.array_equal(sa, sb), ("main row", layer, w, g, p)
            if eng.has_ring(w, layer):
                for p in ring_positions:
                    a, sa = eng.read_row(layer, w, g, p % rc, ring=True, seq=seq)
                    b, sb = orc.row(layer, w, g, p % rc, ring=True)
                    assert np.array_equal(a, b) and np.array_equal(sa, sb), ("ring row", layer, w, g, p)


def attend_both(torch, eng, orc, layer, n, Q, seq=-1):
    Qd = torch.from_numpy(Q).cuda()
    O = torch.empty((Q.shape[0], 24, 256), dtype=torch.float32, device="cuda")
    eng.attend(layer, n, Qd, O, seq=seq)
    eng.sync()
    return O.cpu().numpy(), orc.attend(layer, n, Q)
