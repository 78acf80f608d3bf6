"""GPU parity against the REFERENCE's own decode-attention kernels: mk_kv_step / mk_kv_attend on the caches of
tests/golden/attn_golden.npz (partials the reference's kernels computed on a B200 from identical cache bytes,
tests/golden/make_attn_golden.py) -- KV bytes of the new rows bit-exact, output within 2e-3 max-abs of the merge of the
reference's partials."""
import numpy as np
import pytest

from gpu_util import fill_both
from test_golden import TOL, _attn_cases, load_attn_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", _attn_cases())
@pytest.mark.parametrize("entry", ["step", "attend_static"])
def test_attention_matches_reference_kernels(mk, torch_cuda, name, entry):
    torch = torch_cuda
    c = load_attn_case(name)
    n, T, seed, win = (int(x) for x in c["meta"][:4])
    spec = str(c["spec"])
    eng = mk.Engine(1, n + T + 64, spec, win)
    fill_both(torch, eng, None, 0, 0, n, seed=seed)
    K, V, Q = (torch.from_numpy(np.ascontiguousarray(c[k])).cuda() for k in ("Kn", "Vn", "Q"))
    O = torch.empty((T, 24, 256), dtype=torch.float32, device="cuda")
    if entry == "step":
        eng.step(0, n, K, V, Q, O)
    else:
        eng.append(0, n, K, V)
        eng.attend_static(0, n, Q, O)
    eng.sync()
    rc = eng.ring_rows()
    for w in range(2):  # the new positions' rows: the bytes the reference kernels stored
        for g in range(4):
            for t in range(T):
                a, sa = eng.read_row(0, w, g, n + t)
                assert np.array_equal(a, c["rows_val%d" % w][g, t]) and np.array_equal(sa, c["rows_sc%d" % w][g, t]), (w, g, t)
                if eng.has_ring(w, 0):
                    a, sa = eng.read_row(0, w, g, (n + t) % rc, ring=True)
                    assert np.array_equal(a, c["rows_rval%d" % w][g, t]) and np.array_equal(sa, c["rows_rsc%d" % w][g, t]), (w, g, t)
    O = O.cpu().numpy()
    assert np.isfinite(O).all()
    err = float(np.abs(O - c["ref_merged"]).max())
    assert err <= TOL, (name, entry, err)
    eng.close()
