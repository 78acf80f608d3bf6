"""GPU parity: bytes written by the append / spill / refill kernels against the oracle, bit for bit, through the C ABI."""
import numpy as np
import pytest

import kv_oracle as ko
import kvdata
from gpu_util import assert_rows_equal, fill_both

pytestmark = pytest.mark.gpu

FORMATS = [("", 0), ("K*=5r,V*=5", 2048), ("K*=5r,V*=6", 2048), ("K*=6,V*=5", 2048), ("K*=4,V*=4", 0), ("K*=7,V*=6", 1024),
           ("K*=8,V*=5r", 2048), ("K*=5,V*=8r", 512), ("K*=6r,V*=6r", 2048), ("K*=4r,V*=7", 0)]


@pytest.mark.parametrize("spec,win", FORMATS)
def test_append_bytes_match_oracle(mk, torch_cuda, spec, win):
    torch = torch_cuda
    L = 3700
    eng = mk.Engine(2, L + 8, spec, win)
    orc = ko.Cache(2, L + 8, spec, win)
    for layer in range(2):
        fill_both(torch, eng, orc, layer, 0, L, seed=10 + layer)
    pos = [0, 1, 31, 32, 639, 640, 1919, 2047, 2048, 3231, 3232, 3233, 3500, L - 1]
    for layer in range(2):
        assert_rows_equal(eng, orc, layer, pos, ring_positions=[p for p in pos if p >= L - max(eng.ring_rows(), 1)])
    eng.commit(L)
    assert np.array_equal(eng.state_digest(), orc.digest(L))
    eng.close()


@pytest.mark.parametrize("bits", [4, 5, 6, 7, 8])
@pytest.mark.parametrize("rot", [False, True])
def test_quantizer_edge_rows(mk, torch_cuda, bits, rot):
    torch = torch_cuda
    rows = kvdata.edge_rows()
    rows16 = rows.astype(np.float16)
    n = rows16.shape[0]
    spec = "K*=%d%s,V*=%d%s" % (bits, "r" if rot else "", bits, "r" if rot else "")
    eng = mk.Engine(1, 64, spec, 0)
    K = np.repeat(rows16[:, None, :], 4, axis=1).copy()
    eng.append(0, 0, torch.from_numpy(K).cuda(), torch.from_numpy(K).cuda())
    for i in range(n):
        v = rows16[i].astype(np.float32)
        if rot:
            v = ko.fwht256(v)
        q, s = ko.quant_row(v, bits)
        for w in range(2):
            a, sa = eng.read_row(0, w, 2, i)
            assert np.array_equal(a, q) and np.array_equal(sa, s), (bits, rot, i, w)
    eng.close()


def test_rewritten_rows_and_ring_wrap(mk, torch_cuda):
    # rejected drafts: rows at or past the committed length are rewritten; ring slots wrap at 3232
    torch = torch_cuda
    spec, win = "K*=5r,V*=6", 2048
    eng = mk.Engine(1, 8000, spec, win)
    orc = ko.Cache(1, 8000, spec, win)
    fill_both(torch, eng, orc, 0, 0, 6460, seed=3)
    for step in range(12):
        n = 6460 + 3 * step
        K, V = kvdata.kv_rows(100 + step, 0, n, 8)
        orc.append(0, n, K, V)
        eng.append(0, n, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
        eng.commit(n + 3)
    top = 6460 + 33 + 8
    assert_rows_equal(eng, orc, 0, range(6455, top), ring_positions=range(top - 3232, top))
    eng.close()


def test_spill_mode_rows_equal_eager(mk, torch_cuda):
    """Spill-on-evict (fp16 shadow) must give, for every position that left the window, the bytes eager dual-write gives;
    ring rows are identical for all positions."""
    torch = torch_cuda
    spec, win = "K*=5r,V*=6", 2048
    L = 9000
    eng = mk.Engine(2, L + 64, spec, win, spill=True)
    orc = ko.Cache(2, L + 64, spec, win)
    for layer in range(2):
        fill_both(torch, eng, orc, layer, 0, 5000, seed=20 + layer, chunk=1777)
    # decode-like growth: 1..8 rows per step with an attention call, which is what moves the window
    rng = np.random.default_rng(0)
    n = 5000
    Q = torch.zeros((8, 24, 256), dtype=torch.float16, device="cuda")
    O = torch.empty((8, 24, 256), dtype=torch.float32, device="cuda")
    while n < L - 8:
        T = mk.cap_T(n, 8)
        for layer in range(2):
            K, V = kvdata.kv_rows(50 + layer, layer, n, T)
            orc.append(layer, n, K, V)
            eng.step(layer, n, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda(), Q[:T], O[:T])
        n += int(rng.integers(1, T + 1))
        eng.commit(n)
        if n > 5400 and n < 8200:
            n_skip = 640  # jump ahead with a bulk append so the test stays short
            for layer in range(2):
                fill_both(torch, eng, orc, layer, n, n_skip, seed=70 + layer)
            n += n_skip
            eng.commit(n)
    ws = ko.kv_ws(n, win)
    assert ws > 3000
    for layer in range(2):
        assert_rows_equal(eng, orc, layer, list(range(0, ws, 97)) + [ws - 1], ring_positions=range(max(n - 3000, ws), n, 13))
    eng.close()


def test_refill_after_rewind(mk, torch_cuda):
    torch = torch_cuda
    spec, win = "K*=5r,V*=5", 2048
    for spill in (False, True):
        eng = mk.Engine(2, 7100, spec, win, spill=spill)
        orc = ko.Cache(2, 7100, spec, win)
        for layer in range(2):
            fill_both(torch, eng, orc, layer, 0, 5000, seed=30 + layer)
        eng.commit(5000)
        assert eng.checkpoint() == 5000
        for layer in range(2):
            fill_both(torch, eng, orc, layer, 5000, 2000, seed=40 + layer)
        eng.commit(7000)
        assert eng.checkpoints() == [5000]
        assert not eng.rewind_to(4999)
        assert eng.rewind_to(5000)
        assert orc.ring_rewind(5000) == 5000 - 3232 + 0 - (5000 - 3232) + min(5000, 7000 - 3232) - max(0, 5000 - 3232)
        assert eng.position() == 5000
        for layer in range(2):
            assert_rows_equal(eng, orc, layer, [], ring_positions=range(5000 - 3232, 5000, 7), main=False)
        eng.close()


@pytest.mark.parametrize("bits", [4, 5, 6, 7, 8])
@pytest.mark.parametrize("rot", [0, 1])
def test_append_matches_reference_golden_vectors(mk, torch_cuda, bits, rot):
    """the CUDA append kernel against the committed golden vectors (bytes made by the reference's own device functions)"""
    import os
    torch = torch_cuda
    gpath = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kv_quant_golden.npz")
    if not os.path.exists(gpath):
        pytest.skip("golden vectors not generated")
    g = np.load(gpath)
    rows = g["rows"].astype(np.float16)
    n = rows.shape[0]
    spec = "K*=%d%s,V*=8" % (bits, "r" if rot else "")
    eng = mk.Engine(1, n + 8, spec, 0)
    K = np.repeat(rows[:, None, :], 4, axis=1).copy()
    eng.append(0, 0, torch.from_numpy(K).cuda(), torch.from_numpy(K).cuda())
    q, sc = g["q_%d_%d" % (bits, rot)], g["sc_%d_%d" % (bits, rot)]
    for i in range(n):
        a, sa = eng.read_row(0, 0, 3, i)
        assert np.array_equal(a, q[i]) and np.array_equal(sa, sc[i]), (bits, rot, i)
    eng.close()


def test_step_layers_equals_per_layer_steps(mk, torch_cuda):
    """mk_kv_step_layers is nlayers calls of mk_kv_step: same row bytes, same outputs"""
    torch = torch_cuda
    spec, win, L, T, NL = "K*=5r,V*=6", 2048, 2500, 5, 3
    a = mk.Engine(NL, L + 64, spec, win)
    b = mk.Engine(NL, L + 64, spec, win)
    for l in range(NL):
        K, V = kvdata.kv_rows(7 + l, l, 0, L)
        for e in (a, b):
            e.append(l, 0, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
    Ks = torch.stack([torch.from_numpy(kvdata.kv_rows(30 + l, l, L, T)[0]) for l in range(NL)]).cuda()
    Vs = torch.stack([torch.from_numpy(kvdata.kv_rows(30 + l, l, L, T)[1]) for l in range(NL)]).cuda()
    Qs = torch.stack([torch.from_numpy(kvdata.q_rows(31, l, L, T)) for l in range(NL)]).cuda()
    Oa = torch.zeros((NL, T, 24, 256), dtype=torch.float32, device="cuda")
    Ob = torch.zeros_like(Oa)
    a.step_layers(L, Ks, Vs, Qs, Oa)
    for l in range(NL):
        b.step(l, L, Ks[l], Vs[l], Qs[l], Ob[l])
    # fewer rows than the per-layer buffers hold (layer stride > T rows): the next step with T = 2
    a.step_layers(L + T, Ks[:, :2], Vs[:, :2], Qs[:, :2], Oa[:, :2])
    for l in range(NL):
        b.step(l, L + T, Ks[l, :2], Vs[l, :2], Qs[l, :2], Ob[l, :2])
    a.sync(); b.sync()
    assert torch.equal(Oa, Ob)
    for l in range(NL):
        for side in (0, 1):
            ra, sa = a.read_row(l, side, 2, L + T - 1)
            rb, sb = b.read_row(l, side, 2, L + T - 1)
            assert np.array_equal(ra, rb) and np.array_equal(sa, sb)
    # the same steps in blocks of layers (mk_kv_step_layers_at): layers 0 .. 1, then layer 2
    c = mk.Engine(NL, L + 64, spec, win)
    for l in range(NL):
        K, V = kvdata.kv_rows(7 + l, l, 0, L)
        c.append(l, 0, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
    Oc = torch.zeros_like(Oa)
    for n0, rows in ((L, slice(0, T)), (L + T, slice(0, 2))):
        c.step_layers_at(0, n0, Ks[:2, rows], Vs[:2, rows], Qs[:2, rows], Oc[:2, rows])
        c.step_layers_at(2, n0, Ks[2:, rows], Vs[2:, rows], Qs[2:, rows], Oc[2:, rows])
    c.sync()
    assert torch.equal(Oc, Oa)
    with pytest.raises(mk.EngineError, match="layers must lie"):
        c.step_layers_at(2, L + T + 2, Ks[:2, :1], Vs[:2, :1], Qs[:2, :1], Oc[:2, :1])
    a.close(); b.close(); c.close()


def test_per_layer_spec_items_match_oracle(mk, torch_cuda):
    """items of the MK_KV grammar that name one layer or one side, later items overriding earlier ones (loader.cu:1329-1366): the
    engine's formats, rotations (through the bytes) and rings equal the oracle's, layer by layer, and so do bytes and attention"""
    torch = torch_cuda
    spec, win, NL, L = "K*=5r,V*=6,K1=8,V0=4r,*2=7,V2=5r,K3=6", 640, 4, 1500
    eng = mk.Engine(NL, L + 8, spec, win)
    orc = ko.Cache(NL, L + 8, spec, win)
    want = {(0, 0): 5, (1, 0): 4, (0, 1): 8, (1, 1): 6, (0, 2): 7, (1, 2): 5, (0, 3): 6, (1, 3): 6}
    for (w, l), b in want.items():
        assert eng.bits(w, l) == orc.bits(w, l) == b
        assert eng.has_ring(w, l) == orc.has_ring(w, l) == (b != 8)
    for layer in range(NL):
        fill_both(torch, eng, orc, layer, 0, L, seed=20 + layer)
        assert_rows_equal(eng, orc, layer, [0, 639, 640, L - 1], ring_positions=[L - 600, L - 1])
    eng.commit(L)
    assert np.array_equal(eng.state_digest(), orc.digest(L))
    n, T = L - 4, 4
    for layer in range(NL):
        Q = kvdata.q_rows(9, layer, n, T)
        O = torch.empty((T, 24, 256), dtype=torch.float32, device="cuda")
        eng.attend(layer, n, torch.from_numpy(Q).cuda(), O)
        eng.sync()
        assert np.abs(O.cpu().numpy() - orc.attend(layer, n, Q)).max() <= 2e-3, layer
    eng.close()
