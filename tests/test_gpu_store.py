"""GPU parity: snapshot / restore through the pinned host store, rewind, truncate and side requests leave the cache bit for
bit as the oracle's (the reference's exact-reuse checks, scripts/capi_checks.py:698-822, at tensor level)."""
import numpy as np
import pytest

import kv_oracle as ko
import kvdata
from gpu_util import assert_rows_equal, attend_both, fill_both

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("spill", [False, True])
def test_park_unpark_digest(mk, torch_cuda, spill, monkeypatch):
    torch = torch_cuda
    monkeypatch.setenv("MK_STORE_CHUNK_MIB", "1")  # many chunk crossings
    spec, win, L = "K*=5r,V*=6", 2048, 4100
    eng = mk.Engine(3, L + 64, spec, win, spill=spill)
    orc = ko.Cache(3, L + 64, spec, win)
    for layer in range(3):
        fill_both(torch, eng, orc, layer, 0, L, seed=layer)
    eng.commit(L)
    assert eng.park(0) is None  # no budget: no room
    eng.store_budget(1 << 30)
    need = eng.park_need(0)
    pid = eng.park(0)
    assert pid and pid > 0
    assert eng.park_bytes(pid) == need == len(orc.snapshot(0, L))
    d0 = eng.state_digest()
    assert np.array_equal(d0, orc.digest(L))
    info = eng.store_info()
    assert info["parked"] == 1 and info["last_bytes"] == need and info["kv_token_bytes"] == eng.kv_sizes()["per_token"]
    # clobber the sequence, then bring the parked one back
    eng.reset()
    for layer in range(3):
        fill_both(torch, eng, None, layer, 0, 3000, seed=99)
    eng.commit(3000)
    assert not np.array_equal(eng.state_digest()[:20], d0[:20])
    eng.unpark(pid)
    assert eng.position() == L
    assert np.array_equal(eng.state_digest(), d0)
    assert eng.store_info()["parked"] == 0
    with pytest.raises(mk.EngineError):
        eng.unpark(pid)
    eng.close()


def test_restore_prefix_then_reappend(mk, torch_cuda):
    """conversation-cache round trip, small: park, restore rows [0, P), re-append, decode; everything equals the oracle doing
    unpark + rewind (ring refill) + append"""
    torch = torch_cuda
    spec, win, L, P = "K*=5r,V*=6", 2048, 9000, 4100
    eng = mk.Engine(2, L + 2100, spec, win, spill=True)
    orc = ko.Cache(2, L + 2100, spec, win)
    for layer in range(2):
        fill_both(torch, eng, orc, layer, 0, L, seed=layer)
    eng.commit(L)
    eng.store_budget(2 << 30)
    pid = eng.park(0)
    eng.reset()
    eng.restore_prefix(pid, P, wait=False)
    assert eng.position() == P
    orc.ring_rewind(P)
    for layer in range(2):
        fill_both(torch, eng, orc, layer, P, 700, seed=50 + layer)
    n = P + 700 - 8
    eng.commit(n)
    for layer in range(2):
        Q = kvdata.q_rows(7, layer, n, 8)
        O, Oref = attend_both(torch, eng, orc, layer, n, Q)
        assert np.abs(O - Oref).max() <= 2e-3
        ws = ko.kv_ws(n + 8, win)
        assert_rows_equal(eng, orc, layer, list(range(0, ws, 53)), ring_positions=range(ws, n + 8, 11))
    assert eng.park_drop(pid) and not eng.park_drop(pid)
    eng.close()


def test_exact_checkpoint_restores_rings(mk, torch_cuda):
    torch = torch_cuda
    spec, win = "K*=5r,V*=5", 2048
    eng = mk.Engine(1, 8000, spec, win, exact=True)
    orc = ko.Cache(1, 8000, spec, win)
    fill_both(torch, eng, orc, 0, 0, 5000, seed=1)
    eng.commit(5000)
    eng.checkpoint()
    d0 = eng.state_digest()
    fill_both(torch, eng, None, 0, 5000, 2500, seed=2)
    eng.commit(7500)
    assert eng.rewind_to(5000)
    assert np.array_equal(eng.state_digest(), d0)  # rings exactly as of the checkpoint, not refilled
    assert np.array_equal(d0, orc.digest(5000))
    eng.close()


def test_truncate_refills(mk, torch_cuda):
    torch = torch_cuda
    spec, win = "K*=6,V*=5", 1024
    eng = mk.Engine(1, 6000, spec, win)
    orc = ko.Cache(1, 6000, spec, win)
    fill_both(torch, eng, orc, 0, 0, 5000, seed=1)
    eng.commit(5000)
    eng.truncate(3000)
    orc.ring_rewind(3000)
    assert eng.position() == 3000
    assert np.array_equal(eng.state_digest(), orc.digest(3000))
    with pytest.raises(mk.EngineError):
        eng.truncate(3001)
    eng.close()


def test_side_request_round_trip(mk, torch_cuda, monkeypatch):
    torch = torch_cuda
    monkeypatch.setenv("MK_STORE_CHUNK_MIB", "4")
    spec, win, L = "K*=5r,V*=6", 2048, 5000
    eng = mk.Engine(2, L + 64, spec, win)
    orc = ko.Cache(2, L + 64, spec, win)
    for layer in range(2):
        fill_both(torch, eng, orc, layer, 0, L, seed=layer)
    eng.commit(L)
    d0 = eng.state_digest()
    assert not eng.side_begin()  # store off
    eng.store_budget(1 << 30)
    assert eng.side_begin() and eng.side_active() and eng.position() == 0
    for layer in range(2):
        fill_both(torch, eng, None, layer, 0, 2700, seed=77)  # the side prompt overwrites rows and ring slots
    eng.commit(2700)
    assert eng.side_end() and not eng.side_active()
    assert eng.position() == L and np.array_equal(eng.state_digest(), d0)
    # store too small: the kept sequence is dropped, the engine is reset
    eng.store_budget(16 << 20)  # the kept rows need ~27 MB
    assert eng.side_begin()
    for layer in range(2):
        fill_both(torch, eng, None, layer, 0, 4000, seed=78)
    assert not eng.side_end()
    assert eng.position() == 0
    eng.close()


def test_error_paths_keep_the_engine_usable(mk, torch_cuda):
    torch = torch_cuda
    eng = mk.Engine(1, 256, "", 0)
    K = torch.zeros((4, 4, 256), dtype=torch.float16, device="cuda")
    Q = torch.zeros((1, 24, 256), dtype=torch.float16, device="cuda")
    O = torch.zeros((1, 24, 256), dtype=torch.float32, device="cuda")
    with pytest.raises(mk.EngineError):
        eng.append(0, 255, K, K)  # past the context
    with pytest.raises(mk.EngineError):
        eng.append(1, 0, K, K)  # no such layer
    with pytest.raises(mk.EngineError):
        eng.attend(0, 0, Q, O)  # rows not appended yet
    with pytest.raises(mk.EngineError):
        eng.commit(5)
    eng.append(0, 0, K, K)
    eng.attend(0, 3, Q, O)
    eng.sync()
    assert torch.isfinite(O).all()
    eng.close()


def test_store_exhausted_in_the_middle_of_a_snapshot(mk, torch_cuda, monkeypatch):
    """host_store.cu:246-266: a snapshot that runs out of store room half way gives its chunks back, the call answers "no
    room" (-3 at the C ABI, None here), the sequence and the store are as before, and the same call succeeds once there is room"""
    torch = torch_cuda
    monkeypatch.setenv("MK_STORE_CHUNK_MIB", "1")
    spec, win, L = "K*=5r,V*=6", 2048, 4100
    eng = mk.Engine(2, L + 64, spec, win)
    for layer in range(2):
        fill_both(torch, eng, None, layer, 0, L, seed=layer)
    eng.commit(L)
    d0 = eng.state_digest()
    need = eng.park_need(0)
    assert need > (8 << 20)
    eng.store_budget(5 << 20)  # five chunks: the snapshot takes them one by one and then finds no sixth
    assert eng.park(0) is None
    info = eng.store_info()
    assert info["used"] == 0 and info["parked"] == 0
    assert eng.position() == L and np.array_equal(eng.state_digest(), d0)
    eng.store_budget(need + (2 << 20))
    pid = eng.park(0)
    assert pid and eng.park_bytes(pid) == need
    eng.truncate(0)
    eng.unpark(pid)
    assert np.array_equal(eng.state_digest(), d0)
    eng.close()
