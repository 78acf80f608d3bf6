"""GPU parity of the prompt-state file (state_files.cu:97-238): the engine's file equals the oracle's byte for byte in both write
modes, a load brings back rows, rings and the caller's regions, decoding continues from the restored state as from the original,
and a file that does not match is refused without touching the sequence."""
import hashlib

import numpy as np
import pytest

import kv_oracle as ko
import kvdata
from gpu_util import TOL, assert_rows_equal, attend_both, fill_both

pytestmark = pytest.mark.gpu


def sha(path):
    return hashlib.sha256(open(path, "rb").read()).hexdigest()


@pytest.mark.parametrize("spill", [False, True])
def test_state_file_equals_oracle_and_restores(mk, torch_cuda, tmp_path, spill):
    torch = torch_cuda
    spec, win, layers, L = "K*=5r,V*=6", 2048, 2, 5200  # past the window: the rings have wrapped, spill mode has rows to flush
    eng = mk.Engine(layers, L + 700, spec, win, spill=spill)
    orc = ko.Cache(layers, L + 700, spec, win)
    for l in range(layers):
        fill_both(torch, eng, orc, l, 0, L, seed=60 + l)
    eng.commit(L)
    key = b"state of " + spec.encode() + b"\x00 5200"
    state = torch.arange(1000, dtype=torch.float32, device="cuda")  # a caller's region on the device
    hist = torch.arange(77, dtype=torch.int32)                       # and one on the host
    pe, po = tmp_path / "eng.mks", tmp_path / "orc.mks"
    size = eng.state_save(pe, key, L, extra=[state, hist])
    assert size == pe.stat().st_size
    assert orc.state_save(po, key, L, extra=[state.cpu().numpy().tobytes(), hist.numpy().tobytes()]) == size
    assert sha(pe) == sha(po)
    assert sorted(p.name for p in tmp_path.iterdir()) == ["eng.mks", "orc.mks"]  # no temporary file left

    # a fresh engine takes the state from the file
    eng2 = mk.Engine(layers, L + 700, spec, win, spill=spill)
    state2, hist2 = torch.zeros_like(state), torch.zeros_like(hist)
    assert eng2.state_load(tmp_path / "nothing.mks", key, L, extra=[state2, hist2]) is False
    assert eng2.state_load(pe, key + b"x", L, extra=[state2, hist2]) is False   # another key
    assert eng2.state_load(pe, key, L - 32, extra=[state2, hist2]) is False     # another length
    assert eng2.state_load(pe, key, L, extra=[state2]) is False                 # another set of regions
    assert eng2.position() == 0
    assert eng2.state_load(pe, key, L, extra=[state2, hist2]) is True
    assert eng2.position() == L
    assert torch.equal(state2, state) and torch.equal(hist2, hist)
    assert np.array_equal(eng2.state_digest(), orc.digest(L))
    ws = ko.kv_ws(L, win)
    for l in range(layers):
        assert_rows_equal(eng2, orc, l, [0, 1, ws - 1, ws, L - 1], ring_positions=[ws, L - 700, L - 1])
    # decoding goes on from the restored state: append 8 rows (crossing nothing), attend, against the oracle
    K, V = kvdata.kv_rows(70, 1, L, 8)
    Q = kvdata.q_rows(70, 1, L, 8)
    orc.append(1, L, K, V)
    eng2.append(1, L, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
    got, want = attend_both(torch, eng2, orc, 1, L, Q)
    assert np.abs(got - want).max() <= TOL
    eng.close()
    eng2.close()


def test_state_file_refuses_a_damaged_file_and_a_wrong_state(mk, torch_cuda, tmp_path):
    torch = torch_cuda
    spec, win, L = "K*=6,V*=5r", 640, 900
    eng = mk.Engine(1, L + 64, spec, win)
    fill_both(torch, eng, None, 0, 0, L, seed=5)
    eng.commit(L)
    with pytest.raises(mk.EngineError, match="must equal the rows written"):
        eng.state_save(tmp_path / "a.mks", b"k", L - 100)
    p = tmp_path / "a.mks"
    eng.state_save(p, b"k", L)
    d0 = eng.state_digest()
    b = p.read_bytes()
    (tmp_path / "short.mks").write_bytes(b[:-1])
    (tmp_path / "long.mks").write_bytes(b + b"\x00")
    (tmp_path / "magic.mks").write_bytes(b"MKSTATE2" + b[8:])
    for name in ("short.mks", "long.mks", "magic.mks"):
        assert eng.state_load(tmp_path / name, b"k", L) is False
        assert eng.position() == L and np.array_equal(eng.state_digest(), d0)  # untouched
    assert eng.state_load(p, b"k", L) is True
    assert np.array_equal(eng.state_digest(), d0)
    eng.close()
