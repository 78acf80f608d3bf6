"""The failure path of the decode-attention kernel, without a GPU fault: every device-side wait is bounded, and when one runs out
the kernel sets the status word and returns (mk_shared.cuh:170-203 is the reference's error-word convention, capi.cpp:219-244 its
-1 + reset). Here the limits are set so that the first wait that does not succeed at once gives up; the launch must end, mk_kv_sync
must report -1 with the message, and the same handle must then give a correct attention again. Also: calls a sequence split by
position cannot serve return -1 instead of touching rows it does not hold."""
import numpy as np
import pytest

import kv_oracle as ko
import kvdata
from gpu_util import TOL, attend_both, fill_both

pytestmark = pytest.mark.gpu


def test_expired_wait_returns_error_and_engine_stays_usable(mk, torch_cuda, monkeypatch):
    torch = torch_cuda
    # the limits are the tensor-core kernel's (read when the engine is made); the mma.sync kernel's are compiled in: seconds, by
    # which every copy it issued has landed, so it is never made to give up early
    monkeypatch.setenv("MK_KV_ATTN", "tc")
    spec, win, L, T = "K*=5r,V*=6", 2048, 9000, 8
    eng = mk.Engine(1, L + 64, spec, win)
    orc = ko.Cache(1, L + 64, spec, win)
    fill_both(torch, eng, orc, 0, 0, L, seed=21)
    n = L - T
    Q = kvdata.q_rows(21, 0, n, T)
    Qd = torch.from_numpy(Q).cuda()
    O = torch.zeros((T, 24, 256), dtype=torch.float32, device="cuda")
    try:
        eng.wait_limits_expire_now()
        eng.attend(0, n, Qd, O)  # the staged tiles are not there at the first look: every CTA gives up and runs to its end
        with pytest.raises(mk.EngineError, match="gave up waiting"):
            eng.sync()
    finally:
        eng.wait_limits()  # the defaults again
    # mk_kv_sync reset the engine (the reference's convention): refill, then the same call must be right
    assert eng.position() == 0
    fill_both(torch, eng, None, 0, 0, L, seed=21)
    O2, Oref = attend_both(torch, eng, orc, 0, n, Q)
    assert np.abs(O2 - Oref).max() <= TOL
    eng.close()


def test_split_sequence_refuses_whole_sequence_calls(mk, torch_cuda):
    torch = torch_cuda
    eng = mk.Engine(1, 4096, "K*=5r,V*=6", 2048)
    eng.store_budget(1 << 30)
    eng.set_base(2048)
    K, V = kvdata.kv_rows(3, 0, 2048, 200)
    eng.append(0, 2048, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
    eng.commit(2248)
    Q = torch.zeros((1, 24, 256), dtype=torch.float16, device="cuda")
    O = torch.zeros((1, 24, 256), dtype=torch.float32, device="cuda")
    for call in (lambda: eng.attend(0, 2247, Q, O), lambda: eng.attend_static(0, 2247, Q, O), lambda: eng.truncate(2100),
                 lambda: eng.checkpoint(), lambda: eng.park(), lambda: eng.state_digest(), lambda: eng.side_begin(),
                 lambda: eng.step(0, 2248, torch.from_numpy(K[:1]).cuda(), torch.from_numpy(V[:1]).cuda(), Q, O)):
        with pytest.raises(mk.EngineError, match="split by position"):
            call()
    eng.sync()
    eng.reset()  # a reset keeps the base: the next append below it is refused, at it accepted
    with pytest.raises(mk.EngineError):
        eng.append(0, 0, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
    eng.append(0, 2048, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
    eng.sync()
    eng.close()


def test_attend_behind_overwritten_window_is_refused(mk, torch_cuda):
    """the ring holds the newest rows written: attending at an earlier position after a long append would read later rows"""
    torch = torch_cuda
    eng = mk.Engine(1, 9000, "K*=5r,V*=6", 2048)
    fill_both(torch, eng, None, 0, 0, 8000, seed=4)
    Q = torch.zeros((1, 24, 256), dtype=torch.float16, device="cuda")
    O = torch.zeros((1, 24, 256), dtype=torch.float32, device="cuda")
    with pytest.raises(mk.EngineError, match="overwritten"):
        eng.attend(0, 3000, Q, O)
    eng.commit(8000)
    eng.truncate(3001)  # the refill puts the window's rows back
    eng.attend(0, 3000, Q, O)
    eng.sync()
    eng.close()
