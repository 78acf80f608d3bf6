"""GPU test of mk_kv_attend_static, the attention entry point that never calls the CUDA allocator (its split partials live
in a fixed array inside the library). It must give what mk_kv_attend gives -- both are checked against the oracle under the
path's 2e-3 bar -- on two calls in a row with different inputs: the shared array still holds the first call's partials when the
second one runs. Collected last on purpose."""
import numpy as np
import pytest

import kv_oracle as ko
import kvdata
from gpu_util import TOL, check_flips, fill_both

pytestmark = pytest.mark.gpu


def test_attend_static_matches_attend_twice(mk, torch_cuda):
    torch = torch_cuda
    spec, win = "K*=5r,V*=6", 2048
    eng = mk.Engine(2, 5200, spec, win)
    orc = ko.Cache(2, 5200, spec, win)
    lens = [3000, 700]  # (both inside one window ring: the rows written are counted per sequence, not per layer)
    for layer, L in enumerate(lens):
        fill_both(torch, eng, orc, layer, 0, L, seed=40 + layer)
    cases = []
    for layer, (L, T) in enumerate(zip(lens, (8, 3))):  # second call: fewer chunks and rows than the first left behind
        n = L - T
        Qh = kvdata.q_rows(41, layer, n, T)
        Q = torch.from_numpy(Qh).cuda()
        ref = torch.empty((T, 24, 256), dtype=torch.float32, device="cuda")
        out = torch.full((T, 24, 256), float("nan"), dtype=torch.float32, device="cuda")
        eng.attend(layer, n, Q, ref)
        cases.append((layer, n, Qh, Q, ref, out))
    eng.sync()
    free_before = torch.cuda.mem_get_info()[0]
    for layer, n, Qh, Q, ref, out in cases:
        eng.attend_static(layer, n, Q, out)
    eng.sync()
    assert torch.cuda.mem_get_info()[0] >= free_before  # nothing was taken from the device allocator by the two calls
    for layer, n, Qh, Q, ref, out in cases:
        Oref = orc.attend(layer, n, Qh)
        check_flips(out.cpu().numpy(), Oref, orc, layer, n, Qh, ("static", layer))
        check_flips(ref.cpu().numpy(), Oref, orc, layer, n, Qh, ("attend", layer))
        # the two entry points run different kernels (same arithmetic, another summation order)
        assert np.abs(out.cpu().numpy() - ref.cpu().numpy()).max() <= TOL
    Q9 = torch.zeros((9, 24, 256), dtype=torch.float16, device="cuda")
    O9 = torch.zeros((9, 24, 256), dtype=torch.float32, device="cuda")
    with pytest.raises(mk.EngineError, match="fixed scratch"):
        eng.attend_static(0, 0, Q9, O9)
    eng.close()
