"""GPU test of mk_kv_attend_static, the attention entry point that never calls the CUDA allocator (its split partials live
in a fixed array inside the library). It must give what mk_kv_attend gives, on two calls in a row with different inputs:
the shared array still holds the first call's partials when the second one runs. Collected last on purpose."""
import numpy as np
import pytest

import kvdata

pytestmark = pytest.mark.gpu


def test_attend_static_matches_attend_twice(mk, torch_cuda):
    torch = torch_cuda
    spec, win = "K*=5r,V*=6", 2048
    eng = mk.Engine(2, 5200, spec, win)
    lens = [4100, 700]
    for layer, L in enumerate(lens):
        for a in range(0, L, 2048):
            K, V = kvdata.kv_rows(40 + layer, layer, a, min(2048, L - a))
            eng.append(layer, a, torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda())
    cases = []
    for layer, (L, T) in enumerate(zip(lens, (8, 3))):  # second call: fewer chunks and rows than the first left behind
        n = L - T
        Q = torch.from_numpy(kvdata.q_rows(41, layer, n, T)).cuda()
        ref = torch.empty((T, 24, 256), dtype=torch.float32, device="cuda")
        out = torch.full((T, 24, 256), float("nan"), dtype=torch.float32, device="cuda")
        eng.attend(layer, n, Q, ref)
        cases.append((layer, n, Q, ref, out))
    eng.sync()
    free_before = torch.cuda.mem_get_info()[0]
    for layer, n, Q, ref, out in cases:
        eng.attend_static(layer, n, Q, out)
    eng.sync()
    assert torch.cuda.mem_get_info()[0] >= free_before  # nothing was taken from the device allocator by the two calls
    for layer, n, Q, ref, out in cases:
        assert torch.isfinite(out).all()
        # the two entry points may run different kernels (same arithmetic; an fp16 rounding of P can fall the other way):
        # the bound of the short-context attention tests
        from test_gpu_attend import check_edge
        check_edge(out.cpu().numpy(), ref.cpu().numpy(), kvdata.channel_scales(40 + layer, layer, 1), ("static", layer))
    Q9 = torch.zeros((9, 24, 256), dtype=torch.float16, device="cuda")
    O9 = torch.zeros((9, 24, 256), dtype=torch.float32, device="cuda")
    with pytest.raises(mk.EngineError, match="fixed scratch"):
        eng.attend_static(0, 0, Q9, O9)
    eng.close()
