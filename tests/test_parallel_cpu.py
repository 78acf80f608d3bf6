"""CPU tests of the multi-GPU host logic: slot partition, position ranges, and the partial-softmax combine over a world_size-2
gloo process group (the data path between ranks is one all-gather of (max, sum, un-normalised output) per row)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def test_lpt_partition_balances_bytes(mk):
    P = mk.parallel
    rng = np.random.default_rng(3)
    lengths = np.exp(rng.uniform(np.log(2000), np.log(100000), 32)).astype(int).tolist()
    for n in (1, 2, 4, 8):
        parts = P.lpt_partition(lengths, n)
        assert sorted(i for p in parts for i in p) == list(range(32))
        loads = [sum(P.kv_bytes(lengths[i]) for i in p) for p in parts]
        assert max(loads) <= sum(loads) / n + P.kv_bytes(max(lengths))  # greedy bound
        assert P.lpt_partition(lengths, n) == parts  # deterministic: every rank computes the same deal


def test_split_ranges_cover_and_align(mk):
    P = mk.parallel
    for cap in (100, 4096, 262144 + 64, 101600 + 600):
        for w in (1, 2, 3, 4, 8):
            r = P.split_ranges(cap, w)
            assert r[0][0] == 0 and r[-1][1] == cap and len(r) == w
            for (a, b), (c, d) in zip(r, r[1:]):
                assert b == c and b >= a and (a % 32 == 0 or a == cap) and (b % 32 == 0 or b == cap)


def _partials(q, K, V, lo, hi, T):
    """float64 un-normalised softmax partial of rows over positions [lo, hi): parts [4][48][256], mls [4][48][2]"""
    parts = np.zeros((4, 48, 256), dtype=np.float32)
    mls = np.zeros((4, 48, 2), dtype=np.float32)
    mls[..., 0] = -np.inf
    n = K.shape[0] - T
    for h in range(24):
        g = h // 6
        for t in range(T):
            r = (h % 6) * T + t
            top = min(hi, n + t + 1)
            if top <= lo:
                continue
            s = K[lo:top, g] @ q[t, h] / 16.0
            m = s.max()
            p = np.exp(s - m)
            parts[g, r] = p @ V[lo:top, g]
            mls[g, r] = (m, p.sum())
    return parts, mls


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import importlib
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    P = importlib.import_module("qwen38-megakernel_b200").parallel
    rng = np.random.default_rng(0)  # replicated inputs, as the split-sequence driver assumes
    L, T = 777, 3
    K = rng.standard_normal((L, 4, 256)); V = rng.standard_normal((L, 4, 256)); Q = rng.standard_normal((T, 24, 256))
    lo, hi = P.split_ranges(L, world)[rank]
    part, ml = _partials(Q, K, V, lo, hi, T)
    parts = torch.zeros((world * 4, 48, 256)); mls = torch.zeros((world * 4, 48, 2))  # ranks' partials one after another
    dist.all_gather_into_tensor(parts, torch.from_numpy(part))
    dist.all_gather_into_tensor(mls, torch.from_numpy(ml))
    O = P.combine_partials_np(parts.numpy().reshape(world, 4, 48, 256), mls.numpy().reshape(world, 4, 48, 2), T)
    full_p, full_ml = _partials(Q, K, V, 0, L, T)
    ref = P.combine_partials_np(full_p[None], full_ml[None], T)
    q.put((rank, float(np.abs(O - ref).max())))
    dist.destroy_process_group()


def test_sequence_split_combine_gloo_world2():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("fork")  # (no CUDA in these processes)
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=60) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in res) == [0, 1]
    assert max(e for _, e in res) < 1e-4
