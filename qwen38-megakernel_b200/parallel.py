"""Partitioning of the KV path over the GPUs of one node (one process per GPU, torch.distributed for the plumbing).

Two ways, as the cache shards naturally:
  * independent sequences (slots): every sequence lives wholly on one GPU, dealt by bytes (longest first); no collective;
  * one very long sequence split by position: rank r owns a fixed range of positions; every rank attends the query tokens over
    its own rows with the partition of the whole context, the per-row (max, sum, un-normalised output) partials are
    all-gathered (198 KB per rank and layer at 8 tokens) and merged on every rank by the same merge the single-GPU path uses
    for its split-K partials (reference: qwen38_mk.cu:3048-3064, 4658-4669; the reference itself is single-GPU).
Remote data is only ever read from local memory after the collective delivered it.
"""
import numpy as np

NH, NKV, HD, GQ, AR, ATP = 24, 4, 256, 6, 48, 32


def kv_bytes(length, kbits=5, vbits=6):
    """bytes of one layer's rows of a sequence (values + scales, K and V)"""
    return length * NKV * ((32 * kbits + 16) + (32 * vbits + 16))


def lpt_partition(lengths, n_gpus, cost=kv_bytes):
    """Deals sequences to GPUs, longest first, each to the least loaded GPU. Returns a list of index lists, one per GPU."""
    order = sorted(range(len(lengths)), key=lambda i: (-cost(lengths[i]), i))
    load = [0] * n_gpus
    out = [[] for _ in range(n_gpus)]
    for i in order:
        g = min(range(n_gpus), key=lambda k: (load[k], k))
        out[g].append(i)
        load[g] += cost(lengths[i])
    return out


def split_ranges(capacity, world):
    """Static ownership of positions [0, capacity): rank r owns [lo, hi), multiples of 32, the last rank up to the capacity.
    Ownership cannot follow the attention partition's chunk boundaries: the chunk size grows with the context (32 positions per
    640 of context), rows would have to move between GPUs as the sequence grows. A rank boundary inside a chunk cuts that chunk in
    two pieces whose later one starts its running max afresh; the merge is exact in either case, the fp16 rounding of P is taken
    against another max for the positions after the cut (tests/test_gpu_split.py bounds the effect at 262,152 positions)."""
    per = -(-capacity // world)
    per = -(-per // ATP) * ATP
    out = []
    for r in range(world):
        lo = min(r * per, capacity)
        hi = capacity if r == world - 1 else min((r + 1) * per, capacity)
        out.append((lo, hi))
    return out


def combine_partials_np(parts, mls, T, rot_v=False):
    """numpy statement of the merge: parts [P][4][48][256], mls [P][4][48][2] -> O [T][24][256] (host logic tests)"""
    parts = np.asarray(parts, dtype=np.float32)
    mls = np.asarray(mls, dtype=np.float32)
    O = np.zeros((T, NH, HD), dtype=np.float32)
    for h in range(NH):
        g = h // GQ
        for t in range(T):
            r = (h % GQ) * T + t
            m = mls[:, g, r, 0]
            M = m.max()
            with np.errstate(invalid="ignore"):
                w = np.where(np.isneginf(m), 0.0, np.exp(m - M)).astype(np.float32)
            num = (w[:, None] * parts[:, g, r, :]).sum(0)
            den = (w * mls[:, g, r, 1]).sum()
            O[t, h] = num / den
    if rot_v:
        H = np.array([[(-1) ** bin(i & j).count("1") for j in range(HD)] for i in range(HD)], dtype=np.float32) / 16.0
        O = O @ H
    return O


class SplitSequence:
    """One sequence of up to `capacity` positions split by position over the ranks of a process group.

    Every rank constructs it with the same arguments and calls append / attend with the same (replicated) rows; each rank stores
    only the positions it owns. dist: torch.distributed (initialised, NCCL) or None for a single process."""

    def __init__(self, engine_cls, layers, capacity, kv_spec, kv_win, rank, world, dist=None, spill=False, stream=None):
        self.rank, self.world, self.dist = rank, world, dist
        self.ranges = split_ranges(capacity, world)
        self.lo, self.hi = self.ranges[rank]
        self.eng = engine_cls(layers, max(self.hi - self.lo, ATP), kv_spec, kv_win, spill=spill, stream=stream)
        self.eng.set_base(self.lo - self.lo % ATP)  # (lo is a multiple of 32 unless the rank owns nothing)
        self._bufs = None

    def append(self, layer, pos0, K, V):
        """rows pos0 .. pos0 + n - 1 (replicated on every rank): this rank keeps the ones it owns"""
        n = K.shape[0]
        a, b = max(pos0, self.lo), min(pos0 + n, self.hi)
        if b > a:
            self.eng.append(layer, a, K[a - pos0:b - pos0], V[a - pos0:b - pos0])

    def commit(self, length):
        self.eng.commit(min(max(length, self.lo), self.hi) if length > self.lo else 0)

    def attend(self, layer, n, Q, O):
        import torch
        T = Q.shape[0]
        L = n + T
        if self._bufs is None:
            dev = Q.device
            self._bufs = (torch.empty((NKV, AR, HD), dtype=torch.float32, device=dev), torch.empty((NKV, AR, 2), dtype=torch.float32, device=dev),
                          torch.empty((self.world * NKV, AR, HD), dtype=torch.float32, device=dev),  # the ranks' partials, in order
                          torch.empty((self.world * NKV, AR, 2), dtype=torch.float32, device=dev))
        part, ml, parts, mls = self._bufs
        hi = min(self.hi, L)
        if hi > self.lo:
            self.eng.attend_partial(layer, n, Q, self.lo, hi, part, ml)
        else:  # none of this rank's positions are visible yet: an empty partial
            self.eng.attend_partial(layer, n, Q, self.lo, self.lo, part, ml)
        if self.dist is not None and self.world > 1:
            self.dist.all_gather_into_tensor(parts, part)
            self.dist.all_gather_into_tensor(mls, ml)
        else:
            parts[:NKV].copy_(part)
            mls[:NKV].copy_(ml)
        self.eng.combine(layer, T, self.world, parts, mls, O)

    def step(self, n, K, V, Q, O):
        """One decode step over every layer with ONE exchange: K, V [layers][T][4][256], Q [layers][T][24][256] (replicated on
        every rank), O [layers][T][24][256] fp32. Every rank appends the rows it owns and attends over its own positions for all
        layers (one library call) into one send buffer (the outputs, then the (max, sum) pairs: 3.2 MB at 16 layers), the ranks'
        buffers are all-gathered once per step, and one launch merges every layer."""
        import torch
        layers, T = Q.shape[0], Q.shape[1]
        L = n + T
        key = (layers, str(Q.device))
        if getattr(self, "_step_key", None) != key:
            dev = Q.device
            npart, nml = layers * NKV * AR * HD, layers * NKV * AR * 2
            send = torch.empty(npart + nml, dtype=torch.float32, device=dev)
            recv = torch.empty((self.world, npart + nml), dtype=torch.float32, device=dev)
            self._step_bufs = (send, recv, npart)
            self._step_key = key
        send, recv, npart = self._step_bufs
        part, ml = send[:npart], send[npart:]
        self.eng.step_layers_partial(n, K, V, Q, self.lo, self.hi, self.lo, max(min(self.hi, L), self.lo), part, ml)
        if self.dist is not None and self.world > 1:
            self.dist.all_gather_into_tensor(recv, send)
        else:
            recv[0].copy_(send)
        self.eng.combine_layers_strided(T, self.world, recv[0, :npart], recv[0, npart:], recv.stride(0) * 4, O)

    def close(self):
        self.eng.close()
