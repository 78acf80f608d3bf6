"""ctypes binding of the KV hot path's C ABI (include/mk_kv.h), in the style of the reference's server/mk_engine.py.

Tensor arguments are device pointers: pass torch CUDA tensors (their data_ptr is used) or plain integers.
"""
import ctypes as C
import json
import os

NH, NKV, HD, MAXT = 24, 4, 256, 8
SEQ_MAIN = -1
FLAG_SPILL, FLAG_WIN_ALL, FLAG_EXACT = 1, 2, 4

_DIR = os.path.dirname(os.path.abspath(__file__))


class EngineError(RuntimeError):
    pass


def lib_path():
    return os.environ.get("MK_KV_LIB", os.path.join(_DIR, "libmk_kv.so"))


_lib = None


def load_library():
    """Loads libmk_kv.so and declares every export of include/mk_kv.h. Raises if the library has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise EngineError("libmk_kv.so is not built (%s): run __graft_entry__.build() or make -C %s/csrc" % (path, _DIR))
    L = C.CDLL(path)
    vp, i, ll, cp = C.c_void_p, C.c_int, C.c_longlong, C.c_char_p
    ip, llp, ullp = C.POINTER(C.c_int), C.POINTER(C.c_longlong), C.POINTER(C.c_ulonglong)
    sig = {
        "mk_last_error": (cp, []),
        "mk_kv_abi_sig": (C.c_ulonglong, []),
        "mk_build_info": (cp, []),
        "mk_kv_new": (vp, [i, i, cp, i, i]),
        "mk_free": (None, [vp]),
        "mk_reset": (None, [vp]),
        "mk_kv_set_stream": (i, [vp, vp]),
        "mk_kv_sync": (i, [vp]),
        "mk_kv_wait_limits": (i, [C.c_uint, C.c_uint, C.c_uint]),
        "mk_kv_wait_limits_expire_now": (i, []),
        "mk_kv_append": (i, [vp, i, i, i, i, vp, vp]),
        "mk_kv_attend": (i, [vp, i, i, i, i, vp, vp]),
        "mk_kv_attend_static": (i, [vp, i, i, i, i, vp, vp]),
        "mk_kv_set_base": (i, [vp, i, i]),
        "mk_kv_attend_partial": (i, [vp, i, i, i, i, vp, i, i, vp, vp]),
        "mk_kv_combine": (i, [vp, i, i, i, vp, vp, vp]),
        "mk_kv_step_layers_partial": (i, [vp, i, i, i, i, vp, vp, vp, C.c_size_t, C.c_size_t, i, i, i, i, vp, vp]),
        "mk_kv_combine_layers": (i, [vp, i, i, i, vp, vp, vp, C.c_size_t]),
        "mk_kv_combine_layers_strided": (i, [vp, i, i, i, vp, vp, C.c_size_t, vp, C.c_size_t]),
        "mk_kv_step": (i, [vp, i, i, i, i, vp, vp, vp, vp]),
        "mk_kv_step_layers": (i, [vp, i, i, i, i, vp, vp, vp, vp, C.c_size_t, C.c_size_t, C.c_size_t]),
        "mk_kv_step_layers_at": (i, [vp, i, i, i, i, i, vp, vp, vp, vp, C.c_size_t, C.c_size_t, C.c_size_t]),
        "mk_kv_reserve_batch": (i, [vp, i]),
        "mk_kv_step_batch": (i, [vp, i, ip, i, ip, ip, vp, vp, vp, vp]),
        "mk_kv_attend_batch": (i, [vp, i, ip, i, ip, ip, vp, vp]),
        "mk_kv_commit": (i, [vp, i, i]),
        "mk_kv_position": (i, [vp, i]),
        "mk_kv_cap_T": (i, [i, i]),
        "mk_truncate": (i, [vp, i]),
        "mk_kv_truncate": (i, [vp, i, i]),
        "mk_kv_checkpoint": (i, [vp, i]),
        "mk_checkpoints": (i, [vp, ip, i]),
        "mk_kv_checkpoints": (i, [vp, i, ip, i]),
        "mk_rewind_to": (i, [vp, i]),
        "mk_kv_rewind_to": (i, [vp, i, i]),
        "mk_rewind_to_checkpoint": (i, [vp]),
        "mk_store_budget": (i, [vp, ll]),
        "mk_store_reserve": (i, [vp, ll]),
        "mk_store_info": (i, [vp, llp, i]),
        "mk_kv_sizes": (None, [vp, llp, llp, llp, llp]),
        "mk_park": (i, [vp, i]),
        "mk_kv_park": (i, [vp, i, i]),
        "mk_unpark": (i, [vp, i]),
        "mk_kv_unpark": (i, [vp, i, i]),
        "mk_park_drop": (i, [vp, i]),
        "mk_kv_state_save": (ll, [vp, i, cp, cp, C.c_size_t, i, vp, vp, i]),
        "mk_kv_state_load": (i, [vp, i, cp, cp, C.c_size_t, i, vp, vp, i]),
        "mk_park_need": (ll, [vp, i]),
        "mk_park_bytes": (ll, [vp, i]),
        "mk_kv_restore_prefix": (i, [vp, i, i, i, i]),
        "mk_kv_store_wait": (i, [vp]),
        "mk_side_begin": (i, [vp]),
        "mk_side_end": (i, [vp]),
        "mk_side_end_park": (i, [vp, i, ip]),
        "mk_side_unpark": (i, [vp, i]),
        "mk_side_drop": (i, [vp]),
        "mk_side_active": (i, [vp]),
        "mk_slots_open": (i, [vp, i, i]),
        "mk_slots_open2": (i, [vp, i, i, i]),
        "mk_slots_count": (i, [vp]),
        "mk_state_digest": (i, [vp, ullp, i]),
        "mk_kv_state_digest": (ll, [vp, i, ullp, ll]),
        "mk_kv_read_row": (i, [vp, i, i, i, i, i, i, vp, vp]),
        "mk_kv_write_row": (i, [vp, i, i, i, i, i, i, vp, vp]),
        "mk_kv_unpack_probe": (i, [vp, i, vp, vp, i, vp]),
        "mk_kv_bits": (i, [vp, i, i]),
        "mk_kv_has_ring": (i, [vp, i, i]),
        "mk_kv_ring_rows": (i, [vp]),
        "mk_kv_device_bytes": (ll, [vp]),
        "mk_kv_launches": (ll, [vp]),
        "mk_kv_profile": (ll, [vp, ullp, ll]),
    }
    for name, (res, args) in sig.items():
        f = getattr(L, name)
        f.restype, f.argtypes = res, args
    L._mk_exports = sorted(sig)
    _lib = L
    return L


def cap_T(n, T_req):
    return load_library().mk_kv_cap_T(n, T_req)


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        if not x.is_cuda:
            raise EngineError("expected a CUDA tensor")
        if not x.is_contiguous():
            raise EngineError("expected a contiguous tensor")
        return x.data_ptr()
    raise EngineError("expected a CUDA tensor or a device address")


def _ints(v):
    return (C.c_int * len(v))(*[int(x) for x in v])


class Engine:
    """One KV engine on the current CUDA device (mk_kv_new). kv_spec / kv_win take the reference's MK_KV / MK_KV_WIN."""

    def __init__(self, layers, ctx, kv_spec="", kv_win=0, spill=False, win_all=False, exact=False, stream=None):
        self.L = load_library()
        flags = (FLAG_SPILL if spill else 0) | (FLAG_WIN_ALL if win_all else 0) | (FLAG_EXACT if exact else 0)
        self.h = self.L.mk_kv_new(layers, ctx, kv_spec.encode(), kv_win, flags)
        if not self.h:
            raise EngineError(self.L.mk_last_error().decode())
        self.layers, self.ctx = layers, ctx
        if stream is not None:
            self.set_stream(stream)

    def close(self):
        if getattr(self, "h", None):
            self.L.mk_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _err(self, what):
        return EngineError("%s: %s" % (what, self.L.mk_last_error().decode()))

    def _ck(self, r, what):
        if r < 0:
            raise self._err(what)
        return r

    # ---- plumbing ----
    def set_stream(self, stream):
        """stream: a torch.cuda.Stream, a raw cudaStream_t value, or 0 for the default stream."""
        s = getattr(stream, "cuda_stream", stream)
        self._ck(self.L.mk_kv_set_stream(self.h, s), "set_stream")

    def sync(self):
        self._ck(self.L.mk_kv_sync(self.h), "sync")

    def wait_limits(self, hint_ns=0, rounds=0, polls=0):
        """limits of the attention kernel's device-side waits for the launches that follow (process-wide); all 0: the defaults"""
        self.L.mk_kv_wait_limits(hint_ns, rounds, polls)

    def wait_limits_expire_now(self):
        """the first device-side wait that does not succeed at once gives up (failure-path test)"""
        self.L.mk_kv_wait_limits_expire_now()

    def reset(self):
        self.L.mk_reset(self.h)

    def build_info(self):
        return json.loads(self.L.mk_build_info().decode())

    # ---- hot path ----
    def append(self, layer, pos0, K, V, seq=SEQ_MAIN):
        n = K.shape[0] if hasattr(K, "shape") else None
        if n is None:
            raise EngineError("append needs tensors (use append_raw for addresses)")
        self._ck(self.L.mk_kv_append(self.h, seq, layer, pos0, n, _ptr(K), _ptr(V)), "append")

    def append_raw(self, layer, pos0, n, K, V, seq=SEQ_MAIN):
        self._ck(self.L.mk_kv_append(self.h, seq, layer, pos0, n, _ptr(K), _ptr(V)), "append")

    def attend(self, layer, n, Q, O, seq=SEQ_MAIN):
        self._ck(self.L.mk_kv_attend(self.h, seq, layer, n, Q.shape[0], _ptr(Q), _ptr(O)), "attend")

    def attend_static(self, layer, n, Q, O, seq=SEQ_MAIN):
        """attend() that allocates nothing: partials go to the library's fixed device array (see mk_kv_attend_static)"""
        self._ck(self.L.mk_kv_attend_static(self.h, seq, layer, n, Q.shape[0], _ptr(Q), _ptr(O)), "attend_static")

    def set_base(self, base, seq=SEQ_MAIN):
        """this engine's copy of the sequence holds positions [base, base + ctx) (a sequence split by position over GPUs)"""
        self._ck(self.L.mk_kv_set_base(self.h, seq, base), "set_base")

    def attend_partial(self, layer, n, Q, pos_lo, pos_hi, part_out, ml_out, seq=SEQ_MAIN):
        """un-normalised attention of the T tokens at n over positions [pos_lo, pos_hi): part_out [4][48][256], ml_out [4][48][2]"""
        self._ck(self.L.mk_kv_attend_partial(self.h, seq, layer, n, Q.shape[0], _ptr(Q), pos_lo, pos_hi, _ptr(part_out), _ptr(ml_out)),
                 "attend_partial")

    def combine(self, layer, T, nparts, parts, mls, O):
        """merge of nparts partial results (all-gathered) into O [T][24][256]"""
        self._ck(self.L.mk_kv_combine(self.h, layer, T, nparts, _ptr(parts), _ptr(mls), _ptr(O)), "combine")

    def step_layers_partial(self, n, K, V, Q, own_lo, own_hi, pos_lo, pos_hi, parts, mls, seq=SEQ_MAIN):
        """K, V [layers][T][4][256], Q [layers][T][24][256] (layer stride = the tensors' stride 0); parts [layers][4][48][256],
        mls [layers][4][48][2]"""
        self._ck(self.L.mk_kv_step_layers_partial(self.h, seq, Q.shape[0], n, Q.shape[1], _ptr(K[0]), _ptr(V[0]), _ptr(Q[0]),
                                                  K.stride(0) * K.element_size(), Q.stride(0) * Q.element_size(), own_lo, own_hi, pos_lo, pos_hi,
                                                  _ptr(parts), _ptr(mls)), "step_layers_partial")

    def combine_layers(self, T, nparts, parts, mls, O):
        """parts [nparts][layers][4][48][256], mls [nparts][layers][4][48][2] -> O [layers][T][24][256]"""
        self._ck(self.L.mk_kv_combine_layers(self.h, O.shape[0], T, nparts, _ptr(parts), _ptr(mls), _ptr(O[0]), O.stride(0) * O.element_size()),
                 "combine_layers")

    def combine_layers_strided(self, T, nparts, parts, mls, rank_stride, O):
        """combine_layers when every rank's parts and mls arrays sit in one exchange buffer: parts / mls point at rank 0's arrays, rank p's
        start p * rank_stride bytes later"""
        self._ck(self.L.mk_kv_combine_layers_strided(self.h, O.shape[0], T, nparts, _ptr(parts), _ptr(mls), rank_stride, _ptr(O[0]),
                                                     O.stride(0) * O.element_size()), "combine_layers_strided")

    def step(self, layer, n, K, V, Q, O, seq=SEQ_MAIN):
        self._ck(self.L.mk_kv_step(self.h, seq, layer, n, Q.shape[0], _ptr(K), _ptr(V), _ptr(Q), _ptr(O)), "step")

    def step_layers(self, n, K, V, Q, O, seq=SEQ_MAIN):
        """one decode step over every layer in one call: K, V [layers][T][4][256], Q [layers][T][24][256], O likewise (fp32).
        A layer's rows must be contiguous; the layer stride is free (the first T rows of a larger per-layer buffer are fine)."""
        for x in (K, V, Q, O):
            if not x.is_cuda or not x[0].is_contiguous():
                raise EngineError("step_layers: expected CUDA tensors whose per-layer rows are contiguous")
        self._ck(self.L.mk_kv_step_layers(self.h, seq, K.shape[0], n, Q.shape[1], K.data_ptr(), V.data_ptr(), Q.data_ptr(), O.data_ptr(),
                                          K.stride(0) * K.element_size(), Q.stride(0) * Q.element_size(), O.stride(0) * O.element_size()),
                 "step_layers")

    def step_layers_at(self, layer0, n, K, V, Q, O, seq=SEQ_MAIN):
        """step_layers for layers layer0 .. layer0 + K.shape[0] - 1 (the tensors hold those layers only)"""
        for x in (K, V, Q, O):
            if not x.is_cuda or not x[0].is_contiguous():
                raise EngineError("step_layers_at: expected CUDA tensors whose per-layer rows are contiguous")
        self._ck(self.L.mk_kv_step_layers_at(self.h, seq, layer0, K.shape[0], n, Q.shape[1], K.data_ptr(), V.data_ptr(), Q.data_ptr(), O.data_ptr(),
                                             K.stride(0) * K.element_size(), Q.stride(0) * Q.element_size(), O.stride(0) * O.element_size()),
                 "step_layers_at")

    def reserve_batch(self, njobs):
        self._ck(self.L.mk_kv_reserve_batch(self.h, njobs), "reserve_batch")

    def step_batch(self, seqs, layer, n, T, K, V, Q, O):
        self._ck(self.L.mk_kv_step_batch(self.h, len(seqs), _ints(seqs), layer, _ints(n), _ints(T), _ptr(K), _ptr(V), _ptr(Q),
                                         _ptr(O)), "step_batch")

    def attend_batch(self, seqs, layer, n, T, Q, O):
        self._ck(self.L.mk_kv_attend_batch(self.h, len(seqs), _ints(seqs), layer, _ints(n), _ints(T), _ptr(Q), _ptr(O)),
                 "attend_batch")

    def commit(self, length, seq=SEQ_MAIN):
        self._ck(self.L.mk_kv_commit(self.h, seq, length), "commit")

    def position(self, seq=SEQ_MAIN):
        return self._ck(self.L.mk_kv_position(self.h, seq), "position")

    # ---- rewind ----
    def truncate(self, n, seq=SEQ_MAIN):
        self._ck(self.L.mk_kv_truncate(self.h, seq, n), "truncate")

    def checkpoint(self, seq=SEQ_MAIN):
        return self._ck(self.L.mk_kv_checkpoint(self.h, seq), "checkpoint")

    def checkpoints(self, seq=SEQ_MAIN):
        n = self._ck(self.L.mk_kv_checkpoints(self.h, seq, None, 0), "checkpoints")
        out = (C.c_int * max(n, 1))()
        self.L.mk_kv_checkpoints(self.h, seq, out, n)
        return list(out[:n])

    def rewind_to(self, pos, seq=SEQ_MAIN):
        return self.L.mk_kv_rewind_to(self.h, seq, pos) == 0

    def rewind_to_checkpoint(self):
        return self.L.mk_rewind_to_checkpoint(self.h) == 0

    # ---- host store ----
    def store_budget(self, nbytes):
        self._ck(self.L.mk_store_budget(self.h, int(nbytes)), "store_budget")

    def store_reserve(self, nbytes):
        self._ck(self.L.mk_store_reserve(self.h, int(nbytes)), "store_reserve")

    def store_info(self):
        out = (C.c_longlong * 10)()
        self._ck(self.L.mk_store_info(self.h, out, 10), "store_info")
        keys = ("budget", "allocated", "used", "parked", "last_bytes", "last_us", "side_us", "kv_token_bytes", "side_park_bytes",
                "side_park_us")
        return dict(zip(keys, out))

    def kv_sizes(self):
        a, b, c, d = C.c_longlong(), C.c_longlong(), C.c_longlong(), C.c_longlong()
        self.L.mk_kv_sizes(self.h, C.byref(a), C.byref(b), C.byref(c), C.byref(d))
        return {"per_token": a.value, "rings": b.value, "state": c.value, "checkpoint": d.value}

    def park(self, max_cks=0, seq=SEQ_MAIN):
        """id > 0, 0 for an empty sequence, None when the store has no room"""
        r = self.L.mk_kv_park(self.h, seq, max_cks)
        if r == -3:
            return None
        return self._ck(r, "park")

    def unpark(self, pid, seq=SEQ_MAIN):
        self._ck(self.L.mk_kv_unpark(self.h, seq, pid), "unpark")

    def park_drop(self, pid):
        return self.L.mk_park_drop(self.h, pid) == 0

    def state_save(self, path, key, hend, extra=(), seq=SEQ_MAIN):
        """The reference's prompt-state file (state_files.cu:97-238) of rows 0 .. hend - 1 + the rings + the caller's extra regions
        (torch tensors, device or host). Returns the file's size."""
        import ctypes as C
        key = bytes(key)
        ptrs = (C.c_void_p * max(len(extra), 1))(*[t.data_ptr() for t in extra])
        sizes = (C.c_size_t * max(len(extra), 1))(*[t.numel() * t.element_size() for t in extra])
        r = self.L.mk_kv_state_save(self.h, seq, str(path).encode(), key, len(key), hend, ptrs, sizes, len(extra))
        return self._ck(r, "state_save")

    def state_load(self, path, key, hend, extra=(), seq=SEQ_MAIN):
        """True when the file exists and matches key, hend and every region size: the sequence then holds hend positions."""
        import ctypes as C
        key = bytes(key)
        ptrs = (C.c_void_p * max(len(extra), 1))(*[t.data_ptr() for t in extra])
        sizes = (C.c_size_t * max(len(extra), 1))(*[t.numel() * t.element_size() for t in extra])
        return self._ck(self.L.mk_kv_state_load(self.h, seq, str(path).encode(), key, len(key), hend, ptrs, sizes, len(extra)), "state_load") == 1

    def park_need(self, max_cks=0):
        return self.L.mk_park_need(self.h, max_cks)

    def park_bytes(self, pid):
        return self.L.mk_park_bytes(self.h, pid)

    def restore_prefix(self, pid, pos, seq=SEQ_MAIN, wait=True):
        self._ck(self.L.mk_kv_restore_prefix(self.h, seq, pid, pos, int(wait)), "restore_prefix")

    def store_wait(self):
        self._ck(self.L.mk_kv_store_wait(self.h), "store_wait")

    def side_begin(self):
        r = self._ck(self.L.mk_side_begin(self.h), "side_begin")
        return r == 0

    def side_end(self):
        return self._ck(self.L.mk_side_end(self.h), "side_end") == 1

    def side_end_park(self, max_cks=0):
        """(kept sequence is back, id of the side request's parked conversation or 0)"""
        pid = C.c_int(0)
        r = self._ck(self.L.mk_side_end_park(self.h, max_cks, C.byref(pid)), "side_end_park")
        return r == 1, pid.value

    def side_unpark(self, pid):
        """True: the side request continues parked conversation pid; False: no room in the store (nothing changed)"""
        return self._ck(self.L.mk_side_unpark(self.h, pid), "side_unpark") == 0

    def side_drop(self):
        self._ck(self.L.mk_side_drop(self.h), "side_drop")

    def side_active(self):
        return self.L.mk_side_active(self.h) == 1

    # ---- slots ----
    def slots_open(self, n, ctx=0):
        return self._ck(self.L.mk_slots_open(self.h, n, ctx), "slots_open")

    def slots_count(self):
        return self._ck(self.L.mk_slots_count(self.h), "slots_count")

    # ---- test helpers ----
    def state_digest(self, seq=SEQ_MAIN):
        import numpy as np
        n = self.L.mk_kv_state_digest(self.h, seq, None, 0)
        if n < 0:
            raise self._err("state_digest")
        out = np.zeros(n, dtype=np.uint64)
        self.L.mk_kv_state_digest(self.h, seq, out.ctypes.data_as(C.POINTER(C.c_ulonglong)), n)
        return out

    def read_row(self, layer, side, g, pos, ring=False, seq=SEQ_MAIN):
        import numpy as np
        val = np.zeros(HD, dtype=np.uint8)
        sc = np.zeros(8, dtype=np.uint16)
        n = self._ck(self.L.mk_kv_read_row(self.h, seq, layer, side, g, pos, int(ring), val.ctypes.data, sc.ctypes.data), "read_row")
        return val[:n].copy(), sc

    def write_row(self, layer, side, g, pos, val, sc, ring=False, seq=SEQ_MAIN):
        import numpy as np
        val = np.ascontiguousarray(val, dtype=np.uint8)
        sc = np.ascontiguousarray(sc, dtype=np.uint16)
        self._ck(self.L.mk_kv_write_row(self.h, seq, layer, side, g, pos, int(ring), val.ctypes.data, sc.ctypes.data), "write_row")

    def unpack_probe(self, bits, rows, scales, out):
        """rows uint8 [n][32 bits], scales fp16 [n][8] -> out fp16 [n][256]: the operand values the tensor-core kernel's unpack makes"""
        self._ck(self.L.mk_kv_unpack_probe(self.h, bits, _ptr(rows), _ptr(scales), rows.shape[0], _ptr(out)), "unpack_probe")

    def bits(self, side, layer):
        return self._ck(self.L.mk_kv_bits(self.h, side, layer), "bits")

    def has_ring(self, side, layer):
        return self._ck(self.L.mk_kv_has_ring(self.h, side, layer), "has_ring") == 1

    def ring_rows(self):
        return self._ck(self.L.mk_kv_ring_rows(self.h), "ring_rows")

    def device_bytes(self):
        return self.L.mk_kv_device_bytes(self.h)

    def profile(self):
        """phase stamps of the last decode-attention launch, [CTA][16][20] ns (needs MK_KV_PROFILE=1 at construction)"""
        import numpy as np
        n = self.L.mk_kv_profile(self.h, None, 0)
        if n <= 0:
            return None
        out = np.zeros(n, dtype=np.uint64)
        self.L.mk_kv_profile(self.h, out.ctypes.data_as(C.POINTER(C.c_ulonglong)), n)
        return out.reshape(-1, 16, 20)

    def launches(self):
        return self.L.mk_kv_launches(self.h)
