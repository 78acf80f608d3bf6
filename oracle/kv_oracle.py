"""ctypes binding of the CPU parity oracle (test infrastructure; see kv_oracle.cpp).

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module. It builds the shared library
with g++ on first use if it is missing.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_DIR, "libkv_oracle.so")

NH, NKV, HD = 24, 4, 256


def build(force=False):
    src = os.path.join(_DIR, "kv_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _DIR, "libkv_oracle.so"], check=True, capture_output=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        vp, ip, cp = C.c_void_p, C.c_int, C.c_char_p
        L.orc_last_error.restype = cp
        L.orc_new.restype = vp
        L.orc_new.argtypes = [ip, ip, cp, ip, ip]
        L.orc_free.argtypes = [vp]
        for name in ("orc_ring_rows", "orc_kv_top"):
            getattr(L, name).argtypes = [vp]
        L.orc_bits.argtypes = [vp, ip, ip]
        L.orc_rot.argtypes = [vp, ip, ip]
        L.orc_has_ring.argtypes = [vp, ip, ip]
        L.orc_append.argtypes = [vp, ip, ip, ip, vp, vp]
        L.orc_attend.argtypes = [vp, ip, ip, ip, vp, vp, ip, ip]
        L.orc_attend_cuts.argtypes = [vp, ip, ip, ip, vp, vp, ip, ip, vp]
        L.orc_attend_parts.argtypes = [vp, ip, ip, ip, vp, vp, ip, vp, vp, vp]
        L.orc_merge_parts.restype = None
        L.orc_merge_parts.argtypes = [ip, ip, ip, vp, vp, vp, vp]
        L.orc_buffer.restype = vp
        L.orc_buffer.argtypes = [vp, ip, ip, ip, vp]
        L.orc_ctxp.argtypes = [vp]
        L.orc_refill.argtypes = [vp, ip, ip]
        L.orc_ring_rewind.argtypes = [vp, ip]
        L.orc_row.argtypes = [vp, ip, ip, ip, ip, ip, vp, vp]
        L.orc_digest.restype = C.c_longlong
        L.orc_digest.argtypes = [vp, ip, vp, C.c_longlong]
        L.orc_snapshot.restype = C.c_longlong
        L.orc_snapshot.argtypes = [vp, ip, ip, ip, ip, vp]
        L.orc_state_save.restype = C.c_longlong
        L.orc_state_save.argtypes = [vp, cp, vp, C.c_longlong, ip, ip, vp, vp]
        L.orc_quant_row.argtypes = [vp, ip, vp, vp]
        L.orc_dequant_f32.argtypes = [vp, vp, ip, vp]
        L.orc_dequant_f16.argtypes = [vp, vp, ip, vp]
        L.orc_fwht256.argtypes = [vp]
        L.orc_attn_dims.argtypes = [ip, vp, vp]
        L.orc_parse_spec.argtypes = [cp, ip, vp, vp]
        L.orc_h2f.restype = C.c_float
        L.orc_h2f.argtypes = [C.c_uint]
        L.orc_f2h.restype = C.c_uint
        L.orc_f2h.argtypes = [C.c_float]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def err():
    return lib().orc_last_error().decode()


def kv_ws(L, win):
    return lib().orc_kv_ws(L, win)


def kv_rc(win):
    return lib().orc_kv_rc(win)


def att_cap_T(n, T):
    return lib().orc_att_cap_T(n, T)


def attn_dims(L):
    nch, cs = C.c_int(), C.c_int()
    lib().orc_attn_dims(L, C.byref(nch), C.byref(cs))
    return nch.value, cs.value


def fwht256(v):
    v = np.ascontiguousarray(v, dtype=np.float32).copy()
    assert v.shape[-1] == HD
    flat = v.reshape(-1, HD)
    for i in range(flat.shape[0]):
        lib().orc_fwht256(_p(flat[i]))
    return v


def quant_row(v, bits):
    """v: float32 [256] -> (row bytes uint8 [32*bits], scales uint16 [8])"""
    v = np.ascontiguousarray(v, dtype=np.float32)
    q = np.zeros(32 * bits, dtype=np.uint8)
    sc = np.zeros(8, dtype=np.uint16)
    lib().orc_quant_row(_p(v), bits, _p(q), _p(sc))
    return q, sc


def dequant_row(q, sc, bits, f16=False):
    out = np.zeros(HD, dtype=np.float32)
    q = np.ascontiguousarray(q, dtype=np.uint8)
    sc = np.ascontiguousarray(sc, dtype=np.uint16)
    (lib().orc_dequant_f16 if f16 else lib().orc_dequant_f32)(_p(q), _p(sc), bits, _p(out))
    return out


def parse_spec(spec, layers):
    kvb = np.zeros((2, layers), dtype=np.int32)
    rot = np.zeros((2, layers), dtype=np.int32)
    if lib().orc_parse_spec(spec.encode(), layers, _p(kvb), _p(rot)) != 0:
        raise ValueError(err())
    return kvb, rot


def merge_parts(T, m, l, Op, rot_v=False):
    """the reference's merge of split partials (layout of Cache.attend_parts) -> O fp32 [T][24][256]"""
    m = np.ascontiguousarray(m, dtype=np.float32)
    l = np.ascontiguousarray(l, dtype=np.float32)
    Op = np.ascontiguousarray(Op, dtype=np.float32)
    nc = m.shape[0] // NKV
    O = np.zeros((T, NH, HD), dtype=np.float32)
    lib().orc_merge_parts(T, nc, int(rot_v), _p(m), _p(l), _p(Op), _p(O))
    return O


class Cache:
    """The reference cache state (every row in its main format + the q8 rings), held in host memory."""

    def __init__(self, layers, ctx, spec="", win=0, win_all=False):
        self.h = lib().orc_new(layers, ctx, spec.encode(), win, int(win_all))
        if not self.h:
            raise ValueError(err())
        self.layers, self.ctx, self.win = layers, ctx, win
        self.rc = lib().orc_ring_rows(self.h)

    def close(self):
        if getattr(self, "h", None):
            lib().orc_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass

    def bits(self, w, layer):
        return lib().orc_bits(self.h, w, layer)

    def rot(self, w, layer):
        return bool(lib().orc_rot(self.h, w, layer))

    def has_ring(self, w, layer):
        return bool(lib().orc_has_ring(self.h, w, layer))

    def append(self, layer, pos0, K, V):
        K = np.ascontiguousarray(K, dtype=np.float16)
        V = np.ascontiguousarray(V, dtype=np.float16)
        n = K.shape[0]
        assert K.shape == (n, NKV, HD) and V.shape == (n, NKV, HD)
        if lib().orc_append(self.h, layer, pos0, n, _p(K), _p(V)) != 0:
            raise ValueError(err())

    def attend(self, layer, n, Q, threads=8, split=1):
        Q = np.ascontiguousarray(Q, dtype=np.float16)
        T = Q.shape[0]
        assert Q.shape == (T, NH, HD)
        O = np.zeros((T, NH, HD), dtype=np.float32)
        if lib().orc_attend(self.h, layer, n, T, _p(Q), _p(O), threads, split) != 0:
            raise ValueError(err())
        return O

    def attend_cuts(self, layer, n, Q, cuts, threads=8):
        """attend() with the reference's chunks cut again at the positions `cuts` (a sequence split by position over GPUs)"""
        Q = np.ascontiguousarray(Q, dtype=np.float16)
        T = Q.shape[0]
        O = np.zeros((T, NH, HD), dtype=np.float32)
        c = np.ascontiguousarray(sorted(int(x) for x in cuts), dtype=np.int32)
        if lib().orc_attend_cuts(self.h, layer, n, T, _p(Q), _p(O), threads, len(c), _p(c)) != 0:
            raise ValueError(err())
        return O

    def attend_parts(self, layer, n, Q, threads=8, want_O=True):
        """(O or None, m [items][6T], l [items][6T], Op [items][6T][256], chunks per kv head): the reference partition's split
        partials, item = kv head * chunks + chunk, row = (head % 6) T + t"""
        Q = np.ascontiguousarray(Q, dtype=np.float16)
        T = Q.shape[0]
        nch, _ = attn_dims(n + T)
        R = 6 * T
        m = np.zeros((NKV * nch, R), dtype=np.float32)
        l = np.zeros((NKV * nch, R), dtype=np.float32)
        Op = np.zeros((NKV * nch, R, HD), dtype=np.float32)
        O = np.zeros((T, NH, HD), dtype=np.float32) if want_O else None
        nc = lib().orc_attend_parts(self.h, layer, n, T, _p(Q), _p(O) if want_O else None, threads, _p(m), _p(l), _p(Op))
        if nc < 0:
            raise ValueError(err())
        assert nc == nch
        return O, m, l, Op, nc

    def buffer(self, layer, w, kind):
        """numpy view (uint8) of one of the layer's buffers: kind 0 main values, 1 main scales, 2 ring values, 3 ring scales"""
        nb = C.c_longlong()
        ptr = lib().orc_buffer(self.h, layer, w, kind, C.byref(nb))
        if not ptr:
            return None
        return np.ctypeslib.as_array((C.c_uint8 * nb.value).from_address(ptr))

    @property
    def ctxp(self):
        return lib().orc_ctxp(self.h)

    def refill(self, p0, p1):
        if lib().orc_refill(self.h, p0, p1) != 0:
            raise ValueError(err())

    def ring_rewind(self, P):
        return lib().orc_ring_rewind(self.h, P)

    @property
    def kv_top(self):
        return lib().orc_kv_top(self.h)

    def row(self, layer, w, g, pos, ring=False):
        val = np.zeros(HD, dtype=np.uint8)
        sc = np.zeros(8, dtype=np.uint16)
        n = lib().orc_row(self.h, layer, w, g, pos, int(ring), _p(val), _p(sc))
        if n < 0:
            raise ValueError(err())
        return val[:n].copy(), sc

    def digest(self, n):
        cnt = lib().orc_digest(self.h, n, None, 0)
        out = np.zeros(cnt, dtype=np.uint64)
        lib().orc_digest(self.h, n, _p(out), cnt)
        return out

    def state_save(self, path, key, hend, extra=()):
        """the reference's prompt-state file of rows 0 .. hend - 1 + the rings + the caller's extra regions (bytes objects)"""
        bufs = [np.frombuffer(bytes(e), dtype=np.uint8) for e in extra]
        ptrs = (C.c_void_p * max(len(bufs), 1))(*[b.ctypes.data if b.size else None for b in bufs])
        sizes = (C.c_longlong * max(len(bufs), 1))(*[b.size for b in bufs])
        kb = np.frombuffer(bytes(key), dtype=np.uint8)
        n = lib().orc_state_save(self.h, str(path).encode(), kb.ctypes.data if kb.size else None, kb.size, hend, len(bufs), ptrs, sizes)
        if n < 0:
            raise ValueError("state_save failed")
        return n

    def snapshot(self, a, b, ra=0, rb=None):
        rb = self.rc if rb is None else rb
        size = lib().orc_snapshot(self.h, a, b, ra, rb, None)
        out = np.zeros(size, dtype=np.uint8)
        lib().orc_snapshot(self.h, a, b, ra, rb, _p(out))
        return out
