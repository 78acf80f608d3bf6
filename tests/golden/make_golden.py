#!/usr/bin/env python
"""Generates tests/golden/kv_quant_golden.npz on a GPU box: the bytes the REFERENCE's own quantizer / dequantizer device
functions produce (oracle/_ref/libref_witness.so, built by oracle/build_ref.py from the reference source) for a fixed set
of input rows. The CPU oracle and the CUDA kernels are then both checked against these vectors.

    python tests/golden/make_golden.py [out.npz]
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path[:0] = [os.path.join(ROOT, "tests")]
import kvdata  # noqa: E402


def witness():
    so = os.path.join(ROOT, "oracle", "_ref", "libref_witness.so")
    L = C.CDLL(so)
    L.ref_quant.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    L.ref_dequant.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    return L


def input_rows():
    """fp32 rows whose values are fp16-representable (what the append path feeds the quantizer): corner cases + seeded rows"""
    edge = kvdata.edge_rows().astype(np.float16).astype(np.float32)
    K, V = kvdata.kv_rows(123, 0, 0, 3)
    rnd = np.concatenate([K.reshape(-1, 256), V.reshape(-1, 256)]).astype(np.float32)
    return np.ascontiguousarray(np.concatenate([edge, rnd]))


def run(L, rows, bits, rot):
    n = rows.shape[0]
    q = np.zeros((n, 256), dtype=np.uint8)
    sc = np.zeros((n, 8), dtype=np.uint16)
    assert L.ref_quant(rows.ctypes.data, n, bits, rot, q.ctypes.data, sc.ctypes.data) == 0
    f16 = np.zeros((n, 256), dtype=np.uint16)
    assert L.ref_dequant(q.ctypes.data, sc.ctypes.data, n, bits, f16.ctypes.data) == 0
    return q[:, :32 * bits].copy(), sc, f16


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "kv_quant_golden.npz")
    L = witness()
    rows = input_rows()
    d = {"rows": rows}
    for bits in (4, 5, 6, 7, 8):
        for rot in (0, 1):
            q, sc, f16 = run(L, rows, bits, rot)
            d["q_%d_%d" % (bits, rot)] = q
            d["sc_%d_%d" % (bits, rot)] = sc
            d["f16_%d_%d" % (bits, rot)] = f16
    np.savez_compressed(out, **d)
    print("wrote", out, os.path.getsize(out), "bytes,", rows.shape[0], "rows")


if __name__ == "__main__":
    main()
