"""GPU pin of the CPU oracle: the reference's own quantizer / dequantizer device functions (oracle/_ref, built from the
reference source by oracle/build_ref.py) against the oracle, bit for bit, on fresh seeded rows."""
import os
import sys

import numpy as np
import pytest

import kv_oracle as ko
import kvdata

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def same_half(a, b):
    """fp16 bit patterns equal, up to the sign of a zero product and the payload of a NaN (an overflowed scale times 0)"""
    nan = lambda x: (x & 0x7fff) > 0x7c00
    return (a == b) | (((a & 0x7fff) == 0) & ((b & 0x7fff) == 0)) | (nan(a) & nan(b))


SO = os.path.join(ROOT, "oracle", "_ref", "libref_witness.so")


@pytest.mark.skipif(not os.path.exists(SO), reason="reference witness not built (needs the reference tree at build time)")
@pytest.mark.parametrize("bits", [4, 5, 6, 7, 8])
@pytest.mark.parametrize("rot", [0, 1])
def test_oracle_equals_reference_device_functions(torch_cuda, bits, rot):
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_golden
    L = make_golden.witness()
    K, V = kvdata.kv_rows(77 + bits, 1, 0, 40)
    rows = np.concatenate([kvdata.edge_rows().astype(np.float16).astype(np.float32), K.reshape(-1, 256).astype(np.float32),
                           V.reshape(-1, 256).astype(np.float32)])
    rows = np.ascontiguousarray(rows)
    q, sc, f16 = make_golden.run(L, rows, bits, rot)
    for i in range(rows.shape[0]):
        v = ko.fwht256(rows[i]) if rot else rows[i]
        oq, osc = ko.quant_row(v, bits)
        assert np.array_equal(oq, q[i]) and np.array_equal(osc, sc[i]), (bits, rot, i)
        of = ko.dequant_row(oq, osc, bits, f16=True).astype(np.float16).view(np.uint16)
        assert same_half(of, f16[i]).all(), (bits, rot, i)
