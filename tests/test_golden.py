"""CPU check of the oracle against the committed golden vectors: bytes produced by the reference's own device functions on a
B200 (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

import kv_oracle as ko

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kv_quant_golden.npz")


def same_half(a, b):
    """fp16 bit patterns equal, up to the sign of a zero product and the payload of a NaN (an overflowed scale times 0)"""
    nan = lambda x: (x & 0x7fff) > 0x7c00
    return (a == b) | (((a & 0x7fff) == 0) & ((b & 0x7fff) == 0)) | (nan(a) & nan(b))


@pytest.mark.skipif(not os.path.exists(GOLD), reason="golden vectors not generated yet")
def test_oracle_matches_reference_golden_vectors():
    g = np.load(GOLD)
    rows = g["rows"]
    for bits in (4, 5, 6, 7, 8):
        for rot in (0, 1):
            q, sc, f16 = g["q_%d_%d" % (bits, rot)], g["sc_%d_%d" % (bits, rot)], g["f16_%d_%d" % (bits, rot)]
            for i in range(rows.shape[0]):
                v = ko.fwht256(rows[i]) if rot else rows[i]
                oq, osc = ko.quant_row(v, bits)
                assert np.array_equal(oq, q[i]) and np.array_equal(osc, sc[i]), (bits, rot, i)
                of = ko.dequant_row(oq, osc, bits, f16=True).astype(np.float16).view(np.uint16)
                assert same_half(of, f16[i]).all(), (bits, rot, i)
