"""GPU parity of the unpack step alone (scope row a10): the operand values the tensor-core attention kernel builds from packed rows
are fp16(d * q) of the reference's dequantisers (qwen38_mk.cu:2335-2343, 2457-2468), bit for bit, for every format; the rows are
the oracle's quantizer output on seeded data plus rows of extreme indices and scales."""
import numpy as np
import pytest

import kv_oracle as ko
import kvdata

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", [4, 5, 6, 7, 8])
def test_unpack_operands_bit_exact(mk, torch_cuda, bits):
    torch = torch_cuda
    n = 77  # two full tiles and a ragged one
    K, _ = kvdata.kv_rows(31 + bits, 0, 0, n)
    rb = 32 * bits
    rows = np.zeros((n, rb), dtype=np.uint8)
    sc = np.zeros((n, 8), dtype=np.uint16)
    for i in range(n):
        q, s = ko.quant_row(K[i, i % 4].astype(np.float32), bits)
        rows[i], sc[i] = q, s
    rng = np.random.default_rng(bits)
    rows[5] = 0            # smallest indices
    rows[6] = 0xFF         # largest indices (q8_0: -1)
    rows[7] = rng.integers(0, 256, size=rb, dtype=np.uint8)  # any bytes
    sc[7] = np.array([0x0001, 0x8001, 0x7BFF, 0xFBFF, 0x0000, 0x8000, 0x3C00, 0x0400], dtype=np.uint16)  # subnormal, +-max, +-0, 1, min normal
    eng = mk.Engine(1, 64, "", 0)
    out = torch.zeros((n, 256), dtype=torch.float16, device="cuda")
    eng.unpack_probe(bits, torch.from_numpy(rows).cuda(), torch.from_numpy(sc.view(np.float16)).cuda(), out)
    eng.sync()
    got = out.cpu().numpy().view(np.uint16)
    for i in range(n):
        want = ko.dequant_row(rows[i], sc[i], bits, f16=True).astype(np.float16).view(np.uint16)
        a, b = got[i], want
        same = (a == b) | (((a & 0x7FFF) == 0) & ((b & 0x7FFF) == 0))  # (+0 and -0 are the same operand)
        assert same.all(), (bits, i, np.flatnonzero(~same)[:8], a[~same][:8], b[~same][:8])
    eng.close()
