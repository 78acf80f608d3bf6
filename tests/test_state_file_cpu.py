"""The prompt-state file's layout (state_files.cu:97-238), checked on the CPU: the oracle's writer against a parse of the file written
out by hand here from the cited lines (magic, key, hend, region count, sizes, then the regions in (layer, side, head) order, the rings
with all heads' values before all heads' scales, the caller's regions last)."""
import struct

import numpy as np

import kv_oracle as ko
import kvdata


def parse_state_file(path):
    b = open(path, "rb").read()
    assert b[:8] == b"MKSTATE1"
    pos = 8
    (kn,) = struct.unpack_from("<Q", b, pos); pos += 8
    key = b[pos:pos + kn]; pos += kn
    hend, nr = struct.unpack_from("<QQ", b, pos); pos += 16
    sizes = struct.unpack_from("<%dQ" % nr, b, pos); pos += 8 * nr
    regions = []
    for s in sizes:
        regions.append(b[pos:pos + s]); pos += s
    assert pos == len(b), "the file ends with its last region"
    return key, hend, regions


def test_oracle_state_file_layout(tmp_path):
    spec, win, layers, L = "K*=5r,K0=8,V*=6", 640, 2, 1500  # layer 0's K is q8_0: no ring for it (loader.cu:1490-1503)
    orc = ko.Cache(layers, L + 64, spec, win)
    for l in range(layers):
        K, V = kvdata.kv_rows(40 + l, l, 0, L)
        orc.append(l, 0, K, V)
    extra = [bytes(range(200)), b"", b"\x01\x02\x03"]
    key = b"model x ctx 1564 kvb 8 5r 6 6 win 640\x00tail"
    path = tmp_path / "s.mks"
    size = orc.state_save(path, key, L, extra)
    assert size == path.stat().st_size
    k, hend, R = parse_state_file(path)
    assert k == key and hend == L
    rings = [(l, w) for l in range(layers) for w in range(2) if orc.has_ring(w, l)]
    assert rings == [(0, 1), (1, 0), (1, 1)]
    assert len(R) == layers * 2 * 4 * 2 + 2 * len(rings) + len(extra)
    i = 0
    ctxp = orc.ctxp
    for l in range(layers):
        for w in range(2):
            rb = 32 * orc.bits(w, l)
            val = orc.buffer(l, w, 0).reshape(4, ctxp, rb)
            sc = orc.buffer(l, w, 1).reshape(4, ctxp, 16)  # (bytes: 8 halves per row)
            for g in range(4):
                assert R[i] == val[g, :L].tobytes() and R[i + 1] == sc[g, :L].tobytes(), (l, w, g)
                i += 2
    for l, w in rings:
        assert R[i] == orc.buffer(l, w, 2).tobytes() and R[i + 1] == orc.buffer(l, w, 3).tobytes()
        assert len(R[i]) == 4 * orc.rc * 256 and len(R[i + 1]) == 4 * orc.rc * 16
        i += 2
    assert R[i:] == extra


def test_oracle_state_file_empty_and_overwrite(tmp_path):
    orc = ko.Cache(1, 128, "K*=5r,V*=6", 0)  # no window: no ring regions
    path = tmp_path / "e.mks"
    assert orc.state_save(path, b"", 0) == 8 + 8 + 8 + 8 + 8 * 16
    k, hend, R = parse_state_file(path)
    assert k == b"" and hend == 0 and len(R) == 16 and all(len(r) == 0 for r in R)
    K, V = kvdata.kv_rows(1, 0, 0, 40)
    orc.append(0, 0, K, V)
    orc.state_save(path, b"k", 40)  # replaces the file (written beside it, then renamed)
    k, hend, R = parse_state_file(path)
    assert k == b"k" and hend == 40 and len(R[0]) == 40 * 160 and len(R[1]) == 40 * 16
    assert sorted(p.name for p in tmp_path.iterdir()) == ["e.mks"]
