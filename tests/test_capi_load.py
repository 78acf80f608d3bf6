"""CPU checks of the C-ABI library: it loads, exports every function include/mk_kv.h declares, and follows the error
conventions without a GPU (no compute call is made here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    src = open(os.path.join(ROOT, "include", "mk_kv.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(mk_[A-Za-z0-9_]+)\s*\(", src)))


def test_header_declares_the_reference_names():
    names = declared_functions()
    for n in ("mk_last_error", "mk_free", "mk_reset", "mk_truncate", "mk_rewind_to", "mk_checkpoints", "mk_state_digest",
              "mk_store_budget", "mk_store_reserve", "mk_store_info", "mk_kv_sizes", "mk_park", "mk_unpark", "mk_park_drop",
              "mk_park_need", "mk_park_bytes", "mk_side_begin", "mk_side_end", "mk_side_drop", "mk_side_active", "mk_slots_open",
              "mk_slots_open2", "mk_side_end_park", "mk_side_unpark", "mk_rewind_to_checkpoint", "mk_build_info"):
        assert n in names


def test_library_exports_every_declared_symbol(mk):
    mk.build_library()
    L = ctypes.CDLL(mk.lib_path())
    for n in declared_functions():
        assert hasattr(L, n), "libmk_kv.so does not export " + n
    bound = mk.load_library()
    assert sorted(bound._mk_exports) == declared_functions()


def test_error_conventions_without_compute(mk):
    import torch
    L = mk.load_library()
    assert L.mk_kv_abi_sig() != 0
    assert b"sm_100a" in L.mk_build_info()
    # bad arguments: NULL + a message, before any device work
    assert L.mk_kv_new(0, 128, b"", 0, 0) is None and b"layers" in L.mk_last_error()
    assert L.mk_kv_new(16, 128, b"K*=9", 0, 0) is None and b"MK_KV" in L.mk_last_error()
    assert L.mk_kv_new(16, 128, b"Q1=4", 0, 0) is None
    assert L.mk_kv_append(None, -1, 0, 0, 1, None, None) == -1 and b"null handle" in L.mk_last_error()
    assert L.mk_kv_cap_T(638, 8) == 2 and L.mk_kv_cap_T(640, 8) == 8
    if not torch.cuda.is_available():
        # no silent CPU path: without a device the constructor fails loudly
        with pytest.raises(mk.EngineError):
            mk.Engine(1, 128)
