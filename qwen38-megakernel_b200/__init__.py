"""B200-native KV-cache hot path: quantized append, decode attention over the q8_0 ring + low-bit tier, host snapshots.

The package is a thin ctypes binding of libmk_kv.so (include/mk_kv.h). There is no CPU fallback: importing works
without a GPU, but creating an Engine needs the built library and a CUDA device.
"""
from .engine import Engine, EngineError, lib_path, load_library, cap_T, NH, NKV, HD, MAXT  # noqa: F401
from .build import build_library  # noqa: F401
from . import parallel  # noqa: F401
from . import cache_policy, conversation  # noqa: F401
