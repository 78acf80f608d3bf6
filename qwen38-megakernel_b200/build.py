"""Builds libmk_kv.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
import os
import subprocess

_DIR = os.path.dirname(os.path.abspath(__file__))


def build_library(force=False, verbose=False):
    csrc = os.path.join(_DIR, "csrc")
    args = ["make", "-C", csrc]
    if force:
        args.append("-B")
    r = subprocess.run(args, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(r.stdout)
        print(r.stderr)
    if r.returncode != 0:
        raise RuntimeError("building libmk_kv.so failed:\n" + r.stderr[-4000:])
    return os.path.join(_DIR, "libmk_kv.so")
