#!/usr/bin/env python
"""Builds the reference witness: the reference project's own KV quantizer / dequantizer device functions, cut verbatim out of
its source where it lies (nothing of it is copied into this repository's history), compiled with the small driver
oracle/ref_witness.cu into oracle/_ref/libref_witness.so. The witness runs on a GPU only; tests use it to pin the CPU oracle
and to generate the golden vectors under tests/golden/.

    python oracle/build_ref.py [reference_root]
"""
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAMES = ["kv_store_q8", "kv_store_q4", "fwht256", "kv_store_qn", "q8_to_f16", "q4_to_f16", "kv_hi", "qn_to_f16"]


def cut(src, names):
    lines = src.split("\n")
    pat = re.compile(r"^__device__ .*?\b(" + "|".join(names) + r")\s*\(")
    out, seen, i = [], set(), 0
    while i < len(lines):
        m = pat.match(lines[i])
        if not m:
            i += 1
            continue
        seen.add(m.group(1))
        start = i - 1 if i > 0 and lines[i - 1].startswith("template") else i
        depth, j, opened = 0, i, False
        while j < len(lines):
            depth += lines[j].count("{") - lines[j].count("}")
            opened = opened or "{" in lines[j]
            if opened and depth == 0:
                break
            j += 1
        out.extend(lines[start:j + 1])
        out.append("")
        i = j + 1
    missing = [n for n in names if n not in seen]
    if missing:
        raise SystemExit("build_ref: not found in the reference source: " + " ".join(missing))
    return "\n".join(out) + "\n"


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    src_path = os.path.join(ref, "qwen38_mk.cu")
    if not os.path.exists(src_path):
        print("build_ref: no reference tree at %s: witness not built" % ref)
        return 0
    os.makedirs(OUT, exist_ok=True)
    inc = os.path.join(OUT, "ref_cut.inc")
    with open(inc, "w") as f:
        f.write(cut(open(src_path, encoding="utf-8").read(), NAMES))
    so = os.path.join(OUT, "libref_witness.so")
    # the reference's own flags for device code: -O3 -std=c++17, default -fmad (its Makefile:3-13)
    cmd = ["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-shared", "-I", OUT,
           "-o", so, os.path.join(HERE, "ref_witness.cu")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    os.remove(inc)  # only the binary stays (and only under the git-ignored oracle/_ref)
    if r.returncode != 0:
        print(r.stdout + r.stderr)
        raise SystemExit("build_ref: nvcc failed")
    print("build_ref: built", so)
    return 0


if __name__ == "__main__":
    sys.exit(main())
