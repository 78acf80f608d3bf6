#!/usr/bin/env python
"""Builds the reference witnesses: the reference project's own device code for this path, cut verbatim out of its source where
it lies (nothing of it is copied into this repository's history) and compiled with the small drivers in this directory into
the git-ignored oracle/_ref/:

    libref_witness.so       quantizer / rotation / dequantizer device functions (driver: ref_witness.cu)
    libref_attn_witness.so  the decode-attention kernels, cut by the reference's own script bench/kvattn_gen.py
                            (driver: ref_attn_witness.cu)

The witnesses run on a GPU only; tests use them to pin the CPU oracle and to generate the golden vectors under tests/golden/.

    python oracle/build_ref.py <reference_root>        (or MK_REFERENCE_ROOT=<reference_root>)
"""
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAMES = ["kv_store_q8", "kv_store_q4", "fwht256", "kv_store_qn", "q8_to_f16", "q4_to_f16", "kv_hi", "qn_to_f16"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


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


def nvcc(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        print(r.stdout + r.stderr)
        raise SystemExit("build_ref: nvcc failed")


def build_quant(ref):
    inc = os.path.join(OUT, "ref_cut.inc")
    with open(inc, "w") as f:
        f.write(cut(open(os.path.join(ref, "qwen38_mk.cu"), encoding="utf-8").read(), NAMES))
    so = os.path.join(OUT, "libref_witness.so")
    # the reference's own flags for device code: -O3 -std=c++17, default -fmad (its Makefile:3-13)
    try:
        nvcc(["nvcc", "-O3", "-std=c++17"] + ARCH + ["-Xcompiler", "-fPIC", "-shared", "-I", OUT, "-o", so,
              os.path.join(HERE, "ref_witness.cu")])
    finally:
        os.remove(inc)  # only the binary stays (and only under the git-ignored oracle/_ref)
    print("build_ref: built", so)


def build_attn(ref):
    gen = os.path.join(ref, "bench", "kvattn_gen.py")
    if not os.path.exists(gen):
        print("build_ref: %s is missing: attention witness not built" % gen)
        return
    inc = os.path.join(OUT, "ref_attn_cut.inc")
    subprocess.run([sys.executable, gen, ref, "WORK", inc], check=True, capture_output=True)
    so = os.path.join(OUT, "libref_attn_witness.so")
    # the flags of the reference's own recipe for these kernels (bench/kvattn_bench.cu:5), for sm_100a
    try:
        nvcc(["nvcc", "-O3", "-std=c++17"] + ARCH + ["-Xptxas=-dlcm=cg", "-Xcompiler", "-fPIC", "-shared", "-I", ref, "-I",
              os.path.join(ref, "bench", "stub"), "-I", OUT, "-o", so, os.path.join(HERE, "ref_attn_witness.cu")])
    finally:
        os.remove(inc)
    print("build_ref: built", so)


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MK_REFERENCE_ROOT", "")
    if not ref or not os.path.exists(os.path.join(ref, "qwen38_mk.cu")):
        print("build_ref: no reference tree given (argument or MK_REFERENCE_ROOT): witnesses not built")
        return 0
    os.makedirs(OUT, exist_ok=True)
    build_quant(ref)
    if "--quant-only" not in sys.argv:
        build_attn(ref)
    return 0


if __name__ == "__main__":
    sys.exit(main())
