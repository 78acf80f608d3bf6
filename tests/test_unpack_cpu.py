"""CPU check of the kernels' integer unpackers (csrc/kv_unpack.h is host + device code): builds tests/unpack_check.cpp with g++
and runs it."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_unpackers_decode_every_format(tmp_path):
    exe = str(tmp_path / "unpack_check")
    src = os.path.join(ROOT, "tests", "unpack_check.cpp")
    inc = os.path.join(ROOT, "qwen38-megakernel_b200", "csrc")
    subprocess.run(["g++", "-O2", "-std=c++17", "-I", inc, "-o", exe, src], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
