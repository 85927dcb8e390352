"""The C++ host mirror of the backend interface (include/infr_cuda.hpp): it compiles against the
built library on any machine, and on a B200 a C++ program drives a layer through it and agrees
with the CPU oracle."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "host_mirror_check.cpp")


def build_checker(tmp_path):
    from moe4all_b200 import build
    lib = build.build()
    libdir = os.path.dirname(lib)
    exe = str(tmp_path / "host_mirror_check")
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), SRC, "-o", exe,
           "-L", libdir, "-linfr_cuda", "-Wl,-rpath," + libdir]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_cpp_mirror_compiles_and_links(tmp_path):
    exe = build_checker(tmp_path)
    assert os.path.exists(exe)


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 3])
def test_cpp_mirror_layer_matches_oracle(tmp_path, rows):
    from moe4all_b200 import synth
    from helpers import assert_close, near_tie_rows, oracle_layer

    exe = build_checker(tmp_path)
    ne, E, k, nff = 512, 16, 4, 256
    L = synth.make_layer(41, ne, E, nff, sh_ff=nff, router_std=0.05)
    x = synth.activations(5 + rows, rows, ne)
    inp, out = tmp_path / "layer.bin", tmp_path / "out.bin"
    with open(inp, "wb") as f:
        np.array([rows, ne, E, k, nff, nff, 1, 0], np.int32).tofile(f)
        for a in (L.router.astype(np.float32), L.gate, L.up, L.down, L.sh_gate, L.sh_up, L.sh_down,
                  L.sh_gate_inp.astype(np.float32), np.ascontiguousarray(x, np.float32)):
            np.ascontiguousarray(a).tofile(f)
    r = subprocess.run([exe, str(inp), str(out)], capture_output=True, text=True)
    assert r.returncode == 0 and "OK" in r.stdout, r.stderr + r.stdout
    raw = np.fromfile(out, np.uint8)
    dst = raw[: rows * ne * 4].view(np.float32).reshape(rows, ne)
    ids = raw[rows * ne * 4: rows * ne * 4 + rows * k * 4].view(np.int32).reshape(rows, k)
    ref = oracle_layer(L, x, k)
    ties = set(near_tie_rows(ref, k).tolist())
    for i in range(rows):
        if i not in ties:
            assert ids[i].tolist() == ref.ids[i].tolist()
    assert_close(dst, ref.dst)
