"""CPU-side checks: the oracle reproduces the committed golden vectors, the C-ABI library loads
and exports every symbol the header declares, and descriptors are validated on the host."""
import ctypes
import importlib.util
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden", "moe_cases.npz")


def load_make_golden():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(ROOT, "tests", "golden", "make_golden.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_oracle_matches_golden():
    mg = load_make_golden()
    gold = np.load(GOLDEN)
    for name, c in mg.cases().items():
        _, _, res = mg.run_case(*c)
        assert np.array_equal(res.ids, gold[name + ".ids"]), name
        assert np.array_equal(res.wts.view(np.uint32), gold[name + ".wts"].view(np.uint32)), name
        assert np.array_equal(res.dst.view(np.uint32), gold[name + ".dst"].view(np.uint32)), name
        assert np.abs(gold[name + ".dst"]).max() > 0


def header_symbols():
    text = open(os.path.join(ROOT, "include", "infr_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(infr_cuda_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from moe4all_b200 import build
    from moe4all_b200.backend import EXPORTS

    lib = ctypes.CDLL(build.build())
    declared = header_symbols()
    assert declared, "no declarations parsed from include/infr_cuda.h"
    for sym in declared:
        assert hasattr(lib, sym), f"{sym} is declared in include/infr_cuda.h but not exported"
    assert sorted(EXPORTS) == declared, "backend.EXPORTS and the header disagree"
    assert lib.infr_cuda_name is not None


def test_create_fails_loudly_without_a_gpu():
    import torch
    from moe4all_b200 import BackendError, CudaBackend

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(BackendError):
        CudaBackend(0)


def test_missing_library_is_an_error_not_a_fallback(tmp_path):
    from moe4all_b200 import BackendError, load_library

    with pytest.raises(BackendError):
        load_library(str(tmp_path / "libinfr_cuda.so"))


def test_dtype_geometry():
    # crates/infr-core/src/decode_spec.rs:327, 331
    from moe4all_b200 import DType

    assert DType.Q4K.row_bytes(2048) == 1152 and DType.Q6K.row_bytes(512) == 420
    assert DType.F32.row_bytes(7) == 28
    with pytest.raises(ValueError):
        DType.Q4K.row_bytes(100)


def test_reference_arm_prints_the_contract_line():
    # `bench.py --impl reference` runs the CPU restatement only (no GPU, no CUDA library): one JSON line with the
    # keys the driver reads; the prefill workload's bounded sample keeps this to a second or two
    import json
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--workload", "prefill", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=300, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "moe_prefill_routed_tflops" and line["unit"] == "TFLOP/s"
    assert line["value"] > 0 and line["higher_is_better"] is True and line["vs_baseline"] is None and line["data"] == "synthetic"
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
