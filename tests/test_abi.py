"""The C-ABI shared library: it loads without a GPU, exports every symbol the header declares, and rejects
malformed arguments with status codes (no compute call is made here)."""
import ctypes
import os
import re

import pytest
import torch

import scattermoe_b200
from scattermoe_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "scattermoe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(smoe_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), "library does not export %s" % n
        assert n in _lib.SIGNATURES, "no ctypes signature for %s" % n
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_library_location():
    assert _lib.load().smoe_version() == _lib.ABI_VERSION == 4
    path = scattermoe_b200.library_path()
    assert os.path.dirname(path) == os.path.join(ROOT, "scattermoe_b200"), "the library must live in-tree"


def test_argument_validation_needs_no_device():
    lib = _lib.load()
    # E out of range, negative R: rejected before any CUDA call
    assert lib.smoe_sort_count(None, 4, 0, None, None, None, None, 0, None) == _lib.SMOE_ERR_BAD_ARG
    assert "E=0" in _lib.last_error()
    assert lib.smoe_sort_count(None, -1, 8, None, None, None, None, 0, None) == _lib.SMOE_ERR_BAD_ARG
    assert lib.smoe_sort_count_workspace_bytes(32768, 8) >= 16 * 8 * 4
    assert lib.smoe_offsets_from_sorted(None, -5, 8, None, None) == _lib.SMOE_ERR_BAD_ARG
    # unknown dtype
    rc = lib.smoe_group(256, 4, 4, 1, 256, None, 1, 256, 4, 1, 4, 4, 7, None)   # never dereferenced
    assert rc == _lib.SMOE_ERR_BAD_ARG and "dtype" in _lib.last_error()
    # index length must be rows * fan_out (reference assertion, ops.py:124-125)
    rc = lib.smoe_scatter2scatter(None, 3, 8, 1, None, 0, 0, 0, None, 0, 0, None, 8, 1, None, None, None,
                                  7, 8, 8, 2, 2, 0, 0, 0, 0, None, None)
    assert rc == _lib.SMOE_ERR_BAD_ARG
    with pytest.raises(AssertionError):
        _lib.check(rc, "smoe_scatter2scatter")


def test_cpu_tensors_fail_loudly():
    """No CPU fallback: handing CPU tensors to any op is an error, not a slow path."""
    from scattermoe_b200.kernels import ops
    idx = torch.zeros(4, dtype=torch.int64)
    with pytest.raises(RuntimeError, match="no CPU path"):
        scattermoe_b200.flatten_sort_count(torch.zeros(2, 2, dtype=torch.int64), 4)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.scatter2scatter(torch.zeros(4, 8), torch.zeros(2, 8, 8), idx, idx, 1)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.group(torch.zeros(4, 8), idx)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.group_bwd_W(torch.zeros(4, 8), torch.zeros(4, 8), torch.zeros(2, dtype=torch.int64), 2)


def test_missing_library_is_an_import_error(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib._build, "LIB_PATH", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib._build, "build", lambda *a, **k: (_ for _ in ()).throw(RuntimeError("nvcc not found")))
    with pytest.raises(ImportError, match="no fallback"):
        _lib.load()


def test_reference_arm_of_the_benchmark_runs_on_the_host():
    """`bench.py --impl reference` is the CPU arm: no GPU needed, one JSON line with the contract's keys."""
    import json
    import subprocess
    import sys
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--config", "tiny",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] == "port" and line["value"] > 0
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0


def test_python_constants_match_the_header():
    """Status codes, dtype codes and flag bits are copied by value into the ctypes binding: they must not drift."""
    import re
    import torch
    from scattermoe_b200 import _lib
    text = open(os.path.join(ROOT, "include", "scattermoe_b200.h")).read()
    enum = {m.group(1): int(m.group(2)) for m in re.finditer(r"\b(SMOE_[A-Z0-9_]+)\s*=\s*(\d+)", text)}
    assert enum["SMOE_OK"] == _lib.SMOE_OK and enum["SMOE_ERR_BAD_ARG"] == _lib.SMOE_ERR_BAD_ARG
    assert enum["SMOE_ERR_UNSUPPORTED"] == _lib.SMOE_ERR_UNSUPPORTED
    for name in ("ALLOW_TF32", "FORCE_SIMT", "FORCE_TC", "GATHER_ROWS"):
        assert enum["SMOE_FLAG_" + name] == getattr(_lib, "FLAG_" + name), name
    assert {torch.float32: enum["SMOE_F32"], torch.bfloat16: enum["SMOE_BF16"], torch.float16: enum["SMOE_F16"]} == _lib.DTYPE_CODE
    flags = [v for k, v in enum.items() if k.startswith("SMOE_FLAG_")]
    assert len(set(flags)) == len(flags) and all(v & (v - 1) == 0 for v in flags), "flags are distinct single bits"
