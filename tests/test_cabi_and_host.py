"""CPU-side checks: the C-ABI library loads and exports exactly what the
header declares, the host layer refuses CPU tensors, argument checks."""
import os
import re

import pytest
import torch

import aussm_b200
from aussm_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "aussm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(aussm_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/aussm_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes table and header disagree"
    assert lib.aussm_b200_version() >= 100


def test_workspace_queries_and_options():
    lib = _lib.load()
    assert lib.aussm_b200_unitary_workspace_bytes(0, 1, 1, 1) == 0
    small = lib.aussm_b200_unitary_workspace_bytes(2, 16, 4, 64)
    assert small >= 2 * 16 * 4 * 64 * 4
    # the window workspace is bounded: it does not grow with the sequence length
    a = lib.aussm_b200_unitary_workspace_bytes(16, 1024, 16, 16384)
    b = lib.aussm_b200_unitary_workspace_bytes(16, 1024, 16, 65536)
    assert a == b and a < 10 * 2**30
    assert lib.aussm_b200_scan_unitary_bwd_workspace_bytes(16, 1024, 16, 16384) == 16 * 1024 * 81 * 4
    assert lib.aussm_b200_set_option(b"no_such_option", 1) != 0
    assert b"unknown option" in lib.aussm_b200_last_error()
    assert lib.aussm_b200_set_option(b"window_steps", 0) == 0


def test_no_cpu_fallback():
    x = torch.zeros(1, 2, 16)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        aussm_b200.ssm_adaptive_interface(x, x, torch.zeros(2, 4, 2), torch.zeros(2, 4),
                                          torch.zeros(4, dtype=torch.complex64), torch.zeros(4, dtype=torch.complex64),
                                          torch.zeros(2), x)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        aussm_b200.scan_unitary(torch.zeros(1, 2, 4, 16), x, x, x, *[torch.zeros(4)] * 4, torch.zeros(2))


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "aussm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), f
                assert "oracle/" not in src, f


def test_meta_kernels():
    with torch.device("meta"):
        u = torch.empty(2, 3, 32)
        outs = torch.ops.extension_cpp.ssm_adaptive_unitary.default(
            u, u, torch.empty(3, 4, 3), torch.empty(3, 4), *[torch.empty(4)] * 4, torch.empty(3), u,
            torch.empty(2, 3, 4), torch.empty(2, 3, 4))
    assert outs[0].shape == (2, 3, 32) and outs[1].shape == (2, 3, 4) and outs[2].shape == (2, 3, 4)


def test_bind_process_to_gpu_cpus_never_raises_and_keeps_the_affinity_without_a_gpu():
    import os

    import aussm_b200
    before = os.sched_getaffinity(0)
    n = aussm_b200.bind_process_to_gpu_cpus("cuda:0")
    try:
        assert isinstance(n, int) and n >= 0
        if n == 0:
            assert os.sched_getaffinity(0) == before
    finally:
        os.sched_setaffinity(0, before)
