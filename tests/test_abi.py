"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "thrml_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(thrml_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(T):
    from thrml_rs_b200 import _ffi
    lib = _ffi.lib()
    names = header_symbols()
    assert len(names) >= 45
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/thrml_b200.h but not exported"
    assert sorted(_ffi._SIGNATURES) == names


def test_host_only_entry_points_work_without_a_gpu(T, O):
    assert np.array_equal(T.rng_split(42, 7), O.rng_split(42, 7))
    assert list(T.rng_split(5, 1)) == [5] and len(T.rng_split(5, 0)) == 0
    for side, torus in [(4, False), (4, True), (5, True), (2, True), (32, True)]:
        a, b = T.lattice_edges(side, torus), O.lattice_edges(side, torus)
        assert a[0] == b[0] and np.array_equal(a[1], b[1]) and np.array_equal(a[2], b[2])
    rng = np.random.default_rng(0)
    e = rng.integers(0, 200, (700, 2))
    e = e[e[:, 0] != e[:, 1]]
    ca, na = T.greedy_coloring_arrays(200, e)
    cb, nb = O.greedy_coloring(200, e)
    assert na == nb and np.array_equal(ca, cb)
    assert all(ca[a] != ca[b] for a, b in e)
    assert b"thrml_b200" in T.lib().thrml_version()


def test_device_calls_fail_loudly_without_a_gpu(T):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(T.ThrmlError) as ei:
        T.Context(0)
    assert ei.value.code == -3  # THRML_ERR_CUDA: no CPU fallback


def test_product_does_not_touch_the_oracle():
    pkg = os.path.join(ROOT, "thrml-rs_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cpp", ".h", ".cuh")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"
