"""Committed golden vectors (tests/golden/oracle_golden.npz, written by tests/golden/make_golden.py): the oracle must still
reproduce them on any machine, and the CUDA path must reproduce the same states on a GPU."""
import importlib.util
import os

import numpy as np
import pytest

import models as M

HERE = os.path.dirname(os.path.abspath(__file__))


def _maker():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_oracle_reproduces_golden():
    golden = np.load(os.path.join(HERE, "golden", "oracle_golden.npz"))
    fresh = _maker().build()
    assert sorted(golden.files) == sorted(fresh)
    for k in golden.files:
        assert np.array_equal(golden[k], fresh[k]), k


@pytest.mark.gpu
def test_cuda_path_reproduces_golden(T, O):
    golden = np.load(os.path.join(HERE, "golden", "oracle_golden.npz"))
    assert np.array_equal(T.rng_split(42, 8), golden["rng_split_42_8"])
    for name, desc in _maker().cases(T).items():
        prog = T.Program(M.fill(T.Builder(desc["kinds"], desc.get("dtype_order")), desc))
        st = T.ChainState(prog, 12)
        for i, a in enumerate(M.random_states(desc, 12, 7)):
            st.upload(i, a)
        st.run_blocks(0xC0FFEE, 5)
        for i in range(len(desc["free"])):
            assert np.array_equal(st.download(i, np.uint8), golden[f"{name}_state{i}"]), (name, i)
