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


@pytest.mark.gpu
def test_implicit_engines_reproduce_golden(T):
    """The implicit lattice and Potts engines under their own key -> noise mappings against the frozen oracle states."""
    from thrml_rs_b200 import lattice, potts
    golden = np.load(os.path.join(HERE, "golden", "oracle_golden.npz"))
    mk = _maker()
    desc, info = mk.torus_case()
    H, W, chains = info["H"], info["W"], 8
    init = M.random_states(desc, chains, 7)
    spins = np.zeros((chains, H * W), np.uint8)
    for blk, a in zip(info["blocks"], init):
        spins[:, blk] = a
    for noise in (lattice.NOISE_PACKED, lattice.NOISE_PACKED_TABLE):
        lat = lattice.StripedLattice(H, W, info["J"], info["b"], info["beta"], chains, n_stripes=2, noise=noise)
        lat.upload(spins.reshape(chains, H, W))
        lat.run_blocks(0xC0FFEE, 3)
        got = lat.download().reshape(chains, H * W)
        for i, blk in enumerate(info["blocks"]):
            assert np.array_equal(got[:, blk], golden[f"torus_spin_noise1_state{i}"]), (noise, i)
    desc, info = mk.potts_cube_case()
    side, chains = info["side"], 12
    init = M.random_states(desc, chains, 7)
    cats = np.zeros((chains, side ** 3), np.uint8)
    for blk, a in zip(info["blocks"], init):
        cats[:, blk] = a
    pl = potts.PottsLattice(side, side, side, info["K"], info["tables"], info["unary"], info["beta"], chains)
    pl.upload(cats)
    pl.run_blocks(0xC0FFEE, 3)
    got = pl.download()
    for i, blk in enumerate(info["blocks"]):
        assert np.array_equal(got[:, blk], golden[f"cube_cat_noise1_state{i}"]), i
    # SoftmaxConditional on block 0 through the explicit program
    bld = T.Builder(desc["kinds"])
    for i, (nodes, sb) in enumerate(desc["free"]):
        bld.add_free_block(nodes, superblock=sb, sampler=[2, 1][i])
    for op in desc["ops"]:
        getattr(bld, op[0])(*op[1:])
    bld.compile()
    st = T.ChainState(T.Program(bld), chains)
    for i, a in enumerate(init):
        st.upload(i, a)
    st.run_blocks(0xC0FFEE, 3)
    for i in range(2):
        assert np.array_equal(st.download(i, np.uint8), golden[f"cube_softmax_state{i}"]), i
