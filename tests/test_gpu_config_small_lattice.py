"""The 32 x 32 periodic Ising configuration (J = 0.44, biases N(0, 0.1^2), beta = 1, 256 chains, hinton_init, 200 warm-up
sweeps + 800 more, <s_i> and <s_i s_j> over the 2048 edges), run through the reference-shaped API and through the oracle:
the moment sums agree exactly because every state does."""
import numpy as np
import pytest

import models as M

pytestmark = pytest.mark.gpu


def test_32x32_configuration_matches_oracle(T, O):
    desc, info = M.ising_lattice(T, 32, True, 0x5EED0001, J=0.44, bias_sigma=0.1, beta=1.0)
    assert info["n"] == 1024 and len(info["edges"]) == 2048
    gb, ob = M.build_both(T, O, desc)
    prog = T.Program(gb)
    assert [prog.block_kernel(b) for b in range(2)] == [1, 1]
    chains = 256
    gs, os_ = T.ChainState(prog, chains), O.State(ob, chains, threads=8)
    biases = np.concatenate([info["b"][blk] for blk in info["blocks"]])
    gs.hinton_init([0, 1], biases, 1.0, 7)
    os_.hinton_init([0, 1], biases, 1.0, 7)
    spec = [[(i,) for i in range(1024)], [tuple(e) for e in info["edges"]]]
    gm, om = T.Moments(prog, spec, True), O.Moments(ob, spec, True)
    gs.sample_with_observation(2026, 200, 801, 1, moments=gm)
    os_.sample_with_observation(2026, 200, 801, 1, moments=om)
    for b in range(2):
        assert np.array_equal(gs.download(b), os_.get_block(b))
    for t in range(2):
        a, na = gm.read(t)
        w, nw = om.read(t)
        assert na == nw == 801 * chains and np.array_equal(a, w)
    m1 = gm.read(0)[0] / (801 * chains)
    m2 = gm.read(1)[0] / (801 * chains)
    assert np.all(np.abs(m1) <= 1) and 0.55 < m2.mean() < 0.8  # J = 0.44 sits at the critical coupling: strong nearest-neighbour correlation
