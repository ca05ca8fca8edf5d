"""Sizes at the edges of what the interfaces allow: the largest category count a node type can hold (255,
crates/thrml-core/src/node.rs:8-21: n_categories is a u8), global chain ids up to 2^32 - 1 (the noise counter holds the
chain id in 32 bits), one chain, one node, and the argument checks at those edges."""
import numpy as np
import pytest

import models as M
from test_gpu_parity import assert_states_equal, make_pair, n_blocks_of

pytestmark = pytest.mark.gpu


def test_255_categories_match_oracle(T, O):
    desc, info = M.potts_lattice(T, 4, 255, 11, sigma=0.8, bias_sigma=0.5)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 9, 4)
    gs.run_blocks(5, 3)
    os_.run_blocks(5, 3)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    assert gs.download(0).max() > 200  # the upper categories are reachable: 64 Philox calls per node and chain


def test_largest_chain_ids(T, O):
    """The last 48 chains before 2^32: the noise of chain c depends on c alone, wherever the shard starts."""
    desc, info = M.ising_random_graph(T, 150, 8, 9)
    top = (1 << 32) - 48
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 48, 7, chain_offset=top)
    gs.run_blocks(31, 4)
    os_.run_blocks(31, 4)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    # the same chains as the tail of a longer shard
    longer = T.ChainState(prog, 112, top - 64)
    init = M.random_states(desc, 48, 7)
    pad = M.random_states(desc, 64, 8)
    for i in range(len(init)):
        longer.upload(i, np.concatenate([pad[i], init[i]], axis=0))
    longer.run_blocks(31, 4)
    for i in range(len(init)):
        assert np.array_equal(longer.download(i)[64:], gs.download(i))
    with pytest.raises(T.ThrmlError, match="2\\^32"):
        T.ChainState(prog, 64, top)
    with pytest.raises(T.ThrmlError, match="multiple of 16"):
        T.ChainState(prog, 16, 8)


def test_one_node_one_chain(T, O):
    kinds = np.zeros(1, np.int32)
    desc = dict(kinds=kinds, free=[(np.array([0]), 0)], ops=[("add_discrete_factor", [np.array([0])], [], np.array([[[0.3]]], np.float32))])
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 1, 2)
    gs.run_blocks(3, 40)
    os_.run_blocks(3, 40)
    assert_states_equal(gs, os_, 1)
    got = gs.sample_with_observation(9, 0, 50, 1, obs_blocks=[0])
    want = os_.sample_with_observation(9, 0, 50, 1, obs_blocks=[0])
    assert got.shape == (50, 1, 1) and np.array_equal(got, want)
    assert 0.45 < got.mean() < 0.85  # P(s = 1) = sigmoid(0.6) = 0.646
