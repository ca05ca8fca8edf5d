"""The two multi-sweep kernels that serve queued sweeps of small all-threshold-table programs — the chain-sliced kernel
(four chains of every spin in one CTA's shared memory, no grid barrier) and, for programs too large for that, the
cooperative kernel with a grid barrier per block update — against the oracle and against the launch-per-block path:
same keys, same states, same moment sums, bit for bit."""
import numpy as np
import pytest

import models as M
from test_gpu_parity import assert_states_equal, make_pair, moment_spec, n_blocks_of

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chains", [1, 100, 4100])
def test_run_blocks_uses_one_launch_and_matches_oracle(T, O, chains):
    desc, info = M.ising_random_graph(T, 200, 8, 41)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 3)
    before = gs.launch_counts()
    gs.run_blocks(99, 25)
    os_.run_blocks(99, 25)
    after = gs.launch_counts()
    assert after[1] - before[1] == 1 and after[0] == before[0]
    assert_states_equal(gs, os_, n_blocks_of(desc))


def test_same_states_as_one_launch_per_block(T, O):
    """run_blocks (queued) against sample_blocks called once per sweep key (never queued)."""
    desc, info = M.ising_lattice(T, 12, True, 5)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 48, 8)
    gs2 = T.ChainState(prog, 48)
    for b in range(n_blocks_of(desc)):
        gs2.copy_block_from(gs, b)
    gs.run_blocks(1234, 40)
    for k in T.rng_split(1234, 40):
        gs2.sample_blocks(int(k))
    assert gs.launch_counts()[1] == 1 and gs2.launch_counts()[1] == 0
    for b in range(n_blocks_of(desc)):
        assert np.array_equal(gs.download(b), gs2.download(b))


def test_schedule_longer_than_one_plan(T, O):
    """More block updates than one launch of the chain-sliced kernel carries (16384): the plan is cut into consecutive launches."""
    desc, info = M.ising_lattice(T, 6, True, 9)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 16, 4)
    spec = moment_spec(desc, info)
    gm, om = T.Moments(prog, spec, True), O.Moments(ob, spec, True)
    gs.sample_with_observation(5, 700, 4001, 2, moments=gm)  # (700 + 4000 * 2) sweeps x 2 blocks = 17400 block updates
    os_.sample_with_observation(5, 700, 4001, 2, moments=om)
    assert gs.launch_counts() == (0, 2)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    for t in range(2):
        a, na = gm.read(t)
        b, nb = om.read(t)
        assert na == nb == 4001 * 16 and np.array_equal(a, b)


def big_lattice(T):
    """246 x 246 torus: 60516 spins, more than one CTA's shared memory holds, so queued sweeps take the cooperative kernel."""
    return M.ising_lattice(T, 246, True, 17)


def test_cooperative_kernel_matches_oracle_with_moments(T, O):
    desc, info = big_lattice(T)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 20, 12)
    spec = moment_spec(desc, info)
    gm, om = T.Moments(prog, spec, True), O.Moments(ob, spec, True)
    gs.sample_with_observation(8, 2, 4, 2, moments=gm)
    os_.sample_with_observation(8, 2, 4, 2, moments=om)
    assert gs.launch_counts() == (0, 1)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    for t in range(2):
        a, na = gm.read(t)
        b, nb = om.read(t)
        assert na == nb == 4 * 20 and np.array_equal(a, b)


def test_cooperative_plan_is_cut_at_4096_block_updates(T, O):
    desc, info = big_lattice(T)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 16, 5)
    gs2 = T.ChainState(prog, 16)
    for b in range(n_blocks_of(desc)):
        gs2.copy_block_from(gs, b)
    gs.run_blocks(321, 2100)  # 4200 block updates
    for k in T.rng_split(321, 2100):
        gs2.sample_blocks(int(k))
    assert gs.launch_counts() == (0, 2) and gs2.launch_counts() == (4200, 0)
    for b in range(n_blocks_of(desc)):
        assert np.array_equal(gs.download(b), gs2.download(b))


def test_observer_with_rows_the_kernel_cannot_own_falls_back_per_sample(T, O):
    """A triple row needs the separate observer kernel: the sweeps between observations still ride the persistent
    kernel, the observed sweep is launched block by block."""
    desc, info = M.ising_random_graph(T, 96, 4, 77)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 20, 6)
    spec = [[(i,) for i in range(info["n"])], [(0, 1, 2)]]
    gm, om = T.Moments(prog, spec, True), O.Moments(ob, spec, True)
    gs.sample_with_observation(11, 4, 3, 5, moments=gm)
    os_.sample_with_observation(11, 4, 3, 5, moments=om)
    blocks, persistent = gs.launch_counts()
    assert persistent >= 1 and blocks == 3 * len(desc["free"])
    assert_states_equal(gs, os_, n_blocks_of(desc))
    for t in range(2):
        assert np.array_equal(gm.read(t)[0], om.read(t)[0])


def test_state_observer_and_packed_stream_see_flushed_states(T, O):
    desc, info = M.ising_lattice(T, 8, False, 13)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 40, 2)
    g = gs.sample_with_observation(21, 3, 6, 4, obs_blocks=[0, 1])
    o = os_.sample_with_observation(21, 3, 6, 4, obs_blocks=[0, 1])
    assert np.array_equal(np.asarray(g), np.asarray(o))
    assert gs.launch_counts()[1] >= 1
