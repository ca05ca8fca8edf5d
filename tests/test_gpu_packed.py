"""Bit-packed state format (THRML_OPT_STATE_FORMAT = 1): sweeps of threshold-table programs on the packed mirror give the
oracle's states and moment sums bit for bit, whatever is interleaved with them on the byte copy."""
import numpy as np
import pytest

import models as M

pytestmark = pytest.mark.gpu


def _pair(T, O, desc, chains, offset=0, seed=5):
    gb, ob = M.build_both(T, O, desc)
    prog = T.Program(gb)
    prog.set_option(T.OPT_STATE_FORMAT, 1)
    assert all(prog.block_kernel(b) == 1 for b in range(len(desc["free"])))
    gs, os_ = T.ChainState(prog, chains, offset), O.State(ob, chains, offset)
    for i, a in enumerate(M.random_states(desc, chains, seed)):
        gs.upload(i, a)
        os_.set_block(i, a.astype(np.float32))
    return prog, gs, os_, gb, ob


def _same(gs, os_, n):
    for i in range(n):
        assert np.array_equal(gs.download(i), os_.get_block(i)), i


@pytest.mark.parametrize("chains,offset", [(1024, 0), (1040, 0), (1009, 48), (2100, 4096)])
@pytest.mark.parametrize("case", ["lattice", "graph8"])
def test_packed_sweeps_match_the_oracle(T, O, case, chains, offset):
    desc = {"lattice": M.ising_lattice(T, 8, True, 1)[0], "graph8": M.ising_random_graph(T, 300, 8, 2)[0]}[case]
    n = len(desc["free"]) + len(desc.get("clamped", []))
    prog, gs, os_, gb, ob = _pair(T, O, desc, chains, offset)
    gs.run_blocks(321, 3)
    os_.run_blocks(321, 3)
    assert gs.launch_counts()[1] == 0  # block launches, not the queued kernels
    _same(gs, os_, n)
    # byte-side writes between packed sweeps: one block re-uploaded, then more sweeps through sample_blocks
    fresh = M.random_states(desc, chains, 77)[0]
    gs.upload(0, fresh)
    os_.set_block(0, fresh.astype(np.float32))
    for k in (5, 6):
        gs.sample_blocks(k)
        os_.sample_blocks(k)
    _same(gs, os_, n)


def test_packed_observer_and_format_switch(T, O):
    desc, info = M.ising_random_graph(T, 300, 8, 3)
    chains = 1056
    prog, gs, os_, gb, ob = _pair(T, O, desc, chains)
    edges = info["edges"]
    nn = len(desc["kinds"])
    spec = (np.array([nn, len(edges)], np.int64), np.concatenate([np.arange(nn + 1), nn + 2 * np.arange(1, len(edges) + 1)]).astype(np.int64),
            np.concatenate([np.arange(nn), edges.ravel()]).astype(np.int64))
    gm, om = T.Moments.from_arrays(prog, *spec), O.Moments.from_arrays(ob, *spec)
    gs.sample_with_observation(11, 2, 4, 2, moments=gm)
    os_.sample_with_observation(11, 2, 4, 2, moments=om)
    for t in (0, 1):
        assert np.array_equal(gm.read(t)[0], om.read(t)[0]), t
    assert gm.fused_info()[1] == 0  # every row is owned by an update kernel
    _same(gs, os_, len(desc["free"]))
    # back to the byte format in mid-run, then packed again: the two copies never diverge
    prog.set_option(T.OPT_STATE_FORMAT, 0)
    gs.sample_with_observation(12, 1, 3, 1, moments=gm)
    os_.sample_with_observation(12, 1, 3, 1, moments=om)
    prog.set_option(T.OPT_STATE_FORMAT, 1)
    gs.hinton_init([0], np.zeros(len(desc["free"][0][0]), np.float32), 1.0, 9)
    os_.hinton_init([0], np.zeros(len(desc["free"][0][0]), np.float32), 1.0, 9)
    gs.sample_with_observation(13, 0, 2, 3, moments=gm)
    os_.sample_with_observation(13, 0, 2, 3, moments=om)
    for t in (0, 1):
        assert np.array_equal(gm.read(t)[0], om.read(t)[0]), t
        assert gm.read(t)[1] == om.read(t)[1]
    _same(gs, os_, len(desc["free"]))


def test_packed_sweeps_with_a_clamped_block(T, O):
    """The last colour of the graph is clamped: its rows sit behind the free blocks in the spin class and are read, never written."""
    desc = dict(M.ising_random_graph(T, 300, 8, 6)[0])
    free = list(desc["free"])
    desc["clamped"] = [free.pop()[0]]
    desc["free"] = free
    n = len(desc["free"]) + 1
    prog, gs, os_, gb, ob = _pair(T, O, desc, 1040)
    gs.run_blocks(17, 4)
    os_.run_blocks(17, 4)
    _same(gs, os_, n)


def test_packed_route_is_declined_where_it_does_not_apply(T, O):
    """Fewer than 1009 chains, or a block on another kernel: the option is accepted and the byte kernels run."""
    desc = M.ising_random_graph(T, 200, 12, 4)[0]  # sequential-sum blocks
    gb, ob = M.build_both(T, O, desc)
    prog = T.Program(gb)
    prog.set_option(T.OPT_STATE_FORMAT, 1)
    gs, os_ = T.ChainState(prog, 1040), O.State(ob, 1040)
    for i, a in enumerate(M.random_states(desc, 1040, 5)):
        gs.upload(i, a)
        os_.set_block(i, a.astype(np.float32))
    gs.run_blocks(3, 2)
    os_.run_blocks(3, 2)
    _same(gs, os_, len(desc["free"]))
    with pytest.raises(T.ThrmlError):
        prog.set_option(T.OPT_STATE_FORMAT, 2)
