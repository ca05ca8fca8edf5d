"""Device-side index compilation and colouring against the host compiler and the oracle: every table byte for byte, every
colour equal.  The host compiler is itself pinned to the oracle and to the reference's known answers in test_index_tables."""
import numpy as np
import pytest

import models as M
from test_index_tables import assert_same_tables

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx(T):
    return T.Context(0)


def _host_and_device(T, desc, ctx):
    host = M.fill(T.Builder(desc["kinds"], desc.get("dtype_order")), desc)
    dev = M.fill(T.Builder(desc["kinds"], desc.get("dtype_order")), desc)  # compiled on the host by fill() ...
    dev.compile(ctx)  # ... and again on the device, which replaces every table
    return host, dev


@pytest.mark.parametrize("seed", range(4))
def test_mixed_models(T, O, ctx, seed):
    desc, _ = M.mixed_model(seed, with_clamped=bool(seed % 2), superblock_pair=bool(seed % 3 == 0), two_cat_tails=True)
    host, dev = _host_and_device(T, desc, ctx)
    assert_same_tables(dev, host)
    assert_same_tables(dev, M.fill(O.Model(desc["kinds"], desc.get("dtype_order")), desc))
    for node in range(len(desc["kinds"])):
        assert dev.node_location(node) == host.node_location(node)


def test_lattice_graph_and_potts(T, ctx):
    for desc in (M.ising_lattice(T, 6, True, 3)[0], M.ising_lattice(T, 7, False, 4)[0], M.ising_random_graph(T, 300, 8, 5)[0],
                 M.ising_sparse_random_graph(T, 500, 6, 6)[0], M.potts_lattice(T, 4, 5, 7)[0]):
        assert_same_tables(*_host_and_device(T, desc, ctx))


def test_heads_outside_free_blocks_and_ragged_slot_counts(T, ctx):
    """A star (one node is head of many rows, the rest of one) plus clamped heads: padded slots and ignored rows."""
    n = 40
    kinds = np.zeros(n, np.int32)
    hub_edges = np.stack([np.zeros(30, np.int64), np.arange(1, 31)], 1)
    extra = np.array([[31, 32], [33, 34], [35, 0], [36, 37]], np.int64)  # 36, 37 are clamped; 38, 39 are in no edge
    edges = np.concatenate([hub_edges, extra])
    rng = np.random.default_rng(1)
    desc = dict(kinds=kinds, free=[(np.array([0, 32, 34, 38]), 0), (np.concatenate([np.arange(1, 32), [33, 35, 39]]), 1)],
                clamped=[np.array([36, 37])],
                ops=[("add_ising", np.arange(n), rng.normal(size=n).astype(np.float32), edges, rng.normal(size=len(edges)).astype(np.float32), 0.7)])
    host, dev = _host_and_device(T, desc, ctx)
    assert_same_tables(dev, host)
    assert max(t["k"] for t in dev.tables(0)) == 31  # the hub: 30 spokes + the edge from 35


def test_degenerate_programs(T, ctx):
    """Biases only (no tails anywhere), a block no interaction group touches, and no interaction groups at all."""
    kinds = np.zeros(10, np.int32)
    for ops in ([("add_ising", np.arange(6), np.linspace(-1, 1, 6).astype(np.float32), np.zeros((0, 2), np.int64), np.zeros(0, np.float32), 1.0)], []):
        desc = dict(kinds=kinds, free=[(np.arange(0, 3), 0), (np.arange(3, 6), 1), (np.arange(6, 10), 2)], ops=ops)
        host, dev = _host_and_device(T, desc, ctx)
        assert_same_tables(dev, host)
        assert dev.tables(2) == []


def test_program_from_device_tables_samples_like_the_oracle(T, O, ctx):
    desc, _ = M.ising_random_graph(T, 200, 6, 11)
    bld = M.fill(T.Builder(desc["kinds"]), desc)
    bld.compile(ctx)
    om = M.fill(O.Model(desc["kinds"]), desc)
    st, ost = T.ChainState(T.Program(bld, ctx=ctx), 16), O.State(om, 16)
    for i, a in enumerate(M.random_states(desc, 16, 3)):
        st.upload(i, a)
        ost.set_block(i, a.astype(np.float32))
    st.run_blocks(77, 4)
    ost.run_blocks(77, 4)
    for i in range(len(desc["free"])):
        assert np.array_equal(st.download(i, np.uint8), ost.get_block(i).astype(np.uint8))


def _random_edges(n, m, seed):
    rng = np.random.default_rng(seed)
    return rng.integers(0, n, size=(m, 2)).astype(np.int64)  # duplicates and self-loops included


@pytest.mark.parametrize("n,m,seed", [(1, 0, 0), (50, 0, 1), (64, 400, 2), (5000, 20000, 3), (2000, 150000, 4)])
def test_greedy_colouring_matches_host(T, ctx, n, m, seed):
    from thrml_rs_b200 import engine
    edges = _random_edges(n, m, seed)
    host, n_host = engine.greedy_coloring_arrays(n, edges)
    dev, n_dev = engine.greedy_coloring_arrays(n, edges, ctx)
    assert np.array_equal(host, dev)
    assert n_host == n_dev


def test_greedy_colouring_more_than_64_colours_and_lattice(T, ctx):
    from thrml_rs_b200 import engine
    n = 80  # complete graph: colour(v) = v, beyond the 64-bit mask
    edges = np.array([(a, b) for a in range(n) for b in range(a + 1, n)], np.int64)
    dev, n_dev = engine.greedy_coloring_arrays(n, edges, ctx)
    assert np.array_equal(dev, np.arange(n)) and n_dev == n
    side, ledges, chequer = engine.lattice_edges(32, True)
    dev, n_dev = engine.greedy_coloring_arrays(side * side, ledges, ctx)
    assert np.array_equal(dev, engine.greedy_coloring_arrays(side * side, ledges)[0])
    assert n_dev == 2 and np.array_equal(dev, chequer)


def test_bad_arguments(T, ctx):
    from thrml_rs_b200 import engine
    with pytest.raises(T.ThrmlError):
        engine.greedy_coloring_arrays(4, np.array([[0, 9]]), ctx)
