"""Parity of the CUDA path (through the C ABI) with the CPU oracle on the same seeded inputs.

Bars: index work bit-exact; local fields within 1e-5 relative of the oracle's f64 field (and bit-identical to its f32
field); sampled states bit-exact both with injected noise and with the in-kernel stream — the engine's exp/log are
fixed IEEE sequences, so no |logit - threshold| < 1e-6 escape is needed and none is taken; moment sums exact.
"""
import numpy as np
import pytest

import models as M

pytestmark = pytest.mark.gpu


def make_pair(T, O, desc, chains, seed, chain_offset=0):
    gb, ob = M.build_both(T, O, desc)
    prog = T.Program(gb)
    gs = T.ChainState(prog, chains, chain_offset)
    os_ = O.State(ob, chains, chain_offset)
    init = M.random_states(desc, chains, seed)
    for i, a in enumerate(init):
        gs.upload(i, a)
        os_.set_block(i, a.astype(np.float32))
    return prog, gs, os_, gb, ob


def assert_states_equal(gs, os_, n_blocks):
    for i in range(n_blocks):
        g = gs.download(i)
        o = os_.get_block(i)
        assert np.array_equal(g, o), f"block {i}: {(g != o).sum()} of {g.size} states differ"


def n_blocks_of(desc):
    return len(desc["free"]) + len(desc.get("clamped", []))


def model_cases(T):
    return {
        "lattice": M.ising_lattice(T, 8, True, 1)[0],
        "graph8": M.ising_random_graph(T, 300, 8, 2)[0],
        "graph12": M.ising_random_graph(T, 200, 12, 3)[0],
        "mixed": M.mixed_model(4)[0],
        "mixed_free": M.mixed_model(5, with_clamped=False)[0],
        "mixed_superblock": M.mixed_model(6, superblock_pair=True)[0],
        "potts": M.potts_lattice(T, 6, 5, 7)[0],
    }


CASES = ["lattice", "graph8", "graph12", "mixed", "mixed_free", "mixed_superblock", "potts"]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("chains", [1, 37, 64])
def test_fields(T, O, case, chains):
    desc = model_cases(T)[case]
    prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 11)
    for blk in range(len(desc["free"])):
        g = gs.fields(blk)
        o64, o32 = os_.fields(blk)
        assert np.array_equal(g, o32.reshape(g.shape)), f"block {blk}: f32 fields differ"
        # against the f64 field: 1e-5 relative (the north-star tolerance) wherever the sum does not cancel, and 1e-6 of the
        # summed term magnitudes everywhere (an f32 sum of a dozen terms cannot do better where they cancel)
        terms = sum(np.abs(t["w"]).max(axis=2).__mul__(t["active"]).sum(axis=1) for t in gb.tables(blk))  # [n]
        terms = terms.reshape((1, -1) + (1,) * (g.ndim - 2))
        err = np.abs(g - o64.reshape(g.shape))
        assert np.all(err <= 1e-6 * terms + 1e-30)
        solid = np.abs(o64.reshape(g.shape)) >= 0.01 * terms
        assert np.all(err[solid] <= 1e-5 * np.abs(o64.reshape(g.shape))[solid])


@pytest.mark.parametrize("case", CASES)
def test_noise_injection_states(T, O, case):
    desc = model_cases(T)[case]
    chains, sweeps = 24, 3
    prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 12)
    per_sweep = sum(len(nodes) * max(int(desc["kinds"][nodes[0]]), 1) for nodes, _ in desc["free"]) * chains
    u = np.random.default_rng(5).random(per_sweep * sweeps, dtype=np.float32)
    u = np.clip(u, 1e-7, 1 - 1e-7).astype(np.float32)
    gs.run_blocks(99, sweeps, inj=u)
    os_.run_blocks(99, sweeps, inj=u)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    # one more sweep through sample_blocks
    u1 = u[:per_sweep]
    gs.sample_blocks(7, inj=u1)
    os_.sample_blocks(7, inj=u1)
    assert_states_equal(gs, os_, n_blocks_of(desc))


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("chains", [5, 64, 272])
def test_in_kernel_stream_states(T, O, case, chains):
    desc = model_cases(T)[case]
    prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 13)
    gs.run_blocks(1234, 4)
    os_.run_blocks(1234, 4)
    assert_states_equal(gs, os_, n_blocks_of(desc))


@pytest.mark.parametrize("chains", [130, 1040])
@pytest.mark.parametrize("seed", [21, 22])
def test_general_spin_kernel_on_larger_mixed_models(T, O, seed, chains):
    """Spin blocks with three-spin factors and categorical tails, enough chains for the warp-per-node kernel (several passes
    at 1040 chains, dead lanes at 130)."""
    desc, _ = M.mixed_model(seed, n_spin=90, n_cat=40, K=5, with_clamped=bool(seed % 2))
    prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 17)
    assert prog.block_kernel(0) == 7
    gs.run_blocks(4321, 3)
    os_.run_blocks(4321, 3)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    # the node x four-chain gather kernels on the same program give the same states
    prog.set_option(T.OPT_GATHER_ONLY, 1)
    gg = T.ChainState(prog, chains)
    for i, a in enumerate(M.random_states(desc, chains, 17)):
        gg.upload(i, a)
    gg.run_blocks(4321, 3)
    for i in range(n_blocks_of(desc)):
        assert np.array_equal(gg.download(i), gs.download(i))


@pytest.mark.parametrize("K,chains", [(2, 128), (7, 144), (11, 260), (13, 160), (16, 130), (17, 130), (40, 130)])
def test_categorical_kernels_across_category_counts(T, O, K, chains):
    """Explicit Potts programs on the warp-per-node categorical kernel: every template width, the guard for K below the
    width, the opt-in shared-memory size at K = 16, and K > 16 (register-resident slots, any K) — against the oracle and
    against the gather kernel."""
    desc, _ = M.potts_lattice(T, 6, K, 30 + K)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 19)
    assert all(prog.block_kernel(b) == 5 for b in range(2))
    gs.run_blocks(99, 3)
    os_.run_blocks(99, 3)
    assert_states_equal(gs, os_, 2)
    prog.set_option(T.OPT_GATHER_ONLY, 1)
    gg = T.ChainState(prog, chains)
    for i, a in enumerate(M.random_states(desc, chains, 19)):
        gg.upload(i, a)
    gg.run_blocks(99, 3)
    for i in range(2):
        assert np.array_equal(gg.download(i), gs.download(i))


@pytest.mark.parametrize("K,degree,chains,with_spins", [(4, 12, 130, False), (10, 9, 1040, False), (16, 20, 160, True), (3, 30, 144, True), (16, 30, 132, False)])
def test_many_slot_categorical_kernel(T, O, K, degree, chains, with_spins):
    """Categorical nodes with 10 to 32 active slots (a random regular graph, one table per edge, optionally a spin tail):
    the shared-memory slot kernel against the oracle and against the gather kernel."""
    desc, info = M.potts_random_graph(T, 120, degree, K, 40 + K, with_spins=with_spins)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 23)
    n_cat_blocks = len(info["blocks"])
    assert all(prog.block_kernel(b) == 8 for b in range(n_cat_blocks))
    gs.run_blocks(5, 3)
    os_.run_blocks(5, 3)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    prog.set_option(T.OPT_GATHER_ONLY, 1)
    gg = T.ChainState(prog, chains)
    for i, a in enumerate(M.random_states(desc, chains, 23)):
        gg.upload(i, a)
    gg.run_blocks(5, 3)
    for i in range(n_blocks_of(desc)):
        assert np.array_equal(gg.download(i), gs.download(i))


def test_kernel_selection(T, O):
    cases = model_cases(T)
    prog = T.Program(M.fill(T.Builder(cases["graph8"]["kinds"]), cases["graph8"]))
    assert all(prog.block_kernel(b) == 1 for b in range(len(cases["graph8"]["free"])))
    prog = T.Program(M.fill(T.Builder(cases["graph12"]["kinds"]), cases["graph12"]))
    assert all(prog.block_kernel(b) == 4 for b in range(len(cases["graph12"]["free"])))  # 12 neighbours + a bias: too many for a threshold table
    prog = T.Program(M.fill(T.Builder(cases["mixed"]["kinds"]), cases["mixed"]))
    assert prog.block_kernel(0) == 7  # categorical tails and three-spin factors: the warp-per-node general spin kernel
    prog = T.Program(M.fill(T.Builder(cases["potts"]["kinds"]), cases["potts"]))
    assert all(prog.block_kernel(b) == 5 for b in range(2))  # five active slots per node (8 at most): the register-resident categorical kernel


def test_chain_sharding_is_invisible(T, O):
    """Two states holding chains [0,32) and [32,64) reproduce one state holding [0,64)."""
    desc = model_cases(T)["graph8"]
    gb = M.fill(T.Builder(desc["kinds"]), desc)
    prog = T.Program(gb)
    init = M.random_states(desc, 64, 3)
    full = T.ChainState(prog, 64, 0)
    lo, hi = T.ChainState(prog, 32, 0), T.ChainState(prog, 32, 32)
    for i, a in enumerate(init):
        full.upload(i, a)
        lo.upload(i, a[:32])
        hi.upload(i, a[32:])
    for s in (full, lo, hi):
        s.run_blocks(77, 5)
    for i in range(len(init)):
        f = full.download(i)
        assert np.array_equal(f[:32], lo.download(i)) and np.array_equal(f[32:], hi.download(i))


def test_hinton_init(T, O):
    desc, info = M.ising_lattice(T, 8, True, 21, bias_sigma=1.0, beta=0.7)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 40, 14)
    biases = np.concatenate([info["b"][blk] for blk in info["blocks"]])
    gs.hinton_init([0, 1], biases, 0.7, 5)
    os_.hinton_init([0, 1], biases, 0.7, 5)
    assert_states_equal(gs, os_, 2)
    u = np.random.default_rng(1).random(40 * 64, dtype=np.float32)
    gs.hinton_init([1, 0], np.concatenate([info["b"][info["blocks"][1]], info["b"][info["blocks"][0]]]), 0.7, 5, inj_u=u)
    os_.hinton_init([1, 0], np.concatenate([info["b"][info["blocks"][1]], info["b"][info["blocks"][0]]]), 0.7, 5, inj_u=u)
    assert_states_equal(gs, os_, 2)
    # crates/thrml-models/tests/test_ising.rs:57-98: bias 10 -> (almost) all ones
    gs.hinton_init([0], np.full(32, 10.0, np.float32), 1.0, 9)
    assert gs.download(0).mean() > 0.99
    gs.randomize(3)
    os_.randomize(3)
    assert_states_equal(gs, os_, 2)


def moment_spec(desc, info):
    nodes = list(range(info["n"]))
    return [[(i,) for i in nodes], [tuple(e) for e in info["edges"]]]


@pytest.mark.parametrize("chains", [1, 33, 8100])  # 8100 chains: more than one bit-sliced counter segment per node
def test_moments_and_schedule(T, O, chains):
    desc, info = M.ising_random_graph(T, 120, 6, 31)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 15)
    spec = moment_spec(desc, info)
    gm = T.Moments(prog, spec, True)
    om = O.Moments(ob, spec, True)
    gs.sample_with_observation(2024, 3, 5, 2, moments=gm)
    os_.sample_with_observation(2024, 3, 5, 2, moments=om)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    for t in range(2):
        a, na = gm.read(t)
        b, nb = om.read(t)
        assert na == nb == 5 * chains
        assert np.array_equal(a, b)
    # raw products (no spin transform) and a three-node row
    spec2 = [[(0, 1, 2), (5,), (7, 9)]]
    gm2, om2 = T.Moments(prog, spec2, False), O.Moments(ob, spec2, False)
    gm2.observe(gs)
    om2.observe(os_)
    assert np.array_equal(gm2.read(0)[0], om2.read(0)[0])
    gm.reset()
    assert gm.read(0)[0].sum() == 0 and gm.read(0)[1] == 0


def test_fused_moments_with_leftover_rows(T, O):
    """Rows the update kernels accumulate themselves (single spins, neighbour pairs) mixed with rows they cannot:
    clamped nodes, pairs of clamped nodes, non-neighbours, a triple, repeated rows."""
    desc, info = M.ising_random_graph(T, 160, 8, 61)
    # turn the last block into a clamped block
    clamp_nodes = desc["free"][-1][0]
    desc = dict(desc, free=desc["free"][:-1], clamped=[clamp_nodes])
    edges = [tuple(e) for e in info["edges"]]
    spec = [[(i,) for i in range(info["n"])] + [(3,), (3,)],
            edges + edges[:5] + [(0, 1), (int(clamp_nodes[0]), int(clamp_nodes[-1])), (7, 7)],
            [(0, 5, 9), (2,), edges[0]]]
    for chains, sched in [(33, (2, 4, 3)), (16, (0, 3, 1)), (5, (1, 1, 1))]:
        prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 19)
        gm, om = T.Moments(prog, spec, True), O.Moments(ob, spec, True)
        gs.sample_with_observation(77, *sched, moments=gm)
        os_.sample_with_observation(77, *sched, moments=om)
        assert_states_equal(gs, os_, n_blocks_of(desc))
        for t in range(3):
            a, na = gm.read(t)
            b, nb = om.read(t)
            assert na == nb and np.array_equal(a, b), (chains, sched, t, int((a != b).sum()))


def test_state_observer_schedule(T, O):
    desc = model_cases(T)["mixed"]
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 9, 16)
    for sched in [(2, 4, 3), (0, 1, 5), (4, 0, 1), (0, 3, 0)]:
        g = gs.sample_with_observation(31, *sched, obs_blocks=[2, 0, 3])
        o = os_.sample_with_observation(31, *sched, obs_blocks=[2, 0, 3])
        assert g.shape == o.shape and np.array_equal(g, o)
        assert_states_equal(gs, os_, n_blocks_of(desc))


def test_marginals(T, O):
    desc, info = M.potts_lattice(T, 6, 5, 41)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 50, 17)
    mg = T.Moments.marginals(prog, [0, 1], 5)
    want = np.zeros((36, 5), dtype=np.int64)
    for _ in range(3):
        gs.run_blocks(8, 1)
        os_.run_blocks(8, 1)
        mg.observe(gs)
        st = np.concatenate([os_.get_block(0), os_.get_block(1)], axis=1).astype(np.int64)  # [chains, node]
        for c in range(5):
            want[:, c] += (st == c).sum(axis=0)
    got, n_obs = mg.read(0)
    assert n_obs == 150 and np.array_equal(got.reshape(36, 5), want)


def test_update_weights_reaches_the_kernels(T, O):
    desc, info = M.ising_random_graph(T, 150, 8, 51)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 32, 18)
    J2 = (info["J"] * -1.5).astype(np.float32)
    desc2 = dict(desc, ops=[("add_ising", np.arange(info["n"]), info["b"], info["edges"], J2, info["beta"])])
    gb2, ob2 = M.build_both(T, O, desc2)
    for blk in range(len(desc["free"])):
        prog.update_weights(blk, 1, gb2.tables(blk)[1]["w"].ravel())
    os2 = O.State(ob2, 32)
    for i in range(n_blocks_of(desc)):
        os2.set_block(i, os_.get_block(i))
    gs.run_blocks(5, 3)
    os2.run_blocks(5, 3)
    assert_states_equal(gs, os2, n_blocks_of(desc))


def test_boltzmann_moments_within_4_sigma(T):
    """Exhaustive enumeration of a 3x4 open lattice vs long-run GPU moments: 4 sigma of the Monte-Carlo standard error
    (independent chains, so the error of a chain-average is the across-chain standard deviation / sqrt(chains))."""
    rng = np.random.default_rng(3)
    rows, cols = 3, 4
    n = rows * cols
    edges = np.array([(r * cols + c, r * cols + c + 1) for r in range(rows) for c in range(cols - 1)] + [(r * cols + c, (r + 1) * cols + c) for r in range(rows - 1) for c in range(cols)])
    b = rng.normal(0, 0.3, n).astype(np.float32)
    J = rng.normal(0, 0.5, len(edges)).astype(np.float32)
    colour = np.array([(i // cols + i % cols) % 2 for i in range(n)])
    bld = T.Builder(np.zeros(n, np.int32))
    for c in (0, 1):
        bld.add_free_block(np.flatnonzero(colour == c))
    bld.add_ising(np.arange(n), b, edges, J, 1.0)
    bld.compile()
    prog = T.Program(bld)
    s = np.array([[1 if (cfg >> i) & 1 else -1 for i in range(n)] for cfg in range(1 << n)], dtype=np.float64)
    energy = -(s @ b.astype(np.float64) + ((s[:, edges[:, 0]] * s[:, edges[:, 1]]) @ J.astype(np.float64)))
    p = np.exp(-(energy - energy.min()))
    p /= p.sum()
    exact1 = p @ s
    exact2 = p @ (s[:, edges[:, 0]] * s[:, edges[:, 1]])
    chains, samples = 2048, 200
    st = T.ChainState(prog, chains)
    st.randomize(1)
    obs = st.sample_with_observation(17, 100, samples, 2, obs_blocks=[0, 1])  # [samples, node, chain]
    order = np.concatenate([np.flatnonzero(colour == 0), np.flatnonzero(colour == 1)])
    spins = np.zeros((samples, n, chains))
    spins[:, order, :] = 2.0 * obs - 1.0
    per_chain1 = spins.mean(axis=0)  # [node, chain]
    per_chain2 = (spins[:, edges[:, 0], :] * spins[:, edges[:, 1], :]).mean(axis=0)
    for est, exact in ((per_chain1, exact1), (per_chain2, exact2)):
        mean = est.mean(axis=1)
        sem = est.std(axis=1, ddof=1) / np.sqrt(chains)
        assert np.all(np.abs(mean - exact) < 4 * sem + 1e-9), np.max(np.abs(mean - exact) / sem)


def test_packed_state_streaming_matches_byte_observer(T, O):
    desc = model_cases(T)["graph8"]
    for chains in (37, 64, 200):
        prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 23)
        prog2, gs2, _, _, _ = make_pair(T, O, desc, chains, 23)
        blocks = [1, 0, 3]
        bytes_ = gs.sample_with_observation(11, 2, 5, 2, obs_blocks=blocks)  # [samples][node][chain]
        bits = gs2.sample_states_packed(11, 2, 5, 2, blocks)
        assert bits.shape == (5, bytes_.shape[1], (chains + 31) // 32)
        unpacked = ((bits[:, :, :, None] >> np.arange(32, dtype=np.uint32)) & 1).reshape(5, bytes_.shape[1], -1)[:, :, :chains]
        assert np.array_equal(unpacked.astype(np.uint8), bytes_)
        assert np.all(((bits[:, :, :, None] >> np.arange(32, dtype=np.uint32)) & 1).reshape(5, bytes_.shape[1], -1)[:, :, chains:] == 0)


@pytest.mark.parametrize("degree,chains", [(12, 100), (20, 33), (30, 600)])
def test_sequential_sum_kernel_matches_oracle(T, O, degree, chains):
    """Spin blocks with 9 to 32 active slots per node: the warp-per-node kernel that adds the field entry by entry."""
    desc, info = M.ising_random_graph(T, 260, degree, 100 + degree, w_sigma=0.4, bias_sigma=0.3)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 3)
    assert all(prog.block_kernel(b) == 4 for b in range(len(desc["free"])))
    gs.run_blocks(17, 6)
    os_.run_blocks(17, 6)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    # the observer rides in the update kernel for single spins and neighbour pairs; a triple, a repeated row and a
    # non-neighbour pair go to the separate observer kernel
    e0 = tuple(int(x) for x in info["edges"][0])
    spec = moment_spec(desc, info) + [[(0, 5, 9), (2,), e0, (7, 7)]]
    gm, om = T.Moments(prog, spec, True), O.Moments(ob, spec, True)
    fused, other = gm.fused_info()
    assert fused == info["n"] + len(info["edges"]) and other == 4
    gs.sample_with_observation(5, 1, 3, 2, moments=gm)
    os_.sample_with_observation(5, 1, 3, 2, moments=om)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    for t in range(3):
        assert np.array_equal(gm.read(t)[0], om.read(t)[0])
    # new couplings reach the entry lists
    J2 = (info["J"] * -0.7).astype(np.float32)
    desc2 = dict(desc, ops=[("add_ising", np.arange(info["n"]), info["b"], info["edges"], J2, info["beta"])])
    gb2, ob2 = M.build_both(T, O, desc2)
    for blk in range(len(desc["free"])):
        for t, tab in enumerate(gb2.tables(blk)):
            prog.update_weights(blk, t, tab["w"].ravel())
    os2 = O.State(ob2, chains)
    for i in range(n_blocks_of(desc)):
        os2.set_block(i, os_.get_block(i))
    gs.run_blocks(6, 2)
    os2.run_blocks(6, 2)
    assert_states_equal(gs, os2, n_blocks_of(desc))


@pytest.mark.parametrize("case", ["potts", "mixed_free"])
def test_categorical_screen_and_exact_fallback(T, O, case):
    """Millions of categorical draws: the fast-logarithm screen leaves about one in 10^4 to the exact recomputation, so a
    run of this size takes that path hundreds of times; every state must still equal the oracle's."""
    desc = model_cases(T)[case]
    chains = 8192
    prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 23)
    gs.run_blocks(41, 10)
    os_.run_blocks(41, 10)
    assert_states_equal(gs, os_, n_blocks_of(desc))


@pytest.mark.parametrize("chains", [1, 33, 520])
def test_mixed_degree_blocks_match_oracle(T, O, chains):
    """A sparse random graph with mean degree 6: most nodes keep their threshold tables, the few with more than 8
    neighbours take the sequential sum inside the same launch (kernel kind 6)."""
    desc, info = M.ising_sparse_random_graph(T, 600, 6, 77)
    assert 8 < info["degree"].max() <= 31 and (info["degree"] <= 8).mean() > 0.5
    prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 4)
    kinds = [prog.block_kernel(b) for b in range(len(desc["free"]))]
    assert 6 in kinds and set(kinds) <= {1, 4, 6}
    gs.run_blocks(3, 5)
    os_.run_blocks(3, 5)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    e0 = tuple(int(x) for x in info["edges"][0])
    spec = moment_spec(desc, info) + [[(1, 4, 6), e0]]
    gm, om = T.Moments(prog, spec, True), O.Moments(ob, spec, True)
    assert gm.fused_info() == (info["n"] + len(info["edges"]), 2)
    gs.sample_with_observation(8, 2, 4, 2, moments=gm)
    os_.sample_with_observation(8, 2, 4, 2, moments=om)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    for t in range(3):
        assert np.array_equal(gm.read(t)[0], om.read(t)[0])
    J2 = (info["J"] * 1.7).astype(np.float32)
    desc2 = dict(desc, ops=[("add_ising", np.arange(info["n"]), info["b"], info["edges"], J2, info["beta"])])
    gb2, ob2 = M.build_both(T, O, desc2)
    for blk in range(len(desc["free"])):
        for t, tab in enumerate(gb2.tables(blk)):
            prog.update_weights(blk, t, tab["w"].ravel())
    os2 = O.State(ob2, chains)
    for i in range(n_blocks_of(desc)):
        os2.set_block(i, os_.get_block(i))
    gs.run_blocks(6, 2)
    os2.run_blocks(6, 2)
    assert_states_equal(gs, os2, n_blocks_of(desc))


def test_hub_nodes_continue_in_overflow_rows(T, O):
    """A sparse graph with two hubs (200 and 70 neighbours): their entry lists span several rows of 32; everything else as usual."""
    n = 400
    rng = np.random.default_rng(9)
    a, b = rng.integers(2, n, 900), rng.integers(2, n, 900)
    pairs = [(min(x, y), max(x, y)) for x, y in zip(a, b) if x != y]
    pairs += [(0, j) for j in range(2, 202)] + [(1, j) for j in range(202, 272)]
    edges = np.unique(np.array(pairs, dtype=np.int64), axis=0)
    colour, n_col = T.greedy_coloring_arrays(n, edges)
    blocks = [np.flatnonzero(colour == c) for c in range(n_col)]
    bias = rng.normal(0, 0.1, n).astype(np.float32)
    Jv = rng.normal(0, 0.15, len(edges)).astype(np.float32)
    desc = dict(kinds=np.zeros(n, np.int32), free=[(blk, i) for i, blk in enumerate(blocks)], ops=[("add_ising", np.arange(n), bias, edges, Jv, 1.0)])
    info = dict(n=n, edges=edges)
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 150, 4)
    kinds = [prog.block_kernel(b) for b in range(n_col)]
    assert set(kinds) <= {1, 4, 6} and kinds[int(colour[0])] in (4, 6)
    gs.run_blocks(2, 6)
    os_.run_blocks(2, 6)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    spec = moment_spec(desc, info)
    gm, om = T.Moments(prog, spec, True), O.Moments(ob, spec, True)
    fused, other = gm.fused_info()
    assert fused + other == n + len(edges) and 0 < other <= 2 + 270  # the hubs' own rows and the pairs they would own
    gs.sample_with_observation(4, 1, 3, 2, moments=gm)
    os_.sample_with_observation(4, 1, 3, 2, moments=om)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    for t in range(2):
        assert np.array_equal(gm.read(t)[0], om.read(t)[0])


@pytest.mark.parametrize("degree,chains,extra", [(12, 300, 0.0), (16, 1040, 0.0), (10, 4100, 0.0), (12, 300, 2.0 ** 25), (14, 530, 300000.0),
                                                 (17, 1040, 0.0), (24, 520, 0.0), (31, 300, 2.0 ** 25), (20, 1040, 300000.0), (12, 8100, 0.0), (18, 7700, 0.0)])  # 7700+ chains: two counter segments
def test_split_field_tables_match_oracle(T, O, degree, chains, extra):
    """Sequential-sum nodes with at most 32 neighbour entries, 256 chains or more: the field comes from two (up to 16
    neighbours) or four 256-entry tables and only draws close to the probability take the canonical sum.  `extra` widens
    that window: 0 = the derived bound, 2^25 = every draw through the exact route, 3e5 (2 % of the unit interval) = a mixture."""
    before = dict(T.Program.default_options)
    T.Program.default_options = {**before, T.OPT_SPLIT_MARGIN: extra}
    try:
        desc, info = M.ising_random_graph(T, 260, degree, 300 + degree, w_sigma=0.4, bias_sigma=0.3)
        prog, gs, os_, gb, ob = make_pair(T, O, desc, chains, 3)
    finally:
        T.Program.default_options = before
    assert prog.get_option(T.OPT_SPLIT_MARGIN) == extra
    assert all(prog.block_kernel(b) == 4 for b in range(len(desc["free"])))
    gs.run_blocks(23, 8)
    os_.run_blocks(23, 8)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    e0 = tuple(int(x) for x in info["edges"][0])
    spec = moment_spec(desc, info) + [[(0, 5, 9), e0]]
    gm, om = T.Moments(prog, spec, True), O.Moments(ob, spec, True)
    assert gm.fused_info() == (info["n"] + len(info["edges"]), 2)
    gs.sample_with_observation(5, 1, 3, 2, moments=gm)
    os_.sample_with_observation(5, 1, 3, 2, moments=om)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    for t in range(3):
        assert np.array_equal(gm.read(t)[0], om.read(t)[0])
    # new couplings rebuild the tables (larger ones: wider windows)
    J2 = (info["J"] * -2.5).astype(np.float32)
    desc2 = dict(desc, ops=[("add_ising", np.arange(info["n"]), info["b"], info["edges"], J2, info["beta"])])
    gb2, ob2 = M.build_both(T, O, desc2)
    for blk in range(len(desc["free"])):
        for t, tab in enumerate(gb2.tables(blk)):
            prog.update_weights(blk, t, tab["w"].ravel())
    os2 = O.State(ob2, chains)
    for i in range(n_blocks_of(desc)):
        os2.set_block(i, os_.get_block(i))
    gs.run_blocks(6, 3)
    os2.run_blocks(6, 3)
    assert_states_equal(gs, os2, n_blocks_of(desc))


def test_split_tables_with_isolated_and_leaf_nodes(T, O):
    """Blocks of the sequential-sum kind that also hold nodes with no neighbour at all (a bias only), with one neighbour
    and with no entry at all (zero bias is still an entry; the leaf's weight is exactly zero in one case): all of them
    take the table route with mostly empty configuration bytes."""
    n_core, rng = 240, np.random.default_rng(5)
    core = M.random_regular_graph(n_core, 12, 77)
    leaves = np.array([[int(rng.integers(0, n_core)), n_core + 4 + k] for k in range(6)], dtype=np.int64)
    edges = np.concatenate([np.asarray(core, dtype=np.int64), leaves])
    edges = np.stack([edges.min(axis=1), edges.max(axis=1)], axis=1)
    n = n_core + 10  # nodes n_core .. n_core + 3 are isolated
    colour, n_col = T.greedy_coloring_arrays(n, edges)
    blocks = [np.flatnonzero(colour == c) for c in range(n_col)]
    bias = rng.normal(0, 0.4, n).astype(np.float32)
    bias[n_core] = 0.0
    Jv = rng.normal(0, 0.4, len(edges)).astype(np.float32)
    Jv[-1] = 0.0
    desc = dict(kinds=np.zeros(n, np.int32), free=[(blk, i) for i, blk in enumerate(blocks)], ops=[("add_ising", np.arange(n), bias, edges, Jv, 1.0)])
    prog, gs, os_, gb, ob = make_pair(T, O, desc, 300, 11)
    kinds = [prog.block_kernel(b) for b in range(n_col)]
    assert 4 in kinds and set(kinds) <= {1, 4, 6}
    gs.run_blocks(9, 10)
    os_.run_blocks(9, 10)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    spec = moment_spec(desc, dict(n=n, edges=edges))
    gm, om = T.Moments(prog, spec, True), O.Moments(ob, spec, True)
    gs.sample_with_observation(3, 1, 4, 2, moments=gm)
    os_.sample_with_observation(3, 1, 4, 2, moments=om)
    assert_states_equal(gs, os_, n_blocks_of(desc))
    for t in range(2):
        assert np.array_equal(gm.read(t)[0], om.read(t)[0])
