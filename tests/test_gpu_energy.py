"""Factor energies (DiscreteEBMFactor::factor_energy, FactorizedEBM::energy) on the device against the numpy
restatement, and the use the reference's own tests make of them: the exact Boltzmann distribution of a small mixed
spin / categorical model from enumerated energies, compared with what the sampler produces."""
import itertools

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def small_mixed(T, seed):
    """3 spins (nodes 0-2) and 2 categorical nodes with K = 3 (nodes 3-4); every factor kind the samplers support."""
    rng = np.random.default_rng(seed)
    K = 3
    kinds = np.array([0, 0, 0, K, K], np.int32)
    f = lambda *shape: rng.normal(0, 0.6, shape).astype(np.float32)
    factors = [([[0, 1, 2]], [], f(3, 1, 1)),                      # spin biases
               ([], [[3, 4]], f(2, K, 1)),                         # categorical biases
               ([[0, 1], [1, 2]], [], f(2, 1, 1)),                 # spin-spin
               ([[0, 2]], [[3, 4]], f(2, K, 1)),                   # spin-categorical
               ([], [[3], [4]], f(1, K, K)),                       # categorical-categorical
               ([[0], [1], [2]], [], f(1, 1, 1))]                  # three-spin
    bld = T.Builder(kinds, [0, K])
    for blk in ([0, 2], [1], [3], [4]):
        bld.add_free_block(np.array(blk))
    for sg, cg, w in factors:
        bld.add_discrete_factor([np.array(g) for g in sg], [np.array(g) for g in cg], w)
    bld.compile()
    return T.Program(bld), factors, K


def all_states(K):
    return np.array([list(s) + list(c) for s in itertools.product((0, 1), repeat=3) for c in itertools.product(range(K), repeat=2)], dtype=np.uint8)


def upload_nodes(st, values):
    """values[chain][node] for nodes 0..4 -> blocks ([0, 2], [1], [3], [4])."""
    for b, blk in enumerate(([0, 2], [1], [3], [4])):
        st.upload(b, np.ascontiguousarray(values[:, blk]))


@pytest.mark.parametrize("chains", [1, 72, 203])
def test_factor_energy_matches_numpy(T, O, chains):
    prog, factors, K = small_mixed(T, 5)
    rng = np.random.default_rng(chains)
    vals = np.concatenate([rng.integers(0, 2, (chains, 3)), rng.integers(0, K, (chains, 2))], axis=1).astype(np.uint8)
    st = T.ChainState(prog, chains)
    upload_nodes(st, vals)
    for sg, cg, w in factors:
        got = st.factor_energy(sg, cg, w)
        want = O.factor_energy(w, [vals[:, g] for g in sg], [vals[:, g] for g in cg])
        assert got.shape == (chains,) and np.allclose(got, want, rtol=1e-12, atol=1e-12)


def test_many_rows_are_summed_in_a_fixed_order(T, O):
    """More rows than one reduction chunk (2048), spin-only and with a categorical axis; repeated calls give the same bits."""
    rng = np.random.default_rng(8)
    n_spin, n_cat, K, rows, chains = 50, 30, 5, 5000, 33
    kinds = np.concatenate([np.zeros(n_spin, np.int32), np.full(n_cat, K, np.int32)])
    bld = T.Builder(kinds, [0, K])
    bld.add_free_block(np.arange(n_spin))
    bld.add_free_block(np.arange(n_spin, n_spin + n_cat))
    bld.compile()
    prog = T.Program(bld)
    st = T.ChainState(prog, chains)
    sv, cv = rng.integers(0, 2, (chains, n_spin)).astype(np.uint8), rng.integers(0, K, (chains, n_cat)).astype(np.uint8)
    st.upload(0, sv)
    st.upload(1, cv)
    a, b = rng.integers(0, n_spin, rows), rng.integers(0, n_spin, rows)
    c, d = rng.integers(0, n_cat, rows), rng.integers(0, n_cat, rows)
    w2 = rng.normal(0, 1, (rows, 1, 1)).astype(np.float32)
    got = st.factor_energy([a, b], [], w2)
    assert np.allclose(got, O.factor_energy(w2, [sv[:, a], sv[:, b]], []), rtol=1e-12, atol=1e-9)
    assert np.array_equal(got, st.factor_energy([a, b], [], w2))
    w3 = rng.normal(0, 1, (rows, K, K)).astype(np.float32)
    got = st.factor_energy([a], [n_spin + c, n_spin + d], w3)
    assert np.allclose(got, O.factor_energy(w3, [sv[:, a]], [cv[:, c], cv[:, d]]), rtol=1e-12, atol=1e-9)


def test_argument_errors(T):
    prog, factors, K = small_mixed(T, 5)
    st = T.ChainState(prog, 4)
    with pytest.raises(T.ThrmlError, match="same type"):
        st.factor_energy([[3]], [], np.zeros((1, 1, 1), np.float32))      # categorical node in a spin group
    with pytest.raises(T.ThrmlError, match="not found"):
        st.factor_energy([[17]], [], np.zeros((1, 1, 1), np.float32))
    with pytest.raises(T.ThrmlError, match="shape of the weight tensor"):
        st.factor_energy([[0]], [], np.zeros((1, 3, 1), np.float32))      # a categorical axis without a categorical group
    assert np.array_equal(st.factor_energy([], [], np.zeros((0, 1, 1), np.float32)), np.zeros(4))


def test_api_factorized_ebm_equals_ising_energy(T):
    nodes = [T.Node(T.NodeType.Spin()) for _ in range(6)]
    edges = [(nodes[i], nodes[(i + 1) % 6]) for i in range(6)]
    rng = np.random.default_rng(2)
    b, J = rng.normal(0, 0.4, 6).astype(np.float32), rng.normal(0, 0.7, 6).astype(np.float32)
    ebm = T.IsingEBM(nodes, edges, b, J, 0.8)
    states = rng.integers(0, 2, (9, 6)).astype(np.float32)
    want = ebm.energy_batched(states)
    fact = T.FactorizedEBM(ebm.get_factors(), ebm.node_shape_dtypes())
    blocks = [T.Block(nodes[:4]), T.Block(nodes[4:])]
    got = fact.energy([states[:, :4], states[:, 4:]], blocks)
    assert got.shape == (9,) and np.allclose(got, want, rtol=1e-6, atol=1e-6)
    one = fact.energy([states[0, :4], states[0, 4:]], blocks)
    assert one.shape == (1,) and np.allclose(one, want[0], rtol=1e-6, atol=1e-6)
    f0 = ebm.get_factors()[1]
    assert np.allclose(f0.factor_energy([states[:, :4], states[:, 4:]], blocks) + ebm.get_factors()[0].factor_energy([states[:, :4], states[:, 4:]], blocks), want,
                       rtol=1e-6, atol=1e-6)


def test_reference_known_answer(T):
    """crates/thrml-models/tests/test_ising.rs:23-48 through the factors: 3-spin chain, state (1, 0, 1),
    E = -(0.1 - 0.2 + 0.3 - 0.5 + 0.5) = -0.2 (that test's comment slips a sign and says 0.8; it asserts finiteness only)."""
    nodes = [T.Node(T.NodeType.Spin()) for _ in range(3)]
    ebm = T.IsingEBM(nodes, [(nodes[0], nodes[1]), (nodes[1], nodes[2])], np.array([0.1, 0.2, 0.3], np.float32), np.array([0.5, -0.5], np.float32), 1.0)
    fact = T.FactorizedEBM(ebm.get_factors(), ebm.node_shape_dtypes())
    e = fact.energy([np.array([1.0, 0.0, 1.0], np.float32)], [T.Block(nodes)])
    assert e.shape == (1,) and abs(float(e[0]) + 0.2) < 1e-6


def test_sampler_reaches_the_boltzmann_distribution_of_the_energies(T):
    """The reference's sample-vs-exact check (crates/thrml-models/tests/utils.rs:272-325): probabilities from enumerated
    energies against the empirical distribution of the sampler, here within 4 sigma of the across-chain standard error."""
    prog, factors, K = small_mixed(T, 11)
    states = all_states(K)  # 72 joint configurations
    enum = T.ChainState(prog, len(states))
    upload_nodes(enum, states)
    energy = sum(enum.factor_energy(sg, cg, w) for sg, cg, w in factors)
    p = np.exp(-(energy - energy.min()))
    p /= p.sum()
    chains, samples = 4096, 150
    st = T.ChainState(prog, chains)
    st.randomize(3)
    obs = st.sample_with_observation(29, 60, samples, 2, obs_blocks=[0, 1, 2, 3])  # rows: nodes 0, 2, 1, 3, 4
    vals = np.zeros((samples, 5, chains), dtype=np.int64)
    vals[:, [0, 2, 1, 3, 4], :] = obs
    code = ((vals[:, 0] * 2 + vals[:, 1]) * 2 + vals[:, 2]) * K * K + vals[:, 3] * K + vals[:, 4]  # index into `states`
    freq = np.stack([(code == k).mean(axis=0) for k in range(len(states))])  # [state, chain] time averages
    mean, sem = freq.mean(axis=1), freq.std(axis=1, ddof=1) / np.sqrt(chains)
    assert np.all(np.abs(mean - p) < 4 * sem + 1e-6), float(np.max(np.abs(mean - p) / (sem + 1e-12)))
