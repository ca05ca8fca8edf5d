"""The host-side mirror of the reference API: constructor validation with the reference's error strings (CPU), and the
reference's own smoke tests re-run through the CUDA path (GPU)."""
import numpy as np
import pytest


def spins(T, n):
    return [T.Node(T.NodeType.Spin()) for _ in range(n)]


def test_block_validation(T):
    # crates/thrml-core/tests/test_block.rs:11-153
    with pytest.raises(T.ThrmlError, match="empty"):
        T.Block([])
    with pytest.raises(T.ThrmlError, match="same type"):
        T.Block([T.Node(T.NodeType.Spin()), T.Node(T.NodeType.Categorical(3))])
    a, b = T.Block(spins(T, 2)), T.Block(spins(T, 3))
    assert len(a + b) == 5
    with pytest.raises(T.ThrmlError, match="different node types"):
        a + T.Block([T.Node(T.NodeType.Categorical(3))])
    with pytest.raises(T.ThrmlError, match="twice"):
        T.BlockSpec([a, a], [T.NodeType.Spin()])
    with pytest.raises(T.ThrmlError, match="not found"):
        T.BlockSpec([a], [T.NodeType.Categorical(2)])
    n1, n2 = T.Node(T.NodeType.Spin()), T.Node(T.NodeType.Spin())
    assert n1 != n2 and n1.id != n2.id and n1 == n1


def test_interaction_group_validation(T):
    # crates/thrml-core/tests/test_interaction.rs:17-121
    head = T.Block(spins(T, 3))
    with pytest.raises(T.ThrmlError, match="tail node blocks"):
        T.InteractionGroup(np.zeros((3, 1, 1)), head, [T.Block(spins(T, 2))], 1)
    with pytest.raises(T.ThrmlError, match="leading dimension"):
        T.InteractionGroup(np.zeros((4, 1, 1)), head, [T.Block(spins(T, 3))], 1)
    with pytest.raises(T.ThrmlError, match="n_spin"):
        T.InteractionGroup(np.zeros((3, 1, 1)), head, [T.Block(spins(T, 3))], 2)


def test_factor_validation(T):
    # crates/thrml-models/tests/test_factor.rs:10-49, test_discrete_ebm.rs:20-184
    g3, g2 = T.Block(spins(T, 3)), T.Block(spins(T, 2))
    with pytest.raises(T.ThrmlError, match="same number"):
        T.SpinEBMFactor([g3, g2], np.zeros((3, 1, 1)))
    with pytest.raises(T.ThrmlError, match="leading dimension"):
        T.SpinEBMFactor([g3], np.zeros((4, 1, 1)))
    with pytest.raises(T.ThrmlError, match="At least one"):
        T.DiscreteEBMFactor([], [], np.zeros((1, 1, 1)))
    cat = T.Block([T.Node(T.NodeType.Categorical(4)) for _ in range(3)])
    with pytest.raises(T.ThrmlError, match="shape of the weight tensor"):
        T.CategoricalEBMFactor([cat, cat], np.zeros((3, 4, 1)))


def test_program_validation(T):
    # crates/thrml-samplers/tests/test_program.rs:65-138: sampler count must match the free blocks
    blocks = [T.Block(spins(T, 3)), T.Block(spins(T, 3))]
    spec = T.BlockGibbsSpec([[blocks[0]], [blocks[1]]], [], [T.NodeType.Spin()])
    assert spec.sampling_order == [[0], [1]] and len(spec.free_blocks) == 2
    with pytest.raises(T.ThrmlError, match="Number of samplers"):
        T.BlockSamplingProgram(spec, [T.SpinGibbsConditional()], [])
    spec2 = T.BlockGibbsSpec([[blocks[0], blocks[1]]], [], [T.NodeType.Spin()])
    assert spec2.sampling_order == [[0, 1]]


def test_rng_key_and_schedule(T):
    # crates/thrml-samplers/src/rng.rs:52-86
    keys = T.RngKey.new(42).split(5)
    assert len({k.seed() for k in keys}) == 5
    assert T.RngKey(42).split(10) == T.RngKey(42).split(10)
    assert T.RngKey(9).split(1) == [T.RngKey(9)] and T.RngKey(9).split(0) == []
    a, b = T.RngKey(1).split_two()
    assert a != b
    s = T.SamplingSchedule.new(10, 5, 2)
    assert (s.n_warmup, s.n_samples, s.steps_per_sample) == (10, 5, 2)


def chain_model(T, n=5):
    nodes = spins(T, n)
    edges = [(nodes[i], nodes[i + 1]) for i in range(n - 1)]
    ebm = T.IsingEBM(nodes, edges, np.linspace(-0.2, 0.2, n), np.full(n - 1, 0.5), 1.0)
    even, odd = T.Block(nodes[0::2]), T.Block(nodes[1::2])
    return nodes, edges, ebm, even, odd


@pytest.mark.gpu
def test_run_blocks_shapes(T):
    # crates/thrml-samplers/tests/test_program.rs:141-186: 5 sweeps, shapes preserved
    nodes, edges, ebm, even, odd = chain_model(T)
    prog = T.IsingSamplingProgram(ebm, [even, odd], []).program
    init = [np.zeros(3, np.float32), np.ones(2, np.float32)]
    out = T.run_blocks(T.RngKey(0), prog, init, [], 5)
    assert [o.shape for o in out] == [(3,), (2,)] and all(set(np.unique(o)) <= {0.0, 1.0} for o in out)
    assert T.run_blocks(T.RngKey(0), prog, init, [], 0)[0] is init[0]
    state = [a.copy() for a in init]
    T.sample_blocks(T.RngKey(1), state, [], prog)
    assert [s.shape for s in state] == [(3,), (2,)]


@pytest.mark.gpu
def test_sample_states_and_moments_api(T, O):
    nodes, edges, ebm, even, odd = chain_model(T)
    prog = T.IsingSamplingProgram(ebm, [even, odd], []).program
    sched = T.SamplingSchedule(3, 6, 2)
    init = [np.zeros((4, 3), np.float32), np.ones((4, 2), np.float32)]
    samples = T.sample_states(T.RngKey(5), prog, sched, init, [], [odd, even])
    assert [s.shape for s in samples] == [(6, 4, 2), (6, 4, 3)]
    single = T.sample_states(T.RngKey(5), prog, sched, [a[0] for a in init], [], [even])
    assert single[0].shape == (6, 3) and np.array_equal(single[0], samples[1][:, 0, :])
    m1, m2 = T.estimate_moments(T.RngKey(5), nodes, edges, prog, sched, init, [])
    assert m1.shape == (5,) and m2.shape == (4,)
    # the same schedule through the state observer gives the same averages
    full = np.zeros((6, 4, 5))
    full[:, :, 0::2] = samples[1]
    full[:, :, 1::2] = samples[0]
    sp = 2 * full - 1
    assert np.allclose(m1, sp.mean(axis=(0, 1)), atol=1e-6)
    assert np.allclose(m2, (sp[:, :, :-1] * sp[:, :, 1:]).mean(axis=(0, 1)), atol=1e-6)


@pytest.mark.gpu
def test_clamped_blocks_and_hinton_api(T):
    nodes, edges, ebm, even, odd = chain_model(T)
    prog = T.IsingSamplingProgram(ebm, [even], [odd]).program
    clamp = [np.array([1, 0], np.float32)]
    out = T.run_blocks(T.RngKey(3), prog, [np.zeros(3, np.float32)], clamp, 4)
    assert out[0].shape == (3,)
    # crates/thrml-models/tests/test_ising.rs:57-98: bias 10 -> at least 7 of 10 ones
    big = spins(T, 10)
    ebm2 = T.IsingEBM(big, [], np.full(10, 10.0), np.zeros(0), 1.0)
    init = T.hinton_init(T.RngKey(0), ebm2, [T.Block(big)], [1])
    assert init[0].shape == (1, 10) and init[0].sum() >= 7
    init = T.hinton_init(T.RngKey(0), ebm2, [T.Block(big[:4]), T.Block(big[4:])], [2, 3])
    assert [a.shape for a in init] == [(6, 4), (6, 6)]


@pytest.mark.gpu
def test_potts_factor_program_api(T):
    # crates/thrml-examples/examples/categorical_sampling.rs:108-124: W = beta*I favours equal neighbours
    K, n = 3, 6
    nodes = [T.Node(T.NodeType.Categorical(K)) for _ in range(n)]
    u, v = T.Block(nodes[:-1]), T.Block(nodes[1:])
    w = np.broadcast_to(3.0 * np.eye(K, dtype=np.float32), (n - 1, K, K)).copy()
    factor = T.CategoricalEBMFactor([u, v], w)
    even, odd = T.Block(nodes[0::2]), T.Block(nodes[1::2])
    spec = T.BlockGibbsSpec([[even], [odd]], [], [T.NodeType.Categorical(K)])
    prog = T.FactorSamplingProgram(spec, [T.CategoricalGibbsConditional(K), T.CategoricalGibbsConditional(K)], [factor]).program
    init = [np.zeros((256, 3), np.float32), np.zeros((256, 3), np.float32)]
    out = T.run_blocks(T.RngKey(2), prog, init, [], 30)
    full = np.zeros((256, n))
    full[:, 0::2], full[:, 1::2] = out[0], out[1]
    agree = (full[:, :-1] == full[:, 1:]).mean()
    assert agree > 0.8  # exact: e^3/(e^3+2) = 0.909 per bond


@pytest.mark.gpu
def test_bounded_wait_reports_timeout_and_context_survives(T):
    ctx = T.default_context()
    rc = T.lib().thrml_debug_wait_timeout(ctx.h)
    assert rc == -5  # THRML_ERR_TIMEOUT
    assert b"bounded wait ran out" in T.lib().thrml_last_error()
    # the context still works
    nodes, edges, ebm, even, odd = chain_model(T)
    prog = T.IsingSamplingProgram(ebm, [even, odd], []).program
    out = T.run_blocks(T.RngKey(0), prog, [np.zeros(3, np.float32), np.ones(2, np.float32)], [], 2)
    assert out[0].shape == (3,)


@pytest.mark.gpu
def test_estimate_kl_grad_api(T):
    # crates/thrml-models/src/ising.rs:392-433,531-594: visible data block + hidden block, two phases
    vis, hid = spins(T, 6), spins(T, 4)
    nodes = vis + hid
    edges = [(v, h) for v in vis for h in hid]
    rng = np.random.default_rng(0)
    ebm = T.IsingEBM(nodes, edges, rng.normal(0, 0.1, 10), rng.normal(0, 0.3, 24), 1.0)
    bv, bh = T.Block(vis), T.Block(hid)
    spec = T.IsingTrainingSpec(ebm, [bv], [], [bh], [bv, bh], T.SamplingSchedule(5, 20, 1), T.SamplingSchedule(5, 20, 1))
    data = [rng.integers(0, 2, (8, 6)).astype(np.float32)]
    chains = 64
    init_pos = [np.zeros((chains, 4), np.float32)]
    init_neg = [np.zeros((chains, 6), np.float32), np.zeros((chains, 4), np.float32)]
    key = T.RngKey(3)
    gw, gb = T.estimate_kl_grad(key, spec, nodes, edges, data, [], init_pos, init_neg)
    assert gw.shape == (24,) and gb.shape == (10,)
    # the same gradient from the two estimate_moments calls it is made of
    kp, kn = key.split_two()
    row = data[0][kp.seed() % 8]
    bp, wp = T.estimate_moments(kp, nodes, edges, spec.program_positive.program, spec.schedule_positive, init_pos, [np.broadcast_to(row, (chains, 6)).copy()])
    bn, wn = T.estimate_moments(kn, nodes, edges, spec.program_negative.program, spec.schedule_negative, init_neg, [])
    assert np.array_equal(gw, -(wp - wn)) and np.array_equal(gb, -(bp - bn))
    # clamped visible units reproduce the data row exactly in the positive phase
    assert np.allclose(bp[:6], 2 * row - 1)


@pytest.mark.gpu
def test_ising_energy(T):
    # crates/thrml-models/tests/test_ising.rs:17-55: 3-node chain, b = (0.1, 0.2, 0.3), J = (0.5, -0.5), state (1,0,1):
    # E = -(0.1 - 0.2 + 0.3 - 0.5 + 0.5) = -0.2 (the test's comment says 0.8; the code it calls gives -0.2)
    nodes = spins(T, 3)
    ebm = T.IsingEBM(nodes, [(nodes[0], nodes[1]), (nodes[1], nodes[2])], [0.1, 0.2, 0.3], [0.5, -0.5], 1.0)
    e = ebm.energy([np.array([1.0, 0.0, 1.0], np.float32)])
    assert e.shape == (1,) and abs(e[0] + 0.2) < 1e-6
    # crates/thrml-models/tests/test_ising.rs:185-222: batched energies equal single-state energies within 1e-5
    rng = np.random.default_rng(4)
    big = spins(T, 40)
    edges = [(big[i], big[j]) for i in range(40) for j in range(i + 1, 40) if rng.random() < 0.2]
    b, J = rng.normal(0, 0.5, 40).astype(np.float32), rng.normal(0, 0.5, len(edges)).astype(np.float32)
    ebm = T.IsingEBM(big, edges, b, J, 0.7)
    states = rng.integers(0, 2, (300, 40)).astype(np.float32)
    batched = ebm.energy_batched(states)
    s = 2 * states.astype(np.float64) - 1
    idx = {n: i for i, n in enumerate(big)}
    ea = np.array([idx[a] for a, _ in edges]); eb = np.array([idx[c] for _, c in edges])
    want = -0.7 * (s @ b.astype(np.float64) + (s[:, ea] * s[:, eb]) @ J.astype(np.float64))
    assert np.allclose(batched, want, rtol=1e-6, atol=1e-6)
    assert abs(ebm.energy([states[5]])[0] - batched[5]) < 1e-5


def test_grid_helpers_known_answers(T):
    # crates/thrml-examples/src/lib.rs:255-330: 3 x 4 grid = 12 nodes, 9 + 8 = 17 edges; a 3 x 3 grid two-colours with no
    # monochromatic edge; a 2 x 2 grid gives two blocks of two; a chain of five is two-colourable by the greedy rule
    nodes, edges, grid = T.generate_lattice_graph(3, 4)
    assert len(nodes) == 12 and len(edges) == 17 and len(grid) == 3 and len(grid[0]) == 4
    nodes, edges, grid = T.generate_lattice_graph(3, 3)
    colour = T.bipartite_coloring(grid)
    assert set(colour.tolist()) == {0, 1} and all(colour[a] != colour[b] for a, b in edges)
    nodes, edges, grid = T.generate_lattice_graph(2, 2)
    blocks = T.coloring_to_blocks(nodes, T.bipartite_coloring(grid))
    assert [len(b) for b in blocks] == [2, 2]
    nodes, edges = T.generate_chain_graph(5)
    assert len(edges) == 4 and int(T.greedy_coloring(5, edges).max()) + 1 == 2


@pytest.mark.gpu
def test_softmax_conditional_block(T, O):
    """A block sampled by SoftmaxConditional (softmax.rs:103-222) next to one sampled by CategoricalGibbsConditional: same
    states as the oracle's restatement, and logits that ignore the neighbours."""
    import models as M
    K, side = 5, 6
    desc, info = M.potts_lattice(T, side, K, 3)
    results = []
    for cls in (T.Builder, O.Model):
        bld = cls(desc["kinds"])
        bld.add_free_block(info["blocks"][0], superblock=0, sampler=2)  # SoftmaxConditional
        bld.add_free_block(info["blocks"][1], superblock=1, sampler=1)  # CategoricalGibbsConditional
        for op in desc["ops"]:
            getattr(bld, op[0])(*op[1:])
        bld.compile()
        results.append(bld)
    gb, ob = results
    chains = 70
    prog = T.Program(gb)
    gs, os_ = T.ChainState(prog, chains), O.State(ob, chains)
    init = M.random_states(desc, chains, 2)
    for i, a in enumerate(init):
        gs.upload(i, a)
        os_.set_block(i, a.astype(np.float32))
    th_g, (th64, th32) = gs.fields(0), os_.fields(0)
    assert np.array_equal(th_g, th32)
    assert np.array_equal(th_g[0], th_g[-1])  # no dependence on the chains' neighbour states
    gs.run_blocks(8, 3)
    os_.run_blocks(8, 3)
    for i in range(2):
        assert np.array_equal(gs.download(i), os_.get_block(i))
    # the API mirror accepts the sampler
    cats = [T.Node(T.NodeType.Categorical(3)) for _ in range(4)]
    spec = T.BlockGibbsSpec([[T.Block(cats)]], [], [T.NodeType.Categorical(3)])
    w = np.zeros((4, 3, 1), np.float32)
    w[:, 2, 0] = 40.0
    prog2 = T.BlockSamplingProgram(spec, [T.SoftmaxConditional(3)], [T.InteractionGroup(w, T.Block(cats), [], 0)])
    out = T.run_blocks(T.RngKey(1), prog2, [np.zeros(4, np.float32)], [], 2)
    assert np.array_equal(out[0], np.full(4, 2.0, np.float32))
