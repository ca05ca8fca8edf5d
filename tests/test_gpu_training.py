"""The callers either side of the sampling path that training needs (crates/thrml-models/src/ising.rs:392-433, 531-594;
crates/thrml-examples/examples/train_mnist.rs:616-732): the two-phase KL gradient formed on the device, and the refresh of
a program's weights from the model's parameter vectors without a host-side gather."""
import numpy as np
import pytest

import models as M

pytestmark = pytest.mark.gpu


def _two_phase_models(seed, n_vis=10, n_hid=7, n_cond=4, beta=0.8):
    """Visible (data), hidden and conditioning spins, all-to-all between visible-hidden and conditioning-hidden plus a few
    visible-visible edges.  Returns node id arrays, parameters and the two (free, clamped) block layouts."""
    rng = np.random.default_rng(seed)
    vis, hid, cond = np.arange(n_vis), np.arange(n_vis, n_vis + n_hid), np.arange(n_vis + n_hid, n_vis + n_hid + n_cond)
    n = n_vis + n_hid + n_cond
    edges = [(v, h) for v in vis for h in hid] + [(c, h) for c in cond for h in hid] + [(vis[i], vis[i + 1]) for i in range(0, n_vis - 1, 2)]
    edges = np.array(edges, dtype=np.int64)
    b = rng.normal(0, 0.2, n).astype(np.float32)
    J = rng.normal(0, 0.3, len(edges)).astype(np.float32)
    # the visible-visible edges join an even to an odd unit, so the visible layer takes two colours in the negative phase
    layouts = {"pos": dict(free=[hid], clamped=[vis, cond]), "neg": dict(free=[vis[0::2], vis[1::2], hid], clamped=[cond])}
    return dict(n=n, vis=vis, hid=hid, cond=cond, edges=edges, b=b, J=J, beta=beta, layouts=layouts)


def _build(cls, m, which):
    lay = m["layouts"][which]
    bld = cls(np.zeros(m["n"], np.int32))
    for i, blk in enumerate(lay["free"]):
        bld.add_free_block(blk, superblock=i)
    for blk in lay["clamped"]:
        bld.add_clamped_block(blk)
    bld.add_ising(np.arange(m["n"]), m["b"], m["edges"], m["J"], m["beta"])
    bld.compile()
    return bld


@pytest.mark.parametrize("chains,sched_pos,sched_neg", [(1, (3, 6, 1), (2, 5, 2)), (48, (2, 4, 1), (0, 3, 2)), (300, (1, 1, 1), (1, 2, 1))])
def test_kl_gradient_on_device_matches_oracle(T, O, chains, sched_pos, sched_neg):
    from thrml_rs_b200 import engine as E
    m = _two_phase_models(5)
    rng = np.random.default_rng(chains)
    data_row = rng.integers(0, 2, len(m["vis"])).astype(np.uint8)
    cond_row = rng.integers(0, 2, len(m["cond"])).astype(np.uint8)
    spec = [[(i,) for i in range(m["n"])], [tuple(e) for e in m["edges"]]]
    key = 0xFEED
    k_pos, k_neg = [int(k) for k in T.rng_split(key, 2)]
    sums = {}
    states = {}
    for which, k, sched in (("pos", k_pos, sched_pos), ("neg", k_neg, sched_neg)):
        gb, ob = _build(T.Builder, m, which), _build(O.Model, m, which)
        prog = T.Program(gb)
        gs, os_ = T.ChainState(prog, chains), O.State(ob, chains)
        lay = m["layouts"][which]
        init = [rng.integers(0, 2, (chains, len(blk))).astype(np.uint8) for blk in lay["free"]]
        clamp = [np.broadcast_to(data_row if which == "pos" and i == 0 else cond_row, (chains, len(blk))).copy() for i, blk in enumerate(lay["clamped"])]
        for i, a in enumerate(init + clamp):
            gs.upload(i, a)
            os_.set_block(i, a.astype(np.float32))
        om = O.Moments(ob, spec, True)
        os_.sample_with_observation(k, *sched, moments=om)
        sums[which] = [om.read(t)[0].astype(np.float64) / (sched[1] * chains) for t in range(2)]
        states[which] = (gs, T.Moments(prog, spec, True), prog)
    gw, gb_ = E.estimate_kl_grad(states["pos"][0], states["neg"][0], states["pos"][1], states["neg"][1], key, sched_pos, sched_neg, m["beta"])
    want_b = (sums["pos"][0].astype(np.float32) - sums["neg"][0].astype(np.float32)) * np.float32(-m["beta"])
    want_w = (sums["pos"][1].astype(np.float32) - sums["neg"][1].astype(np.float32)) * np.float32(-m["beta"])
    assert gw.dtype == np.float32 and np.array_equal(gw, want_w) and np.array_equal(gb_, want_b)
    # clamped data: the positive phase reproduces the data row exactly in the bias moments
    pos_mean = states["pos"][1].read(0)[0][: len(m["vis"])] / (sched_pos[1] * chains)
    assert np.array_equal(pos_mean, 2.0 * data_row - 1.0)


def test_kl_gradient_api_with_conditioning_block_and_chains(T):
    """The API mirror with a batch of chains and a conditioning block given once (a 1-D array stands for every chain)."""
    from thrml_rs_b200.api import Node, NodeType
    vis, hid, cond = [[Node(NodeType.Spin()) for _ in range(k)] for k in (6, 4, 3)]
    nodes = vis + hid + cond
    edges = [(v, h) for v in vis for h in hid] + [(c, h) for c in cond for h in hid]
    rng = np.random.default_rng(1)
    ebm = T.IsingEBM(nodes, edges, rng.normal(0, 0.1, len(nodes)), rng.normal(0, 0.3, len(edges)), 0.7)
    bv, bh, bc = T.Block(vis), T.Block(hid), T.Block(cond)
    spec = T.IsingTrainingSpec(ebm, [bv], [bc], [bh], [bv, bh], T.SamplingSchedule(2, 6, 1), T.SamplingSchedule(2, 6, 1))
    data = [rng.integers(0, 2, (5, 6)).astype(np.float32)]
    cond_vals = [rng.integers(0, 2, 3).astype(np.float32)]
    chains = 40
    init_pos = [rng.integers(0, 2, (chains, 4)).astype(np.float32)]
    init_neg = [rng.integers(0, 2, (chains, 6)).astype(np.float32), rng.integers(0, 2, (chains, 4)).astype(np.float32)]
    key = T.RngKey(11)
    gw, gb = T.estimate_kl_grad(key, spec, nodes, edges, data, cond_vals, init_pos, init_neg)
    kp, kn = key.split_two()
    row = data[0][kp.seed() % 5]
    bp, wp = T.estimate_moments(kp, nodes, edges, spec.program_positive.program, spec.schedule_positive, init_pos, [row, cond_vals[0]])
    bn, wn = T.estimate_moments(kn, nodes, edges, spec.program_negative.program, spec.schedule_negative, init_neg, cond_vals)
    assert np.array_equal(gw, (wp - wn) * np.float32(-0.7)) and np.array_equal(gb, (bp - bn) * np.float32(-0.7))
    assert np.array_equal(bp[10:], 2 * cond_vals[0] - 1) and np.array_equal(bn[10:], 2 * cond_vals[0] - 1)
    # an SGD step: new parameters reach both existing programs through the device-side refresh
    ebm.update_weights(ebm.weights - 0.1 * gw, ebm.biases - 0.1 * gb)
    spec.refresh_weights()
    gw2, gb2 = T.estimate_kl_grad(key, spec, nodes, edges, data, cond_vals, init_pos, init_neg)
    fresh = T.IsingTrainingSpec(ebm, [bv], [bc], [bh], [bv, bh], spec.schedule_positive, spec.schedule_negative)
    gw3, gb3 = T.estimate_kl_grad(key, fresh, nodes, edges, data, cond_vals, init_pos, init_neg)
    assert np.array_equal(gw2, gw3) and np.array_equal(gb2, gb3) and not np.array_equal(gw2, gw)


@pytest.mark.parametrize("make,kinds", [(lambda T: M.ising_random_graph(T, 300, 8, 4), {1}), (lambda T: M.ising_random_graph(T, 260, 12, 5, w_sigma=0.4, bias_sigma=0.3), {4}),
                                        (lambda T: M.ising_sparse_random_graph(T, 400, 6, 6), {1, 4, 6})])
def test_update_group_equals_a_program_built_with_the_new_weights(T, O, make, kinds):
    desc, info = make(T)
    chains = 272
    prog = T.Program(M.fill(T.Builder(desc["kinds"]), desc))
    assert {prog.block_kernel(b) for b in range(len(desc["free"]))} <= kinds
    rng = np.random.default_rng(9)
    b2 = rng.normal(0, 0.3, info["n"]).astype(np.float32)
    J2 = rng.normal(0, 0.4, len(info["edges"])).astype(np.float32)
    beta2 = 1.3
    prog.update_group(0, b2, scale=beta2)   # the bias factor's group
    prog.update_group(1, J2, scale=beta2)   # the edge factor's group (its rows repeat J once per endpoint)
    desc2 = dict(desc, ops=[("add_ising", np.arange(info["n"]), b2, info["edges"], J2, beta2)])
    ob = M.fill(O.Model(desc2["kinds"]), desc2)
    gs, os_ = T.ChainState(prog, chains), O.State(ob, chains)
    for i, a in enumerate(M.random_states(desc, chains, 3)):
        gs.upload(i, a)
        os_.set_block(i, a.astype(np.float32))
    gs.run_blocks(21, 4)
    os_.run_blocks(21, 4)
    for i in range(len(desc["free"])):
        assert np.array_equal(gs.download(i), os_.get_block(i)), i
    with pytest.raises(T.ThrmlError, match="interaction group"):
        prog.update_group(7, b2)
    with pytest.raises(T.ThrmlError, match="wdim"):
        prog.update_group(0, np.zeros((info["n"], 2), np.float32))
