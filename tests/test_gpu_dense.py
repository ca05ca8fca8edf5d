"""The dense bipartite (RBM-style) path: tcgen05 GEMM + sampling epilogue, integer tensor-core pair correlations, CD-1.

Tolerances.  The tensor cores add the same exact products (bf16 coupling x +-1) as the gather kernel but in another order.
The fields the kernel draws from are read back out of tensor memory (thrml_fields_debug on a dense block) and compared
with the oracle's f64 fields: within 1e-5 relative wherever the sum does not cancel, within 1e-6 of the summed term
magnitudes everywhere.  A sampled spin may differ from the oracle's only where the uniform lies inside the window those
two f32 fields' own measured errors open around the threshold: |logit(u) - 2 gamma_f64| <= 2 (|gamma_gpu - gamma_f64| +
|gamma_oracle_f32 - gamma_f64|) + 2e-6.  Pair correlations are integer counts and must match exactly.
"""
import numpy as np
import pytest

import fullsize_checks as F
import models as M

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def single_cta_tiles(T):
    """This file exercises the one-CTA tiles; tests/test_gpu_dense_pair.py re-runs the same checks with CTA pairs."""
    before = dict(T.Program.default_options)
    T.Program.default_options = {**before, T.OPT_DENSE_TILES: 0}
    yield
    T.Program.default_options = before


def to_bf16(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def spin_uniforms(n_nodes, chains, key, chain_offset=0):
    """u[chain][node] of the dense path's key -> noise mapping."""
    return F.spin_uniforms(n_nodes, np.arange(chains) + chain_offset, key, mapping=2)


def rbm(T, n_v, n_h, seed, sigma=0.1):
    rng = np.random.default_rng(seed)
    W = to_bf16(rng.normal(0, sigma, (n_v, n_h)))
    b = rng.normal(0, 0.2, n_v + n_h).astype(np.float32)
    vis, hid = np.arange(n_v), np.arange(n_v, n_v + n_h)
    edges = np.stack([np.repeat(vis, n_h), np.tile(hid, n_v)], axis=1)
    desc = dict(kinds=np.zeros(n_v + n_h, np.int32), free=[(vis, 0), (hid, 1)], ops=[("add_ising", np.arange(n_v + n_h), b, edges, W.ravel(), 1.0)])
    return desc, W, b


def check_update(gs, os_, block, key, W_in, chains, n_blocks):
    """GPU dense update of `block` vs the oracle from the same state; returns the mismatch count."""
    o64, o32 = os_.fields(block)
    gf = gs.fields(block).astype(np.float64)  # bias + f32 accumulator, out of tensor memory
    scale = (np.abs(W_in).sum(axis=0) if block == 1 else np.abs(W_in).sum(axis=1)) + 0.2
    err = np.abs(gf - o64)
    assert (err / scale[None, :]).max() <= 1e-6
    big = np.abs(o64) >= 0.01 * scale[None, :]
    assert (err[big] / np.abs(o64[big])).max() <= 1e-5
    gs.sample_single_block(block, key)
    os_.sample_single_block(block, key)
    g, o = gs.download(block), os_.get_block(block)
    bad = np.argwhere(g != o)
    if len(bad):
        u = spin_uniforms(g.shape[1], chains, key)
        for c, i in bad:
            uu = min(max(u[c, i], 1e-12), 1 - 1e-12)
            gap = abs(np.log(uu / (1 - uu)) - 2 * o64[c, i])
            assert gap <= 2 * (err[c, i] + abs(float(o32[c, i]) - o64[c, i])) + 2e-6, (c, i, gap)
    assert len(bad) <= max(2, g.size // 20000)
    # resynchronise so later steps compare like with like
    gs.upload(block, o.astype(np.uint8))
    return len(bad)


@pytest.mark.parametrize("n_v,n_h,chains", [(100, 200, 200), (784, 300, 256), (64, 128, 128), (130, 70, 37)])
def test_dense_update_matches_oracle(T, O, n_v, n_h, chains):
    desc, W, b = rbm(T, n_v, n_h, 3)
    gb, ob = M.build_both(T, O, desc)
    prog = T.Program(gb)
    assert prog.enable_dense(False) == 2
    assert [prog.block_kernel(i) for i in range(2)] == [3, 3]
    gs, os_ = T.ChainState(prog, chains), O.State(ob, chains)
    os_.set_spin_noise(2)  # blocks on the dense path draw their noise under that path's own mapping
    for i, a in enumerate(M.random_states(desc, chains, 5)):
        gs.upload(i, a)
        os_.set_block(i, a.astype(np.float32))
    total = 0
    for step, blk in enumerate([1, 0, 1, 0, 1]):
        total += check_update(gs, os_, blk, 1000 + step, W, chains, 2)
    # the conditional means follow the logistic law: mean_c h_j ~ mean_c sigmoid(2 gamma_j)
    o64, _ = os_.fields(1)
    gs.sample_single_block(1, 77)
    h = gs.download(1)
    p = 1 / (1 + np.exp(-2 * o64))
    z = (h.mean(axis=0) - p.mean(axis=0)) / np.sqrt((p * (1 - p)).mean(axis=0) / chains + 1e-12)
    assert np.abs(z).max() < 5.5
    gs.pair_tmem_check()


def test_dense_refuses_inexact_weights_unless_allowed(T, O):
    desc, W, b = rbm(T, 40, 48, 9)
    desc["ops"][0] = ("add_ising", np.arange(88), b, desc["ops"][0][3], (W.ravel() * np.float32(1.0001)).astype(np.float32), 1.0)
    prog = T.Program(M.fill(T.Builder(desc["kinds"]), desc))
    with pytest.raises(T.ThrmlError, match="bf16"):
        prog.enable_dense(False)
    assert prog.enable_dense(True) == 2


def test_sparse_blocks_do_not_qualify(T):
    desc, _ = M.ising_random_graph(T, 300, 8, 2)
    prog = T.Program(M.fill(T.Builder(desc["kinds"]), desc))
    assert prog.enable_dense(True) == 0


@pytest.mark.parametrize("n_a,n_b,chains", [(100, 200, 200), (784, 130, 1000), (64, 64, 4096), (5, 300, 33)])
def test_pair_correlation_is_exact(T, n_a, n_b, chains):
    kinds = np.zeros(n_a + n_b, np.int32)
    bld = T.Builder(kinds)
    bld.add_free_block(np.arange(n_a))
    bld.add_free_block(np.arange(n_a, n_a + n_b))
    bld.compile()
    st = T.ChainState(T.Program(bld), chains)
    rng = np.random.default_rng(n_a + chains)
    a = (rng.random((chains, n_a)) < 0.13).astype(np.uint8)
    b = (rng.random((chains, n_b)) < 0.6).astype(np.uint8)
    st.upload(0, a)
    st.upload(1, b)
    got = st.pair_correlation(0, 1)
    sa, sb = 2 * a.astype(np.int64) - 1, 2 * b.astype(np.int64) - 1
    want = ((sa.T @ sb).astype(np.float32) / np.float32(chains)).astype(np.float32)
    assert np.array_equal(got, want)
    got_t = st.pair_correlation(1, 0)
    assert np.array_equal(got_t, want.T)
    st.pair_tmem_check()


def test_cd1_step_composition_and_statistics(T, O):
    n_v, n_h, chains = 96, 160, 512
    desc, W, b = rbm(T, n_v, n_h, 11)
    gb, ob = M.build_both(T, O, desc)
    prog = T.Program(gb)
    prog.enable_dense(False)
    rng = np.random.default_rng(2)
    v0 = (rng.random((chains, n_v)) < 0.13).astype(np.uint8)
    st = T.ChainState(prog, chains)
    pos, neg = st.cd1_step(0, 1, v0, 99)
    v1, h1 = st.download(0, np.uint8), st.download(1, np.uint8)
    # the same step composed from its parts
    k0, k1 = [int(k) for k in T.rng_split(99, 2)]
    st2 = T.ChainState(prog, chains)
    st2.upload(0, v0)
    st2.sample_single_block(1, k0)
    h0 = st2.download(1, np.uint8)
    pos2 = st2.pair_correlation(0, 1)
    st2.sample_blocks(k1)
    neg2 = st2.pair_correlation(0, 1)
    assert np.array_equal(pos, pos2) and np.array_equal(neg, neg2)
    assert np.array_equal(v1, st2.download(0, np.uint8)) and np.array_equal(h1, st2.download(1, np.uint8))
    s = lambda x: 2.0 * x - 1.0
    assert np.array_equal(pos, (s(v0).T @ s(h0) / chains).astype(np.float32))
    assert np.array_equal(neg, (s(v1).T @ s(h1) / chains).astype(np.float32))
    # against the oracle's chain (same keys, same noise mapping): statistics agree within Monte-Carlo error
    os_ = O.State(ob, chains)
    os_.set_spin_noise(2)
    os_.set_block(0, v0.astype(np.float32))
    os_.set_block(1, np.zeros((chains, n_h), np.float32))
    os_.sample_single_block(1, k0)
    oh0 = os_.get_block(1)
    assert (oh0 != h0).mean() < 1e-3
    os_.sample_blocks(k1)
    oneg = s(os_.get_block(0)).T @ s(os_.get_block(1)) / chains
    assert np.abs(oneg - neg).max() < 6 / np.sqrt(chains)


def test_moment_observer_survives_enabling_the_dense_path(T, O):
    """An observer built while the blocks still ran the gather kernels keeps giving exact sums after the program switches
    them to the tensor-core kernel (its fused row maps are then ignored)."""
    desc, W, b = rbm(T, 48, 64, 21)
    gb, ob = M.build_both(T, O, desc)
    prog = T.Program(gb)
    spec = [[(i,) for i in range(112)], [(0, 48), (5, 60), (47, 111)]]
    mom = T.Moments(prog, spec, True)
    assert prog.enable_dense(False) == 2
    st = T.ChainState(prog, 64)
    for i, a in enumerate(M.random_states(desc, 64, 2)):
        st.upload(i, a)
    st.sample_with_observation(8, 1, 3, 1, moments=mom)
    v, h = st.download(0).astype(np.int64), st.download(1).astype(np.int64)
    # the last observation is the current state; check its contribution through a fresh observer
    mom2 = T.Moments(prog, spec, True)
    mom2.observe(st)
    s_all = 2 * np.concatenate([v, h], axis=1) - 1
    assert np.array_equal(mom2.read(0)[0], s_all.sum(axis=0))
    # an identical chain observed by an observer built after the switch accumulates the same sums
    st_b, mom_b = T.ChainState(prog, 64), T.Moments(prog, spec, True)
    for i, a in enumerate(M.random_states(desc, 64, 2)):
        st_b.upload(i, a)
    st_b.sample_with_observation(8, 1, 3, 1, moments=mom_b)
    for t in range(2):
        assert np.array_equal(mom.read(t)[0], mom_b.read(t)[0]) and mom.read(t)[1] == mom_b.read(t)[1] == 3 * 64
    assert np.array_equal(mom2.read(1)[0], np.array([(s_all[:, a] * s_all[:, c]).sum() for a, c in spec[1]]))


def test_cd1_step_from_a_resident_data_state(T):
    """thrml_cd1_step_from reads the visible data in place from another state: same correlations and same final state as
    copying the data block over and running thrml_cd1_step; the data state is left untouched."""
    n_v, n_h, chains = 96, 160, 300
    desc, W, b = rbm(T, n_v, n_h, 13)
    prog = T.Program(M.fill(T.Builder(desc["kinds"]), desc))
    assert prog.enable_dense(False) == 2
    rng = np.random.default_rng(4)
    v0 = (rng.random((chains, n_v)) < 0.13).astype(np.uint8)
    data, a, c = T.ChainState(prog, chains), T.ChainState(prog, chains), T.ChainState(prog, chains)
    data.upload(0, v0)
    for key in (41, 42):  # two steps in a row from the same data
        pos_a, neg_a = a.cd1_step(0, 1, None, key, data=data)
        c.copy_block_from(data, 0)
        pos_c, neg_c = c.cd1_step(0, 1, None, key)
        assert np.array_equal(pos_a, pos_c) and np.array_equal(neg_a, neg_c)
        for blk in (0, 1):
            assert np.array_equal(a.download(blk, np.uint8), c.download(blk, np.uint8))
        assert np.array_equal(data.download(0, np.uint8), v0)
