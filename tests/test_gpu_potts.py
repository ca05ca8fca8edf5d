"""Implicit 3-D Potts lattice against the oracle's explicit factor program on the same torus: identical states and
category marginals."""
import numpy as np
import pytest

import models as M

pytestmark = pytest.mark.gpu


def explicit_potts(nx, ny, nz, K, tables, unary, beta):
    n = nx * ny * nz
    idx = np.arange(n).reshape(nx, ny, nz)
    colour = (np.add.outer(np.add.outer(np.arange(nx), np.arange(ny)), np.arange(nz)) % 2).ravel()
    blocks = [np.flatnonzero(colour == c) for c in (0, 1)]
    ops = [("add_discrete_factor", [], [np.arange(n)], (np.float32(beta) * unary).reshape(n, K, 1).astype(np.float32))]
    for d in range(3):
        u = idx.ravel()
        v = np.roll(idx, -1, axis=d).ravel()
        w = np.broadcast_to((np.float32(beta) * tables[d]).astype(np.float32), (n, K, K)).copy()
        ops.append(("add_discrete_factor", [], [u, v], w))
    return dict(kinds=np.full(n, K, np.int32), free=[(blocks[0], 0), (blocks[1], 1)], ops=ops), blocks


@pytest.mark.parametrize("noise", [0, 1])
@pytest.mark.parametrize("shape,K,chains", [((4, 4, 4), 3, 8), ((2, 4, 6), 10, 37), ((6, 2, 4), 5, 64), ((4, 2, 4), 7, 20),
                                            ((4, 4, 4), 5, 8192)])  # the last: millions of draws, hundreds of near-ties sent to the exact path
def test_potts_lattice_matches_explicit_program(T, O, shape, K, chains, noise):
    """noise 0: the explicit program's key -> noise mapping; noise 1: the Potts engine's own (one call per category and chain
    quad), which the oracle restates for its explicit program (set_cat_noise)."""
    check_against_explicit_program(T, O, shape, K, chains, 0.3, 0.1, noise)


@pytest.mark.parametrize("noise", [0, 1])
@pytest.mark.parametrize("shape,K,chains,sigma,usigma", [((2, 4, 6), 10, 4096, 3.0, 1.0), ((4, 4, 2), 8, 4096, 1.0, 4.0), ((2, 2, 4), 10, 4096, 30.0, 0.1)])
def test_potts_strong_couplings(T, O, shape, K, chains, sigma, usigma, noise):
    """Large table and unary magnitudes: the pre-added direction tables round differently from the canonical six adds by
    an amount that grows with the magnitudes, and the near-tie window has to grow with it."""
    check_against_explicit_program(T, O, shape, K, chains, sigma, usigma, noise)


def check_against_explicit_program(T, O, shape, K, chains, sigma, usigma, noise=1):
    from thrml_rs_b200 import potts
    nx, ny, nz = shape
    n = nx * ny * nz
    rng = np.random.default_rng(n + K)
    tables = rng.normal(0, sigma, (3, K, K)).astype(np.float32)
    unary = rng.normal(0, usigma, (n, K)).astype(np.float32)
    beta = 0.8
    desc, blocks = explicit_potts(nx, ny, nz, K, tables, unary, beta)
    om = M.fill(O.Model(desc["kinds"]), desc)
    os_ = O.State(om, chains)
    os_.set_cat_noise(noise)
    cats = rng.integers(0, K, (chains, n)).astype(np.uint8)
    for bi, blk in enumerate(blocks):
        os_.set_block(bi, cats[:, blk].astype(np.float32))
    lat = potts.PottsLattice(nx, ny, nz, K, tables, unary, beta, chains, noise=noise)
    lat.upload(cats)
    assert np.array_equal(lat.download(), cats)
    want = np.zeros((n, K), dtype=np.int64)
    for step in range(3):
        lat.run_blocks(70 + step, 2)
        os_.run_blocks(70 + step, 2)
        got = lat.download()
        for bi, blk in enumerate(blocks):
            assert np.array_equal(got[:, blk], os_.get_block(bi)), (step, bi)
        lat.observe_marginals()
        for c in range(K):
            want[:, c] += (got == c).sum(axis=0)
    counts, n_obs = lat.read_marginals()
    assert n_obs == 3 * chains and np.array_equal(counts, want)


def test_potts_randomize_and_schedule(T, O):
    from thrml_rs_b200 import potts
    K, chains = 4, 16
    tables = np.stack([2.0 * np.eye(K, dtype=np.float32)] * 3)
    lat = potts.PottsLattice(4, 4, 4, K, tables, None, 1.0, chains)
    lat.randomize(9)
    s0 = lat.download()
    assert s0.max() == K - 1 and s0.min() == 0
    lat.sample_with_marginals(5, 10, 4, 2)
    counts, n_obs = lat.read_marginals()
    assert n_obs == 4 * chains and np.all(counts.sum(axis=1) == n_obs)
    lat.reset_marginals()
    counts0, n0 = lat.read_marginals()
    assert n0 == 0 and not counts0.any()
    s = lat.download().reshape(chains, 4, 4, 4)
    agree = np.mean([(s == np.roll(s, -1, axis=a)).mean() for a in (1, 2, 3)])
    assert agree > 0.6  # T = 2 I favours equal neighbours (uniform would give 0.25)


@pytest.mark.parametrize("K,chains", [(5, 48), (3, 128), (10, 256), (16, 384), (12, 1024), (20, 128)])
def test_library_drivers_match_per_colour_calls(T, K, chains):
    """thrml_potts_run_blocks / thrml_potts_sample_with_marginals = the same key schedule driven colour by colour.  With
    full warps of chains (a multiple of 128) and at most 16 categories the library's schedule counts the categories inside
    the update kernels; the per-colour calls below always use the separate observer kernel."""
    from thrml_rs_b200 import potts
    rng = np.random.default_rng(4)
    tables = rng.normal(0, 0.4, (3, K, K)).astype(np.float32)
    unary = rng.normal(0, 0.2, (6 * 4 * 8, K)).astype(np.float32)
    a = potts.PottsLattice(6, 4, 8, K, tables, unary, 0.8, chains)
    b = potts.PottsLattice(6, 4, 8, K, tables, unary, 0.8, chains)
    a.randomize(3)
    b.randomize(3)
    a.sample_with_marginals(21, 2, 3, 2)
    k_warm, k_samp = [int(k) for k in T.rng_split(21, 2)]
    for k in T.rng_split(k_warm, 2):
        b.sample_blocks(int(k))
    b.observe_marginals()
    for ks in T.rng_split(k_samp, 2):
        for k in T.rng_split(int(ks), 2):
            b.sample_blocks(int(k))
        b.observe_marginals()
    assert np.array_equal(a.download(), b.download())
    ca, na = a.read_marginals()
    cb, nb = b.read_marginals()
    assert na == nb == 3 * chains and np.array_equal(ca, cb)
