"""Implicit bit-packed lattice engine against the oracle's explicit Ising program on the same torus: same states bit for
bit, whole or in stripes; observables against numpy."""
import numpy as np
import pytest

import models as M

pytestmark = pytest.mark.gpu


def torus_model(H, W, J, b, beta):
    idx = np.arange(H * W).reshape(H, W)
    pairs = np.concatenate([np.stack([idx.ravel(), np.roll(idx, -1, axis=1).ravel()], 1), np.stack([idx.ravel(), np.roll(idx, -1, axis=0).ravel()], 1)])
    e = np.unique(np.sort(pairs, axis=1), axis=0)  # ascending (min, max), duplicates erased: make_nearest_neighbor_lattice's edge set
    colour = (np.add.outer(np.arange(H), np.arange(W)) % 2).ravel()
    blocks = [np.flatnonzero(colour == c) for c in (0, 1)]
    n = H * W
    desc = dict(kinds=np.zeros(n, np.int32), free=[(blocks[0], 0), (blocks[1], 1)],
                ops=[("add_ising", np.arange(n), np.full(n, b, np.float32), e, np.full(len(e), J, np.float32), beta)])
    return desc, blocks, e


@pytest.mark.parametrize("noise", [0, 1, 2])
@pytest.mark.parametrize("H,W,chains,stripes", [(8, 64, 16, 1), (6, 128, 4, 1), (8, 64, 16, 2), (12, 64, 8, 3), (4, 192, 32, 2), (16, 256, 64, 1)])
def test_lattice_matches_explicit_program(T, O, H, W, chains, stripes, noise):
    """noise 0: the explicit program's key -> noise mapping; noise 1: the lattice engine's packed mapping, which the oracle
    restates for its explicit program (set_spin_noise).  Fields, thresholds and the draw rule are the same in both."""
    from thrml_rs_b200 import lattice
    J, b, beta = 0.4407, 0.07, 0.9
    desc, blocks, edges = torus_model(H, W, J, b, beta)
    om = M.fill(O.Model(desc["kinds"]), desc)
    os_ = O.State(om, chains)
    os_.set_spin_noise(min(noise, 1))  # 2 = mapping 1 through the table route
    rng = np.random.default_rng(H * W + chains)
    spins = rng.integers(0, 2, (chains, H, W)).astype(np.uint8)
    flat = spins.reshape(chains, H * W)
    for bi, blk in enumerate(blocks):
        os_.set_block(bi, flat[:, blk].astype(np.float32))
    lat = lattice.StripedLattice(H, W, J, b, beta, chains, n_stripes=stripes, noise=noise)
    lat.upload(spins)
    assert np.array_equal(lat.download(), spins)
    for step, n_iters in enumerate([1, 3]):
        lat.run_blocks(40 + step, n_iters)
        os_.run_blocks(40 + step, n_iters)
        got = lat.download().reshape(chains, H * W)
        for bi, blk in enumerate(blocks):
            assert np.array_equal(got[:, blk], os_.get_block(bi)), (step, bi)
    # observables
    s = 2.0 * lat.download().astype(np.int64) - 1
    want_m = s.sum(axis=(1, 2))
    want_b = (s * np.roll(s, -1, axis=1)).sum(axis=(1, 2)) + (s * np.roll(s, -1, axis=2)).sum(axis=(1, 2))
    obs = lat.observe()
    assert np.array_equal(obs[0], want_m) and np.array_equal(obs[1], want_b)


def test_lattice_randomize_matches_explicit_randomize(T, O):
    from thrml_rs_b200 import lattice
    H, W, chains = 4, 64, 8
    desc, blocks, _ = torus_model(H, W, 0.3, 0.0, 1.0)
    prog = T.Program(M.fill(T.Builder(desc["kinds"]), desc))
    st = T.ChainState(prog, chains)
    st.randomize(5)
    lat = lattice.StripedLattice(H, W, 0.3, 0.0, 1.0, chains, noise=lattice.NOISE_PROGRAM)
    lat.randomize(5)
    got = lat.download().reshape(chains, H * W)
    for bi, blk in enumerate(blocks):
        assert np.array_equal(got[:, blk], st.download(bi, np.uint8))


def test_lattice_argument_checks(T):
    from thrml_rs_b200 import lattice
    with pytest.raises(T.ThrmlError, match="multiple of 64"):
        lattice.LatticeStripe(8, 60, 0, 8, 0.4, 0.0, 1.0, 16)
    with pytest.raises(T.ThrmlError, match="n_chains"):
        lattice.LatticeStripe(8, 64, 0, 8, 0.4, 0.0, 1.0, 6)
    with pytest.raises(T.ThrmlError, match="out of range"):
        lattice.LatticeStripe(8, 64, 4, 8, 0.4, 0.0, 1.0, 16)


@pytest.mark.parametrize("noise", [0, 1, 2])
@pytest.mark.parametrize("H,W,chains", [(8, 64, 16), (6, 192, 4), (16, 128, 32), (4, 64, 256)])
def test_library_sweep_driver_bits_and_series(T, H, W, chains, noise):
    """thrml_lattice_run_blocks on a whole lattice = the per-colour calls driven from the host; the bit-packed transfers
    round-trip; the recorded series holds, per sweep, the sums thrml_lattice_observe would report; moments follow."""
    from thrml_rs_b200 import lattice
    J, b, beta = (0.4407, 0.05, 1.0) if chains != 32 else (1.7, -0.6, 1.0)  # the second set saturates some thresholds (probabilities near 0 and 1)
    rng = np.random.default_rng(H + W)
    spins = rng.integers(0, 2, (chains, H, W)).astype(np.uint8)
    host_driven = lattice.StripedLattice(H, W, J, b, beta, chains, n_stripes=1, noise=noise)
    host_driven.upload(spins)
    lib = lattice.DistributedStripe(H, W, J, b, beta, chains, None, noise=noise)
    bits = np.packbits(spins.reshape(chains, H, W // 32, 32), axis=3, bitorder="little").view("<u4").reshape(chains, H, W // 32)
    lib.upload_bits(bits)
    assert np.array_equal(lib.download_local(), spins)
    assert np.array_equal(lib.stripe.download_bits(), bits)
    want_series = []
    for k in T.rng_split(31, 3):
        host_driven.sample_blocks(int(k))
        want_series.append(host_driven.observe())
    lib.run_blocks(31, 3, record=True)
    assert np.array_equal(lib.download_local(), host_driven.download())
    series = lib.series()
    assert series.shape == (3, 2, chains) and np.array_equal(series, np.stack(want_series))
    mom, n_rec = lib.moments()
    N = H * W
    m = series[:, 0, :] / N
    e = -(float(np.float32(J)) * series[:, 1, :] + float(np.float32(b)) * series[:, 0, :]) / N  # the handle keeps J and b as f32
    assert n_rec == 3
    assert np.allclose(mom, np.stack([m.mean(0), (m * m).mean(0), e.mean(0), (e * e).mean(0)]), rtol=1e-12, atol=1e-15)
    lib.series_reset()
    lib.run_blocks(32, 1, record=True)
    assert lib.series().shape == (1, 2, chains)
    # the series keeps growing past its first allocation
    lib.series_reset()
    lib.run_blocks(33, 1100, record=True)
    s = 2 * lib.download_local().astype(np.int64) - 1
    last = np.stack([s.sum(axis=(1, 2)), (s * np.roll(s, -1, axis=1)).sum(axis=(1, 2)) + (s * np.roll(s, -1, axis=2)).sum(axis=(1, 2))])
    series = lib.series()
    assert series.shape[0] == 1100 and np.array_equal(series[-1], last)


def test_partial_stripe_needs_a_communicator(T):
    from thrml_rs_b200 import lattice
    s = lattice.LatticeStripe(8, 64, 0, 4, 0.4, 0.0, 1.0, 16)
    from thrml_rs_b200._ffi import check
    with pytest.raises(T.ThrmlError, match="communicator"):
        check(T.lib().thrml_lattice_run_blocks(s.h, 1, 1, None, 0))
