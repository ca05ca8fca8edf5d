"""Parity checks at the benchmark configurations' own sizes.

Chains are independent and every kernel keys its noise by the global chain id, so the CPU oracle can follow any slice of
the chains of a full-size device state at a cost of seconds: the device runs all chains, the oracle runs a few of them
from the same start with the same keys, and the states of those chains must agree bit for bit.  Observer sums are
checked against numpy on the downloaded device state.  Used by tests/test_gpu_fullsize.py (asserting) and by bench.py's
CPU leg (reporting a `parity_check` object); each function returns a dict whose "ok" says whether every comparison held.
"""
import time

import numpy as np


def sparse_ising_check(T, O, model, program, state, chains, chain_base=0, slice_chains=16, sweeps=2, edge_sample=200_000, oracle_model=None, threads=16):
    """Sparse Ising program (bench.py's model dict): hinton_init, `sweeps` sweeps with the fused moment observer on the
    device; the first and the last `slice_chains` chains followed by the oracle; one more sweep whose observation is
    compared with numpy sums over all chains of the downloaded state.  `state` is overwritten."""
    from thrml_rs_b200 import workloads as W
    t0 = time.time()
    n, blocks = model["n"], model["blocks"]
    n_blocks = len(blocks)
    biases = np.concatenate([model["b"][blk] for blk in blocks])
    spec = W.ising_moment_arrays(model)
    om = oracle_model if oracle_model is not None else W.fill_ising(O.Model(np.zeros(n, np.int32)), model)
    K_INIT, K_RUN, K_OBS = 0xC2C2_0001, 0xC2C2_0002, 0xC2C2_0003
    state.hinton_init(list(range(n_blocks)), biases, model["beta"], K_INIT)
    mom = T.Moments.from_arrays(program, *spec)
    state.sample_with_observation(K_RUN, 1, sweeps, 1, moments=mom)  # 1 + (sweeps - 1) sweeps, `sweeps` observations
    out = {"workload": "sparse_ising", "nodes": int(n), "chains": int(chains), "state_bytes": int(n) * int(-(-chains // 16) * 16), "sweeps": int(sweeps),
           "slices": [], "kernels": sorted({int(program.block_kernel(b)) for b in range(n_blocks)})}
    ok = True
    starts = sorted({0, max(chains - slice_chains, 0) // 16 * 16})
    o_sums = None
    for start in starts:
        cnt = min(slice_chains, chains - start)
        os_ = O.State(om, cnt, chain_base + start, threads=threads)
        os_.hinton_init(list(range(n_blocks)), biases, model["beta"], K_INIT)
        omom = O.Moments.from_arrays(om, *spec)
        os_.sample_with_observation(K_RUN, 1, sweeps, 1, moments=omom)
        bad = 0
        for b in range(n_blocks):
            bad += int(np.count_nonzero(state.download_chains(b, start, cnt) != os_.get_block(b).astype(np.uint8)))
        out["slices"].append({"first_chain": int(chain_base + start), "chains": int(cnt), "mismatched_spins": bad})
        ok &= bad == 0
        if chains <= slice_chains:  # the slice is the whole state: the sums must agree too
            o_sums = [omom.read(t)[0] for t in range(2)]
    if o_sums is not None:
        same = all(np.array_equal(mom.read(t)[0], o_sums[t]) for t in range(2))
        out["moment_sums_equal_oracle"] = bool(same)
        ok &= same
    # one observation against numpy on the downloaded state: all <s_i>, a sample of the <s_i s_j>
    mom2 = T.Moments.from_arrays(program, *spec)
    obs = state.sample_with_observation(K_OBS, 1, 1, 1, moments=mom2, obs_blocks=list(range(n_blocks)))[0]  # [row][chain], rows = blocks concatenated
    row_of = np.empty(n, dtype=np.int64)
    row_of[np.concatenate(blocks)] = np.arange(n)
    ones = obs.sum(axis=1, dtype=np.int64)
    m1_want = (2 * ones - chains)[row_of]
    m1, n_obs = mom2.read(0)
    m2, _ = mom2.read(1)
    edges = model["edges"]
    rng = np.random.default_rng(5)
    pick = np.sort(rng.choice(len(edges), size=min(edge_sample, len(edges)), replace=False))
    m2_bad = 0
    for lo in range(0, len(pick), 16384):
        e = edges[pick[lo:lo + 16384]]
        differ = (obs[row_of[e[:, 0]]] ^ obs[row_of[e[:, 1]]]).sum(axis=1, dtype=np.int64)
        m2_bad += int(np.count_nonzero(m2[pick[lo:lo + 16384]] != chains - 2 * differ))
    m1_bad = int(np.count_nonzero(m1 != m1_want))
    out["moments_vs_numpy"] = {"observations": int(n_obs), "first_moment_rows_checked": int(n), "first_moment_mismatches": m1_bad,
                               "second_moment_rows_checked": int(len(pick)), "second_moment_mismatches": m2_bad}
    ok &= m1_bad == 0 and m2_bad == 0 and n_obs == chains
    out["ok"] = bool(ok)
    out["seconds"] = round(time.time() - t0, 1)
    return out


def potts_check(T, O, side=64, K=10, chains=1024, slice_chains=8, sweeps=2, seed=0x5EED0004, ctx=None):
    """Implicit Potts lattice at side^3 nodes x `chains` chains against the oracle's explicit factor program on the first
    and last `slice_chains` chains; category marginals against numpy on the downloaded state."""
    from thrml_rs_b200 import potts
    t0 = time.time()
    n = side ** 3
    rng = np.random.default_rng(seed)
    tables = rng.normal(0, 0.3, (3, K, K)).astype(np.float32)
    unary = rng.normal(0, 0.1, (n, K)).astype(np.float32)
    lat = potts.PottsLattice(side, side, side, K, tables, unary, 1.0, chains, 0, ctx)
    lat.randomize(5)
    start_state = lat.download()
    lat.run_blocks(77, sweeps)
    lat.observe_marginals()
    final = lat.download()
    counts, n_obs = lat.read_marginals()
    idx = np.arange(n).reshape(side, side, side)
    colour = (np.add.outer(np.add.outer(np.arange(side), np.arange(side)), np.arange(side)) % 2).ravel()
    blocks = [np.flatnonzero(colour == c) for c in (0, 1)]
    om = O.Model(np.full(n, K, np.int32))
    for blk in blocks:
        om.add_free_block(blk)
    om.add_discrete_factor([], [np.arange(n)], unary.reshape(n, K, 1))
    for d in range(3):
        om.add_discrete_factor([], [idx.ravel(), np.roll(idx, -1, axis=d).ravel()], np.broadcast_to(tables[d], (n, K, K)).copy())
    om.compile()
    out = {"workload": "potts", "side": side, "categories": K, "chains": chains, "sweeps": sweeps, "slices": []}
    ok = True
    for start in sorted({0, (chains - slice_chains) // 16 * 16}):
        cnt = min(slice_chains, chains - start)
        os_ = O.State(om, cnt, start, threads=cnt)
        os_.set_cat_noise(1)  # the implicit engine's own key -> noise mapping (its default)
        for bi, blk in enumerate(blocks):
            os_.set_block(bi, start_state[start:start + cnt][:, blk].astype(np.float32))
        os_.run_blocks(77, sweeps)
        bad = sum(int(np.count_nonzero(final[start:start + cnt][:, blk] != os_.get_block(bi).astype(np.uint8))) for bi, blk in enumerate(blocks))
        out["slices"].append({"first_chain": int(start), "chains": int(cnt), "mismatched_nodes": bad})
        ok &= bad == 0
    want = np.stack([(final == k).sum(axis=0) for k in range(K)], axis=1)
    bad = int(np.count_nonzero(counts != want))
    out["marginals_vs_numpy"] = {"observations": int(n_obs), "cells_checked": int(want.size), "mismatches": bad}
    ok &= bad == 0 and n_obs == chains
    out["ok"] = bool(ok)
    out["seconds"] = round(time.time() - t0, 1)
    return out


def lattice_check(T, O, side=2048, chains=16, sweeps=2, stripes=4, ctx=None, J=0.4407, b=0.0, beta=1.0, noise=1):
    """Bit-packed implicit lattice at side^2 spins, held whole and as `stripes` stripes, against the oracle's explicit
    Ising program on the same torus (every chain) under the same key -> noise mapping (1 = the lattice engine's packed
    mapping, 0 = the explicit program's); the recorded observable series against numpy on the final state."""
    from thrml_rs_b200 import lattice
    t0 = time.time()
    n = side * side
    whole = lattice.DistributedStripe(side, side, J, b, beta, chains, None, ctx, noise=noise)
    whole.randomize(11)
    start = whole.download_local()  # [chain][row][col]
    whole.run_blocks(99, sweeps, record=True)
    final = whole.download_local()
    series = whole.series()
    out = {"workload": "lattice", "side": side, "chains": chains, "sweeps": sweeps, "noise_mapping": "packed" if noise == 1 else "program"}
    ok = True
    if stripes > 1:
        part = lattice.StripedLattice(side, side, J, b, beta, chains, n_stripes=stripes, ctx=ctx, noise=noise)
        part.upload(start)
        part.run_blocks(99, sweeps)
        bad = int(np.count_nonzero(part.download() != final))
        out["striped_vs_whole_mismatches"] = bad
        out["stripes"] = stripes
        ok &= bad == 0
    # oracle: the explicit program on the same torus
    _, edges, colour = T.lattice_edges(side, True)
    blocks = [np.flatnonzero(colour == c) for c in (0, 1)]
    om = O.Model(np.zeros(n, np.int32))
    for blk in blocks:
        om.add_free_block(blk)
    om.add_ising(np.arange(n), np.full(n, b, np.float32), edges, np.full(len(edges), J, np.float32), beta)
    om.compile()
    os_ = O.State(om, chains, 0, threads=chains)
    os_.set_spin_noise(noise)
    flat0, flat1 = start.reshape(chains, n), final.reshape(chains, n)
    for bi, blk in enumerate(blocks):
        os_.set_block(bi, flat0[:, blk].astype(np.float32))
    os_.run_blocks(99, sweeps)
    bad = sum(int(np.count_nonzero(flat1[:, blk] != os_.get_block(bi).astype(np.uint8))) for bi, blk in enumerate(blocks))
    out["oracle_chains"] = chains
    out["mismatched_spins_vs_oracle"] = bad
    ok &= bad == 0
    s = 2 * final.astype(np.int64) - 1
    want = np.stack([s.sum(axis=(1, 2)), (s * np.roll(s, -1, axis=1)).sum(axis=(1, 2)) + (s * np.roll(s, -1, axis=2)).sum(axis=(1, 2))])
    good = len(series) == sweeps and np.array_equal(series[-1], want)
    out["series_last_record_equals_numpy"] = bool(good)
    ok &= good
    out["ok"] = bool(ok)
    out["seconds"] = round(time.time() - t0, 1)
    return out


def _philox(c0, c1, c2, c3, k0, k1):
    c0, c1, c2, c3 = [np.asarray(x, dtype=np.uint64) for x in np.broadcast_arrays(c0, c1, c2, c3)]
    k0, k1 = np.uint64(k0), np.uint64(k1)
    m32 = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c0
        p1 = np.uint64(0xCD9E8D57) * c2
        c0, c1, c2, c3 = ((p1 >> np.uint64(32)) ^ c1 ^ k0) & m32, p1 & m32, ((p0 >> np.uint64(32)) ^ c3 ^ k1) & m32, p0 & m32
        k0 = (k0 + np.uint64(0x9E3779B9)) & m32
        k1 = (k1 + np.uint64(0xBB67AE85)) & m32
    return c0, c1, c2, c3


def spin_uniforms(n_nodes, chain_ids, key, mapping=0):
    """u[chain][node] (24-bit uniforms) for the given global chain ids.  mapping 0: the gather kernels' (one 32-bit word per
    draw, word c & 3 of Philox(n, c >> 2, 0, tag)); mapping 2: the dense path's (top 16 bits = half n & 1 of word (n >> 1) & 3
    of Philox(n >> 3, c, 1, tag), low 16 bits = low half of word c & 3 of Philox(n, c >> 2, 2, tag))."""
    node = np.arange(n_nodes, dtype=np.uint64)[None, :]
    chain = np.asarray(chain_ids, dtype=np.uint64)[:, None]
    k0, k1 = key & 0xFFFFFFFF, key >> 32
    TAG = 0x5350494E
    pick = lambda words, sel: np.choose((sel + np.zeros((len(chain_ids), n_nodes), dtype=np.uint64)).astype(np.int64), words)
    if mapping == 0:
        r = pick(_philox(node, chain >> np.uint64(2), 0, TAG, k0, k1), chain & np.uint64(3))
    else:
        tw = pick(_philox(node >> np.uint64(3), chain, 1, TAG, k0, k1), (node >> np.uint64(1)) & np.uint64(3))
        top = (tw >> (np.uint64(16) * (node & np.uint64(1)))) & np.uint64(0xFFFF)
        low = pick(_philox(node, chain >> np.uint64(2), 2, TAG, k0, k1), chain & np.uint64(3)) & np.uint64(0xFFFF)
        r = (top << np.uint64(16)) | low
    return (r >> np.uint64(8)).astype(np.float64) * 2.0 ** -24


def dense_check(T, O, n_visible=784, n_hidden=4096, chains=1024, slice_chains=16, tiles=2, ctx=None):
    """Dense bipartite path at the RBM configuration's layer sizes.  (1) The local fields the tensor-core kernel draws
    from (bias + the f32 accumulator read out of tensor memory) against the oracle's f64 fields on two chain slices.
    (2) The draws of both layers against the oracle's sampler on the same slices: a draw may differ only where the uniform
    lies inside the window the two f32 fields' own errors open around the threshold; the window actually needed is
    reported beside the count of draws that fall within 1e-6 of their threshold."""
    from thrml_rs_b200 import workloads as W
    t0 = time.time()
    model = W.rbm_ising(n_visible, n_hidden)
    program = T.Program(W.fill_ising(T.Builder(np.zeros(model["n"], np.int32)), model), ctx)
    assert program.enable_dense(False) == 2
    program.set_option(T.OPT_DENSE_TILES, tiles)
    om = W.fill_ising(O.Model(np.zeros(model["n"], np.int32)), model)
    rng = np.random.default_rng(17)
    init = [(rng.random((chains, n_visible)) < 0.13).astype(np.uint8), rng.integers(0, 2, (chains, n_hidden)).astype(np.uint8)]
    state = T.ChainState(program, chains)
    for b, a in enumerate(init):
        state.upload(b, a)
    Wm = model["W"].astype(np.float64)
    sum_abs = [np.abs(Wm).sum(axis=1) + np.abs(model["b"][:n_visible]), np.abs(Wm).sum(axis=0) + np.abs(model["b"][n_visible:])]  # per node of block 0 / 1
    out = {"workload": "rbm", "visible": n_visible, "hidden": n_hidden, "chains": chains, "tiles": {0: "single", 1: "pair", 2: "auto"}[tiles], "blocks": []}
    ok = True
    starts = sorted({0, (chains - slice_chains) // 16 * 16})
    for block, key in ((1, 0xD0D0_0001), (0, 0xD0D0_0002)):
        g_fields = state.fields(block)  # all chains, from tensor memory
        rec = {"block": "hidden" if block == 1 else "visible", "reduction_length": int(n_visible if block == 1 else n_hidden)}
        worst_abs = worst_rel = worst_scaled = 0.0
        mism = within_1e6 = draws = 0
        window_needed = 0.0
        slices = []
        for start in starts:
            cnt = min(slice_chains, chains - start)
            os_ = O.State(om, cnt, start, threads=cnt)
            os_.set_spin_noise(2)  # the dense path's key -> noise mapping
            for b in range(2):
                os_.set_block(b, state.download_chains(b, start, cnt).astype(np.float32))
            o64, o32 = os_.fields(block)
            g = g_fields[start:start + cnt].astype(np.float64)
            err = np.abs(g - o64)
            big = np.abs(o64) >= 0.01 * sum_abs[block][None, :]  # sums that do not cancel: the relative bound applies
            worst_abs = max(worst_abs, float(err.max()))
            worst_rel = max(worst_rel, float((err[big] / np.abs(o64[big])).max()) if big.any() else 0.0)
            worst_scaled = max(worst_scaled, float((err / sum_abs[block][None, :]).max()))
            slices.append((start, cnt, os_, o64, o32, g))
        rec.update({"max_abs_field_error": worst_abs, "max_rel_field_error_where_not_cancelling": worst_rel, "max_field_error_over_sum_abs_terms": worst_scaled})
        ok &= worst_rel <= 1e-5 and worst_scaled <= 1e-6
        state.sample_single_block(block, key)
        for start, cnt, os_, o64, o32, g in slices:
            os_.sample_single_block(block, key)
            got, want = state.download_chains(block, start, cnt), os_.get_block(block).astype(np.uint8)
            u = np.clip(spin_uniforms(got.shape[1], np.arange(start, start + cnt), key, mapping=2), 1e-12, 1 - 1e-12)
            gap = np.abs(np.log(u / (1 - u)) - 2 * o64)
            draws += got.size
            within_1e6 += int(np.count_nonzero(gap < 1e-6))
            bad = got != want
            mism += int(bad.sum())
            if bad.any():
                allowed = 2 * (np.abs(g - o64) + np.abs(o32.astype(np.float64) - o64)) + 2e-6
                ok &= bool(np.all(gap[bad] <= allowed[bad]))
                window_needed = max(window_needed, float(gap[bad].max()))
        rec.update({"draws_checked": draws, "draws_within_1e-6_of_threshold": within_1e6, "mismatched_draws": mism, "largest_gap_of_a_mismatch": window_needed})
        out["blocks"].append(rec)  # the next block's oracles are rebuilt from the device state, so a differing draw does not propagate
    out["ok"] = bool(ok)
    out["seconds"] = round(time.time() - t0, 1)
    return out


def mixed_check(T, O, model, program, state, chains, slice_chains=16, sweeps=2, threads=16):
    """Spin / category checkerboard (bench.py --workload mixed): `sweeps` sweeps from a seeded random start on the device, the
    first and last `slice_chains` chains followed by the oracle from the same start.  `state` is overwritten."""
    from thrml_rs_b200 import workloads as W
    t0 = time.time()
    n_blocks = len(model["blocks"])
    state.randomize(0xC6C6_0001)
    start = {}
    starts = sorted({0, max(chains - slice_chains, 0) // 16 * 16})
    for s0 in starts:
        cnt = min(slice_chains, chains - s0)
        start[s0] = [state.download_chains(b, s0, cnt) for b in range(n_blocks)]
    state.run_blocks(0xC6C6_0002, sweeps)
    om = W.fill_factors(O.Model(model["kinds"], model["dtype_order"]), model)
    out = {"workload": "mixed", "nodes": int(model["n"]), "chains": int(chains), "sweeps": int(sweeps), "slices": [],
           "kernels": [int(program.block_kernel(b)) for b in range(n_blocks)]}
    ok = True
    for s0 in starts:
        cnt = min(slice_chains, chains - s0)
        os_ = O.State(om, cnt, s0, threads=threads)
        for b in range(n_blocks):
            os_.set_block(b, start[s0][b].astype(np.float32))
        os_.run_blocks(0xC6C6_0002, sweeps)
        bad = sum(int(np.count_nonzero(state.download_chains(b, s0, cnt) != os_.get_block(b).astype(np.uint8))) for b in range(n_blocks))
        out["slices"].append({"first_chain": int(s0), "chains": int(cnt), "mismatched_nodes": bad})
        ok &= bad == 0
    out["ok"] = bool(ok)
    out["seconds"] = round(time.time() - t0, 1)
    return out
