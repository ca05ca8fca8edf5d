"""Seeded model descriptions fed identically to the library's Builder and the oracle's Model (same method names)."""
import numpy as np


def fill(bld, desc):
    """desc: dict(free=[(nodes, superblock)], clamped=[nodes], ops=[(method, args...)]).  Returns bld compiled."""
    for nodes, sb in desc["free"]:
        bld.add_free_block(nodes, superblock=sb)
    for nodes in desc.get("clamped", []):
        bld.add_clamped_block(nodes)
    for op in desc["ops"]:
        getattr(bld, op[0])(*op[1:])
    bld.compile()
    return bld


def ising_lattice(T, side, torus, seed, J=0.44, bias_sigma=0.1, beta=1.0):
    rng = np.random.default_rng(seed)
    side, edges, colour = T.lattice_edges(side, torus)
    n = side * side
    b = rng.normal(0, bias_sigma, n).astype(np.float32)
    Jv = np.full(len(edges), J, dtype=np.float32)
    blocks = [np.flatnonzero(colour == c) for c in (0, 1)]
    desc = dict(kinds=np.zeros(n, np.int32), free=[(blocks[0], 0), (blocks[1], 1)], ops=[("add_ising", np.arange(n), b, edges, Jv, beta)])
    return desc, dict(n=n, edges=edges, b=b, J=Jv, blocks=blocks, beta=beta)


def random_regular_graph(n, degree, seed):
    """Configuration model: `degree` stubs per node, seeded shuffle, consecutive stubs paired, self-loops and duplicate
    edges erased; edges returned sorted by (min,max)."""
    rng = np.random.default_rng(seed)
    stubs = np.repeat(np.arange(n, dtype=np.int64), degree)
    rng.shuffle(stubs)
    a, b = stubs[0::2], stubs[1::2]
    lo, hi = np.minimum(a, b), np.maximum(a, b)
    keep = lo != hi
    e = np.unique(np.stack([lo[keep], hi[keep]], axis=1), axis=0)
    return e


def ising_random_graph(T, n, degree, seed, w_sigma=None, bias_sigma=0.05, beta=1.0):
    rng = np.random.default_rng(seed + 1)
    edges = random_regular_graph(n, degree, seed)
    colour, n_col = T.greedy_coloring_arrays(n, edges)
    w_sigma = w_sigma if w_sigma is not None else 1.0 / np.sqrt(degree)
    Jv = rng.normal(0, w_sigma, len(edges)).astype(np.float32)
    b = rng.normal(0, bias_sigma, n).astype(np.float32)
    blocks = [np.flatnonzero(colour == c) for c in range(n_col)]
    desc = dict(kinds=np.zeros(n, np.int32), free=[(blk, i) for i, blk in enumerate(blocks)], ops=[("add_ising", np.arange(n), b, edges, Jv, beta)])
    return desc, dict(n=n, edges=edges, b=b, J=Jv, blocks=blocks, beta=beta, colour=colour)


def ising_sparse_random_graph(T, n, mean_degree, seed, w_sigma=0.3, bias_sigma=0.1, beta=1.0):
    """Erdos-Renyi-like Ising model: n * mean_degree / 2 random distinct edges, so degrees spread around the mean
    (a few nodes far above it); greedy-coloured blocks."""
    rng = np.random.default_rng(seed)
    m = n * mean_degree // 2
    a, b = rng.integers(0, n, 2 * m), rng.integers(0, n, 2 * m)
    lo, hi = np.minimum(a, b), np.maximum(a, b)
    edges = np.unique(np.stack([lo[lo != hi], hi[lo != hi]], axis=1), axis=0)[:m]
    colour, n_col = T.greedy_coloring_arrays(n, edges)
    Jv = rng.normal(0, w_sigma, len(edges)).astype(np.float32)
    bias = rng.normal(0, bias_sigma, n).astype(np.float32)
    blocks = [np.flatnonzero(colour == c) for c in range(n_col)]
    desc = dict(kinds=np.zeros(n, np.int32), free=[(blk, i) for i, blk in enumerate(blocks)], ops=[("add_ising", np.arange(n), bias, edges, Jv, beta)])
    degree = np.bincount(edges.ravel(), minlength=n)
    return desc, dict(n=n, edges=edges, b=bias, J=Jv, blocks=blocks, beta=beta, colour=colour, degree=degree)


def potts_lattice(T, side, K, seed, sigma=0.3, bias_sigma=0.1):
    """2-D periodic Potts model: unary [n,K,1] factor plus one [E,K,K] pair factor per direction with a shared table."""
    rng = np.random.default_rng(seed)
    n = side * side
    idx = np.arange(n).reshape(side, side)
    colour = (np.add.outer(np.arange(side), np.arange(side)) % 2).ravel()
    blocks = [np.flatnonzero(colour == c) for c in (0, 1)]
    unary = rng.normal(0, bias_sigma, (n, K, 1)).astype(np.float32)
    ops = [("add_discrete_factor", [], [np.arange(n)], unary)]
    for axis in (0, 1):
        tab = rng.normal(0, sigma, (K, K)).astype(np.float32)
        u = idx.ravel()
        v = np.roll(idx, -1, axis=axis).ravel()
        w = np.broadcast_to(tab, (n, K, K)).copy()
        ops.append(("add_discrete_factor", [], [u, v], w))
    desc = dict(kinds=np.full(n, K, np.int32), free=[(blocks[0], 0), (blocks[1], 1)], ops=ops)
    return desc, dict(n=n, K=K, blocks=blocks)


def potts_random_graph(T, n, degree, K, seed, sigma=0.3, with_spins=False):
    """K-state nodes on a random regular graph with one [K, K] table per edge and a unary factor: degree + 1 active slots per
    node.  with_spins adds a block of spins coupled to the categorical nodes through [K]-weight factors with a spin tail."""
    rng = np.random.default_rng(seed)
    edges = random_regular_graph(n, degree, seed)
    colour, n_col = T.greedy_coloring_arrays(n, edges)
    blocks = [np.flatnonzero(colour == c) for c in range(n_col)]
    n_all = n + (n if with_spins else 0)
    kinds = np.concatenate([np.full(n, K, np.int32), np.zeros(n_all - n, np.int32)])
    ops = [("add_discrete_factor", [], [np.arange(n)], rng.normal(0, 0.1, (n, K, 1)).astype(np.float32)),
           ("add_discrete_factor", [], [edges[:, 0], edges[:, 1]], rng.normal(0, sigma, (len(edges), K, K)).astype(np.float32))]
    free = [(blk, i) for i, blk in enumerate(blocks)]
    if with_spins:
        spins = np.arange(n, 2 * n)
        free.append((spins, n_col))
        ops.append(("add_discrete_factor", [spins], [np.arange(n)], rng.normal(0, 0.4, (n, K, 1)).astype(np.float32)))
    desc = dict(kinds=kinds, free=free, ops=ops, dtype_order=[K, 0] if with_spins else None)
    return desc, dict(n=n, K=K, edges=edges, blocks=blocks)


def mixed_model(seed, n_spin=12, n_cat=10, K=4, with_clamped=True, superblock_pair=False, two_cat_tails=False):
    """Spins and categorical nodes with spin-spin, spin-cat, cat-cat and three-spin factors, random blocks."""
    rng = np.random.default_rng(seed)
    n = n_spin + n_cat
    kinds = np.concatenate([np.zeros(n_spin, np.int32), np.full(n_cat, K, np.int32)])
    spins, cats = np.arange(n_spin), np.arange(n_spin, n)
    sp = rng.permutation(spins)
    ct = rng.permutation(cats)
    free = [(np.sort(sp[: n_spin // 3]), 0), (np.sort(sp[n_spin // 3: 2 * n_spin // 3]), 0 if superblock_pair else 1), (np.sort(ct[: n_cat // 2]), 2)]
    rest_spin, rest_cat = np.sort(sp[2 * n_spin // 3:]), np.sort(ct[n_cat // 2:])
    clamped = []
    if with_clamped:
        clamped = [rest_spin, rest_cat]
    else:
        free += [(rest_spin, 3), (rest_cat, 4)]
    ops = []
    ops.append(("add_discrete_factor", [spins], [], rng.normal(0, 0.3, (n_spin, 1, 1)).astype(np.float32)))
    ops.append(("add_discrete_factor", [], [cats], rng.normal(0, 0.3, (n_cat, K, 1)).astype(np.float32)))
    m = 14
    ops.append(("add_discrete_factor", [rng.integers(0, n_spin, m), rng.integers(0, n_spin, m)], [], rng.normal(0, 0.5, (m, 1, 1)).astype(np.float32)))
    m = 9
    ops.append(("add_discrete_factor", [rng.integers(0, n_spin, m), rng.integers(0, n_spin, m), rng.integers(0, n_spin, m)], [], rng.normal(0, 0.4, (m, 1, 1)).astype(np.float32)))
    m = 11
    ops.append(("add_discrete_factor", [rng.integers(0, n_spin, m)], [rng.integers(n_spin, n, m)], rng.normal(0, 0.5, (m, K, 1)).astype(np.float32)))
    m = 13
    ops.append(("add_discrete_factor", [], [rng.integers(n_spin, n, m), rng.integers(n_spin, n, m)], rng.normal(0, 0.5, (m, K, K)).astype(np.float32)))
    if two_cat_tails:  # index compilation only: the samplers honour one categorical tail per group
        m = 7
        ops.append(("add_discrete_factor", [rng.integers(0, n_spin, m)], [rng.integers(n_spin, n, m), rng.integers(n_spin, n, m)], rng.normal(0, 0.5, (m, K, K)).astype(np.float32)))
    desc = dict(kinds=kinds, free=free, clamped=clamped, ops=ops, dtype_order=[0, K])
    return desc, dict(n_spin=n_spin, n_cat=n_cat, K=K)


def build_both(T, O, desc):
    order = desc.get("dtype_order")
    gb = fill(T.Builder(desc["kinds"], order), desc)
    ob = fill(O.Model(desc["kinds"], order), desc)
    return gb, ob


def random_states(desc, chains, seed):
    """Per block (free ++ clamped) a uint8 [chains, n] array of valid values."""
    rng = np.random.default_rng(seed)
    out = []
    for nodes in [f[0] for f in desc["free"]] + list(desc.get("clamped", [])):
        kind = int(desc["kinds"][nodes[0]])
        hi = 2 if kind == 0 else kind
        out.append(rng.integers(0, hi, (chains, len(nodes))).astype(np.uint8))
    return out
