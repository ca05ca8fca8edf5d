"""Seeded synthetic inputs for the benchmark configurations (the reference ships no datasets for this path)."""
import numpy as np

from . import engine as _eng


def random_regular_edges(n_nodes, degree, seed):
    """Configuration model: `degree` stubs per node, seeded Fisher-Yates shuffle of the stub list, consecutive stubs
    paired, self-loops and duplicate edges erased.  Edges come back sorted by (min, max)."""
    rng = np.random.default_rng(seed)
    stubs = np.repeat(np.arange(n_nodes, dtype=np.int64), degree)
    rng.shuffle(stubs)
    a, b = stubs[0::2], stubs[1::2]
    lo, hi = np.minimum(a, b), np.maximum(a, b)
    code = np.unique(lo[lo != hi] * n_nodes + hi[lo != hi])
    return np.stack([code // n_nodes, code % n_nodes], axis=1)


def random_graph_edges(n_nodes, mean_degree, seed):
    """Erdos-Renyi-like graph: n * mean_degree / 2 endpoint pairs drawn uniformly, self-loops and duplicates erased, so
    degrees are Poisson-distributed around the mean.  Edges come back sorted by (min, max)."""
    rng = np.random.default_rng(seed)
    m = n_nodes * mean_degree // 2
    a, b = rng.integers(0, n_nodes, m), rng.integers(0, n_nodes, m)
    lo, hi = np.minimum(a, b), np.maximum(a, b)
    code = np.unique(lo[lo != hi] * n_nodes + hi[lo != hi])
    return np.stack([code // n_nodes, code % n_nodes], axis=1)


def sparse_ising(n_nodes=1 << 20, degree=8, seed=0x5EED0002, bias_sigma=0.05, beta=1.0, regular=True, ctx=None):
    """Sparse random Ising model, `degree`-regular (at most `degree` neighbours per node) or, with regular=False, a
    random graph with that mean degree: couplings N(0, 1/degree), biases N(0, bias_sigma^2), blocks from greedy colouring
    in node order (ascending node index inside each colour).  With a device context the colouring runs on that device."""
    edges = random_regular_edges(n_nodes, degree, seed) if regular else random_graph_edges(n_nodes, degree, seed)
    rng = np.random.default_rng(seed + 1)
    J = rng.normal(0.0, np.sqrt(1.0 / degree), len(edges)).astype(np.float32)
    b = rng.normal(0.0, bias_sigma, n_nodes).astype(np.float32)
    colour, n_colours = _eng.greedy_coloring_arrays(n_nodes, edges, ctx)
    blocks = [np.flatnonzero(colour == c).astype(np.int64) for c in range(n_colours)]
    return dict(n=n_nodes, edges=edges, J=J, b=b, beta=float(beta), colour=colour, blocks=blocks)


def fill_ising(builder, model, ctx=None):
    """Feed a sparse_ising() model to a builder (the library's or any object with the same methods); with a device context
    the library's builder compiles its slot tables on that device."""
    for i, blk in enumerate(model["blocks"]):
        builder.add_free_block(blk, superblock=i)
    builder.add_ising(np.arange(model["n"], dtype=np.int64), model["b"], model["edges"], model["J"], model["beta"])
    builder.compile() if ctx is None else builder.compile(ctx)
    return builder


def ising_moment_arrays(model):
    """CSR form of MomentAccumulatorObserver::ising_moment_spec(all nodes, all edges)."""
    n, e = model["n"], len(model["edges"])
    rows_per_type = np.array([n, e], dtype=np.int64)
    row_ptr = np.concatenate([np.arange(n + 1, dtype=np.int64), n + 2 * np.arange(1, e + 1, dtype=np.int64)])
    members = np.concatenate([np.arange(n, dtype=np.int64), model["edges"].astype(np.int64).ravel()])
    return rows_per_type, row_ptr, members


def to_bf16(x):
    """Round f32 values to the nearest bf16 value (ties to even), returned as f32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def rbm_ising(n_visible=784, n_hidden=4096, seed=0x5EED0003, w_sigma=0.01, bias_sigma=0.01):
    """Bipartite RBM-style Ising model: dense couplings N(0, w_sigma^2) held as bf16 values, biases N(0, bias_sigma^2);
    two blocks (visible, hidden); edges (v, h) in row-major order."""
    rng = np.random.default_rng(seed)
    W = to_bf16(rng.normal(0.0, w_sigma, (n_visible, n_hidden)))
    b = rng.normal(0.0, bias_sigma, n_visible + n_hidden).astype(np.float32)
    vis = np.arange(n_visible, dtype=np.int64)
    hid = np.arange(n_visible, n_visible + n_hidden, dtype=np.int64)
    edges = np.stack([np.repeat(vis, n_hidden), np.tile(hid, n_visible)], axis=1)
    return dict(n=n_visible + n_hidden, n_visible=n_visible, n_hidden=n_hidden, W=W, b=b, edges=edges, J=W.ravel().copy(), beta=1.0, blocks=[vis, hid])


def spin_category_checkerboard(side=512, K=4, seed=0x5EED0006):
    """Mixed discrete EBM on a periodic side x side grid: spins on one checkerboard colour, K-state nodes on the other, so every
    spin has four categorical neighbours (factors with a [K] weight row and a categorical tail for the spin, a spin tail for
    the category) and the other way round; spins of even rows also carry a three-spin term with their two diagonal spins
    of the next row.  Three blocks: spins of even rows, spins of odd rows, all K-state nodes.  Returns the pieces a builder
    takes: kinds, dtype_order, blocks, factor ops (method name and arguments)."""
    rng = np.random.default_rng(seed)
    idx = np.arange(side * side, dtype=np.int64).reshape(side, side)
    colour = np.add.outer(np.arange(side), np.arange(side)) % 2
    row = idx // side
    spins, cats = np.sort(idx[colour == 0]), np.sort(idx[colour == 1])
    even, odd = np.sort(idx[(colour == 0) & (row % 2 == 0)]), np.sort(idx[(colour == 0) & (row % 2 == 1)])
    kinds = np.where(colour.ravel() == 0, 0, K).astype(np.int32)
    ops = [("add_discrete_factor", [spins], [], rng.normal(0, 0.2, (spins.size, 1, 1)).astype(np.float32)),
           ("add_discrete_factor", [], [cats], rng.normal(0, 0.2, (cats.size, K, 1)).astype(np.float32))]
    for axis in (1, 0):
        a, b = idx.ravel(), np.roll(idx, -1, axis=axis).ravel()
        m = colour.ravel()[a] == 0  # a is the spin of the pair
        ops.append(("add_discrete_factor", [a[m]], [b[m]], rng.normal(0, 0.4, (int(m.sum()), K, 1)).astype(np.float32)))
        ops.append(("add_discrete_factor", [b[~m]], [a[~m]], rng.normal(0, 0.4, (int((~m).sum()), K, 1)).astype(np.float32)))
    r, c = even // side, even % side
    below = ((r + 1) % side) * side
    ops.append(("add_discrete_factor", [even, below + (c + 1) % side, below + (c - 1) % side], [], rng.normal(0, 0.3, (even.size, 1, 1)).astype(np.float32)))
    return dict(n=side * side, side=side, K=K, kinds=kinds, dtype_order=[0, K], blocks=[even, odd, cats], ops=ops)


def fill_factors(builder, model, ctx=None):
    """Feed a spin_category_checkerboard() model to a builder (the library's or any object with the same methods)."""
    for i, blk in enumerate(model["blocks"]):
        builder.add_free_block(blk, superblock=i)
    for op in model["ops"]:
        getattr(builder, op[0])(*op[1:])
    builder.compile() if ctx is None else builder.compile(ctx)
    return builder
