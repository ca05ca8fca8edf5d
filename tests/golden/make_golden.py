"""Generates tests/golden/oracle_golden.npz from the CPU oracle: seeded small models, their compiled index tables, states
after fixed keys and sweep counts, moment sums, key splits and noise words.  The fixture freezes today's behaviour so that a
later change to the oracle or to the engine's key -> noise mapping is caught on any machine (the CUDA path is compared with
the same file on a GPU).  Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import __graft_entry__ as graft  # noqa: E402


def cases(T):
    import models as M
    return {"lattice": M.ising_lattice(T, 6, True, 101)[0], "graph": M.ising_random_graph(T, 120, 8, 102)[0], "mixed": M.mixed_model(103)[0],
            "potts": M.potts_lattice(T, 4, 4, 104)[0]}


def run_case(O, M, desc, chains=12):
    om = M.fill(O.Model(desc["kinds"], desc.get("dtype_order")), desc)
    st = O.State(om, chains)
    for i, a in enumerate(M.random_states(desc, chains, 7)):
        st.set_block(i, a.astype(np.float32))
    st.run_blocks(0xC0FFEE, 5)
    n_free = len(desc["free"])
    states = [st.get_block(i).astype(np.uint8) for i in range(n_free)]
    tables = []
    for b in range(n_free):
        for t in om.tables(b):
            tables += [t["rows"].ravel(), t["idx"].ravel(), t["active"].ravel().astype(np.int32)]
    return states, np.concatenate(tables).astype(np.int64)


def torus_case():
    """8 x 64 periodic Ising lattice, one coupling and one bias: the model both the explicit program and the implicit bit-packed
    lattice engine can run."""
    H, W, J, b, beta = 8, 64, 0.4407, 0.07, 0.9
    idx = np.arange(H * W).reshape(H, W)
    pairs = np.concatenate([np.stack([idx.ravel(), np.roll(idx, -1, axis=1).ravel()], 1), np.stack([idx.ravel(), np.roll(idx, -1, axis=0).ravel()], 1)])
    e = np.unique(np.sort(pairs, axis=1), axis=0)
    colour = (np.add.outer(np.arange(H), np.arange(W)) % 2).ravel()
    blocks = [np.flatnonzero(colour == c) for c in (0, 1)]
    n = H * W
    desc = dict(kinds=np.zeros(n, np.int32), free=[(blocks[0], 0), (blocks[1], 1)],
                ops=[("add_ising", np.arange(n), np.full(n, b, np.float32), e, np.full(len(e), J, np.float32), beta)])
    return desc, dict(H=H, W=W, J=J, b=b, beta=beta, blocks=blocks)


def potts_cube_case():
    """4 x 4 x 4 periodic Potts model, K = 3, shared direction tables: explicit factor program and implicit Potts engine alike."""
    side, K, beta = 4, 3, 0.8
    rng = np.random.default_rng(105)
    tables = rng.normal(0, 0.3, (3, K, K)).astype(np.float32)
    unary = rng.normal(0, 0.1, (side ** 3, K)).astype(np.float32)
    n = side ** 3
    idx = np.arange(n).reshape(side, side, side)
    colour = (np.add.outer(np.add.outer(np.arange(side), np.arange(side)), np.arange(side)) % 2).ravel()
    blocks = [np.flatnonzero(colour == c) for c in (0, 1)]
    ops = [("add_discrete_factor", [], [np.arange(n)], (np.float32(beta) * unary).reshape(n, K, 1).astype(np.float32))]
    for d in range(3):
        ops.append(("add_discrete_factor", [], [idx.ravel(), np.roll(idx, -1, axis=d).ravel()], np.broadcast_to((np.float32(beta) * tables[d]).astype(np.float32), (n, K, K)).copy()))
    desc = dict(kinds=np.full(n, K, np.int32), free=[(blocks[0], 0), (blocks[1], 1)], ops=ops)
    return desc, dict(side=side, K=K, beta=beta, tables=tables, unary=unary, blocks=blocks)


def run_mapped(O, M, desc, chains, sweeps, spin_noise=0, cat_noise=0, samplers=None):
    """States after `sweeps` sweeps under an engine-specific key -> noise mapping (or sampler kinds), from seeded random states."""
    om = O.Model(desc["kinds"], desc.get("dtype_order"))
    for i, (nodes, sb) in enumerate(desc["free"]):
        om.add_free_block(nodes, superblock=sb, sampler=None if samplers is None else samplers[i])
    for op in desc["ops"]:
        getattr(om, op[0])(*op[1:])
    om.compile()
    st = O.State(om, chains)
    st.set_spin_noise(spin_noise)
    st.set_cat_noise(cat_noise)
    for i, a in enumerate(M.random_states(desc, chains, 7)):
        st.set_block(i, a.astype(np.float32))
    st.run_blocks(0xC0FFEE, sweeps)
    return [st.get_block(i).astype(np.uint8) for i in range(len(desc["free"]))]


def build():
    graft.build()
    T = graft.load_package()
    from oracle import oracle as O
    import models as M
    out = {"rng_split_42_8": O.rng_split(42, 8), "rng_split_max": O.rng_split(2 ** 64 - 1, 3),
           "philox": np.array([O.philox([i, 2 * i, 7, 0x5350494E], [0xDEADBEEF, i]) for i in range(8)], dtype=np.uint32),
           "det_sigmoid": np.array([O.det_sigmoid(float(x)) for x in np.linspace(-30, 30, 61)], dtype=np.float32),
           "det_log": np.array([O.det_log(float(x)) for x in np.geomspace(1e-7, 20, 61)], dtype=np.float32)}
    for name, desc in cases(T).items():
        states, tables = run_case(O, M, desc)
        out[f"{name}_tables"] = tables
        for i, s in enumerate(states):
            out[f"{name}_state{i}"] = s
    # the engine-specific key -> noise mappings and the third sampler kind
    torus, _ = torus_case()
    for mapping in (1, 2):  # 1: the implicit lattice engine's bit-sliced mapping, 2: the dense path's
        for i, s in enumerate(run_mapped(O, M, torus, 8, 3, spin_noise=mapping)):
            out[f"torus_spin_noise{mapping}_state{i}"] = s
    cube, _ = potts_cube_case()
    for i, s in enumerate(run_mapped(O, M, cube, 12, 3, cat_noise=1)):  # the implicit Potts engine's mapping
        out[f"cube_cat_noise1_state{i}"] = s
    for i, s in enumerate(run_mapped(O, M, cube, 12, 3, samplers=[2, 1])):  # block 0 sampled by SoftmaxConditional
        out[f"cube_softmax_state{i}"] = s
    return out


if __name__ == "__main__":
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_golden.npz"), **build())
    print("written")
