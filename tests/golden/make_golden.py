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
    return out


if __name__ == "__main__":
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_golden.npz"), **build())
    print("written")
