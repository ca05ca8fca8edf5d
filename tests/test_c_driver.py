"""A host in plain C (tests/c_driver.c) against include/thrml_b200.h: the header is valid C99, the program links with
nothing but the shared library, and on a GPU its results equal the oracle's."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "thrml-rs_b200")


def build_driver(tmp_path):
    exe = str(tmp_path / "c_driver")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-O1", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "c_driver.c"),
                    "-L", LIBDIR, "-lthrml_b200", "-Wl,-rpath," + LIBDIR, "-o", exe], check=True)
    return exe


def test_c_host_compiles_and_links(T, tmp_path):
    build_driver(tmp_path)


@pytest.mark.gpu
def test_c_host_matches_oracle(T, O, tmp_path):
    chains, key = 48, 11
    exe = build_driver(tmp_path)
    run = subprocess.run([exe, str(chains), str(key)], capture_output=True, text=True)
    assert run.returncode == 0, run.stderr
    out = run.stdout.split()
    checksum, n_obs, t1, w1, t2, w2 = (int(x) for x in out)
    side, edges, colour = T.lattice_edges(16, True)
    n = side * side
    bias = np.array([0.05 * ((i * 37) % 11 - 5) for i in range(n)], dtype=np.float32)
    J = np.array([0.3 + 0.01 * (e % 7) for e in range(len(edges))], dtype=np.float32)
    blocks = [np.flatnonzero(colour == c) for c in (0, 1)]
    om = O.Model(np.zeros(n, np.int32))
    for c, blk in enumerate(blocks):
        om.add_free_block(blk, superblock=c)
    om.add_ising(np.arange(n), bias, edges, J, 1.0)
    om.compile()
    st = O.State(om, chains)
    st.hinton_init([0, 1], np.concatenate([bias[blk] for blk in blocks]), 1.0, key)
    spec = [[(i,) for i in range(n)], [tuple(int(x) for x in e) for e in edges]]
    mom = O.Moments(om, spec, True)
    st.sample_with_observation(key + 1, 20, 31, 2, moments=mom)
    h = 1469598103934665603
    for c in range(2):
        for v in st.get_block(c).astype(np.uint8).ravel():  # [chain][node]
            h = ((h ^ int(v)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    s1, n1 = mom.read(0)
    s2, n2 = mom.read(1)
    assert n_obs == n1 == n2 == 31 * chains
    assert (t1, w1) == (int(s1.sum()), int((np.arange(1, n + 1) * s1).sum()))
    assert (t2, w2) == (int(s2.sum()), int((np.arange(1, len(edges) + 1) * s2).sum()))
    assert checksum == h
