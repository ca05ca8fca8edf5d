"""Synthetic workload generators (thrml-rs_b200/workloads.py): the library's host compiler and the oracle compile the same
tables from them, and the oracle can sweep them — all on the CPU."""
import numpy as np

from test_index_tables import assert_same_tables


def test_sparse_ising_generator(T, O):
    from thrml_rs_b200 import workloads as W
    for regular in (True, False):
        model = W.sparse_ising(512, 8, 7, regular=regular)
        assert sorted(np.concatenate(model["blocks"]).tolist()) == list(range(512))
        colour = model["colour"]
        e = model["edges"]
        assert np.all(colour[e[:, 0]] != colour[e[:, 1]])  # a proper colouring
        if regular:
            assert np.bincount(e.ravel(), minlength=512).max() <= 8
        gb = W.fill_ising(T.Builder(np.zeros(512, np.int32)), model)
        ob = W.fill_ising(O.Model(np.zeros(512, np.int32)), model)
        assert_same_tables(gb, ob)
        rows_per_type, row_ptr, members = W.ising_moment_arrays(model)
        assert rows_per_type.tolist() == [512, len(e)] and row_ptr[-1] == len(members) == 512 + 2 * len(e)


def test_checkerboard_generator(T, O):
    from thrml_rs_b200 import workloads as W
    model = W.spin_category_checkerboard(8, 4)
    assert [len(b) for b in model["blocks"]] == [16, 16, 32]
    gb = W.fill_factors(T.Builder(model["kinds"], model["dtype_order"]), model)
    ob = W.fill_factors(O.Model(model["kinds"], model["dtype_order"]), model)
    assert_same_tables(gb, ob)
    # spins of even rows: a bias, four categorical neighbours, one three-spin term; the 4-state nodes: a bias and four spins
    assert sum(int(t["active"].reshape(16, -1).sum(axis=1).max()) for t in gb.tables(0)) == 6
    assert sum(int(t["active"].reshape(32, -1).sum(axis=1).max()) for t in gb.tables(2)) == 5
    st = O.State(ob, 4)
    st.randomize(1)
    st.run_blocks(2, 2)
    assert st.get_block(2).max() <= 3


def test_rbm_generator_values_are_bf16(T):
    from thrml_rs_b200 import workloads as W
    m = W.rbm_ising(8, 16, 3)
    assert m["edges"].shape == (128, 2) and np.array_equal(W.to_bf16(m["W"]), m["W"])
    assert np.all(m["W"].view(np.uint32) & 0xFFFF == 0)
