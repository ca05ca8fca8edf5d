"""Index compilation: the library's builder against the oracle, bit for bit, and against the reference's own
known answers (crates/thrml-core/tests/test_block.rs, crates/thrml-models/tests/test_factor.rs, test_discrete_ebm.rs)
and the hand-derived 5-spin chain tables."""
import numpy as np
import pytest

import models as M


def assert_same_tables(gb, ob):
    assert gb.counts() == ob.counts()
    n_free, _, n_groups, _ = gb.counts()
    for g in range(n_groups):
        a, b = gb.group(g), ob.group(g)
        assert a["n_spin"] == b["n_spin"]
        for key in ("head", "tails", "w"):
            assert np.array_equal(a[key], b[key]), (g, key)
    for blk in range(n_free):
        ta, tb = gb.tables(blk), ob.tables(blk)
        assert len(ta) == len(tb)
        for x, y in zip(ta, tb):
            for key in ("k", "wdim", "n_spin", "source_group"):
                assert x[key] == y[key], (blk, key)
            for key in ("rows", "active", "idx", "tail_sd"):
                assert np.array_equal(x[key], y[key]), (blk, key)
            assert x["w"].tobytes() == y["w"].tobytes(), (blk, "w")


@pytest.mark.parametrize("seed", range(6))
def test_mixed_models_match_oracle(T, O, seed):
    desc, _ = M.mixed_model(seed, with_clamped=bool(seed % 2), superblock_pair=bool(seed % 3 == 0), two_cat_tails=True)
    gb, ob = M.build_both(T, O, desc)
    assert_same_tables(gb, ob)
    for node in range(len(desc["kinds"])):
        assert gb.node_location(node) == ob.node_location(node)


def test_lattice_and_random_graph_match_oracle(T, O):
    desc, _ = M.ising_lattice(T, 6, True, 3)
    assert_same_tables(*M.build_both(T, O, desc))
    desc, info = M.ising_random_graph(T, 500, 8, 5)
    gb, ob = M.build_both(T, O, desc)
    assert_same_tables(gb, ob)
    # every node's slots are its incident edges: first those where it is edge.0, then edge.1, each in edge order
    edges = info["edges"]
    for blk, nodes in enumerate(info["blocks"]):
        tab = gb.tables(blk)[1]
        for i, nd in enumerate(nodes[:20]):
            first = [e for e in range(len(edges)) if edges[e, 0] == nd]
            second = [len(edges) + e for e in range(len(edges)) if edges[e, 1] == nd]
            want = first + second
            assert list(tab["rows"][i][: len(want)]) == want
            assert tab["active"][i].sum() == len(want)


def test_blockspec_positions_kat(T):
    # crates/thrml-core/tests/test_block.rs:131-153: blocks of 3 and 4 spins -> positions [0,1,2] and [3,4,5,6], class 0
    n1 = [T.Node(T.NodeType.Spin()) for _ in range(3)]
    n2 = [T.Node(T.NodeType.Spin()) for _ in range(4)]
    b1, b2 = T.Block(n1), T.Block(n2)
    spec = T.BlockSpec([b1, b2], [T.NodeType.Spin()])
    assert spec.get_node_locations(b1) == (0, [0, 1, 2])
    assert spec.get_node_locations(b2) == (0, [3, 4, 5, 6])


def test_blockspec_two_classes(T):
    s = [T.Node(T.NodeType.Spin()) for _ in range(2)]
    c = [T.Node(T.NodeType.Categorical(3)) for _ in range(3)]
    s2 = [T.Node(T.NodeType.Spin()) for _ in range(2)]
    bs, bc, bs2 = T.Block(s), T.Block(c), T.Block(s2)
    spec = T.BlockSpec([bs, bc, bs2], [T.NodeType.Spin(), T.NodeType.Categorical(3)])
    assert spec.get_node_locations(bs) == (0, [0, 1])
    assert spec.get_node_locations(bc) == (1, [0, 1, 2])
    assert spec.get_node_locations(bs2) == (0, [2, 3])
    spec = T.BlockSpec([bs, bc], [T.NodeType.Categorical(3), T.NodeType.Spin()])
    assert spec.get_node_locations(bs)[0] == 1 and spec.get_node_locations(bc)[0] == 0


def test_five_spin_chain_tables(T, O):
    """Chain 0-1-2-3-4 with blocks even=[0,2,4], odd=[1,3] (the model of crates/thrml-models/tests/test_ising.rs:100-136),
    tables derived by hand from program.rs:88-318."""
    b = np.array([0.1, 0.2, 0.3, 0.4, 0.5], np.float32)
    J = np.array([1.0, 2.0, 3.0, 4.0], np.float32)
    edges = np.array([[0, 1], [1, 2], [2, 3], [3, 4]])
    desc = dict(kinds=np.zeros(5, np.int32), free=[(np.array([0, 2, 4]), 0), (np.array([1, 3]), 1)], ops=[("add_ising", np.arange(5), b, edges, J, 1.0)])
    gb, ob = M.build_both(T, O, desc)
    assert_same_tables(gb, ob)
    assert [gb.node_location(i)[1] for i in range(5)] == [0, 3, 1, 4, 2]
    g = gb.group(1)
    assert list(g["head"]) == [0, 1, 2, 3, 1, 2, 3, 4] and list(g["tails"][0]) == [1, 2, 3, 4, 0, 1, 2, 3] and g["n_spin"] == 1
    assert list(g["w"].ravel()) == [1, 2, 3, 4, 1, 2, 3, 4]
    even_bias, even_edge = gb.tables(0)
    assert even_bias["k"] == 1 and list(even_bias["rows"].ravel()) == [0, 2, 4]
    assert even_edge["k"] == 2
    assert even_edge["rows"].tolist() == [[0, 0], [2, 5], [7, 0]]
    assert even_edge["active"].tolist() == [[1, 0], [1, 1], [1, 0]]
    assert even_edge["w"][:, :, 0].tolist() == [[1, 1], [3, 2], [4, 1]]
    assert even_edge["idx"][0].tolist() == [[3, 0], [4, 3], [4, 0]]
    odd_bias, odd_edge = gb.tables(1)
    assert odd_edge["rows"].tolist() == [[1, 4], [3, 6]]
    assert odd_edge["w"][:, :, 0].tolist() == [[2, 1], [4, 3]]
    assert odd_edge["idx"][0].tolist() == [[1, 0], [2, 1]]


def test_factor_group_structure(T):
    # crates/thrml-models/tests/test_factor.rs:52-157: 3 spin groups -> one merged group, head/tails equal length, W rows == head
    groups = [T.Block([T.Node(T.NodeType.Spin()) for _ in range(4)]) for _ in range(3)]
    f = T.SpinEBMFactor(groups, np.ones((4, 1, 1), np.float32))
    igs = f.to_interaction_groups()
    assert len(igs) >= 1
    for ig in igs:
        assert all(len(t) == len(ig.head_nodes) for t in ig.tail_nodes)
        assert ig.interaction.shape[0] == len(ig.head_nodes)
    assert len(igs[0].head_nodes) == 12 and len(igs[0].tail_nodes) == 2 and igs[0].n_spin == 2
    # crates/thrml-models/tests/test_discrete_ebm.rs:187-230: 2 spin + 2 categorical groups -> at least 2 groups
    sg = [T.Block([T.Node(T.NodeType.Spin()) for _ in range(3)]) for _ in range(2)]
    cg = [T.Block([T.Node(T.NodeType.Categorical(3)) for _ in range(3)]) for _ in range(2)]
    f = T.DiscreteEBMFactor(sg, cg, np.arange(27, dtype=np.float32).reshape(3, 3, 3))
    igs = f.to_interaction_groups()
    assert len(igs) == 3
    assert igs[0].n_spin == 1 and len(igs[0].tail_nodes) == 3
    # second categorical head sees the transposed table (discrete_ebm.rs:534-542)
    assert np.array_equal(igs[2].interaction, np.arange(27, dtype=np.float32).reshape(3, 3, 3).transpose(0, 2, 1))
    # Ising: bias factor + edge factor = 2 factors (crates/thrml-examples/examples/ising_chain.rs:102-106)
    nodes = [T.Node(T.NodeType.Spin()) for _ in range(3)]
    ebm = T.IsingEBM(nodes, [(nodes[0], nodes[1]), (nodes[1], nodes[2])], np.zeros(3), np.ones(2), 1.0)
    assert len(ebm.get_factors()) == 2


def test_square_factor_merges_groups(T):
    # crates/thrml-models/tests/test_discrete_ebm.rs:63-66,180-183 ("square"), discrete_ebm.rs:902-987 (merge by (tails, n_spin))
    import pytest
    cg = [T.Block([T.Node(T.NodeType.Categorical(3)) for _ in range(4)]) for _ in range(2)]
    with pytest.raises(T.ThrmlError, match="square"):
        T.SquareDiscreteEBMFactor([], cg, np.zeros((4, 3, 2), np.float32))
    w = np.arange(36, dtype=np.float32).reshape(4, 3, 3)
    plain = T.CategoricalEBMFactor(cg, w).to_interaction_groups()
    merged = T.SquareDiscreteEBMFactor([], cg, w).to_interaction_groups()
    assert len(plain) == 2 and len(merged) == 1
    m = merged[0]
    assert len(m.head_nodes) == 8 and len(m.tail_nodes) == 1 and m.n_spin == 0
    assert m.head_nodes.nodes() == cg[0].nodes() + cg[1].nodes() and m.tail_nodes[0].nodes() == cg[1].nodes() + cg[0].nodes()
    assert np.array_equal(m.interaction[:4], w) and np.array_equal(m.interaction[4:], w.transpose(0, 2, 1))
