"""Pins for the CPU oracle: the reference's own known-answer tests, and published vectors for the third-party
algorithms its path uses."""
import math

import numpy as np


def test_spin_product_kat(O):
    # crates/thrml-models/tests/test_discrete_ebm.rs:232-278
    assert list(O.spin_product([[1, 0, 1], [1, 1, 0]])) == [1.0, -1.0, -1.0]
    assert list(O.spin_product([])) == [1.0]


def test_batch_gather_kat(O):
    # crates/thrml-models/tests/test_discrete_ebm.rs:281-316: [2,3,3], idx [0,1],[2,0] -> [3,40]
    w = np.array([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 20, 30, 40, 50, 60, 70, 80, 90], np.float32).reshape(2, 3, 3)
    assert list(O.batch_gather(w, [[0, 1], [2, 0]])) == [3.0, 40.0]
    # crates/thrml-models/tests/discrete_ebm_batch_gather_test.rs:6-95: weights 1..24 as [2,3,4], idx [0,1],[2,3] -> [3,20];
    # weights 1..12 as [4,3,1], idx [0,1,2,0],[0,0,0,0] -> [1,5,9,10]
    w = np.arange(1, 25, dtype=np.float32).reshape(2, 3, 4)
    assert list(O.batch_gather(w, [[0, 1], [2, 3]])) == [3.0, 20.0]
    w = np.arange(1, 13, dtype=np.float32).reshape(4, 3, 1)
    assert list(O.batch_gather(w, [[0, 1, 2, 0], [0, 0, 0, 0]])) == [1.0, 5.0, 9.0, 10.0]


def test_lattice_counts_kat(O):
    # crates/thrml-models/src/graph_utils.rs:250-328: 4x4 open -> 24 edges, torus -> 32, blocks of 8; odd side rounds up
    side, e, colour = O.lattice_edges(4, False)
    assert (side, len(e), int((colour == 0).sum()), int((colour == 1).sum())) == (4, 24, 8, 8)
    side, e, colour = O.lattice_edges(4, True)
    assert (side, len(e)) == (4, 32)
    side, e, _ = O.lattice_edges(5, True)
    assert (side, len(e)) == (6, 72)
    side, e, _ = O.lattice_edges(32, True)
    assert (side, len(e)) == (32, 2048)
    assert all(a < b for a, b in e) and [tuple(x) for x in e] == sorted(tuple(x) for x in e)


def test_greedy_coloring_kat(O):
    # crates/thrml-examples/src/lib.rs:265-301: 5-chain -> 2 colours; lattice colouring is proper
    colour, nc = O.greedy_coloring(5, [[0, 1], [1, 2], [2, 3], [3, 4]])
    assert nc == 2 and list(colour) == [0, 1, 0, 1, 0]
    side, e, _ = O.lattice_edges(6, False)
    colour, nc = O.greedy_coloring(36, e)
    assert nc == 2 and all(colour[a] != colour[b] for a, b in e)


def test_categorical_sample_kat(O):
    # crates/thrml-samplers/src/softmax.rs:873-898: logits +-10 -> categories [2, 1]
    logits = np.array([[-10, -10, 10, -10], [-10, 10, -10, -10]], np.float32)
    rng = np.random.default_rng(0)
    for _ in range(20):
        u = rng.uniform(1e-3, 1 - 1e-3, (2, 4)).astype(np.float32)
        assert list(O.categorical_sample(logits, u)) == [2.0, 1.0]
    # ties -> lowest index (crates/thrml-kernels/src/gumbel_argmax/kernel.rs:75-84)
    assert list(O.categorical_sample(np.zeros((1, 3), np.float32), np.full((1, 3), 0.5, np.float32))) == [0.0]


def test_sigmoid_bernoulli_fused_equals_unfused(O):
    # crates/thrml-kernels/src/sigmoid_bernoulli/mod.rs:35-56: identical uniforms -> identical samples (u<p vs u<=p differ only at u==p)
    rng = np.random.default_rng(1)
    g = rng.normal(0, 2, 1000).astype(np.float32)
    u = rng.random(1000).astype(np.float32)
    assert np.array_equal(O.sigmoid_bernoulli(g, u, True), O.sigmoid_bernoulli(g, u, False))
    assert list(O.sigmoid_bernoulli(np.array([0.0], np.float32), np.array([0.5], np.float32), True)) == [1.0]
    assert list(O.sigmoid_bernoulli(np.array([0.0], np.float32), np.array([0.5], np.float32), False)) == [0.0]


def test_chacha_published_vectors(O):
    # ChaCha8 / ChaCha20 keystream for the all-zero 256-bit key and nonce (eSTREAM / RFC 7539 reference vectors)
    assert O.chacha_block(np.zeros(8, np.uint32), 0, 0, 8).tobytes().hex().startswith("3e00ef2f895f40d67f5bb8e81f09a5a12c840ec3ce9a7f3b181be188ef711a1e")
    assert O.chacha_block(np.zeros(8, np.uint32), 0, 0, 20).tobytes().hex().startswith("76b8e0ada0f13d90405d6ae55386bd28bdd219b8a08ded1aa836efcc8b770dc7")


def test_rng_key_split_properties(O):
    # crates/thrml-samplers/src/rng.rs:52-86 (uniqueness, determinism) and :21-26 (n == 0, n == 1)
    keys = O.rng_split(42, 5)
    assert len(set(int(k) for k in keys)) == 5
    assert np.array_equal(O.rng_split(42, 10), O.rng_split(42, 10))
    assert len(O.rng_split(42, 0)) == 0 and list(O.rng_split(42, 1)) == [42]
    assert np.array_equal(O.rng_split(42, 5), O.rng_split(42, 10)[:5])


def test_philox_published_vectors(O):
    # Random123 known-answer vectors for philox4x32-10
    assert [int(x) for x in O.philox([0, 0, 0, 0], [0, 0])] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert [int(x) for x in O.philox([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2)] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert [int(x) for x in O.philox([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0])] == [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]


def test_deterministic_math_close_to_libm(O):
    rng = np.random.default_rng(2)
    for x in np.concatenate([np.linspace(-90, 90, 2001), rng.normal(0, 3, 2000)]).astype(np.float32):
        q = 1.0 / (1.0 + math.exp(-float(x)))
        assert abs(O.det_sigmoid(float(x)) - q) <= 3e-7 * q + 1e-37
    for u in np.concatenate([rng.random(2000), 1 - 2.0 ** -np.arange(1, 25), 2.0 ** -np.arange(1, 30), np.linspace(1e-7, 17, 500)]).astype(np.float32):
        if u > 0 and u != 1:
            assert abs(O.det_log(float(u)) - math.log(float(u))) <= 2e-7 * abs(math.log(float(u)))


def test_batch_gather_strided_shapes(O):
    # crates/thrml-kernels/tests/test_batch_gather_extended.rs:12-117: 3 to 8 index dimensions, explicit strides; the
    # reference asserts the output length only.  Values follow out[b] = W_flat[b*batch_stride + sum idx*stride].
    w = np.arange(120, dtype=np.float32)
    out = O.batch_gather_strided(w, [[0, 1, 2], [1, 0, 3]], [60, 20, 1], 60)
    assert len(out) == 2 and out[0] == 22.0
    for batch, n_idx, strides, bstride, size in [(4, 4, [16, 4, 2, 1], 64, 4 * 64), (3, 5, [32, 16, 8, 4, 1], 160, 3 * 160), (2, 6, [64, 32, 16, 8, 4, 1], 384, 2 * 384),
                                                 (4, 7, [64, 32, 16, 8, 4, 2, 1], 256, 4 * 256), (2, 8, [128, 64, 32, 16, 8, 4, 2, 1], 512, 2 * 512)]:
        out = O.batch_gather_strided(np.ones(size, np.float32), np.zeros((batch, n_idx), np.int32), strides, bstride)
        assert len(out) == batch and np.all(out == 1.0)


def test_gumbel_argmax_scan_equals_tensor_ops(O):
    # crates/thrml-kernels/src/gumbel_argmax/mod.rs:35-59: the serial scan (fused kernel) and the tensor-op formulation
    # argmax(logits - ln(-ln u)) pick the same categories on identical uniforms
    rng = np.random.default_rng(3)
    logits = rng.normal(0, 5, (100, 100)).astype(np.float32)
    u = rng.uniform(1e-6, 1 - 1e-6, (100, 100)).astype(np.float32)
    scan = O.categorical_sample(logits, u, use_libm=True)
    tensor_ops = np.argmax(logits - np.log(-np.log(u.astype(np.float64))), axis=1)
    assert np.array_equal(scan.astype(np.int64), tensor_ops)
    assert np.array_equal(O.categorical_sample(logits, u, use_libm=False).astype(np.int64), tensor_ops)


def test_factor_energy_restatement(O):
    # crates/thrml-models/tests/test_ising.rs:23-48: 3-spin chain, biases (0.1, 0.2, 0.3), weights (0.5, -0.5), beta 1,
    # state (1, 0, 1): E = -(0.1 - 0.2 + 0.3 - 0.5 + 0.5) = -0.2 = bias factor + edge factor (discrete_ebm.rs:552-592 per
    # factor).  The comment in that test slips a sign and says 0.8; the test itself only asserts a finite value.
    state = np.array([1, 0, 1])
    e_bias = O.factor_energy(np.array([0.1, 0.2, 0.3]).reshape(3, 1, 1), [state], [])
    e_edge = O.factor_energy(np.array([0.5, -0.5]).reshape(2, 1, 1), [state[[0, 1]], state[[1, 2]]], [])
    assert abs(e_bias - (-0.2)) < 1e-12 and abs(e_edge) < 1e-12
    assert abs(O.factor_energy(np.array([0.5, -0.5]).reshape(2, 1, 1), [np.array([1, 0]), np.array([1, 1])], []) + 1.0) < 1e-12
    assert abs(O.factor_energy(np.array([0.5, -0.5]).reshape(2, 1, 1), [np.array([1, 0]), np.array([1, 0])], []) - 0.0) < 1e-12
    assert abs(O.factor_energy(np.array([0.5, -0.25]).reshape(2, 1, 1), [np.array([1, 0]), np.array([0, 0])], []) - 0.75) < 1e-12
    # categorical axes: W[row, c1, c2] picked per row, spins as signs; a batch of two chains
    w = np.arange(2 * 3 * 3, dtype=np.float64).reshape(2, 3, 3)
    e = O.factor_energy(w, [np.array([[1, 0], [0, 0]])], [np.array([[2, 0], [1, 1]]), np.array([[1, 2], [0, 2]])])
    assert np.allclose(e, [-(w[0, 2, 1] - w[1, 0, 2]), -(-w[0, 1, 0] - w[1, 1, 2])])
    w1 = np.arange(6, dtype=np.float64).reshape(2, 3, 1)
    assert O.factor_energy(w1, [], [np.array([2, 1])]) == -(w1[0, 2, 0] + w1[1, 1, 0])


def test_softmax_conditional_logits_ignore_neighbours(O):
    """SoftmaxConditional (softmax.rs:147-222): per-category weights summed over active slots; interactions whose weights
    are not [rows, K, 1] are skipped and neighbour states never enter.  Checked against numpy on a small model."""
    K, n = 4, 6
    rng = np.random.default_rng(0)
    unary_a = rng.normal(0, 1, (n, K, 1)).astype(np.float32)
    unary_b = rng.normal(0, 1, (3, K, 1)).astype(np.float32)
    pair = rng.normal(0, 1, (n - 1, K, K)).astype(np.float32)
    m = O.Model(np.full(n, K, np.int32))
    m.add_free_block(np.arange(n), sampler=2)
    m.add_discrete_factor([], [np.arange(n)], unary_a)
    m.add_discrete_factor([], [np.array([0, 2, 2])], unary_b)            # node 2 heads two rows of this group
    m.add_discrete_factor([], [np.arange(n - 1), np.arange(1, n)], pair)  # [rows, K, K]: skipped by this sampler
    m.compile()
    st = O.State(m, 3)
    st.set_block(0, rng.integers(0, K, (3, n)).astype(np.float32))
    _, th = st.fields(0)
    want = unary_a[:, :, 0].copy()
    want[0] += unary_b[0, :, 0]
    want[2] += unary_b[1, :, 0] + unary_b[2, :, 0]
    assert np.allclose(th, np.broadcast_to(want, (3, n, K)), rtol=0, atol=1e-6)
    # the draw is the usual Gumbel-argmax of those logits: overwhelming logits decide it
    m2 = O.Model(np.full(2, 3, np.int32))
    m2.add_free_block(np.arange(2), sampler=2)
    m2.add_discrete_factor([], [np.arange(2)], np.array([[[-30.0], [30.0], [-30.0]], [[30.0], [-30.0], [-30.0]]], np.float32))
    m2.compile()
    s2 = O.State(m2, 5)
    s2.sample_blocks(1)
    assert np.array_equal(s2.get_block(0), np.broadcast_to(np.array([1.0, 0.0], np.float32), (5, 2)))
