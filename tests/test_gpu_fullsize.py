"""Parity at the sizes the benchmark configurations name (tests/fullsize_checks.py explains the method): the device
runs every chain of the full-size state, the oracle follows a few of them.

  sparse 8-regular Ising, 2^20 spins x 4096 chains (4 GiB of state: row offsets pass 2^32)   -> k_spin_lut + fused observer
  Potts 64^3, K = 10, 1024 chains                                                             -> k_potts_update
  2-D Ising 2048^2 bit-packed, 16 chains, whole and in four stripes                           -> k_lattice_update
  RBM 784 x 4096, 1024 chains: fields out of tensor memory vs the oracle's f64 fields        -> k_dense_gemm
"""
import numpy as np
import pytest

import fullsize_checks as F

pytestmark = pytest.mark.gpu


def test_sparse_ising_full_size_chain_slices(T, O):
    from thrml_rs_b200 import workloads as W
    model = W.sparse_ising(1 << 20, 8, 0x5EED0002)
    chains = 4096
    program = T.Program(W.fill_ising(T.Builder(np.zeros(model["n"], np.int32)), model))
    state = T.ChainState(program, chains)
    res = F.sparse_ising_check(T, O, model, program, state, chains)
    assert res["state_bytes"] >= 1 << 32
    assert res["kernels"] == [1]
    assert res["ok"], res


def test_sparse_ising_full_size_with_chain_offset(T, O):
    """The shard a rank of an 8-GPU run holds: 512 chains whose global ids start at 3584.  Colouring and slot tables come
    from the device here, the oracle compiles the same blocks on the host."""
    from thrml_rs_b200 import workloads as W
    ctx = T.default_context()
    model = W.sparse_ising(1 << 18, 8, 0x5EED0002, ctx=ctx)
    program = T.Program(W.fill_ising(T.Builder(np.zeros(model["n"], np.int32)), model, ctx=ctx), ctx)
    state = T.ChainState(program, 512, chain_offset=3584)
    res = F.sparse_ising_check(T, O, model, program, state, 512, chain_base=3584)
    assert res["ok"], res


def test_potts_64_cubed(T, O):
    res = F.potts_check(T, O, side=64, K=10, chains=1024)
    assert res["ok"], res


@pytest.mark.parametrize("side,noise", [(2048, 1), (1024, 0)])
def test_lattice_whole_and_striped(T, O, side, noise):
    res = F.lattice_check(T, O, side=side, chains=16, sweeps=2, stripes=4, noise=noise)
    assert res["ok"], res


@pytest.mark.parametrize("tiles", [2, 0])
def test_rbm_layer_sizes_fields_and_draws(T, O, tiles):
    res = F.dense_check(T, O, n_visible=784, n_hidden=4096, chains=1024, tiles=tiles)
    assert res["ok"], res
    for blk in res["blocks"]:
        assert blk["mismatched_draws"] <= 2, res


def test_mixed_checkerboard_256(T, O):
    """The general spin kernel and the warp-per-node categorical kernel at 256^2 nodes x 2048 chains, chain slices against the oracle."""
    from thrml_rs_b200 import workloads as W
    ctx = T.default_context()
    model = W.spin_category_checkerboard(256, 4)
    program = T.Program(W.fill_factors(T.Builder(model["kinds"], model["dtype_order"]), model, ctx=ctx), ctx)
    state = T.ChainState(program, 2048)
    res = F.mixed_check(T, O, model, program, state, 2048)
    assert res["kernels"] == [7, 7, 5]
    assert res["ok"], res
