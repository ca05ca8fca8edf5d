"""The dense kernels with CTA pairs sharing 256-row tiles (tcgen05 cta_group::2): the same checks as the one-CTA
tiles, plus equality of the two tilings where the arithmetic is exact (integer correlations)."""
import numpy as np
import pytest

import test_gpu_dense as D

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def pair_mode(T):
    before = dict(T.Program.default_options)
    T.Program.default_options = {**before, T.OPT_DENSE_TILES: 1}
    yield
    T.Program.default_options = before


# tile widths: 128 columns for narrow blocks, 208 where that pads least (784 -> 832), 256 for wide ones; chains below and
# above one 256-row tile, ragged in both directions
@pytest.mark.parametrize("n_v,n_h,chains", [(64, 128, 128), (100, 200, 200), (784, 300, 256), (130, 70, 37), (96, 2100, 600)])
def test_dense_update_matches_oracle(T, O, n_v, n_h, chains):
    D.test_dense_update_matches_oracle(T, O, n_v, n_h, chains)


@pytest.mark.parametrize("n_a,n_b,chains", [(64, 64, 4096), (100, 200, 200), (784, 130, 1000), (5, 300, 33), (300, 2100, 700)])
def test_pair_correlation_is_exact(T, n_a, n_b, chains):
    D.test_pair_correlation_is_exact(T, n_a, n_b, chains)


def test_cd1_step_composition_and_statistics(T, O):
    D.test_cd1_step_composition_and_statistics(T, O)


@pytest.mark.parametrize("n_a,n_b,chains", [(300, 2100, 2200), (784, 512, 2048), (2100, 300, 2100), (40, 512, 4096)])
def test_auto_mode_correlations(T, n_a, n_b, chains):
    """Mode 2 picks the tiling per launch; when only the second block fills 256-row tiles well the operands are swapped and
    the epilogue writes the transposed result.  Integer arithmetic: every route gives the same exact matrix."""
    T.Program.default_options = {T.OPT_DENSE_TILES: 2}
    D.test_pair_correlation_is_exact(T, n_a, n_b, chains)


def test_auto_mode_update_and_cd1(T, O):
    T.Program.default_options = {T.OPT_DENSE_TILES: 2}
    D.test_dense_update_matches_oracle(T, O, 96, 2100, 300)   # long reduction for the visible layer: pair tiles there only
    D.test_cd1_step_composition_and_statistics(T, O)
