"""thrml_rs_b200 — B200-native block-Gibbs sampling engine behind the thrml-rs sampling API.

The directory name contains a hyphen, so the package is imported under the module name `thrml_rs_b200` through
`__graft_entry__.load_package()` (tests and bench.py do this) or by putting an importlib spec on it directly.
"""
from ._ffi import ThrmlError, lib  # noqa: F401
from .engine import (OPT_DENSE_TILES, OPT_GATHER_ONLY, OPT_SPLIT_MARGIN, OPT_STATE_FORMAT, Builder, ChainState, Comm, Context, Moments, Program, default_context, greedy_coloring_arrays,  # noqa: F401
                     lattice_edges, pack_chains, rng_split)
from .api import (Block, BlockGibbsSpec, BlockSamplingProgram, BlockSpec, CategoricalEBMFactor,  # noqa: F401
                  CategoricalGibbsConditional, DiscreteEBMFactor, FactorizedEBM, FactorSamplingProgram, InteractionGroup, IsingEBM,
                  IsingSamplingProgram, IsingTrainingSpec, MomentAccumulatorObserver, Node, NodeType, RngKey, SamplingSchedule,
                  SoftmaxConditional, SpinEBMFactor, SpinGibbsConditional, SquareDiscreteEBMFactor, StateObserver, coloring_to_blocks, estimate_kl_grad, estimate_moments,
                  bipartite_coloring, generate_chain_graph, generate_lattice_graph, greedy_coloring, hinton_init, make_nearest_neighbor_lattice, run_blocks, sample_blocks,
                  sample_states, sample_with_observation)

lib()  # fail at import time when the compiled library is absent: there is no other compute path
