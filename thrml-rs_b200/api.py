"""Host-side mirror of thrml-rs's sampling API: same names, argument meaning and error behaviour, driving the
C ABI instead of Burn tensors.

States are numpy arrays: a block state is `[n]` (one chain, as in the reference) or `[chains, n]` (a batch of
independent chains, the shape hinton_init returns).  Spins are 0/1, categories are integer indices.  Errors raise
ThrmlError (a ValueError) whose text carries the reference's own message.
"""
import itertools
from dataclasses import dataclass

import numpy as np

from . import engine as _eng
from ._ffi import ThrmlError

_node_counter = itertools.count()  # NODE_COUNTER, crates/thrml-core/src/node.rs:30


@dataclass(frozen=True)
class NodeType:
    """crates/thrml-core/src/node.rs:8-21.  kind 0 = Spin, K >= 1 = Categorical{n_categories: K}."""
    kind: int

    @staticmethod
    def Spin():
        return NodeType(0)

    @staticmethod
    def Categorical(n_categories):
        if not 1 <= int(n_categories) <= 255:
            raise ThrmlError(-1, "n_categories must fit in u8 and be at least 1")
        return NodeType(int(n_categories))


class Node:
    """crates/thrml-core/src/node.rs:24-51: identity = (fresh id from a global counter, type)."""
    __slots__ = ("id", "node_type")

    def __init__(self, node_type):
        self.id = next(_node_counter)
        self.node_type = node_type

    def __hash__(self):
        return hash((self.id, self.node_type.kind))

    def __eq__(self, other):
        return isinstance(other, Node) and self.id == other.id and self.node_type == other.node_type

    def __repr__(self):
        return f"Node({self.id}, {self.node_type.kind})"


class Block:
    """crates/thrml-core/src/block.rs:5-65: ordered, non-empty, single-type node list."""

    def __init__(self, nodes):
        nodes = list(nodes)
        if not nodes:
            raise ThrmlError(-1, "Block cannot be empty")
        t = nodes[0].node_type
        if any(n.node_type != t for n in nodes):
            raise ThrmlError(-1, "All nodes in a block must be of the same type")
        self._nodes = nodes
        self._type = t

    def node_type(self):
        return self._type

    def nodes(self):
        return self._nodes

    def __len__(self):
        return len(self._nodes)

    def __iter__(self):
        return iter(self._nodes)

    def __getitem__(self, i):
        return self._nodes[i]

    def __add__(self, other):
        if self._type != other._type:
            raise ThrmlError(-1, "Cannot add blocks of different node types")
        return Block(self._nodes + other._nodes)

    def __eq__(self, other):
        return isinstance(other, Block) and self._nodes == other._nodes


class _Dense:
    """Global Node objects -> dense ids of one builder."""

    def __init__(self):
        self.ids = {}
        self.kinds = []

    def of(self, node):
        i = self.ids.get(node)
        if i is None:
            i = len(self.kinds)
            self.ids[node] = i
            self.kinds.append(node.node_type.kind)
        return i

    def many(self, nodes):
        return np.fromiter((self.of(n) for n in nodes), dtype=np.int64, count=len(nodes))


class BlockSpec:
    """crates/thrml-core/src/blockspec.rs:5-89.  node_shape_dtypes: ordered list (or dict keys) of NodeTypes."""

    def __init__(self, blocks, node_shape_dtypes):
        self.blocks = list(blocks)
        self.node_shape_dtypes = list(node_shape_dtypes)
        self._dense = _Dense()
        for b in self.blocks:
            self._dense.many(b.nodes())
        self._builder = _eng.Builder(self._dense.kinds or [0], [t.kind for t in self.node_shape_dtypes])
        for b in self.blocks:  # placed as clamped blocks: a plain BlockSpec has no samplers
            self._builder.add_clamped_block(self._dense.many(b.nodes()))
        self._builder.compile()

    def get_node_locations(self, block):
        locs = []
        sd = None
        for n in block.nodes():
            if n not in self._dense.ids:
                raise ThrmlError(-1, "Node not found in global location map")
            sd, pos = self._builder.node_location(self._dense.ids[n])
            locs.append(pos)
        return sd, locs


class InteractionGroup:
    """crates/thrml-core/src/interaction.rs:107-181 (tensor interactions): weights [rows, d1, d2]."""

    def __init__(self, interaction, head_nodes, tail_nodes, n_spin):
        w = np.asarray(interaction, dtype=np.float32)
        if w.ndim != 3:
            raise ThrmlError(-1, "interaction tensor must have shape [n_nodes, dim1, dim2]")
        for t in tail_nodes:
            if len(t) != len(head_nodes):
                raise ThrmlError(-1, "All tail node blocks must have the same length as head_nodes")
        if w.shape[0] != len(head_nodes):
            raise ThrmlError(-1, "All arrays in interaction must have leading dimension equal to the length of head_nodes")
        if n_spin > len(tail_nodes):
            raise ThrmlError(-1, "n_spin cannot exceed number of tail blocks")
        self.interaction = w
        self.head_nodes = head_nodes
        self.tail_nodes = list(tail_nodes)
        self.n_spin = int(n_spin)


class RngKey:
    """crates/thrml-samplers/src/rng.rs:10-51."""
    __slots__ = ("_seed",)

    def __init__(self, seed):
        self._seed = int(seed) & 0xFFFFFFFFFFFFFFFF

    @staticmethod
    def new(seed):
        return RngKey(seed)

    def split(self, n):
        return [RngKey(int(k)) for k in _eng.rng_split(self._seed, n)]

    def split_two(self):
        a, b = self.split(2)
        return a, b

    def seed(self):
        return self._seed

    def __eq__(self, other):
        return isinstance(other, RngKey) and other._seed == self._seed

    def __hash__(self):
        return hash(self._seed)

    def __repr__(self):
        return f"RngKey({self._seed})"


@dataclass(frozen=True)
class SamplingSchedule:
    """crates/thrml-samplers/src/schedule.rs:4-20."""
    n_warmup: int
    n_samples: int
    steps_per_sample: int

    @staticmethod
    def new(n_warmup, n_samples, steps_per_sample):
        return SamplingSchedule(n_warmup, n_samples, steps_per_sample)


class SpinGibbsConditional:
    """crates/thrml-samplers/src/spin_gibbs.rs:41-100."""
    kind = _eng.SAMPLER_SPIN


class CategoricalGibbsConditional:
    """crates/thrml-samplers/src/softmax.rs:228-271."""
    kind = _eng.SAMPLER_CATEGORICAL

    def __init__(self, n_categories, n_spin=0):
        self.n_categories = n_categories
        self.n_spin = n_spin


class SoftmaxConditional:
    """crates/thrml-samplers/src/softmax.rs:103-222: logits = the per-category weights of the block's interactions summed
    over active slots; neighbour states are not read and interactions whose weights are not `[rows, K, 1]` are skipped."""
    kind = _eng.SAMPLER_SOFTMAX

    def __init__(self, n_categories):
        self.n_categories = n_categories


class BlockGibbsSpec:
    """crates/thrml-samplers/src/program.rs:17-64."""

    def __init__(self, free_super_blocks, clamped_blocks, node_shape_dtypes):
        self.superblocks = [list(sb) for sb in free_super_blocks]
        self.free_blocks = [b for sb in self.superblocks for b in sb]
        self.sampling_order = []
        i = 0
        for sb in self.superblocks:
            self.sampling_order.append(list(range(i, i + len(sb))))
            i += len(sb)
        self.clamped_blocks = list(clamped_blocks)
        self.node_shape_dtypes = list(node_shape_dtypes)
        self.spec = BlockSpec(self.free_blocks + self.clamped_blocks, self.node_shape_dtypes)


class BlockSamplingProgram:
    """crates/thrml-samplers/src/program.rs:70-318: the index compiler runs on the host at construction; the device
    program is created on first use."""

    def __init__(self, gibbs_spec, samplers, interaction_groups, ctx=None):
        if len(samplers) != len(gibbs_spec.free_blocks):
            raise ThrmlError(-1, f"Number of samplers ({len(samplers)}) must match number of free blocks ({len(gibbs_spec.free_blocks)})")
        self.gibbs_spec = gibbs_spec
        self.samplers = list(samplers)
        self._dense = _Dense()
        for b in gibbs_spec.free_blocks + gibbs_spec.clamped_blocks:
            self._dense.many(b.nodes())
        flat = []
        for g in interaction_groups:
            head = self._dense.many(g.head_nodes.nodes())
            tails = [self._dense.many(t.nodes()) for t in g.tail_nodes]
            flat.append((head, tails, g.n_spin, g.interaction))
        self.builder = _eng.Builder(self._dense.kinds, [t.kind for t in gibbs_spec.node_shape_dtypes])
        bi = 0
        for sb_i, sb in enumerate(gibbs_spec.superblocks):
            for b in sb:
                self.builder.add_free_block(self._dense.many(b.nodes()), superblock=sb_i, sampler=self.samplers[bi].kind)
                bi += 1
        for b in gibbs_spec.clamped_blocks:
            self.builder.add_clamped_block(self._dense.many(b.nodes()))
        for head, tails, n_spin, w in flat:
            self.builder.add_group(head, tails, n_spin, w)
        self.builder.compile()
        self._ctx = ctx
        self._program = None

    @property
    def device_program(self):
        if self._program is None:
            self._program = _eng.Program(self.builder, self._ctx)
        return self._program

    def dense_id(self, node):
        if node not in self._dense.ids:
            raise ThrmlError(-1, "Node not found in global location map")
        return self._dense.ids[node]

    def block_index(self, block):
        for i, b in enumerate(self.gibbs_spec.free_blocks + self.gibbs_spec.clamped_blocks):
            if b is block or b == block:
                return i
        raise ThrmlError(-1, "block is not part of this program")


# ---------------------------------------------------------------------------------------------------------
# Drivers: crates/thrml-samplers/src/sampling.rs
# ---------------------------------------------------------------------------------------------------------
def _batch_of(states):
    """(chains, batched): batched when any entry is `[chains, n]`; 1-D entries then stand for every chain."""
    for s in states:
        s = np.asarray(s)
        if s.ndim == 2:
            return s.shape[0], True
    return 1, False


def _make_state(program, state_free, state_clamp, chain_offset=0):
    n_free = len(program.gibbs_spec.free_blocks)
    n_clamp = len(program.gibbs_spec.clamped_blocks)
    if len(state_free) != n_free or len(state_clamp) != n_clamp:
        raise ThrmlError(-1, "state lists must have one entry per free / clamped block")
    chains, batched = _batch_of(list(state_free) + list(state_clamp))
    st = _eng.ChainState(program.device_program, chains, chain_offset)
    for i, s in enumerate(list(state_free) + list(state_clamp)):
        s = np.asarray(s)
        if s.ndim == 2 and s.shape[0] != chains:
            raise ThrmlError(-1, "batched block states must share the leading dimension")
        if s.ndim == 1 and batched:  # one row for every chain (a clamped or conditioning block given once)
            s = np.broadcast_to(s, (chains, s.shape[0]))
        st.upload(i, np.ascontiguousarray(s).reshape(chains, -1))
    return st, chains, batched


def _read_free(st, program, batched):
    out = []
    for i in range(len(program.gibbs_spec.free_blocks)):
        a = st.download(i)
        out.append(a if batched else a[0])
    return out


def sample_blocks(key, state_free, clamp_state, program, noise=None):
    """sampling.rs:28-63: one sweep; `state_free` (a list) is updated in place."""
    st, _, batched = _make_state(program, state_free, clamp_state)
    st.sample_blocks(key.seed(), noise)
    state_free[:] = _read_free(st, program, batched)


def run_blocks(key, program, init_chain_state, state_clamp, n_iters, noise=None):
    """sampling.rs:81-106."""
    if n_iters == 0:
        return list(init_chain_state)
    st, _, batched = _make_state(program, init_chain_state, state_clamp)
    st.run_blocks(key.seed(), n_iters, noise)
    return _read_free(st, program, batched)


class StateObserver:
    """crates/thrml-observers/src/state_observer.rs:12-50."""

    def __init__(self, blocks_to_sample):
        self.blocks_to_sample = list(blocks_to_sample)

    def init(self):
        return None


class MomentAccumulatorObserver:
    """crates/thrml-observers/src/moment.rs:29-148: running sums of prod f(x) over node tuples; the carry is a list
    of one f64 array per moment type (exact integer sums)."""

    def __init__(self, moment_spec, transform_to_spin):
        self.moment_spec = [[list(row) for row in t] for t in moment_spec]
        self.transform_to_spin = bool(transform_to_spin)
        seen = {}
        for t in self.moment_spec:
            for row in t:
                for n in row:
                    seen.setdefault(n, len(seen))
        self.flat_nodes_list = list(seen)
        self.flat_to_full_moment_slices = [[[seen[n] for n in row] for row in t] for t in self.moment_spec]

    @staticmethod
    def ising_moment_spec(first_moment_nodes, second_moment_edges):
        spec = []
        if first_moment_nodes:
            spec.append([[n] for n in first_moment_nodes])
        if second_moment_edges:
            spec.append([[a, b] for a, b in second_moment_edges])
        return spec

    def init(self):
        return [np.zeros(len(t), dtype=np.float64) for t in self.moment_spec]


def sample_with_observation(key, program, schedule, init_chain_state, state_clamp, observation_carry_init, f_observe, noise=None):
    """sampling.rs:178-320.  Returns (final carry, samples); samples = one `[n_samples, n]` array per observed block
    (`[n_samples, chains, n]` for a batch), empty for a moment observer."""
    st, chains, batched = _make_state(program, init_chain_state, state_clamp)
    if isinstance(f_observe, MomentAccumulatorObserver):
        spec = [[[program.dense_id(n) for n in row] for row in t] for t in f_observe.moment_spec]
        mom = _eng.Moments(program.device_program, spec, f_observe.transform_to_spin)
        st.sample_with_observation(key.seed(), schedule.n_warmup, schedule.n_samples, schedule.steps_per_sample, moments=mom, inj=noise)
        carry = [np.asarray(c, dtype=np.float64) + mom.read(t)[0] for t, c in enumerate(observation_carry_init)]
        return carry, []
    blocks = [program.block_index(b) for b in f_observe.blocks_to_sample]
    obs = st.sample_with_observation(key.seed(), schedule.n_warmup, schedule.n_samples, schedule.steps_per_sample, obs_blocks=blocks, inj=noise)
    out, row = [], 0
    for b in blocks:
        n = program.device_program.block_len(b)
        a = obs[:, row:row + n, :].transpose(0, 2, 1).astype(np.float32)  # [samples, chains, n]
        out.append(a if batched else a[:, 0, :])
        row += n
    return observation_carry_init, out


def sample_states(key, program, schedule, init_state_free, state_clamp, nodes_to_sample, noise=None):
    """sampling.rs:128-156."""
    observer = StateObserver(list(nodes_to_sample))
    _, samples = sample_with_observation(key, program, schedule, init_state_free, state_clamp, None, observer, noise)
    return samples


# ---------------------------------------------------------------------------------------------------------
# Models: crates/thrml-models/src/{discrete_ebm,factor,ising}.rs
# ---------------------------------------------------------------------------------------------------------
class DiscreteEBMFactor:
    """discrete_ebm.rs:294-548."""

    def __init__(self, spin_node_groups, categorical_node_groups, weights):
        self.spin_node_groups = list(spin_node_groups)
        self.categorical_node_groups = list(categorical_node_groups)
        w = np.asarray(weights, dtype=np.float32)
        if w.ndim != 3:
            raise ThrmlError(-1, "weights must be a rank-3 tensor [b, x_1, x_2]")
        groups = self.spin_node_groups + self.categorical_node_groups
        if not groups:
            raise ThrmlError(-1, "At least one node group must be provided")
        n = len(groups[0])
        if any(len(g) != n for g in groups):
            raise ThrmlError(-1, "Every block in node_groups must contain the same number of nodes")
        if w.shape[0] != n:
            raise ThrmlError(-1, "The leading dimension of weights must have the same length as the number of nodes in each node group")
        eff = 3
        while eff > 1 and w.shape[eff - 1] == 1:
            eff -= 1
        if eff < 1 + len(self.categorical_node_groups):
            raise ThrmlError(-1, f"The shape of the weight tensor must be [b, x_1, ..., x_k], where k is the length of categorical_node_groups ({len(self.categorical_node_groups)})")
        self.weights = w

    def node_groups(self):
        return self.spin_node_groups + self.categorical_node_groups

    def to_interaction_groups(self):
        """discrete_ebm.rs:379-510, evaluated by the library's builder."""
        dense = _Dense()
        sg = [dense.many(g.nodes()) for g in self.spin_node_groups]
        cg = [dense.many(g.nodes()) for g in self.categorical_node_groups]
        inv = {i: n for n, i in dense.ids.items()}
        b = _eng.Builder(dense.kinds)
        n0 = b.counts()[2]
        made = b.add_discrete_factor(sg, cg, self.weights)
        out = []
        for g in range(n0, n0 + made):
            d = b.group(g)
            head = Block([inv[int(i)] for i in d["head"]])
            tails = [Block([inv[int(i)] for i in t]) for t in d["tails"]]
            out.append(InteractionGroup(d["w"], head, tails, d["n_spin"]))
        return out


def _energy_state(state, blocks, node_shape_dtypes, ctx):
    """A device state holding `state` (one array per block, `[n]` or `[chains, n]`) (no interactions; the blocks only
    give the layout): the block_state_to_global step of ebm.rs:117-121 for energy evaluation."""
    blocks = list(blocks)
    arrays = [np.atleast_2d(np.asarray(a)) for a in state]
    if len(arrays) != len(blocks):
        raise ThrmlError(-1, "Number of states not equal to number of blocks")
    spec = BlockGibbsSpec([[b] for b in blocks], [], node_shape_dtypes)
    samplers = [SpinGibbsConditional() if b.node_type().kind == 0 else CategoricalGibbsConditional(b.node_type().kind) for b in blocks]
    prog = BlockSamplingProgram(spec, samplers, [], ctx)
    st = _eng.ChainState(prog.device_program, arrays[0].shape[0])
    for i, (a, b) in enumerate(zip(arrays, blocks)):
        if a.shape[1] != len(b):
            raise ThrmlError(-1, "Block/state length mismatch")
        st.upload(i, a)
    return prog, st


def _factor_energy_on(factor, prog, st):
    sg = [[prog.dense_id(n) for n in g.nodes()] for g in factor.spin_node_groups]
    cg = [[prog.dense_id(n) for n in g.nodes()] for g in factor.categorical_node_groups]
    w = factor.weights
    if len(cg) < 2:  # a trailing axis of length 1 carries no index (discrete_ebm.rs:577-583)
        w = w.reshape(w.shape[0], -1, 1)
    return st.factor_energy(sg, cg, w)


def _factor_energy(self, state, blocks, node_shape_dtypes=None, ctx=None):
    """discrete_ebm.rs:552-592: E = -sum_rows W[row, categories...] * prod(2 s - 1) for the state given per block
    (`blocks` plays the BlockSpec's role).  `[n]` block states give a one-element array like the reference; `[chains, n]`
    states give one energy per chain."""
    types = node_shape_dtypes or list(dict.fromkeys(b.node_type() for b in blocks))
    prog, st = _energy_state(state, blocks, types, ctx)
    return _factor_energy_on(self, prog, st).astype(np.float32)


DiscreteEBMFactor.factor_energy = _factor_energy


class FactorizedEBM:
    """ebm.rs:93-130: an EBM that is the sum of its factors' energies."""

    def __init__(self, factors, node_shape_dtypes):
        self.factor_list = list(factors)
        self.node_shape_dtypes = list(node_shape_dtypes)

    def factors(self):
        return self.factor_list

    def energy(self, state, blocks, ctx=None):
        prog, st = _energy_state(state, blocks, self.node_shape_dtypes, ctx)
        total = np.zeros(st.n_chains, dtype=np.float64)
        for f in self.factor_list:
            total += _factor_energy_on(f, prog, st)
        return total.astype(np.float32)


class SpinEBMFactor(DiscreteEBMFactor):
    """discrete_ebm.rs:742-790."""

    def __init__(self, node_groups, weights):
        super().__init__(node_groups, [], weights)


class CategoricalEBMFactor(DiscreteEBMFactor):
    """discrete_ebm.rs:792-851."""

    def __init__(self, node_groups, weights):
        super().__init__([], node_groups, weights)


class SquareDiscreteEBMFactor(DiscreteEBMFactor):
    """discrete_ebm.rs:858-987: a factor whose category dimensions are all equal; its interaction groups with the same
    (number of tails, n_spin) are concatenated into one.  The reference iterates a HashMap of buckets; here buckets
    come out in first-seen order."""

    def __init__(self, spin_node_groups, categorical_node_groups, weights):
        w = np.asarray(weights, dtype=np.float32)
        if w.ndim == 3 and any(d != w.shape[1] for d in w.shape[1:]):
            raise ThrmlError(-1, "Interaction tensor is not square")
        super().__init__(spin_node_groups, categorical_node_groups, w)

    def to_interaction_groups(self):
        base = super().to_interaction_groups()
        buckets = {}
        for g in base:
            buckets.setdefault((len(g.tail_nodes), g.n_spin), []).append(g)
        merged = []
        for (n_tail, n_spin), bucket in buckets.items():
            if len(bucket) == 1:
                merged.append(bucket[0])
                continue
            head = Block([n for g in bucket for n in g.head_nodes.nodes()])
            tails = [Block([n for g in bucket for n in g.tail_nodes[i].nodes()]) for i in range(n_tail)]
            merged.append(InteractionGroup(np.concatenate([g.interaction for g in bucket], axis=0), head, tails, n_spin))
        return merged


class FactorSamplingProgram:
    """factor.rs:133-185."""

    def __init__(self, gibbs_spec, samplers, factors, other_interaction_groups=(), ctx=None):
        groups = []
        for f in factors:
            groups.extend(f.to_interaction_groups())
        groups.extend(other_interaction_groups)
        self.program = BlockSamplingProgram(gibbs_spec, samplers, groups, ctx)


class IsingEBM:
    """ising.rs:22-149: E(s) = -beta (sum b_i s_i + sum J_ij s_i s_j)."""

    def __init__(self, nodes, edges, biases, weights, beta):
        self.nodes = list(nodes)
        self.edges = list(edges)
        self.biases = np.asarray(biases, dtype=np.float32).reshape(-1)
        self.weights = np.asarray(weights, dtype=np.float32).reshape(-1)
        self.beta = np.float32(np.asarray(beta, dtype=np.float32).reshape(-1)[0])
        self._node_type = self.nodes[0].node_type if self.nodes else NodeType.Spin()

    def update_weights(self, new_weights, new_biases):
        self.weights = np.asarray(new_weights, dtype=np.float32).reshape(-1)
        self.biases = np.asarray(new_biases, dtype=np.float32).reshape(-1)

    def beta_value(self):
        return float(self.beta)

    def get_factors(self):
        factors = []
        if self.nodes:
            factors.append(SpinEBMFactor([Block(self.nodes)], (self.beta * self.biases).reshape(-1, 1, 1)))
        if self.edges:
            b0 = Block([e[0] for e in self.edges])
            b1 = Block([e[1] for e in self.edges])
            factors.append(SpinEBMFactor([b0, b1], (self.beta * self.weights).reshape(-1, 1, 1)))
        return factors

    def node_shape_dtypes(self):
        return [self._node_type]

    def energy_batched(self, states, ctx=None):
        """ising.rs:227-321: states `[batch, n_nodes]` (0/1, node order = self.nodes) -> energies `[batch]`."""
        states = np.asarray(states, dtype=np.float32)
        states = states.reshape(-1, len(self.nodes))
        spec = BlockGibbsSpec([[Block(self.nodes)]], [], self.node_shape_dtypes())
        prog = BlockSamplingProgram(spec, [SpinGibbsConditional()], [], ctx)
        st = _eng.ChainState(prog.device_program, states.shape[0])
        st.upload(0, states)
        ids = [prog.dense_id(n) for n in self.nodes]
        edges = np.array([[prog.dense_id(a), prog.dense_id(b)] for a, b in self.edges], dtype=np.int64).reshape(-1, 2)
        return st.ising_energy(ids, self.biases, edges, self.weights, self.beta_value()).astype(np.float32)

    def energy(self, state, blocks=None, ctx=None):
        """ising.rs:150-225: energy of one state given as the first block's tensor in node order."""
        first = state[0] if isinstance(state, (list, tuple)) else state
        return self.energy_batched(np.asarray(first).reshape(1, -1), ctx)


class IsingSamplingProgram:
    """ising.rs:329-389: every free block is its own superblock; SpinGibbsConditional everywhere."""

    def __init__(self, ebm, free_blocks, clamped_blocks, ctx=None):
        gibbs_spec = BlockGibbsSpec([[b] for b in free_blocks], clamped_blocks, ebm.node_shape_dtypes())
        samplers = [SpinGibbsConditional() for _ in gibbs_spec.free_blocks]
        groups = []
        for f in ebm.get_factors():
            groups.extend(f.to_interaction_groups())
        self.program = BlockSamplingProgram(gibbs_spec, samplers, groups, ctx)
        self._has_bias_group = bool(ebm.nodes)

    def refresh_weights(self, ebm):
        """The explicit counterpart of IsingEBM::update_weights (ising.rs:71-86) for a program that already exists: the
        reference's programs keep the beta-scaled weights they were built with (train_mnist.rs:600-612 rebuilds them), here
        the device tables re-read b[N] and J[E] through thrml_program_update_group — N + E floats cross the host link."""
        dp, beta, g = self.program.device_program, ebm.beta_value(), 0
        if self._has_bias_group:
            dp.update_group(g, ebm.biases, scale=beta)
            g += 1
        if ebm.edges:
            dp.update_group(g, ebm.weights, scale=beta)


def hinton_init(key, model, blocks, batch_shape, ctx=None, noise=None):
    """ising.rs:602-673: per block a `[batch, block_len]` array with P(s=1) = sigmoid(beta * b)."""
    batch = int(np.prod(batch_shape)) if len(batch_shape) else 1
    node_map = {n: i for i, n in enumerate(model.nodes)}
    spec = BlockGibbsSpec([[b] for b in blocks], [], [blocks[0].node_type()] if blocks else [NodeType.Spin()])
    prog = BlockSamplingProgram(spec, [SpinGibbsConditional() for _ in blocks], [], ctx)
    st = _eng.ChainState(prog.device_program, batch)
    biases = np.concatenate([[model.biases[node_map.get(n, 0)] for n in b.nodes()] for b in blocks]).astype(np.float32)
    st.hinton_init(list(range(len(blocks))), biases, model.beta_value(), key.seed(), noise)
    return [st.download(i) for i in range(len(blocks))]


def estimate_moments(key, first_moment_nodes, second_moment_edges, program, schedule, init_state, clamped_data):
    """ising.rs:455-505: (<s_i>, <s_i s_j>) = accumulated sums / n_samples (and / chains for a batch)."""
    observer = MomentAccumulatorObserver(MomentAccumulatorObserver.ising_moment_spec(list(first_moment_nodes), list(second_moment_edges)), True)
    carry, _ = sample_with_observation(key, program, schedule, init_state, clamped_data, observer.init(), observer)
    chains, _ = _batch_of(list(init_state) + list(clamped_data))
    denom = float(schedule.n_samples) * chains
    node_m = carry[0] / denom if first_moment_nodes else np.zeros(0)
    edge_m = (carry[1] if first_moment_nodes else carry[0]) / denom if second_moment_edges else np.zeros(0)
    return node_m.astype(np.float32), edge_m.astype(np.float32)


class IsingTrainingSpec:
    """ising.rs:392-433: the positive program clamps data + conditioning blocks, the negative one only conditioning."""

    def __init__(self, ebm, data_blocks, conditioning_blocks, positive_sampling_blocks, negative_sampling_blocks, schedule_positive, schedule_negative, ctx=None):
        self.ebm = ebm
        self.program_positive = IsingSamplingProgram(ebm, list(positive_sampling_blocks), list(data_blocks) + list(conditioning_blocks), ctx)
        self.program_negative = IsingSamplingProgram(ebm, list(negative_sampling_blocks), list(conditioning_blocks), ctx)
        self.schedule_positive = schedule_positive
        self.schedule_negative = schedule_negative

    def refresh_weights(self):
        """Push the EBM's current biases, couplings and beta into both programs' device tables."""
        self.program_positive.refresh_weights(self.ebm)
        self.program_negative.refresh_weights(self.ebm)


def estimate_kl_grad(key, training_spec, bias_nodes, weight_edges, data, conditioning_values, init_state_positive, init_state_negative):
    """ising.rs:531-594: grad = -beta (<.>_data - <.>_model), returned as (grad_weights, grad_biases).  `data` is one
    `[batch, n]` array per data block; like the reference, the positive phase clamps the single row `key_pos % batch`
    (ising.rs:549-559).  Chains batch through the init states as everywhere else; 1-D clamped or conditioning arrays then
    stand for every chain.  Both phases and the difference run on the device (thrml_estimate_kl_grad)."""
    key_pos, _ = key.split_two()
    clamped_pos = []
    for d in data:
        d = np.asarray(d)
        clamped_pos.append(d[key_pos.seed() % d.shape[0]])
    cond = [np.asarray(c) for c in conditioning_values]
    clamped_pos += cond
    prog_pos, prog_neg = training_spec.program_positive.program, training_spec.program_negative.program
    st_pos, _, _ = _make_state(prog_pos, init_state_positive, clamped_pos)
    st_neg, _, _ = _make_state(prog_neg, init_state_negative, cond)
    spec = MomentAccumulatorObserver.ising_moment_spec(list(bias_nodes), list(weight_edges))
    if len(spec) != 2:  # ising_moment_spec drops an empty type; the device entry wants both, possibly empty
        spec = [[(n,) for n in bias_nodes], [tuple(e) for e in weight_edges]]
    moms = []
    for prog in (prog_pos, prog_neg):
        moms.append(_eng.Moments(prog.device_program, [[[prog.dense_id(n) for n in row] for row in t] for t in spec], True))
    sp, sn = training_spec.schedule_positive, training_spec.schedule_negative
    return _eng.estimate_kl_grad(st_pos, st_neg, moms[0], moms[1], key.seed(), (sp.n_warmup, sp.n_samples, sp.steps_per_sample),
                                 (sn.n_warmup, sn.n_samples, sn.steps_per_sample), training_spec.ebm.beta_value())


# ---------------------------------------------------------------------------------------------------------
# Input builders: crates/thrml-models/src/graph_utils.rs:177-243, crates/thrml-examples/src/lib.rs:114-205
# ---------------------------------------------------------------------------------------------------------
def make_nearest_neighbor_lattice(side_len, torus):
    """Returns (nodes, edges as index pairs sorted by (min,max), upper block, lower block)."""
    if side_len <= 0:
        raise ThrmlError(-1, "side_len must be positive")
    side, edges, colour = _eng.lattice_edges(side_len, torus)
    nodes = [Node(NodeType.Spin()) for _ in range(side * side)]
    upper = Block([n for n, c in zip(nodes, colour) if c == 0])
    lower = Block([n for n, c in zip(nodes, colour) if c == 1])
    return nodes, edges, upper, lower


def generate_lattice_graph(rows, cols, node_type=None):
    """lib.rs:34-71: `rows x cols` grid with 4-connectivity, no wrap-around.  Returns (nodes, edges, node_grid): nodes in
    row-major creation order, edges as index pairs in the reference's insertion order (for each cell: right, then down),
    node_grid[row][col] = index into nodes."""
    if node_type is None:
        node_type = NodeType.Spin()
    nodes = [Node(node_type) for _ in range(rows * cols)]
    grid = [[r * cols + c for c in range(cols)] for r in range(rows)]
    edges = []
    for r in range(rows):
        for c in range(cols):
            if c + 1 < cols:
                edges.append((grid[r][c], grid[r][c + 1]))
            if r + 1 < rows:
                edges.append((grid[r][c], grid[r + 1][c]))
    return nodes, np.array(edges, dtype=np.int64).reshape(-1, 2), grid


def generate_chain_graph(length, node_type=None):
    """lib.rs:83-101: a path of `length` nodes.  Returns (nodes, edges as index pairs)."""
    if node_type is None:
        node_type = NodeType.Spin()
    nodes = [Node(node_type) for _ in range(length)]
    return nodes, np.array([(i, i + 1) for i in range(max(length - 1, 0))], dtype=np.int64).reshape(-1, 2)


def bipartite_coloring(node_grid):
    """lib.rs:160-173: checkerboard colouring of a grid, colour = (row + col) % 2, as an array indexed by node index."""
    n = sum(len(r) for r in node_grid)
    colour = np.zeros(n, dtype=np.int32)
    for r, row in enumerate(node_grid):
        for c, idx in enumerate(row):
            colour[idx] = (r + c) % 2
    return colour


def greedy_coloring(n_nodes, edges, ctx=None):
    """lib.rs:114-147 on index arrays: colour per node (on the device of `ctx` when one is given)."""
    return _eng.greedy_coloring_arrays(n_nodes, edges, ctx)[0]


def coloring_to_blocks(nodes, coloring):
    """lib.rs:177-205 with ascending node index inside each colour (the reference's HashMap order is unspecified)."""
    n_colours = int(max(coloring)) + 1 if len(coloring) else 0
    groups = [[] for _ in range(n_colours)]
    for n, c in zip(nodes, coloring):
        groups[int(c)].append(n)
    return [Block(g) for g in groups if g]
