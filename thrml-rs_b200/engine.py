"""Thin object wrappers over the C ABI handles: Context, Builder (host index compiler), Program, ChainState, Moments.

These keep device state resident between calls; the reference-shaped functions in samplers.py / models.py are
written on top of them.
"""
import ctypes as C
import os

import numpy as np

from . import _ffi
from ._ffi import check, f32, i32, i64, lib, ptr

SAMPLER_SPIN = 0
SAMPLER_CATEGORICAL = 1
SAMPLER_SOFTMAX = 2

_default_ctx = {}


class Context:
    """One CUDA device + one stream (thrml_ctx)."""

    def __init__(self, device_id=0):
        self.h = C.c_void_p()
        check(lib().thrml_ctx_create(C.c_int32(device_id), C.byref(self.h)))
        self.device_id = device_id

    def synchronize(self):
        check(lib().thrml_ctx_synchronize(self.h))

    @property
    def stream(self):
        return lib().thrml_ctx_stream(self.h)

    def close(self):
        if self.h:
            lib().thrml_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def default_context(device_id=None):
    """Process-wide context; one process drives one GPU (LOCAL_RANK selects it under torchrun)."""
    if device_id is None:
        device_id = int(os.environ.get("LOCAL_RANK", "0"))
    if device_id not in _default_ctx:
        _default_ctx[device_id] = Context(device_id)
    return _default_ctx[device_id]


class Comm:
    """One rank of the library's NCCL communicator (thrml_comm); one process per GPU.

    `Comm.unique_id()` is called on rank 0 and the 128 bytes are handed to the other ranks by the host's own means;
    `Comm.from_torch(dist, ctx)` does that through an initialised torch.distributed group (any backend)."""

    def __init__(self, ctx, unique_id, rank, world_size):
        self.ctx, self.rank, self.world_size = ctx, int(rank), int(world_size)
        uid = np.ascontiguousarray(np.frombuffer(bytes(unique_id), dtype=np.uint8))
        if uid.size != 128:
            raise ValueError("a communicator id is 128 bytes")
        self.h = C.c_void_p()
        check(lib().thrml_comm_create(ctx.h, ptr(uid), C.c_int32(rank), C.c_int32(world_size), C.byref(self.h)))

    @staticmethod
    def unique_id():
        uid = np.zeros(128, dtype=np.uint8)
        check(lib().thrml_comm_unique_id(ptr(uid)))
        return uid.tobytes()

    @classmethod
    def from_torch(cls, dist, ctx):
        """Rank 0 draws the id, torch.distributed broadcasts it, every rank joins."""
        rank, world = dist.get_rank(), dist.get_world_size()
        box = [cls.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return cls(ctx, box[0], rank, world)

    def info(self):
        r, w, v = C.c_int32(), C.c_int32(), C.c_int32()
        check(lib().thrml_comm_info(self.h, C.byref(r), C.byref(w), C.byref(v)))
        return dict(rank=r.value, world_size=w.value, nccl_version=v.value)

    def close(self):
        h, self.h = getattr(self, "h", None), None
        if h and lib is not None:
            lib().thrml_comm_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def rng_split(key, n):
    out = np.zeros(max(int(n), 0), dtype=np.uint64)
    check(lib().thrml_rng_split(C.c_uint64(int(key)), C.c_int64(int(n)), ptr(out)))
    return out


def lattice_edges(side_len, torus):
    side, ne = C.c_int64(), C.c_int64()
    check(lib().thrml_lattice_edges(C.c_int64(side_len), C.c_int32(int(torus)), C.byref(side), C.byref(ne), None, None))
    edges = np.zeros((ne.value, 2), dtype=np.int64)
    colour = np.zeros(side.value * side.value, dtype=np.int32)
    check(lib().thrml_lattice_edges(C.c_int64(side_len), C.c_int32(int(torus)), C.byref(side), C.byref(ne), ptr(edges), ptr(colour)))
    return side.value, edges, colour


def greedy_coloring_arrays(n_nodes, edges, ctx=None):
    """Colour per node and the colour count; with a device context the dataflow form runs on that device (same colours)."""
    edges = i64(edges).reshape(-1, 2)
    colour = np.zeros(n_nodes, dtype=np.int32)
    nc = C.c_int32()
    if ctx is None:
        check(lib().thrml_greedy_coloring(C.c_int64(n_nodes), C.c_int64(len(edges)), ptr(edges), ptr(colour), C.byref(nc)))
    else:
        check(lib().thrml_greedy_coloring_device(ctx.h, C.c_int64(n_nodes), C.c_int64(len(edges)), ptr(edges), ptr(colour), C.byref(nc), None))
    return colour, nc.value


def pack_chains(state):
    """`[chain][node]` 0/1 bytes -> uint32 `[node][ceil(chains / 32)]` with chain c at bit c & 31 of word c // 32."""
    a = np.ascontiguousarray(state, dtype=np.uint8)
    chains, n = a.shape
    words = (chains + 31) // 32
    padded = np.zeros((n, words * 32), dtype=np.uint8)
    padded[:, :chains] = a.T
    return np.packbits(padded, axis=1, bitorder="little").view("<u4").reshape(n, words)


class Builder:
    """Host-side index compiler (thrml_builder): blocks + interaction groups -> per-block slot tables."""

    def __init__(self, kinds, dtype_order=None):
        self.kinds = i32(kinds)
        if dtype_order is None:
            dtype_order = list(dict.fromkeys(int(k) for k in self.kinds))
        order = i32(dtype_order)
        self.h = C.c_void_p()
        check(lib().thrml_builder_create(ptr(self.kinds), C.c_int64(len(self.kinds)), ptr(order), C.c_int32(len(order)), C.byref(self.h)))
        self.free_blocks = []
        self.clamped_blocks = []

    def __del__(self):
        h, self.h = getattr(self, "h", None), None
        if h and lib is not None:  # module globals are already cleared when the interpreter is shutting down
            lib().thrml_builder_destroy(h)

    def add_free_block(self, nodes, superblock=None, sampler=None):
        nodes = i64(nodes)
        if superblock is None:
            superblock = len(self.free_blocks)
        if sampler is None:
            sampler = SAMPLER_SPIN if (len(nodes) == 0 or self.kinds[nodes[0]] == 0) else SAMPLER_CATEGORICAL
        check(lib().thrml_builder_add_free_block(self.h, ptr(nodes), C.c_int64(len(nodes)), C.c_int32(superblock), C.c_int32(sampler)))
        self.free_blocks.append(nodes)

    def add_clamped_block(self, nodes):
        nodes = i64(nodes)
        check(lib().thrml_builder_add_clamped_block(self.h, ptr(nodes), C.c_int64(len(nodes))))
        self.clamped_blocks.append(nodes)

    def add_group(self, head, tails, n_spin, w):
        head = i64(head)
        rows = len(head)
        tails = i64(np.array(tails, dtype=np.int64).reshape(-1, rows)) if len(tails) else np.zeros((0, rows), dtype=np.int64)
        w = f32(w)
        if w.ndim != 3:
            w = w.reshape(rows, 1, 1) if w.size == rows else w.reshape(rows, -1, 1)
        check(lib().thrml_builder_add_interaction_group(self.h, ptr(head), C.c_int64(rows), ptr(tails), C.c_int32(tails.shape[0]), C.c_int32(n_spin), ptr(w),
                                                        C.c_int32(w.shape[1]), C.c_int32(w.shape[2])))

    def add_discrete_factor(self, spin_groups, cat_groups, w):
        w = f32(w)
        rows = w.shape[0]
        sg = i64(np.array(spin_groups, dtype=np.int64).reshape(-1, rows)) if len(spin_groups) else np.zeros((0, rows), dtype=np.int64)
        cg = i64(np.array(cat_groups, dtype=np.int64).reshape(-1, rows)) if len(cat_groups) else np.zeros((0, rows), dtype=np.int64)
        n_out = C.c_int32()
        check(lib().thrml_builder_add_discrete_factor(self.h, ptr(sg), C.c_int32(sg.shape[0]), ptr(cg), C.c_int32(cg.shape[0]), C.c_int64(rows), ptr(w),
                                                      C.c_int32(w.shape[1]), C.c_int32(w.shape[2]), C.byref(n_out)))
        return n_out.value

    def add_ising(self, nodes, biases, edges, weights, beta):
        nodes, biases = i64(nodes), f32(biases)
        edges, weights = i64(edges).reshape(-1, 2), f32(weights)
        check(lib().thrml_builder_add_ising(self.h, ptr(nodes), C.c_int64(len(nodes)), ptr(biases), ptr(edges), C.c_int64(len(edges)), ptr(weights), C.c_float(beta)))

    def compile(self, ctx=None):
        """Index compilation; with a device context the slot tables are built on that device (identical tables)."""
        if ctx is None:
            check(lib().thrml_builder_compile(self.h))
        else:
            check(lib().thrml_builder_compile_device(self.h, ctx.h))

    def counts(self):
        a, b, c, d = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
        check(lib().thrml_builder_counts(self.h, C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
        return a.value, b.value, c.value, d.value

    def node_location(self, node):
        sd, pos = C.c_int32(), C.c_int64()
        check(lib().thrml_builder_node_location(self.h, C.c_int64(int(node)), C.byref(sd), C.byref(pos)))
        return sd.value, pos.value

    def group(self, g):
        rows, nt, ns, d1, d2 = C.c_int64(), C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
        check(lib().thrml_builder_group_shape(self.h, C.c_int32(g), C.byref(rows), C.byref(nt), C.byref(ns), C.byref(d1), C.byref(d2)))
        head = np.zeros(rows.value, dtype=np.int64)
        tails = np.zeros((nt.value, rows.value), dtype=np.int64)
        w = np.zeros((rows.value, d1.value, d2.value), dtype=np.float32)
        check(lib().thrml_builder_group_data(self.h, C.c_int32(g), ptr(head), ptr(tails), ptr(w)))
        return dict(head=head, tails=tails, n_spin=ns.value, w=w)

    def tables(self, block):
        nt, n = C.c_int32(), C.c_int64()
        check(lib().thrml_builder_block_tables(self.h, C.c_int32(block), C.byref(nt), C.byref(n)))
        out = []
        for t in range(nt.value):
            k, wdim, ns, ntl, src = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
            check(lib().thrml_builder_table_shape(self.h, C.c_int32(block), C.c_int32(t), C.byref(k), C.byref(wdim), C.byref(ns), C.byref(ntl), C.byref(src)))
            nk = n.value * k.value
            rows = np.zeros(nk, dtype=np.int32)
            active = np.zeros(nk, dtype=np.uint8)
            w = np.zeros(nk * wdim.value, dtype=np.float32)
            idx = np.zeros((ntl.value, nk), dtype=np.int32)
            tsd = np.zeros(ntl.value, dtype=np.int32)
            check(lib().thrml_builder_table_data(self.h, C.c_int32(block), C.c_int32(t), ptr(rows), ptr(active), ptr(w), ptr(idx), ptr(tsd)))
            out.append(dict(k=k.value, wdim=wdim.value, n_spin=ns.value, source_group=src.value, rows=rows.reshape(n.value, k.value),
                            active=active.reshape(n.value, k.value), w=w.reshape(n.value, k.value, wdim.value), idx=idx.reshape(ntl.value, n.value, k.value), tail_sd=tsd))
        return out


OPT_DENSE_TILES = 1
OPT_SPLIT_MARGIN = 2
OPT_GATHER_ONLY = 3
OPT_STATE_FORMAT = 4


class Program:
    """Compiled tables resident on the device (thrml_program)."""

    # Options applied to every program this class creates afterwards ({option id: value}); a host-side convenience of
    # this wrapper (tests use it to run every kernel route) — the library itself keeps options per program handle.
    default_options = {}

    def __init__(self, builder, ctx=None):
        self.ctx = ctx or default_context()
        self.builder = builder
        self.h = C.c_void_p()
        check(lib().thrml_program_create(self.ctx.h, builder.h, C.byref(self.h)))
        for opt, value in self.default_options.items():
            self.set_option(opt, value)

    def set_option(self, option, value):
        check(lib().thrml_program_set_option(self.h, C.c_int32(option), C.c_double(value)))

    def get_option(self, option):
        v = C.c_double()
        check(lib().thrml_program_get_option(self.h, C.c_int32(option), C.byref(v)))
        return v.value

    def __del__(self):
        h, self.h = getattr(self, "h", None), None
        if h and lib is not None:  # module globals are already cleared when the interpreter is shutting down
            lib().thrml_program_destroy(h)

    def update_weights(self, block, table, w):
        w = f32(w)
        check(lib().thrml_program_update_weights(self.h, C.c_int32(block), C.c_int32(table), ptr(w)))

    def update_group(self, group, w, period=None, scale=1.0):
        """thrml_program_update_group: refresh on the device every table compiled from interaction group `group` from the
        group's parameter rows `w` (`[period]` or `[period, wdim]`)."""
        w = f32(w)
        w = w.reshape(w.shape[0], -1)
        check(lib().thrml_program_update_group(self.h, C.c_int32(group), ptr(w), C.c_int64(w.shape[0] if period is None else period), C.c_int32(w.shape[1]), C.c_float(scale)))

    def enable_dense(self, allow_bf16_rounding=False):
        """Switch every qualifying bipartite spin block to the tensor-core kernel; returns how many were switched."""
        n = C.c_int32()
        check(lib().thrml_program_enable_dense(self.h, C.c_int32(int(allow_bf16_rounding)), C.byref(n)))
        return n.value

    def block_kernel(self, block):
        k = C.c_int32()
        check(lib().thrml_program_block_kernel(self.h, C.c_int32(block), C.byref(k)))
        return k.value

    def block_len(self, block):
        nf = len(self.builder.free_blocks)
        return len(self.builder.free_blocks[block]) if block < nf else len(self.builder.clamped_blocks[block - nf])

    def block_kind(self, block):
        nf = len(self.builder.free_blocks)
        nodes = self.builder.free_blocks[block] if block < nf else self.builder.clamped_blocks[block - nf]
        return int(self.builder.kinds[nodes[0]])


class ChainState:
    """n_chains chains of the program's global state on the device (thrml_state)."""

    def __init__(self, program, n_chains, chain_offset=0):
        self.program = program
        self.n_chains = int(n_chains)
        self.h = C.c_void_p()
        check(lib().thrml_state_create(program.h, C.c_int64(n_chains), C.c_int64(chain_offset), C.byref(self.h)))

    def __del__(self):
        h, self.h = getattr(self, "h", None), None
        if h and lib is not None:  # module globals are already cleared when the interpreter is shutting down
            lib().thrml_state_destroy(h)

    def upload(self, block, host):
        n = self.program.block_len(block)
        host = np.asarray(host)
        if host.dtype == np.uint8:
            host = np.ascontiguousarray(host).reshape(self.n_chains, n)
            check(lib().thrml_state_upload_u8(self.h, C.c_int32(block), ptr(host)))
        else:
            host = f32(host).reshape(self.n_chains, n)
            check(lib().thrml_state_upload_f32(self.h, C.c_int32(block), ptr(host)))

    def upload_many(self, blocks, hosts):
        """thrml_state_upload_u8_many: several blocks' `[chain][node]` byte arrays, one host wait for all of them."""
        blocks = i32(blocks)
        hosts = [np.ascontiguousarray(h, dtype=np.uint8).reshape(self.n_chains, self.program.block_len(int(b))) for b, h in zip(blocks, hosts)]
        ptrs = (C.c_void_p * len(hosts))(*[h.ctypes.data for h in hosts])
        check(lib().thrml_state_upload_u8_many(self.h, ptr(blocks), C.c_int32(len(hosts)), ptrs))

    def upload_packed(self, blocks, bits):
        """thrml_state_upload_packed: spin blocks as bits, `bits[i]` = uint32 `[node][ceil(chains / 32)]`, bit c & 31 of word
        c // 32 = chain c (the layout `sample_states_packed` returns and `pack_chains` produces)."""
        blocks = i32(blocks)
        words = (self.n_chains + 31) // 32
        bits = [np.ascontiguousarray(b, dtype=np.uint32).reshape(self.program.block_len(int(k)), words) for k, b in zip(blocks, bits)]
        ptrs = (C.c_void_p * len(bits))(*[b.ctypes.data for b in bits])
        check(lib().thrml_state_upload_packed(self.h, ptr(blocks), C.c_int32(len(bits)), ptrs))

    def upload_static(self, block, host):
        """thrml_state_upload_u8_static: the same upload staged in the library's fixed 4 MiB device array, for hosts that
        must not allocate device memory while running.  Blocks above 4 MiB (nodes x chains) raise ThrmlError."""
        n = self.program.block_len(block)
        host = np.ascontiguousarray(host, dtype=np.uint8).reshape(self.n_chains, n)
        check(lib().thrml_state_upload_u8_static(self.h, C.c_int32(block), ptr(host)))

    def copy_block_from(self, other, block):
        check(lib().thrml_state_copy_block(self.h, other.h, C.c_int32(block)))

    def download(self, block, dtype=np.float32):
        n = self.program.block_len(block)
        out = np.zeros((self.n_chains, n), dtype=dtype)
        if dtype == np.uint8:
            check(lib().thrml_state_download_u8(self.h, C.c_int32(block), ptr(out)))
        else:
            check(lib().thrml_state_download_f32(self.h, C.c_int32(block), ptr(out)))
        return out

    def download_chains(self, block, chain_begin, n_chains):
        """uint8 `[n_chains][node]` of chains chain_begin .. chain_begin + n_chains - 1 of one block."""
        out = np.zeros((int(n_chains), self.program.block_len(block)), dtype=np.uint8)
        check(lib().thrml_state_download_chains_u8(self.h, C.c_int32(block), C.c_int64(chain_begin), C.c_int64(n_chains), ptr(out)))
        return out

    def hinton_init(self, blocks, biases, beta, key, inj_u=None):
        blocks, biases = i32(blocks), f32(biases)
        inj = f32(inj_u).ravel() if inj_u is not None else None
        check(lib().thrml_hinton_init(self.h, ptr(blocks), C.c_int32(len(blocks)), ptr(biases), C.c_float(beta), C.c_uint64(int(key)), ptr(inj)))

    def randomize(self, key):
        check(lib().thrml_state_randomize(self.h, C.c_uint64(int(key))))

    def sample_blocks(self, key, inj=None):
        nz, keep = _ffi.make_noise(inj)
        check(lib().thrml_sample_blocks(self.h, C.c_uint64(int(key)), C.byref(nz) if nz else None))

    def run_blocks(self, key, n_iters, inj=None):
        nz, keep = _ffi.make_noise(inj)
        check(lib().thrml_run_blocks(self.h, C.c_uint64(int(key)), C.c_int64(n_iters), C.byref(nz) if nz else None))

    def ising_energy(self, nodes, biases, edges, weights, beta):
        """Per-chain Ising energy of the current state (f64)."""
        nodes, biases = i64(nodes), f32(biases)
        edges, weights = i64(edges).reshape(-1, 2), f32(weights)
        out = np.zeros(self.n_chains, dtype=np.float64)
        check(lib().thrml_ising_energy(self.h, C.c_int64(len(nodes)), ptr(nodes), ptr(biases), C.c_int64(len(edges)), ptr(edges), ptr(weights), C.c_float(beta), ptr(out)))
        return out

    def factor_energy(self, spin_groups, cat_groups, weights):
        """Per-chain energy of one discrete factor (f64): node-id lists per group, weights `[rows, d1, d2]`."""
        w = f32(weights)
        w = w.reshape(w.shape[0], -1, 1) if w.ndim < 3 else w
        groups = [i64(g) for g in list(spin_groups) + list(cat_groups)]
        nodes = np.ascontiguousarray(np.stack(groups)) if groups else np.zeros((0, w.shape[0]), dtype=np.int64)
        out = np.zeros(self.n_chains, dtype=np.float64)
        check(lib().thrml_factor_energy(self.h, C.c_int64(w.shape[0]), C.c_int32(len(spin_groups)), C.c_int32(len(cat_groups)), ptr(nodes), ptr(w),
                                        C.c_int32(w.shape[1]), C.c_int32(w.shape[2]), ptr(out)))
        return out

    def sample_single_block(self, block, key):
        check(lib().thrml_sample_single_block(self.h, C.c_int32(block), C.c_uint64(int(key))))

    def pair_correlation(self, block_a, block_b):
        out = np.zeros((self.program.block_len(block_a), self.program.block_len(block_b)), dtype=np.float32)
        check(lib().thrml_pair_correlation(self.h, C.c_int32(block_a), C.c_int32(block_b), ptr(out)))
        return out

    def cd1_step(self, visible_block, hidden_block, v0, key, want_stats=True, data=None, out=None, comm=None):
        """One CD-1 step.  v0: host `[chain][visible]` bytes to upload first (None = keep the current visible state);
        data: another ChainState whose visible block is the data (read in place, thrml_cd1_step_from); out: optional pair of
        caller-owned f32 `[n_visible][n_hidden]` arrays for the two correlation matrices (pinned memory copies faster);
        comm: chains sharded over the communicator's ranks, the matrices are means over all of them (thrml_cd1_step_comm)."""
        nv, nh = self.program.block_len(visible_block), self.program.block_len(hidden_block)
        v0 = np.ascontiguousarray(v0, dtype=np.uint8).reshape(self.n_chains, nv) if v0 is not None else None
        pos, neg = out if out is not None else ((np.zeros((nv, nh), dtype=np.float32), np.zeros((nv, nh), dtype=np.float32)) if want_stats else (None, None))
        if comm is not None:
            check(lib().thrml_cd1_step_comm(self.h, data.h if data is not None else None, C.c_int32(visible_block), C.c_int32(hidden_block), C.c_uint64(int(key)), comm.h,
                                            ptr(pos), ptr(neg)))
        elif data is not None:
            check(lib().thrml_cd1_step_from(self.h, data.h, C.c_int32(visible_block), C.c_int32(hidden_block), C.c_uint64(int(key)), ptr(pos), ptr(neg)))
        else:
            check(lib().thrml_cd1_step(self.h, C.c_int32(visible_block), C.c_int32(hidden_block), ptr(v0), C.c_uint64(int(key)), ptr(pos), ptr(neg)))
        return pos, neg

    def fields(self, block):
        n = self.program.block_len(block)
        kind = self.program.block_kind(block)
        shape = (self.n_chains, n, kind) if kind > 0 else (self.n_chains, n)
        out = np.zeros(shape, dtype=np.float32)
        check(lib().thrml_fields_debug(self.h, C.c_int32(block), ptr(out)))
        return out

    def pair_tmem_check(self):
        """Bring-up check of the CTA-pair kernels: raises if the two CTAs of the last pair launch disagreed on their
        tensor-memory base."""
        check(lib().thrml_debug_pair_tmem_check(self.h))

    def launch_counts(self):
        """(per-block update launches, persistent multi-sweep launches) issued by this state so far."""
        a, b = C.c_int64(), C.c_int64()
        check(lib().thrml_state_launch_counts(self.h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def sample_states_packed(self, key, n_warmup, n_samples, steps_per_sample, obs_blocks):
        """Samples of the listed spin blocks as bits: uint32 [samples][observed node][ceil(chains/32)]."""
        ob = i32(obs_blocks)
        rows = sum(self.program.block_len(int(b)) for b in ob)
        out = np.zeros((max(int(n_samples), 1), rows, (self.n_chains + 31) // 32), dtype=np.uint32)
        check(lib().thrml_sample_states_packed(self.h, C.c_uint64(int(key)), C.c_int64(n_warmup), C.c_int64(n_samples), C.c_int64(steps_per_sample), ptr(ob),
                                               C.c_int32(len(ob)), ptr(out)))
        return out

    def sample_with_observation(self, key, n_warmup, n_samples, steps_per_sample, moments=None, obs_blocks=None, inj=None):
        nz, keep = _ffi.make_noise(inj)
        obs, ob = None, None
        if obs_blocks is not None:
            ob = i32(obs_blocks)
            rows = sum(self.program.block_len(int(b)) for b in ob)
            obs = np.zeros((max(int(n_samples), 1), rows, self.n_chains), dtype=np.uint8)
        check(lib().thrml_sample_with_observation(self.h, C.c_uint64(int(key)), C.c_int64(n_warmup), C.c_int64(n_samples), C.c_int64(steps_per_sample),
                                                  moments.h if moments is not None else None, ptr(ob), C.c_int32(0 if ob is None else len(ob)), ptr(obs),
                                                  C.byref(nz) if nz else None))
        return obs


def estimate_kl_grad(pos_state, neg_state, moments_pos, moments_neg, key, schedule_pos, schedule_neg, beta):
    """thrml_estimate_kl_grad: both phases and -beta (mean_pos - mean_neg) on the device; schedules are
    (n_warmup, n_samples, steps_per_sample).  Returns (grad_w, grad_b) as f32 arrays."""
    n_b, n_w = int(moments_pos.rows_per_type[0]), int(moments_pos.rows_per_type[1])
    gw, gb = np.zeros(max(n_w, 1), dtype=np.float32), np.zeros(max(n_b, 1), dtype=np.float32)
    check(lib().thrml_estimate_kl_grad(pos_state.h, neg_state.h, moments_pos.h, moments_neg.h, C.c_uint64(int(key)), *[C.c_int64(int(x)) for x in schedule_pos],
                                       *[C.c_int64(int(x)) for x in schedule_neg], C.c_float(beta), ptr(gw), ptr(gb)))
    return gw[:n_w], gb[:n_b]


class Moments:
    """Moment accumulator on the device (thrml_moments).  spec: list of moment types, each a list of node-id tuples."""

    def __init__(self, program, spec, transform_to_spin=True):
        self.program = program
        self.rows_per_type = np.array([len(t) for t in spec], dtype=np.int64)
        flat, ptrs = [], [0]
        for t in spec:
            for row in t:
                flat.extend(int(x) for x in row)
                ptrs.append(len(flat))
        self.row_ptr = np.array(ptrs, dtype=np.int64)
        self.members = np.array(flat, dtype=np.int64) if flat else np.zeros(1, dtype=np.int64)
        self.h = C.c_void_p()
        check(lib().thrml_moments_create(program.h, C.c_int32(len(spec)), ptr(self.rows_per_type), ptr(self.row_ptr), ptr(self.members),
                                         C.c_int32(int(transform_to_spin)), C.byref(self.h)))

    @classmethod
    def from_arrays(cls, program, rows_per_type, row_ptr, members, transform_to_spin=True):
        self = cls.__new__(cls)
        self.program = program
        self.rows_per_type = i64(rows_per_type)
        self.row_ptr = i64(row_ptr)
        self.members = i64(members)
        self.h = C.c_void_p()
        check(lib().thrml_moments_create(program.h, C.c_int32(len(self.rows_per_type)), ptr(self.rows_per_type), ptr(self.row_ptr), ptr(self.members),
                                         C.c_int32(int(transform_to_spin)), C.byref(self.h)))
        return self

    @classmethod
    def marginals(cls, program, blocks, K):
        self = cls.__new__(cls)
        self.program = program
        blocks = i32(blocks)
        n = sum(program.block_len(int(b)) for b in blocks)
        self.rows_per_type = np.array([n * K], dtype=np.int64)
        self.h = C.c_void_p()
        check(lib().thrml_marginals_create(program.h, ptr(blocks), C.c_int32(len(blocks)), C.c_int32(K), C.byref(self.h)))
        return self

    def __del__(self):
        h, self.h = getattr(self, "h", None), None
        if h and lib is not None:  # module globals are already cleared when the interpreter is shutting down
            lib().thrml_moments_destroy(h)

    def reset(self):
        check(lib().thrml_moments_reset(self.h))

    def observe(self, state):
        check(lib().thrml_moments_observe(self.h, state.h))

    def read(self, t, out=None):
        """(int64 sums of moment type t, observations x chains).  `out` may be a caller-owned int64 array (pinned host
        memory makes the copy run at link speed)."""
        if out is None:
            out = np.zeros(int(self.rows_per_type[t]), dtype=np.int64)
        assert out.dtype == np.int64 and out.size >= int(self.rows_per_type[t])
        n = C.c_int64()
        check(lib().thrml_moments_read(self.h, C.c_int32(t), ptr(out), C.byref(n)))
        return out, n.value

    def allreduce(self, comm):
        """thrml_moments_allreduce: the one collective of the chain-parallel path (sums and observation count, in place)."""
        check(lib().thrml_moments_allreduce(self.h, comm.h))

    def fused_info(self):
        """(rows accumulated by the update kernels, rows left to the observer kernel)."""
        a, b = C.c_int64(), C.c_int64()
        check(lib().thrml_moments_fused_info(self.h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def device_buffer(self):
        p, cnt = C.c_void_p(), C.c_int64()
        check(lib().thrml_moments_device_buffer(self.h, C.byref(p), C.byref(cnt)))
        return p.value, cnt.value
