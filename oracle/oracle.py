"""ctypes binding of the CPU oracle (oracle/liboracle.so).  Test infrastructure: imported only by tests/,
__graft_entry__.smoke() and bench.py's CPU-baseline legs, never by the product package."""
import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None

i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
i64p = np.ctypeslib.ndpointer(np.int64, flags="C_CONTIGUOUS")
f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")


def lib():
    global _lib
    if _lib is None:
        path = _build.OUT
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(_build.SRC):
            _build.build()
        _lib = C.CDLL(path)
        _lib.orc_last_error.restype = C.c_char_p
        _lib.orc_det_sigmoid.restype = C.c_float
        _lib.orc_det_sigmoid.argtypes = [C.c_float]
        _lib.orc_det_log.restype = C.c_float
        _lib.orc_det_log.argtypes = [C.c_float]
        _lib.orc_u24.restype = C.c_float
        _lib.orc_u24.argtypes = [C.c_uint32]
        _lib.orc_u23_open.restype = C.c_float
        _lib.orc_u23_open.argtypes = [C.c_uint32]
        _lib.orc_spin_product.restype = C.c_int64
    return _lib


class OracleError(RuntimeError):
    pass


def _chk(rc):
    if rc != 0:
        raise OracleError(lib().orc_last_error().decode())


def _p(a, ct):
    return a.ctypes.data_as(C.POINTER(ct)) if a is not None else None


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def rng_split(key, n):
    out = np.zeros(max(n, 0), dtype=np.uint64)
    lib().orc_rng_split(C.c_uint64(key), C.c_int64(n), _p(out, C.c_uint64))
    return out


def chacha_block(key8, counter, stream, rounds):
    key8 = np.ascontiguousarray(key8, dtype=np.uint32)
    out = np.zeros(16, dtype=np.uint32)
    lib().orc_chacha_block(_p(key8, C.c_uint32), C.c_uint64(counter), C.c_uint64(stream), C.c_int(rounds), _p(out, C.c_uint32))
    return out


def philox(ctr4, key2):
    ctr4 = np.ascontiguousarray(ctr4, dtype=np.uint32)
    key2 = np.ascontiguousarray(key2, dtype=np.uint32)
    out = np.zeros(4, dtype=np.uint32)
    lib().orc_philox(_p(ctr4, C.c_uint32), _p(key2, C.c_uint32), _p(out, C.c_uint32))
    return out


def det_sigmoid(x):
    return float(lib().orc_det_sigmoid(C.c_float(x)))


def det_log(x):
    return float(lib().orc_det_log(C.c_float(x)))


def spin_product(lists):
    n_lists = len(lists)
    n = len(lists[0]) if n_lists else 0
    vals = np.ascontiguousarray(np.array(lists, dtype=np.uint8).reshape(n_lists, n))
    out = np.zeros(max(n, 1), dtype=np.float32)
    cnt = lib().orc_spin_product(_p(vals, C.c_uint8), C.c_int32(n_lists), C.c_int64(n), _p(out, C.c_float))
    return out[:cnt]


def batch_gather(w, idx_lists):
    w = _f32(w)
    batch = w.shape[0]
    dims = np.array(w.shape[1:], dtype=np.int32)
    idx = np.ascontiguousarray(np.array(idx_lists, dtype=np.int32).reshape(len(dims), batch))
    out = np.zeros(batch, dtype=np.float32)
    _chk(lib().orc_batch_gather(_p(w, C.c_float), C.c_int64(batch), _p(dims, C.c_int32), C.c_int32(len(dims)), _p(idx, C.c_int32), _p(out, C.c_float)))
    return out


def batch_gather_strided(w, idx, strides, batch_stride):
    w = _f32(w).ravel()
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    strides = _i64(strides)
    out = np.zeros(idx.shape[0], dtype=np.float32)
    _chk(lib().orc_batch_gather_strided(_p(w, C.c_float), C.c_int64(w.size), C.c_int64(idx.shape[0]), C.c_int32(idx.shape[1]), _p(idx, C.c_int32), _p(strides, C.c_int64),
                                        C.c_int64(batch_stride), _p(out, C.c_float)))
    return out


def factor_energy(weights, spin_vals, cat_vals):
    """DiscreteEBMFactor::factor_energy (crates/thrml-models/src/discrete_ebm.rs:552-592) restated with numpy in f64:
    E = -sum_rows W[row, c_1, ...] * prod_groups (2 s - 1).  spin_vals / cat_vals: lists of `[rows]` (or
    `[chains, rows]`) arrays gathered per node group; weights `[rows, d1, d2]`.  Returns a scalar or `[chains]`."""
    w = np.asarray(weights, dtype=np.float64)
    rows = w.shape[0]
    w = w.reshape(rows, -1) if len(cat_vals) == 0 else w
    idx = np.arange(rows)
    if len(cat_vals) == 0:
        g = w[:, 0]
    elif len(cat_vals) == 1:
        g = w.reshape(rows, w.shape[1], -1)[idx, np.asarray(cat_vals[0], dtype=np.int64), 0]
    else:
        g = w[idx, np.asarray(cat_vals[0], dtype=np.int64), np.asarray(cat_vals[1], dtype=np.int64)]
    prod = 1.0
    for sv in spin_vals:
        prod = prod * (2.0 * np.asarray(sv, dtype=np.float64) - 1.0)
    return -np.sum(g * prod, axis=-1)


def lattice_edges(side_len, torus):
    side = C.c_int64()
    ne = C.c_int64()
    _chk(lib().orc_lattice_edges(C.c_int64(side_len), C.c_int32(int(torus)), C.byref(side), C.byref(ne), None, None))
    edges = np.zeros((ne.value, 2), dtype=np.int64)
    colour = np.zeros(side.value * side.value, dtype=np.int32)
    _chk(lib().orc_lattice_edges(C.c_int64(side_len), C.c_int32(int(torus)), C.byref(side), C.byref(ne), _p(edges, C.c_int64), _p(colour, C.c_int32)))
    return side.value, edges, colour


def greedy_coloring(n, edges):
    edges = _i64(edges).reshape(-1, 2)
    colour = np.zeros(n, dtype=np.int32)
    nc = C.c_int32()
    _chk(lib().orc_greedy_coloring(C.c_int64(n), C.c_int64(len(edges)), _p(edges, C.c_int64), _p(colour, C.c_int32), C.byref(nc)))
    return colour, nc.value


def categorical_sample(logits, u, use_libm=False):
    logits = _f32(logits)
    u = _f32(u)
    n, K = logits.shape
    out = np.zeros(n, dtype=np.float32)
    _chk(lib().orc_categorical_sample(_p(logits, C.c_float), _p(u, C.c_float), C.c_int64(n), C.c_int32(K), _p(out, C.c_float), C.c_int32(int(use_libm))))
    return out


def sigmoid_bernoulli(gamma, u, inclusive=True):
    gamma = _f32(gamma)
    u = _f32(u)
    out = np.zeros(gamma.shape, dtype=np.float32)
    _chk(lib().orc_sigmoid_bernoulli(_p(gamma, C.c_float), _p(u, C.c_float), C.c_int64(gamma.size), _p(out, C.c_float), C.c_int32(int(inclusive))))
    return out


class Model:
    """Index compiler of the oracle: the same call sequence as the library's builder."""

    def __init__(self, kinds, dtype_order=None):
        kinds = np.ascontiguousarray(kinds, dtype=np.int32)
        if dtype_order is None:
            dtype_order = list(dict.fromkeys(int(k) for k in kinds))
        order = np.ascontiguousarray(dtype_order, dtype=np.int32)
        self.kinds = kinds
        self.h = C.c_void_p()
        _chk(lib().orc_model_create(_p(kinds, C.c_int32), C.c_int64(len(kinds)), _p(order, C.c_int32), C.c_int32(len(order)), C.byref(self.h)))
        self.free_blocks = []
        self.clamped_blocks = []

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_model_destroy(self.h)
            self.h = None

    def add_free_block(self, nodes, superblock=None, sampler=None):
        nodes = _i64(nodes)
        if superblock is None:
            superblock = len(self.free_blocks)
        if sampler is None:
            sampler = 0 if (len(nodes) == 0 or self.kinds[nodes[0]] == 0) else 1
        _chk(lib().orc_model_add_free_block(self.h, _p(nodes, C.c_int64), C.c_int64(len(nodes)), C.c_int32(superblock), C.c_int32(sampler)))
        self.free_blocks.append(nodes)

    def add_clamped_block(self, nodes):
        nodes = _i64(nodes)
        _chk(lib().orc_model_add_clamped_block(self.h, _p(nodes, C.c_int64), C.c_int64(len(nodes))))
        self.clamped_blocks.append(nodes)

    def add_group(self, head, tails, n_spin, w):
        head = _i64(head)
        rows = len(head)
        tails = _i64(np.array(tails, dtype=np.int64).reshape(-1, rows)) if len(tails) else np.zeros((0, rows), dtype=np.int64)
        w = _f32(w).reshape(rows, *(np.shape(w)[1:] if np.ndim(w) == 3 else (1, 1)))
        _chk(lib().orc_model_add_group(self.h, _p(head, C.c_int64), C.c_int64(rows), _p(tails, C.c_int64), C.c_int32(tails.shape[0]), C.c_int32(n_spin),
                                       _p(w, C.c_float), C.c_int32(w.shape[1]), C.c_int32(w.shape[2])))

    def add_discrete_factor(self, spin_groups, cat_groups, w):
        w = _f32(w)
        rows = w.shape[0]
        sg = _i64(np.array(spin_groups, dtype=np.int64).reshape(-1, rows)) if len(spin_groups) else np.zeros((0, rows), dtype=np.int64)
        cg = _i64(np.array(cat_groups, dtype=np.int64).reshape(-1, rows)) if len(cat_groups) else np.zeros((0, rows), dtype=np.int64)
        n_out = C.c_int32()
        _chk(lib().orc_model_add_discrete_factor(self.h, _p(sg, C.c_int64), C.c_int32(sg.shape[0]), _p(cg, C.c_int64), C.c_int32(cg.shape[0]), C.c_int64(rows),
                                                 _p(w, C.c_float), C.c_int32(w.shape[1]), C.c_int32(w.shape[2]), C.byref(n_out)))
        return n_out.value

    def add_ising(self, nodes, biases, edges, weights, beta):
        nodes = _i64(nodes)
        biases = _f32(biases)
        edges = _i64(edges).reshape(-1, 2)
        weights = _f32(weights)
        _chk(lib().orc_model_add_ising(self.h, _p(nodes, C.c_int64), C.c_int64(len(nodes)), _p(biases, C.c_float), _p(edges, C.c_int64), C.c_int64(len(edges)),
                                       _p(weights, C.c_float), C.c_float(beta)))

    def compile(self):
        _chk(lib().orc_model_compile(self.h))

    def counts(self):
        a, b, c, d = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
        _chk(lib().orc_model_counts(self.h, C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
        return a.value, b.value, c.value, d.value

    def node_location(self, node):
        sd, pos = C.c_int32(), C.c_int64()
        _chk(lib().orc_model_node_location(self.h, C.c_int64(node), C.byref(sd), C.byref(pos)))
        return sd.value, pos.value

    def group(self, g):
        rows, nt, ns, d1, d2 = C.c_int64(), C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
        _chk(lib().orc_model_group_shape(self.h, C.c_int32(g), C.byref(rows), C.byref(nt), C.byref(ns), C.byref(d1), C.byref(d2)))
        head = np.zeros(rows.value, dtype=np.int64)
        tails = np.zeros((nt.value, rows.value), dtype=np.int64)
        w = np.zeros((rows.value, d1.value, d2.value), dtype=np.float32)
        _chk(lib().orc_model_group_data(self.h, C.c_int32(g), _p(head, C.c_int64), _p(tails, C.c_int64), _p(w, C.c_float)))
        return dict(head=head, tails=tails, n_spin=ns.value, w=w)

    def tables(self, block):
        nt, n = C.c_int32(), C.c_int64()
        _chk(lib().orc_model_block_tables(self.h, C.c_int32(block), C.byref(nt), C.byref(n)))
        out = []
        for t in range(nt.value):
            k, wdim, ns, ntl, src = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
            _chk(lib().orc_model_table_shape(self.h, C.c_int32(block), C.c_int32(t), C.byref(k), C.byref(wdim), C.byref(ns), C.byref(ntl), C.byref(src)))
            nk = n.value * k.value
            rows = np.zeros(nk, dtype=np.int32)
            active = np.zeros(nk, dtype=np.uint8)
            w = np.zeros(nk * wdim.value, dtype=np.float32)
            idx = np.zeros((ntl.value, nk), dtype=np.int32)
            tsd = np.zeros(ntl.value, dtype=np.int32)
            _chk(lib().orc_model_table_data(self.h, C.c_int32(block), C.c_int32(t), _p(rows, C.c_int32), _p(active, C.c_uint8), _p(w, C.c_float), _p(idx, C.c_int32), _p(tsd, C.c_int32)))
            out.append(dict(k=k.value, wdim=wdim.value, n_spin=ns.value, source_group=src.value, rows=rows.reshape(n.value, k.value),
                            active=active.reshape(n.value, k.value), w=w.reshape(n.value, k.value, wdim.value), idx=idx.reshape(ntl.value, n.value, k.value), tail_sd=tsd))
        return out


class State:
    def __init__(self, model, n_chains, chain_offset=0, threads=1):
        self.model = model
        self.n_chains = n_chains
        self.h = C.c_void_p()
        _chk(lib().orc_state_create(model.h, C.c_int64(n_chains), C.c_int64(chain_offset), C.byref(self.h)))
        lib().orc_state_set_threads(self.h, C.c_int32(threads))

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_state_destroy(self.h)
            self.h = None

    def set_spin_noise(self, mapping):
        """0 = one 32-bit word per (spin, chain) (the gather kernels' mapping), 1 = the implicit lattice engine's bit-sliced
        mapping, 2 = the dense (tensor-core) path's mapping."""
        lib().orc_state_set_spin_noise(self.h, C.c_int32(mapping))

    def set_cat_noise(self, mapping):
        """0 = the explicit categorical kernels' mapping, 1 = the implicit Potts engine's (one call per category and chain quad)."""
        lib().orc_state_set_cat_noise(self.h, C.c_int32(mapping))

    def _block_len(self, block):
        nf = len(self.model.free_blocks)
        return len(self.model.free_blocks[block]) if block < nf else len(self.model.clamped_blocks[block - nf])

    def set_block(self, block, host):
        host = _f32(host).reshape(self.n_chains, self._block_len(block))
        _chk(lib().orc_state_set_block(self.h, C.c_int32(block), _p(host, C.c_float)))

    def get_block(self, block):
        out = np.zeros((self.n_chains, self._block_len(block)), dtype=np.float32)
        _chk(lib().orc_state_get_block(self.h, C.c_int32(block), _p(out, C.c_float)))
        return out

    def fields(self, block):
        n = self._block_len(block)
        kind = int(self.model.kinds[self.model.free_blocks[block][0]])
        width = n * max(kind, 1)
        o64 = np.zeros((self.n_chains, width), dtype=np.float64)
        o32 = np.zeros((self.n_chains, width), dtype=np.float32)
        _chk(lib().orc_fields(self.h, C.c_int32(block), _p(o64, C.c_double), _p(o32, C.c_float)))
        if kind > 0:
            return o64.reshape(self.n_chains, n, kind), o32.reshape(self.n_chains, n, kind)
        return o64, o32

    def sample_blocks(self, key, inj=None):
        inj = _f32(inj).ravel() if inj is not None else None
        _chk(lib().orc_sample_blocks(self.h, C.c_uint64(key), _p(inj, C.c_float), C.c_int64(0 if inj is None else inj.size)))

    def sample_single_block(self, block, key):
        _chk(lib().orc_sample_single_block(self.h, C.c_int32(block), C.c_uint64(key)))

    def run_blocks(self, key, n_iters, inj=None):
        inj = _f32(inj).ravel() if inj is not None else None
        _chk(lib().orc_run_blocks(self.h, C.c_uint64(key), C.c_int64(n_iters), _p(inj, C.c_float), C.c_int64(0 if inj is None else inj.size)))

    def hinton_init(self, blocks, biases, beta, key, inj_u=None):
        blocks = np.ascontiguousarray(blocks, dtype=np.int32)
        biases = _f32(biases)
        inj_u = _f32(inj_u).ravel() if inj_u is not None else None
        _chk(lib().orc_hinton_init(self.h, _p(blocks, C.c_int32), C.c_int32(len(blocks)), _p(biases, C.c_float), C.c_float(beta), C.c_uint64(key), _p(inj_u, C.c_float)))

    def randomize(self, key):
        _chk(lib().orc_state_randomize(self.h, C.c_uint64(key)))

    def sample_with_observation(self, key, n_warmup, n_samples, steps_per_sample, moments=None, obs_blocks=None, inj=None):
        inj = _f32(inj).ravel() if inj is not None else None
        obs = None
        ob = None
        if obs_blocks is not None:
            ob = np.ascontiguousarray(obs_blocks, dtype=np.int32)
            rows = sum(self._block_len(int(b)) for b in ob)
            obs = np.zeros((max(n_samples, 1), rows, self.n_chains), dtype=np.uint8)
        _chk(lib().orc_sample_with_observation(self.h, C.c_uint64(key), C.c_int64(n_warmup), C.c_int64(n_samples), C.c_int64(steps_per_sample),
                                               moments.h if moments is not None else None, _p(ob, C.c_int32), C.c_int32(0 if ob is None else len(ob)),
                                               _p(obs, C.c_uint8), _p(inj, C.c_float), C.c_int64(0 if inj is None else inj.size)))
        return obs


class Moments:
    def __init__(self, model, spec, transform_to_spin=True):
        """spec: list (moment types) of lists (rows) of node-id tuples."""
        self.rows_per_type = np.array([len(t) for t in spec], dtype=np.int64)
        flat, ptr = [], [0]
        for t in spec:
            for row in t:
                flat.extend(int(x) for x in row)
                ptr.append(len(flat))
        self.row_ptr = np.array(ptr, dtype=np.int64)
        self.members = np.array(flat, dtype=np.int64) if flat else np.zeros(0, dtype=np.int64)
        self.h = C.c_void_p()
        _chk(lib().orc_moments_create(model.h, C.c_int32(len(spec)), _p(self.rows_per_type, C.c_int64), _p(self.row_ptr, C.c_int64), _p(self.members, C.c_int64),
                                      C.c_int32(int(transform_to_spin)), C.byref(self.h)))

    @classmethod
    def from_arrays(cls, model, rows_per_type, row_ptr, members, transform_to_spin=True):
        self = cls.__new__(cls)
        self.rows_per_type = _i64(rows_per_type)
        self.row_ptr = _i64(row_ptr)
        self.members = _i64(members)
        self.h = C.c_void_p()
        _chk(lib().orc_moments_create(model.h, C.c_int32(len(self.rows_per_type)), _p(self.rows_per_type, C.c_int64), _p(self.row_ptr, C.c_int64),
                                      _p(self.members, C.c_int64), C.c_int32(int(transform_to_spin)), C.byref(self.h)))
        return self

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_moments_destroy(self.h)
            self.h = None

    def observe(self, state):
        _chk(lib().orc_moments_observe(self.h, state.h))

    def read(self, t):
        out = np.zeros(int(self.rows_per_type[t]), dtype=np.int64)
        n = C.c_int64()
        _chk(lib().orc_moments_read(self.h, C.c_int32(t), _p(out, C.c_int64), C.byref(n)))
        return out, n.value
