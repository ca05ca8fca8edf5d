"""Implicit 3-D Potts lattice (thrml_potts): handle wrapper.  The sweep and schedule drivers live in the library
(thrml_potts_run_blocks, thrml_potts_sample_with_marginals); key handling mirrors sample_blocks / run_blocks /
sample_with_observation (crates/thrml-samplers/src/sampling.rs:28-320): per sweep key.split(2) gives the two colours'
block keys.
"""
import ctypes as C

import numpy as np

from . import engine as _eng
from ._ffi import check, f32, lib, ptr


NOISE_PROGRAM = 0  # the explicit factor program's key -> noise mapping: states equal FactorSamplingProgram's on the same torus
NOISE_QUAD = 1     # the engine's own mapping (default): one generator call per category serves four chains


class PottsLattice:
    def __init__(self, nx, ny, nz, n_categories, tables, unary, beta, n_chains, chain_offset=0, ctx=None, noise=NOISE_QUAD):
        self.ctx = ctx or _eng.default_context()
        self.shape, self.K, self.n_chains = (nx, ny, nz), n_categories, n_chains
        self.n = nx * ny * nz
        tables = f32(tables).reshape(3, n_categories, n_categories)
        unary = f32(unary).reshape(self.n, n_categories) if unary is not None else None
        self.h = C.c_void_p()
        check(lib().thrml_potts_create(self.ctx.h, C.c_int32(nx), C.c_int32(ny), C.c_int32(nz), C.c_int32(n_categories), ptr(tables), ptr(unary), C.c_float(beta),
                                       C.c_int64(n_chains), C.c_int64(chain_offset), C.byref(self.h)))
        check(lib().thrml_potts_set_noise(self.h, C.c_int32(noise)))

    def __del__(self):
        h, self.h = getattr(self, "h", None), None
        if h and lib is not None:  # module globals are already cleared when the interpreter is shutting down
            lib().thrml_potts_destroy(h)

    def randomize(self, key):
        check(lib().thrml_potts_randomize(self.h, C.c_uint64(int(key))))

    def upload(self, cats):
        a = np.ascontiguousarray(cats, dtype=np.uint8).reshape(self.n_chains, self.n)
        check(lib().thrml_potts_upload(self.h, ptr(a)))

    def download(self):
        out = np.zeros((self.n_chains, self.n), dtype=np.uint8)
        check(lib().thrml_potts_download(self.h, ptr(out)))
        return out

    def sample_blocks(self, key):
        k = _eng.rng_split(key, 2)
        for colour in (0, 1):
            check(lib().thrml_potts_update(self.h, C.c_int32(colour), C.c_uint64(int(k[colour]))))

    def run_blocks(self, key, n_iters):
        """thrml_potts_run_blocks (asynchronous)."""
        check(lib().thrml_potts_run_blocks(self.h, C.c_uint64(int(key)), C.c_int64(n_iters)))

    def observe_marginals(self):
        check(lib().thrml_potts_observe_marginals(self.h))

    def sample_with_marginals(self, key, n_warmup, n_samples, steps_per_sample):
        """thrml_potts_sample_with_marginals: sample_with_observation with the category-marginal observer."""
        check(lib().thrml_potts_sample_with_marginals(self.h, C.c_uint64(int(key)), C.c_int64(n_warmup), C.c_int64(n_samples), C.c_int64(steps_per_sample)))

    def allreduce_marginals(self, comm):
        check(lib().thrml_potts_marginals_allreduce(self.h, comm.h))

    def read_marginals(self):
        out = np.zeros((self.n, self.K), dtype=np.int32)
        n = C.c_int64()
        check(lib().thrml_potts_read_marginals(self.h, ptr(out), C.byref(n)))
        return out, n.value

    def reset_marginals(self):
        check(lib().thrml_potts_reset_marginals(self.h))

    def synchronize(self):
        check(lib().thrml_potts_synchronize(self.h))
