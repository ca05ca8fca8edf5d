"""Implicit bit-packed Ising lattice (thrml_lattice): stripes, halo refresh, sweep driver.

`LatticeStripe` wraps one stripe handle.  `StripedLattice` drives several stripes inside one process (device-to-device
halo copies; used to test that striping is invisible); `DistributedStripe` is one stripe per process, swept by the
library's own driver (thrml_lattice_run_blocks: NCCL point-to-point halo rows between ring neighbours).  Key handling
mirrors run_blocks / sample_blocks (crates/thrml-samplers/src/sampling.rs:28-106): keys = key.split(n_iters), then per
sweep key.split(2) gives the two colours' block keys.
"""
import ctypes as C

import numpy as np

from . import engine as _eng
from ._ffi import check, lib, ptr


NOISE_PROGRAM = 0  # the explicit program's key -> noise mapping: states equal IsingSamplingProgram's on the same torus
NOISE_PACKED = 1   # the lattice engine's own mapping (default): two generator calls give the top bytes of 32 spins as bit planes
NOISE_PACKED_TABLE = 2  # the same mapping, thresholds looked up spin by spin (the route for thresholds the bit-sliced compare cannot take)


class LatticeStripe:
    def __init__(self, height, width, row_begin, n_rows, coupling, bias, beta, n_chains, chain_offset=0, ctx=None, noise=NOISE_PACKED):
        self.ctx = ctx or _eng.default_context()
        self.height, self.width, self.row_begin, self.n_rows, self.n_chains = height, width, row_begin, n_rows, n_chains
        self.h = C.c_void_p()
        check(lib().thrml_lattice_create(self.ctx.h, C.c_int64(height), C.c_int64(width), C.c_int64(row_begin), C.c_int64(n_rows), C.c_float(coupling),
                                         C.c_float(bias), C.c_float(beta), C.c_int64(n_chains), C.c_int64(chain_offset), C.byref(self.h)))
        check(lib().thrml_lattice_set_noise(self.h, C.c_int32(noise)))

    def __del__(self):
        h, self.h = getattr(self, "h", None), None
        if h and lib is not None:  # module globals are already cleared when the interpreter is shutting down
            lib().thrml_lattice_destroy(h)

    def randomize(self, key):
        check(lib().thrml_lattice_randomize(self.h, C.c_uint64(int(key))))

    def upload(self, spins):
        """spins: uint8 [chain][stripe row][column] of 0/1."""
        a = np.ascontiguousarray(spins, dtype=np.uint8).reshape(self.n_chains, self.n_rows, self.width)
        check(lib().thrml_lattice_upload(self.h, ptr(a)))

    def download(self):
        out = np.zeros((self.n_chains, self.n_rows, self.width), dtype=np.uint8)
        check(lib().thrml_lattice_download(self.h, ptr(out)))
        return out

    def upload_bits(self, bits):
        """bits: uint32 [chain][stripe row][width / 32], bit k of word v = column 32 v + k."""
        a = np.ascontiguousarray(bits, dtype=np.uint32).reshape(self.n_chains, self.n_rows, self.width // 32)
        check(lib().thrml_lattice_upload_bits(self.h, ptr(a)))

    def download_bits(self):
        out = np.zeros((self.n_chains, self.n_rows, self.width // 32), dtype=np.uint32)
        check(lib().thrml_lattice_download_bits(self.h, ptr(out)))
        return out

    def update(self, colour, block_key, row_begin=0, row_end=None):
        check(lib().thrml_lattice_update(self.h, C.c_int32(colour), C.c_uint64(int(block_key)), C.c_int64(row_begin), C.c_int64(self.n_rows if row_end is None else row_end)))

    def wrap_halo(self, colour):
        check(lib().thrml_lattice_wrap_halo(self.h, C.c_int32(colour)))

    def copy_halo_from(self, which_dst, src, which_src, colour):
        check(lib().thrml_lattice_copy_halo(self.h, C.c_int32(which_dst), src.h, C.c_int32(which_src), C.c_int32(colour)))

    def halo_info(self, colour):
        p = [C.c_void_p() for _ in range(4)]
        n = C.c_int64()
        check(lib().thrml_lattice_halo_info(self.h, C.c_int32(colour), C.byref(p[0]), C.byref(p[1]), C.byref(p[2]), C.byref(p[3]), C.byref(n)))
        return dict(send_top=p[0].value, send_bottom=p[1].value, recv_top=p[2].value, recv_bottom=p[3].value, row_bytes=n.value)

    def observe(self):
        """(sum of spins, sum of bond products) per chain over this stripe, int64 [2][chains]."""
        out = np.zeros((2, self.n_chains), dtype=np.int64)
        check(lib().thrml_lattice_observe(self.h, ptr(out)))
        return out

    def synchronize(self):
        check(lib().thrml_lattice_synchronize(self.h))


def stripe_rows(height, n_stripes):
    """Row ranges of `n_stripes` equal stripes (height must divide evenly into stripes of at least two rows)."""
    if height % n_stripes or height // n_stripes < 2:
        raise ValueError("height must split into equal stripes of at least two rows")
    per = height // n_stripes
    return [(i * per, per) for i in range(n_stripes)]


class StripedLattice:
    """All stripes of a lattice inside one process (one stripe = the whole lattice, or several on one device)."""

    def __init__(self, height, width, coupling, bias, beta, n_chains, n_stripes=1, ctx=None, noise=NOISE_PACKED):
        self.height, self.width, self.n_chains = height, width, n_chains
        self.stripes = [LatticeStripe(height, width, r0, n, coupling, bias, beta, n_chains, 0, ctx, noise) for r0, n in stripe_rows(height, n_stripes)]

    def refresh_halos(self, colour):
        n = len(self.stripes)
        if n == 1:
            self.stripes[0].wrap_halo(colour)
            return
        for i, s in enumerate(self.stripes):
            s.copy_halo_from(0, self.stripes[(i - 1) % n], 1, colour)  # halo above <- last row of the stripe above
            s.copy_halo_from(1, self.stripes[(i + 1) % n], 0, colour)  # halo below <- first row of the stripe below

    def upload(self, spins):
        spins = np.asarray(spins, dtype=np.uint8).reshape(self.n_chains, self.height, self.width)
        for s in self.stripes:
            s.upload(spins[:, s.row_begin:s.row_begin + s.n_rows, :])
        self.refresh_halos(0)
        self.refresh_halos(1)

    def randomize(self, key):
        for s in self.stripes:
            s.randomize(key)
        self.refresh_halos(0)
        self.refresh_halos(1)

    def download(self):
        return np.concatenate([s.download() for s in self.stripes], axis=1)

    def sample_blocks(self, key):
        k = _eng.rng_split(key, 2)
        for colour in (0, 1):
            for s in self.stripes:
                s.update(colour, int(k[colour]))
            self.refresh_halos(colour)

    def run_blocks(self, key, n_iters):
        if n_iters <= 0:
            return
        for k in _eng.rng_split(key, n_iters):
            self.sample_blocks(int(k))

    def observe(self):
        return sum(s.observe() for s in self.stripes)

    def synchronize(self):
        for s in self.stripes:
            s.synchronize()


class DistributedStripe:
    """One stripe per process (rank r of `comm` holds rows [r H / world, (r + 1) H / world)).  Everything that runs per
    sweep — the colour updates, the boundary-rows-first halo exchange over NCCL, the observable series — is the
    library's thrml_lattice_run_blocks; this class only holds the handles.  `comm` = None for a single process holding
    the whole lattice."""

    def __init__(self, height, width, coupling, bias, beta, n_chains, comm=None, ctx=None, noise=NOISE_PACKED):
        self.comm = comm
        self.rank = comm.rank if comm is not None else 0
        self.world = comm.world_size if comm is not None else 1
        r0, n = stripe_rows(height, self.world)[self.rank]
        self.stripe = LatticeStripe(height, width, r0, n, coupling, bias, beta, n_chains, 0, ctx, noise)
        self.n_chains = n_chains

    def _comm(self):
        return self.comm.h if self.comm is not None else None

    def refresh_halos(self):
        check(lib().thrml_lattice_refresh_halos(self.stripe.h, self._comm()))

    def randomize(self, key):
        self.stripe.randomize(key)
        self.refresh_halos()

    def upload(self, spins):
        """spins: uint8 [chain][row][column] of the WHOLE lattice; this rank keeps its rows."""
        s = self.stripe
        s.upload(np.asarray(spins, dtype=np.uint8)[:, s.row_begin:s.row_begin + s.n_rows, :])
        self.refresh_halos()

    def upload_bits(self, bits):
        """bits: uint32 [chain][row][width / 32] of THIS rank's rows."""
        self.stripe.upload_bits(bits)
        self.refresh_halos()

    def run_blocks(self, key, n_iters, record=False):
        check(lib().thrml_lattice_run_blocks(self.stripe.h, C.c_uint64(int(key)), C.c_int64(n_iters), self._comm(), C.c_int32(int(record))))

    def sample_blocks(self, key):
        """One sweep with the sweep key itself (run_blocks over one iteration would split it once more)."""
        k = _eng.rng_split(key, 2)
        n = self.stripe.n_rows
        if self.world == 1:
            for colour in (0, 1):
                self.stripe.update(colour, int(k[colour]))
                self.stripe.wrap_halo(colour)
            return
        raise NotImplementedError("multi-rank stripes sweep through run_blocks")

    def series(self):
        """Whole-lattice (sum of spins, sum of bond products) per recorded sweep and chain: int64 [records][2][chains]."""
        n = C.c_int64()
        check(lib().thrml_lattice_read_series(self.stripe.h, self._comm(), None, C.c_int64(0), C.byref(n)))
        out = np.zeros((n.value, 2, self.n_chains), dtype=np.int64)
        if n.value:
            check(lib().thrml_lattice_read_series(self.stripe.h, self._comm(), ptr(out), C.c_int64(n.value), C.byref(n)))
        return out

    def moments(self):
        """(<m>, <m^2>, <e>, <e^2>) per chain over the recorded sweeps, float64 [4][chains], and the record count."""
        out = np.zeros((4, self.n_chains), dtype=np.float64)
        n = C.c_int64()
        check(lib().thrml_lattice_moments(self.stripe.h, self._comm(), ptr(out), C.byref(n)))
        return out, n.value

    def series_reset(self):
        check(lib().thrml_lattice_series_reset(self.stripe.h))

    def observe_local(self):
        return self.stripe.observe()

    def download_local(self):
        return self.stripe.download()

    def synchronize(self):
        self.stripe.synchronize()
