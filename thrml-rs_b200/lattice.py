"""Implicit bit-packed Ising lattice (thrml_lattice): stripes, halo refresh, sweep driver.

`LatticeStripe` wraps one stripe handle.  `StripedLattice` drives the stripes of one process (a whole lattice, or several
stripes on one device); `run_distributed_sweeps` drives one stripe per process with the halo rows exchanged point to
point over torch.distributed (NCCL over NVLink on a multi-GPU box, gloo on CPU tensors is not applicable: stripes live on
GPUs).  Key handling mirrors run_blocks / sample_blocks (crates/thrml-samplers/src/sampling.rs:28-106): keys =
key.split(n_iters), then per sweep key.split(2) gives the two colours' block keys.
"""
import ctypes as C

import numpy as np

from . import engine as _eng
from ._ffi import check, lib, ptr


class LatticeStripe:
    def __init__(self, height, width, row_begin, n_rows, coupling, bias, beta, n_chains, chain_offset=0, ctx=None):
        self.ctx = ctx or _eng.default_context()
        self.height, self.width, self.row_begin, self.n_rows, self.n_chains = height, width, row_begin, n_rows, n_chains
        self.h = C.c_void_p()
        check(lib().thrml_lattice_create(self.ctx.h, C.c_int64(height), C.c_int64(width), C.c_int64(row_begin), C.c_int64(n_rows), C.c_float(coupling),
                                         C.c_float(bias), C.c_float(beta), C.c_int64(n_chains), C.c_int64(chain_offset), C.byref(self.h)))

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

    def __init__(self, height, width, coupling, bias, beta, n_chains, n_stripes=1, ctx=None):
        self.height, self.width, self.n_chains = height, width, n_chains
        self.stripes = [LatticeStripe(height, width, r0, n, coupling, bias, beta, n_chains, 0, ctx) for r0, n in stripe_rows(height, n_stripes)]

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


def _as_tensor(torch, addr, nbytes):
    class _View:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (addr, False), "version": 3}

    return torch.as_tensor(_View(), device="cuda")


class DistributedStripe:
    """One stripe per process; halo rows travel with torch.distributed point-to-point operations (ring of stripes)."""

    def __init__(self, height, width, coupling, bias, beta, n_chains, torch, dist, ctx=None):
        self.torch, self.dist = torch, dist
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        r0, n = stripe_rows(height, self.world)[self.rank]
        self.stripe = LatticeStripe(height, width, r0, n, coupling, bias, beta, n_chains, 0, ctx)
        self.stream = torch.cuda.ExternalStream(self.stripe.ctx.stream)
        self.side = torch.cuda.Stream()
        self.views = []
        for colour in (0, 1):
            info = self.stripe.halo_info(colour)
            self.views.append({k: _as_tensor(torch, info[k], info["row_bytes"]) for k in ("send_top", "send_bottom", "recv_top", "recv_bottom")})

    def refresh_halos(self, colour):
        v, dist = self.views[colour], self.dist
        up, down = (self.rank - 1) % self.world, (self.rank + 1) % self.world
        with self.torch.cuda.stream(self.stream):
            if self.world == 1:
                self.stripe.wrap_halo(colour)
                return
            # My first row goes up and lands in the upper stripe's lower halo; my last row goes down into the lower
            # stripe's upper halo.  With two stripes both neighbours are the same process and point-to-point messages
            # between one pair match in issue order, so the receives are listed in the order the peer sends:
            # its first row (my lower halo) before its last row (my upper halo).
            ops = [dist.P2POp(dist.isend, v["send_top"], up), dist.P2POp(dist.isend, v["send_bottom"], down),
                   dist.P2POp(dist.irecv, v["recv_bottom"], down), dist.P2POp(dist.irecv, v["recv_top"], up)]
            for req in dist.batch_isend_irecv(ops):
                req.wait()

    def randomize(self, key):
        self.stripe.randomize(key)
        self.refresh_halos(0)
        self.refresh_halos(1)

    def sample_blocks(self, key):
        """One sweep.  Per colour the two boundary rows are updated first and sent while the interior rows are still
        being updated: the exchange runs on a side stream and the next colour waits for it."""
        k = _eng.rng_split(key, 2)
        n = self.stripe.n_rows
        torch = self.torch
        for colour in (0, 1):
            if self.world == 1 or n < 4:
                self.stripe.update(colour, int(k[colour]))
                self.refresh_halos(colour)
                continue
            self.stripe.update(colour, int(k[colour]), 0, 1)
            self.stripe.update(colour, int(k[colour]), n - 1, n)
            self.side.wait_stream(self.stream)             # boundary rows are final
            self._exchange(colour, self.side)
            self.stripe.update(colour, int(k[colour]), 1, n - 1)
            self.stream.wait_stream(self.side)             # halos of this colour are in place before the other colour reads them

    def _exchange(self, colour, stream):
        v, dist = self.views[colour], self.dist
        up, down = (self.rank - 1) % self.world, (self.rank + 1) % self.world
        with self.torch.cuda.stream(stream):
            ops = [dist.P2POp(dist.isend, v["send_top"], up), dist.P2POp(dist.isend, v["send_bottom"], down),
                   dist.P2POp(dist.irecv, v["recv_bottom"], down), dist.P2POp(dist.irecv, v["recv_top"], up)]
            for req in dist.batch_isend_irecv(ops):
                req.wait()

    def run_blocks(self, key, n_iters):
        for k in _eng.rng_split(key, n_iters) if n_iters > 0 else []:
            self.sample_blocks(int(k))

    def observe(self):
        """Whole-lattice sums: the stripes' sums added with one small allreduce."""
        self.stream.synchronize()
        local = self.torch.from_numpy(self.stripe.observe()).cuda()
        if self.world > 1:
            self.dist.all_reduce(local)
        return local.cpu().numpy()


def distributed_self_check(torch, dist, ctx=None, height=64, width=128, chains=16, sweeps=3):
    """Small lattice sampled once as stripes over all ranks and once whole on every rank: the observables must agree
    exactly (the states are a function of the keys alone, however the rows are sharded)."""
    whole = StripedLattice(height, width, 0.4407, 0.05, 1.0, chains, 1, ctx)
    whole.randomize(3)
    whole.run_blocks(4, sweeps)
    want = whole.observe()
    part = DistributedStripe(height, width, 0.4407, 0.05, 1.0, chains, torch, dist, ctx)
    part.randomize(3)
    part.run_blocks(4, sweeps)
    got = part.observe()
    return bool(np.array_equal(got, want))
