"""Two ranks on two GPUs (skipped on a single-GPU machine), everything multi-GPU going through the library's own
communicator (thrml_comm over NCCL): chain-sharded moment sums combined by thrml_moments_allreduce equal the
single-device sums (int32 and int64 transport), Potts marginals likewise, and a lattice split into two stripes whose
halo rows travel inside thrml_lattice_run_blocks equals the whole lattice, state and observable series; the CD-1 step with
its chains sharded (thrml_cd1_step_comm) returns the correlation matrices of the unsharded step."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LATTICES = [(64, 128, 16, 5), (4, 64, 8, 3), (8, 192, 4, 4)]  # (H, W, chains, sweeps): overlapped exchange, two-row stripes, four-row stripes


def _rbm_case(T, ctx=None):
    """64 visible x 96 hidden spins with bf16-valued couplings, 256 chains: a program on the dense path and its data."""
    rng = np.random.default_rng(12)
    nv, nh, chains = 64, 96, 256
    W = (np.round(rng.normal(0, 0.3, (nv, nh)) * 64) / 64).astype(np.float32)
    b = rng.normal(0, 0.2, nv + nh).astype(np.float32)
    vis, hid = np.arange(nv), np.arange(nv, nv + nh)
    edges = np.stack([np.repeat(vis, nh), np.tile(hid, nv)], 1)
    bld = T.Builder(np.zeros(nv + nh, np.int32))
    bld.add_free_block(vis, superblock=0)
    bld.add_free_block(hid, superblock=1)
    bld.add_ising(np.arange(nv + nh), b, edges, W.ravel(), 1.0)
    bld.compile()
    prog = T.Program(bld, ctx) if ctx is not None else T.Program(bld)
    assert prog.enable_dense(False) == 2
    v0 = (rng.random((chains, nv)) < 0.3).astype(np.uint8)
    return prog, v0, chains


def _potts_inputs():
    rng = np.random.default_rng(8)
    K = 4
    return K, rng.normal(0, 0.4, (3, K, K)).astype(np.float32), rng.normal(0, 0.2, (4 * 4 * 6, K)).astype(np.float32)


def _worker(rank, world, port, out_dir):
    os.environ.update(LOCAL_RANK=str(rank), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as graft
    T = graft.load_package()
    from thrml_rs_b200 import lattice, potts, sharding
    import models as M
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)  # only carries the communicator id
    ctx = T.default_context(rank)
    comm = T.Comm.from_torch(dist, ctx)
    info = comm.info()
    assert info["rank"] == rank and info["world_size"] == world and info["nccl_version"] > 20000
    out = {}
    # chain-sharded moments: few observations (int32 transport) and a forged observation count beyond 2^31 (int64 transport)
    desc, ginfo = M.ising_random_graph(T, 200, 8, 9)
    prog = T.Program(M.fill(T.Builder(desc["kinds"]), desc), ctx)
    total = 96
    n_local, start = sharding.shard_chains(total, rank, world)
    init = M.random_states(desc, total, 4)
    spec = [[(i,) for i in range(ginfo["n"])], [tuple(e) for e in ginfo["edges"]]]
    for tag, forged in (("i32", 0), ("i64", 1 << 31)):
        st = T.ChainState(prog, n_local, start)
        for i, a in enumerate(init):
            st.upload(i, a[start:start + n_local])
        mom = T.Moments(prog, spec, True)
        st.sample_with_observation(5, 2, 6, 1, moments=mom)
        if forged:
            from thrml_rs_b200._ffi import check
            check(T.lib().thrml_moments_add_observations(mom.h, forged))
        mom.allreduce(comm)
        s0, n_obs = mom.read(0)
        out[f"sums_{tag}"] = np.concatenate([s0, mom.read(1)[0]])
        out[f"n_obs_{tag}"] = np.array([n_obs])
    # Potts marginals, chains sharded
    K, tables, unary = _potts_inputs()
    pl = potts.PottsLattice(4, 4, 6, K, tables, unary, 1.0, n_local, start, ctx)
    pl.randomize(6)
    pl.sample_with_marginals(12, 1, 3, 1)
    pl.allreduce_marginals(comm)
    counts, n_obs = pl.read_marginals()
    out["potts_counts"], out["potts_n_obs"] = counts, np.array([n_obs])
    # CD-1 with the chains sharded: 128 of the 256 chains per rank
    rprog, v0, rchains = _rbm_case(T, ctx)
    half = rchains // world
    data, chain = T.ChainState(rprog, half, rank * half), T.ChainState(rprog, half, rank * half)
    data.upload(0, v0[rank * half:(rank + 1) * half])
    pos, neg = chain.cd1_step(0, 1, None, 99, data=data, comm=comm)
    out["cd1_pos"], out["cd1_neg"] = pos, neg
    # striped lattices
    for li, (H, W, chains, sweeps) in enumerate(LATTICES):
        spins = np.random.default_rng(H * W).integers(0, 2, (chains, H, W)).astype(np.uint8)
        part = lattice.DistributedStripe(H, W, 0.4407, 0.03, 1.0, chains, comm, ctx)
        part.upload(spins)
        part.run_blocks(4, sweeps, record=True)
        out[f"lat{li}_rows_{rank}"] = part.download_local()
        series = part.series()
        mom, n_rec = part.moments()
        if rank == 0:
            out[f"lat{li}_series"], out[f"lat{li}_moments"] = series, mom
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **out)
    comm.close()
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpus_through_the_library_communicator(T, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    import models as M
    from thrml_rs_b200 import lattice, potts
    port = 29600 + (os.getpid() % 1000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    desc, info = M.ising_random_graph(T, 200, 8, 9)
    prog = T.Program(M.fill(T.Builder(desc["kinds"]), desc))
    st = T.ChainState(prog, 96)
    for i, a in enumerate(M.random_states(desc, 96, 4)):
        st.upload(i, a)
    spec = [[(i,) for i in range(info["n"])], [tuple(e) for e in info["edges"]]]
    mom = T.Moments(prog, spec, True)
    st.sample_with_observation(5, 2, 6, 1, moments=mom)
    want = np.concatenate([mom.read(0)[0], mom.read(1)[0]])
    for r in (r0, r1):  # the result lands on every rank
        assert np.array_equal(r["sums_i32"], want) and r["n_obs_i32"][0] == 6 * 96
        assert np.array_equal(r["sums_i64"], want) and r["n_obs_i64"][0] == 6 * 96 + 2 * (1 << 31)
    K, tables, unary = _potts_inputs()
    pl = potts.PottsLattice(4, 4, 6, K, tables, unary, 1.0, 96)
    pl.randomize(6)
    pl.sample_with_marginals(12, 1, 3, 1)
    counts, n_obs = pl.read_marginals()
    for r in (r0, r1):
        assert np.array_equal(r["potts_counts"], counts) and r["potts_n_obs"][0] == n_obs == 3 * 96
    rprog, v0, rchains = _rbm_case(T)
    data, chain = T.ChainState(rprog, rchains), T.ChainState(rprog, rchains)
    data.upload(0, v0)
    pos, neg = chain.cd1_step(0, 1, None, 99, data=data)
    for r in (r0, r1):  # 128 chains per rank: a power of two, so the sharded means are the unsharded ones bit for bit
        assert np.array_equal(r["cd1_pos"], pos) and np.array_equal(r["cd1_neg"], neg)
    for li, (H, W, chains, sweeps) in enumerate(LATTICES):
        spins = np.random.default_rng(H * W).integers(0, 2, (chains, H, W)).astype(np.uint8)
        whole = lattice.DistributedStripe(H, W, 0.4407, 0.03, 1.0, chains, None)
        whole.upload(spins)
        whole.run_blocks(4, sweeps, record=True)
        got = np.concatenate([r0[f"lat{li}_rows_0"], r1[f"lat{li}_rows_1"]], axis=1)
        assert np.array_equal(got, whole.download_local()), (H, W)
        assert np.array_equal(r0[f"lat{li}_series"], whole.series())
        assert np.allclose(r0[f"lat{li}_moments"], whole.moments()[0], rtol=1e-12, atol=1e-15)
