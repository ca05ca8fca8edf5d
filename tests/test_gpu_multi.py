"""Two ranks on two GPUs over NCCL (skipped on a single-GPU machine): chain-sharded moment sums combined with one
allreduce equal the single-device sums, and a lattice split into two stripes with NCCL halo rows equals the whole lattice."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    os.environ.update(LOCAL_RANK=str(rank), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as graft
    T = graft.load_package()
    from thrml_rs_b200 import lattice, sharding
    import models as M
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ctx = T.default_context(rank)
    # chain-sharded moments
    desc, info = M.ising_random_graph(T, 200, 8, 9)
    prog = T.Program(M.fill(T.Builder(desc["kinds"]), desc), ctx)
    total = 96
    n_local, start = sharding.shard_chains(total, rank, world)
    st = T.ChainState(prog, n_local, start)
    init = M.random_states(desc, total, 4)
    for i, a in enumerate(init):
        st.upload(i, a[start:start + n_local])
    spec = [[(i,) for i in range(info["n"])], [tuple(e) for e in info["edges"]]]
    mom = T.Moments(prog, spec, True)
    st.sample_with_observation(5, 2, 6, 1, moments=mom)
    ptr, cnt = mom.device_buffer()

    class _View:
        __cuda_array_interface__ = {"shape": (cnt,), "typestr": "<i8", "data": (ptr, False), "version": 3}

    t = torch.as_tensor(_View(), device="cuda")
    sharding.allreduce_sums(t, dist)
    torch.cuda.synchronize()
    sums = np.concatenate([mom.read(0)[0], mom.read(1)[0]])
    # striped lattice
    ok = lattice.distributed_self_check(torch, dist, ctx)
    if rank == 0:
        np.save(os.path.join(out_dir, "sums.npy"), sums)
        np.save(os.path.join(out_dir, "lattice_ok.npy"), np.array([ok]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpus_nccl(T, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    import models as M
    port = 29600 + (os.getpid() % 1000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    got = np.load(tmp_path / "sums.npy")
    assert bool(np.load(tmp_path / "lattice_ok.npy")[0])
    desc, info = M.ising_random_graph(T, 200, 8, 9)
    prog = T.Program(M.fill(T.Builder(desc["kinds"]), desc))
    st = T.ChainState(prog, 96)
    for i, a in enumerate(M.random_states(desc, 96, 4)):
        st.upload(i, a)
    spec = [[(i,) for i in range(info["n"])], [tuple(e) for e in info["edges"]]]
    mom = T.Moments(prog, spec, True)
    st.sample_with_observation(5, 2, 6, 1, moments=mom)
    want = np.concatenate([mom.read(0)[0], mom.read(1)[0]])
    assert np.array_equal(got, want)
