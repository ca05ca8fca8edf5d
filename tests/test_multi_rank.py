"""World-size-2 run of the chain-parallel path on CPU (gloo): each rank samples its shard of the chains with the
global chain ids the sharding helper assigns, the moment sums are combined by one allreduce, and the result equals a
single-rank run over all chains.  The per-rank sampler here is the oracle (no GPU in this test); the same property
is checked for the CUDA path on one device in test_gpu_parity.py::test_chain_sharding_is_invisible."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, total_chains, out_path):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as graft
    T = graft.load_package()
    from thrml_rs_b200 import sharding
    from oracle import oracle as O
    import models as M
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    # the product's communicator bootstrap: rank 0 draws the id inside the library (NCCL loaded at run time), the host
    # group broadcasts it, every rank ends up with the same 128 bytes (joining the communicator itself needs GPUs)
    box = [T.Comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    uid = box[0]
    assert isinstance(uid, bytes) and len(uid) == 128 and any(uid)
    ids = [None] * world
    dist.all_gather_object(ids, uid)
    assert all(i == uid for i in ids)
    from thrml_rs_b200 import lattice
    rows = lattice.stripe_rows(64, world)
    assert rows[rank] == (rank * 64 // world, 64 // world)
    desc, info = M.ising_random_graph(T, 80, 6, 9)
    om = M.fill(O.Model(desc["kinds"]), desc)
    n_local, start = sharding.shard_chains(total_chains, rank, world)
    init = M.random_states(desc, total_chains, 4)
    st = O.State(om, n_local, start)
    for i, a in enumerate(init):
        st.set_block(i, a[start:start + n_local].astype(np.float32))
    spec = [[(i,) for i in range(info["n"])], [tuple(e) for e in info["edges"]]]
    mom = O.Moments(om, spec, True)
    st.sample_with_observation(5, 2, 4, 1, moments=mom)
    sums = torch.from_numpy(np.concatenate([mom.read(0)[0], mom.read(1)[0]]))
    sharding.allreduce_sums(sums, dist)
    if rank == 0:
        np.save(out_path, sums.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_chain_sharding(T, O, tmp_path):
    import torch.multiprocessing as mp
    import models as M
    from thrml_rs_b200 import sharding
    total = 40
    assert [sharding.shard_chains(total, r, 2) for r in range(2)] == [(16, 0), (24, 16)]
    assert [sharding.shard_chains(4096 * 8, r, 8) for r in (0, 7)] == [(4096, 0), (4096, 4096 * 7)]
    assert [sharding.shard_chains(160, r, 8) for r in range(8)] == [(32, 0), (32, 32)] + [(16, 64 + 16 * i) for i in range(6)]
    # fewer than one 16-chain unit per rank: every rank raises before any collective, none is left with zero chains
    for r in range(8):
        with pytest.raises(ValueError, match="cannot be sharded"):
            sharding.shard_chains(96, r, 8)
    with pytest.raises(ValueError, match="cannot be sharded"):
        sharding.shard_chains(10, 1, 2)
    out = str(tmp_path / "sums.npy")
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, total, out), nprocs=2, join=True)
    got = np.load(out)
    desc, info = M.ising_random_graph(T, 80, 6, 9)
    om = M.fill(O.Model(desc["kinds"]), desc)
    st = O.State(om, total, 0)
    for i, a in enumerate(M.random_states(desc, total, 4)):
        st.set_block(i, a.astype(np.float32))
    spec = [[(i,) for i in range(info["n"])], [tuple(e) for e in info["edges"]]]
    mom = O.Moments(om, spec, True)
    st.sample_with_observation(5, 2, 4, 1, moments=mom)
    want = np.concatenate([mom.read(0)[0], mom.read(1)[0]])
    assert np.array_equal(got, want)
