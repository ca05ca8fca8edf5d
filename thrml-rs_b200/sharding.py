"""Chain sharding for multi-GPU runs: one process per GPU, chains split evenly, program replicated, the in-kernel
random stream keyed by the global chain id, one allreduce(sum) of the moment accumulators at read-out."""


def shard_chains(total_chains, rank, world_size, align=16):
    """(local chain count, global id of local chain 0).  Shard starts are multiples of `align` (the state layout works
    in 16-chain words), the last rank takes the remainder."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError("rank out of range")
    per = -(-total_chains // world_size)
    per = -(-per // align) * align
    start = min(rank * per, total_chains)
    stop = min(start + per, total_chains)
    return stop - start, start


def allreduce_sums(tensor, dist):
    """The single collective of the chain-parallel path: sum the int64 moment accumulators over ranks, in place."""
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM)
    return tensor
