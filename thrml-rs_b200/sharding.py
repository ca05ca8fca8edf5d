"""Chain sharding for multi-GPU runs: one process per GPU, chains split evenly, program replicated, the in-kernel
random stream keyed by the global chain id, one allreduce(sum) of the moment accumulators at read-out."""


def shard_chains(total_chains, rank, world_size, align=16):
    """(local chain count, global id of local chain 0).  Shard starts are multiples of `align` (the state layout works
    in 16-chain words): the 16-chain units are dealt out evenly, the first ranks take one more when they do not divide,
    and the last rank also takes the chains beyond the last whole unit.  Fewer than one unit per rank is an error on
    every rank alike."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError("rank out of range")
    if total_chains < align * world_size:
        # every rank raises the same error before any collective: a rank left without chains could not create a state
        # and would leave the others waiting in the allreduce
        raise ValueError(f"{total_chains} chains cannot be sharded over {world_size} ranks in units of {align}: use at most {max(total_chains // align, 1)} ranks")
    units = total_chains // align  # whole units; the remainder rides with the last rank
    base, extra = divmod(units, world_size)
    start = align * (rank * base + min(rank, extra))
    stop = total_chains if rank == world_size - 1 else start + align * (base + (1 if rank < extra else 0))
    return stop - start, start


def allreduce_sums(tensor, dist):
    """The single collective of the chain-parallel path: sum the int64 moment accumulators over ranks, in place."""
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM)
    return tensor
