"""Partitioning of the multi-GPU workloads.  Every fused pair runs on one GPU and nothing is
exchanged between GPUs on the data path, so "multi-GPU" means handing out independent units:

  * the pair sweep: pair i goes to rank i mod world (the reference's sweep enumerates (K1, K2)
    pairs and runs them one after another, scripts/profile_test_suite.py:13-47);
  * a batch-sharded operator pair: rank r gets images [r*n/world, (r+1)*n/world) (the remainder
    spread over the first ranks) and its own copy of the weights.

Results are combined on the host (gather of per-rank dicts, max of per-rank times).
"""


def assign_pairs(names, world, rank):
    """Names of the sweep entries rank `rank` of `world` measures, in sweep order."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank / world")
    return [n for i, n in enumerate(names) if i % world == rank]


def shard_batch(n, world, rank):
    """(first image, image count) of rank `rank`'s contiguous shard of a batch of n images."""
    if world < 1 or not 0 <= rank < world or n < 0:
        raise ValueError("bad rank / world / batch")
    base, extra = divmod(n, world)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


def merge_results(per_rank):
    """Union of the per-rank result dicts; a name reported by two ranks is a partitioning bug."""
    out = {}
    for d in per_rank:
        for k, v in d.items():
            if k in out:
                raise ValueError("pair %s measured on two ranks" % k)
            out[k] = v
    return out


def max_over_ranks(values):
    """Job time of a sharded workload: the slowest rank."""
    return max(values)
