"""Host-side plan of the data-parallel step (no device code): how the batch is sharded and which contiguous gradient
ranges are all-reduced in which order.  Used by the trainer (GPU, NCCL) and by the CPU/gloo tests of the N > 1 logic.

The path shards by batch rows only: rank r owns rows [r*B/W, (r+1)*B/W) of the global batch and full replicas of all
parameters.  Every rank's loss is the mean over ITS rows, so the full-batch gradient is the SUM of the per-rank
gradients times 1/W; the sum is the all-reduce, the 1/W lives in the fused optimizer (`grad_scale`)."""
from __future__ import annotations


def shard_rows(global_batch: int, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) rows of the global batch owned by `rank`; the batch must divide evenly (weak scaling keeps the
    per-rank batch fixed, so it always does)."""
    if global_batch % world:
        raise ValueError(f"global batch {global_batch} is not divisible by world size {world}")
    per = global_batch // world
    return rank * per, (rank + 1) * per


def shard_epoch_order(order, rank: int, world: int):
    """The samples of one epoch that `rank` trains on: every rank draws the SAME permutation `order` (same seed) and
    takes the positions rank, rank + world, ... of it, after trimming the tail so that all ranks get equally many
    samples (a data-parallel step needs every rank to have a batch).  Together the shards cover each kept sample once."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a world of {world}")
    keep = (len(order) // world) * world
    return order[:keep][rank::world]


def layer_buckets_packed(sizes) -> list[tuple[int, int]]:
    """(offset, count) of [dW_l, db_l] for every layer in the PACKED parameter order
    [W_0 {in,out}, b_0, W_1, b_1, ...] (Module::named_parameters order)."""
    out, off = [], 0
    for a, b in zip(sizes[:-1], sizes[1:]):
        n = a * b + b
        out.append((off, n))
        off += n
    return out


def reduce_order(n_layers: int) -> list[int]:
    """Buckets are reduced head first: layer L-1's gradients are final first, so its all-reduce overlaps the
    backward of layers L-2 ... 0."""
    return list(range(n_layers - 1, -1, -1))


def allreduce_gradients(flat_grads, sizes, group=None) -> None:
    """Sum the per-layer buckets of a flat packed gradient tensor across ranks, in backward order (in place)."""
    import torch.distributed as dist

    buckets = layer_buckets_packed(sizes)
    for layer in reduce_order(len(buckets)):
        off, n = buckets[layer]
        dist.all_reduce(flat_grads[off:off + n], op=dist.ReduceOp.SUM, group=group)


COMM_OK, COMM_FAILED = 0, 8  # 8 = ODL_ERR_COMM of the C ABI


def guarded(collective, *args, **kwargs) -> tuple[int, str]:
    """Run a collective step and turn what a broken process group raises -- a peer that left, a time-out of the
    group's own watchdog, a transport error -- into (status, message) instead of an exception from deep inside the
    step, so that a training loop can stop cleanly, checkpoint and rebuild the group.  The process group's `timeout=`
    bounds the wait; nothing here waits on its own."""
    try:
        collective(*args, **kwargs)
        return COMM_OK, ""
    except Exception as e:  # torch raises RuntimeError / DistBackendError / DistNetworkError depending on the backend
        return COMM_FAILED, f"{type(e).__name__}: {e}"
