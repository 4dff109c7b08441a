"""Row-sharded reductions over the GPUs of one node: one process per GPU, torch.distributed (NCCL).

The reference has no multi-GPU form of these primitives. Rows shard contiguously:
  * outputs per row (row norms, row argmin) are disjoint slices - no communication;
  * outputs per column and per key are reduced locally WITHOUT final_op, all-reduced
    (sum / min / max) and finished with final_op on every rank.
"""
import torch
import torch.distributed as dist

from . import linalg

_RED = {"add": dist.ReduceOp.SUM, "min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX}


def shard_rows(n_rows, rank, world):
    """Contiguous block [r0, r1) of rank `rank`: sizes differ by at most one row and the blocks
    tile [0, n_rows) in rank order."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank / world size")
    base, extra = divmod(n_rows, world)
    r0 = rank * base + min(rank, extra)
    return r0, r0 + base + (1 if rank < extra else 0)


def combine_partials(partial, reduce_op="add", group=None):
    """All-reduces a per-rank partial vector / table in place (any device torch.distributed
    supports for the group's backend) and returns it."""
    if reduce_op not in _RED:
        raise ValueError("only add / min / max partials can be combined across ranks")
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=_RED[reduce_op], group=group)
    return partial


def reduce_columns(shard, total_rows, init=0.0, main_op="identity", reduce_op="add", final_op="identity",
                   final_scalar=1.0, group=None):
    """Column reduction of a row-sharded row-major matrix; every rank gets the full result.
    `total_rows` is the row count of the whole matrix (what a mean divides by is the caller's
    final_scalar; it is accepted here so call sites read like the single-GPU call)."""
    del total_rows
    part = linalg.reduce(shard, linalg.ALONG_COLUMNS, init=init, main_op=main_op, reduce_op=reduce_op)
    combine_partials(part, reduce_op, group)
    linalg.apply_final(part, final_op, final_scalar)
    return part


def reduce_rows(shard, **kw):
    """Row-wise reduction of this rank's rows: the result is this rank's slice of the output."""
    return linalg.reduce(shard, linalg.ALONG_ROWS, **kw)


def reduce_rows_by_key(shard, keys_shard, n_unique_keys, weights_shard=None, with_counts=True, group=None):
    """Keyed row sums of a row-sharded matrix (keys and weights sharded with the rows): local
    tables, then one all-reduce for the sums and one for the int64 counts."""
    counts = torch.zeros(n_unique_keys, dtype=torch.int64, device=shard.device) if with_counts else None
    sums = linalg.reduce_rows_by_key(shard, keys_shard, n_unique_keys, d_weights=weights_shard, counts=counts)
    combine_partials(sums, "add", group)
    if counts is not None:
        combine_partials(counts, "add", group)
    return sums, counts
