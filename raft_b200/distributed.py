"""Row-sharded reductions over the GPUs of one node: one process per GPU, torch.distributed (NCCL).

The reference has no multi-GPU form of these primitives. Rows shard contiguously:
  * outputs per row (row norms, row argmin) are disjoint slices - no communication;
  * outputs per column and per key are reduced locally WITHOUT final_op, all-reduced
    (sum / min / max) and finished with final_op on every rank. The collective is the one the
    reference wraps as comms_t::allreduce (cpp/include/raft/comms/detail/std_comms.hpp:366-375).
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


def _active(group):
    return dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


def combine_partials(partial, reduce_op="add", group=None):
    """All-reduces a per-rank partial vector / table in place (any device torch.distributed
    supports for the group's backend) and returns it."""
    if reduce_op not in _RED:
        raise ValueError("only add / min / max partials can be combined across ranks")
    if _active(group):
        dist.all_reduce(partial, op=_RED[reduce_op], group=group)
    return partial


def combine_partials_grouped(partials, reduce_op="add", group=None):
    """All-reduces several per-rank partials of possibly different dtypes (a table of sums and a
    vector of int64 counts) as ONE grouped collective - one launch instead of one per tensor, the
    ncclGroupStart / ncclGroupEnd pairing of a single-process caller. Backends without grouping
    (gloo) get one call per tensor. Returns the list."""
    if reduce_op not in _RED:
        raise ValueError("only add / min / max partials can be combined across ranks")
    partials = [p for p in partials if p is not None]
    if not _active(group) or not partials:
        return partials
    manager = getattr(dist, "_coalescing_manager", None)
    if manager is not None and partials[0].is_cuda and len(partials) > 1:
        with manager(group=group, device=partials[0].device, async_ops=False):
            for p in partials:
                dist.all_reduce(p, op=_RED[reduce_op], group=group)
    else:
        for p in partials:
            dist.all_reduce(p, op=_RED[reduce_op], group=group)
    return partials


def _init_for_rank(init, reduce_op, group):
    """A sum's start value enters the total once: rank 0 keeps it, the others start from zero
    (min / max start values are idempotent and stay)."""
    if reduce_op == "add" and _active(group) and dist.get_rank(group) != 0:
        return 0.0
    return init


def reduce_columns(shard, total_rows, init=0.0, main_op="identity", reduce_op="add", final_op="identity",
                   final_scalar=1.0, group=None, out=None, workspace=None):
    """Column reduction of a row-sharded row-major matrix; every rank gets the full result.
    `total_rows` is the row count of the whole matrix (what a mean divides by is the caller's
    final_scalar; it is accepted here so call sites read like the single-GPU call). `out` and
    `workspace` (see linalg.reduce_workspace_bytes) make the call allocation-free."""
    del total_rows
    part = linalg.reduce(shard, linalg.ALONG_COLUMNS, out, init=_init_for_rank(init, reduce_op, group),
                         main_op=main_op, reduce_op=reduce_op, workspace=workspace)
    combine_partials(part, reduce_op, group)
    linalg.apply_final(part, final_op, final_scalar)
    return part


def reduce_rows(shard, **kw):
    """Row-wise reduction of this rank's rows: the result is this rank's slice of the output."""
    return linalg.reduce(shard, linalg.ALONG_ROWS, **kw)


def reduce_rows_by_key(shard, keys_shard, n_unique_keys, weights_shard=None, with_counts=True, group=None,
                       sums=None, counts=None, workspace=None):
    """Keyed row sums of a row-sharded matrix (keys and weights sharded with the rows): local
    tables, then ONE grouped all-reduce of the sums and the int64 counts. `sums`, `counts` and
    `workspace` (see linalg.reduce_rows_by_key_workspace_bytes) make the call allocation-free."""
    if counts is None and with_counts:
        counts = torch.zeros(n_unique_keys, dtype=torch.int64, device=shard.device)
    sums = linalg.reduce_rows_by_key(shard, keys_shard, n_unique_keys, d_sums=sums, d_weights=weights_shard,
                                     counts=counts, workspace=workspace)
    combine_partials_grouped([sums, counts], "add", group)
    return sums, counts
