"""Row-sharded reductions over the GPUs of one node: one process per GPU, torch.distributed (NCCL).

The reference has no multi-GPU form of these primitives. Rows shard contiguously:
  * outputs per row (row norms, row argmin) are disjoint slices - no communication;
  * outputs per column and per key are reduced locally WITHOUT final_op, all-reduced
    (sum / min / max) and finished with final_op on every rank. The collective is the one the
    reference wraps as comms_t::allreduce (cpp/include/raft/comms/detail/std_comms.hpp:366-375).
"""
import ctypes

import torch
import torch.distributed as dist

from . import _lib as L
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
    """All-reduces several per-rank partials. Tensors of one dtype go out as ONE grouped collective (one
    launch, the ncclGroupStart / ncclGroupEnd pairing of a single-process caller); NCCL groups through
    torch.distributed only take tensors of identical type, so a table of fp32 sums and a vector of int64
    counts are two calls, back to back on the communicator's stream. Returns the list."""
    if reduce_op not in _RED:
        raise ValueError("only add / min / max partials can be combined across ranks")
    partials = [p for p in partials if p is not None]
    if not _active(group) or not partials:
        return partials
    by_type = {}
    for p in partials:
        by_type.setdefault((p.dtype, p.device), []).append(p)
    manager = getattr(dist, "_coalescing_manager", None)
    for (_, device), same in by_type.items():
        if manager is not None and device.type == "cuda" and len(same) > 1:
            with manager(group=group, device=device, async_ops=False):
                for p in same:
                    dist.all_reduce(p, op=_RED[reduce_op], group=group)
        else:
            for p in same:
                dist.all_reduce(p, op=_RED[reduce_op], group=group)
    return partials


class PeerExchange:
    """Exchange areas for the one-kernel all-reduce over peer memory (b2r_peer_allreduce_sum): one area
    per rank, created on the rank's current CUDA device and opened by every other rank of `group`
    through CUDA IPC (the ranks must be processes of ONE node whose GPUs can reach one another).
    Construction is a collective set-up step (allocation, handle exchange); the all-reduce itself is one
    asynchronous launch on the current stream and allocates nothing. Every rank must make the same
    sequence of all_reduce_sum calls. `max_payload_bytes` bounds fp32 sums + int64 counts of one call."""

    def __init__(self, max_payload_bytes, group=None, wait_limit_ms=None):
        if not _active(group):
            raise RuntimeError("PeerExchange needs an initialised process group of at least two ranks")
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.lib = L.load()
        self.device = torch.device("cuda", torch.cuda.current_device())
        area = ctypes.c_void_p()
        L.check(self.lib.b2r_peer_area_create(self.world, self.rank, int(max_payload_bytes), ctypes.byref(area)),
                "b2r_peer_area_create")
        self.area = area
        handle = ctypes.create_string_buffer(64)
        L.check(self.lib.b2r_peer_area_ipc_handle(self.area, handle), "b2r_peer_area_ipc_handle")
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        for r, h in enumerate(handles):
            if r != self.rank:
                L.check(self.lib.b2r_peer_area_open(self.area, r, ctypes.create_string_buffer(h, 64)),
                        "b2r_peer_area_open")
        if wait_limit_ms is not None:
            L.check(self.lib.b2r_peer_area_set_wait_limit_ms(self.area, int(wait_limit_ms)),
                    "b2r_peer_area_set_wait_limit_ms")
        # nobody may push into an area that is not mapped everywhere yet
        dist.barrier(group=group, device_ids=[self.device.index])

    def all_reduce_sum(self, sums=None, counts=None, scale=1.0):
        """In place: `sums` (fp32, contiguous) and `counts` (int64, contiguous) become their sums over all
        ranks; the fp32 sums are multiplied by `scale` afterwards (the deferred final_op of a mean)."""
        for t, dt in ((sums, torch.float32), (counts, torch.int64)):
            if t is not None and (t.dtype != dt or not t.is_contiguous() or not t.is_cuda):
                raise ValueError("PeerExchange takes contiguous CUDA tensors: fp32 sums, int64 counts")
        with torch.cuda.device(self.device):
            st = self.lib.b2r_peer_allreduce_sum(
                self.area, sums.data_ptr() if sums is not None else None, sums.numel() if sums is not None else 0,
                counts.data_ptr() if counts is not None else None, counts.numel() if counts is not None else 0,
                float(scale), torch.cuda.current_stream(self.device).cuda_stream)
        L.check(st, "b2r_peer_allreduce_sum")

    def status(self, clear=True):
        """Synchronises the device and returns L.OK, or L.ERR_TIMEOUT if a wait of an earlier call ran out."""
        torch.cuda.synchronize(self.device)
        out = ctypes.c_int32(0)
        with torch.cuda.device(self.device):
            L.check(self.lib.b2r_peer_area_status(self.area, ctypes.byref(out), 1 if clear else 0),
                    "b2r_peer_area_status")
        return out.value

    def close(self):
        if self.area is not None:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group, device_ids=[self.device.index])  # no peer still pushes into this area
            with torch.cuda.device(self.device):
                self.lib.b2r_peer_area_destroy(self.area)
            self.area = None


def _init_for_rank(init, reduce_op, group):
    """A sum's start value enters the total once: rank 0 keeps it, the others start from zero
    (min / max start values are idempotent and stay)."""
    if reduce_op == "add" and _active(group) and dist.get_rank(group) != 0:
        return 0.0
    return init


def reduce_columns(shard, total_rows, init=0.0, main_op="identity", reduce_op="add", final_op="identity",
                   final_scalar=1.0, group=None, out=None, workspace=None, peer=None):
    """Column reduction of a row-sharded row-major matrix; every rank gets the full result.
    `total_rows` is the row count of the whole matrix (what a mean divides by is the caller's
    final_scalar; it is accepted here so call sites read like the single-GPU call). `out` and
    `workspace` (see linalg.reduce_workspace_bytes) make the call allocation-free. With `peer`
    (a PeerExchange) fp32 sums are combined, and a scaling final_op applied, by ONE kernel over peer
    memory instead of the library all-reduce and a final_op launch."""
    del total_rows
    part = linalg.reduce(shard, linalg.ALONG_COLUMNS, out, init=_init_for_rank(init, reduce_op, group),
                         main_op=main_op, reduce_op=reduce_op, workspace=workspace)
    if (peer is not None and reduce_op == "add" and part.dtype == torch.float32 and
            final_op in ("identity", "mul_const", "div_const")):
        scale = 1.0 if final_op == "identity" else (final_scalar if final_op == "mul_const" else 1.0 / final_scalar)
        peer.all_reduce_sum(sums=part, scale=scale)
        return part
    combine_partials(part, reduce_op, group)
    linalg.apply_final(part, final_op, final_scalar)
    return part


def reduce_rows(shard, **kw):
    """Row-wise reduction of this rank's rows: the result is this rank's slice of the output."""
    return linalg.reduce(shard, linalg.ALONG_ROWS, **kw)


def reduce_rows_by_key(shard, keys_shard, n_unique_keys, weights_shard=None, with_counts=True, group=None,
                       sums=None, counts=None, workspace=None, peer=None):
    """Keyed row sums of a row-sharded matrix (keys and weights sharded with the rows): local
    tables, then the all-reduce of the sums and the one of the int64 counts - or, with `peer` (a
    PeerExchange) and fp32 sums, ONE kernel over peer memory for both. `sums`, `counts` and
    `workspace` (see linalg.reduce_rows_by_key_workspace_bytes) make the call allocation-free."""
    if counts is None and with_counts:
        counts = torch.zeros(n_unique_keys, dtype=torch.int64, device=shard.device)
    sums = linalg.reduce_rows_by_key(shard, keys_shard, n_unique_keys, d_sums=sums, d_weights=weights_shard,
                                     counts=counts, workspace=workspace)
    if peer is not None and sums.dtype == torch.float32:
        peer.all_reduce_sum(sums=sums, counts=counts)
    else:
        combine_partials_grouped([sums, counts], "add", group)
    return sums, counts
