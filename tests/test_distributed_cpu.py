"""Host-side logic of the row-sharded reductions on CPU: the row partition, and the cross-rank
combination of per-rank partials over a world-size-2 gloo group (partials come from the CPU
oracle here; on GPUs they come from the kernels)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from raft_b200 import distributed as D


@pytest.mark.parametrize("n,world", [(0, 1), (1, 4), (10, 3), (1_000_000, 8), (7, 8), (16_777_216, 8)])
def test_shard_rows_tiles_the_range(n, world):
    blocks = [D.shard_rows(n, r, world) for r in range(world)]
    assert blocks[0][0] == 0 and blocks[-1][1] == n
    for (a0, a1), (b0, b1) in zip(blocks, blocks[1:]):
        assert a1 == b0 and a0 <= a1
    sizes = [b - a for a, b in blocks]
    assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        D.shard_rows(n, world, world)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import oracle as o
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, d, nkeys = 1001, 33, 17
        full = o.synth((n, d), np.float32, 2, "uniform", 0, 1)
        keys = o.synth((n,), np.int32, 5, "int", 0, nkeys)
        r0, r1 = D.shard_rows(n, rank, world)
        # column sum and mean: fp64 partials, SUM
        part = torch.from_numpy(o.reduce(full[r0:r1], apply=1))
        D.combine_partials(part, "add")
        ok = np.allclose(part.numpy(), o.reduce(full, apply=1), rtol=1e-12)
        # a sum's start value enters the total ONCE (rank 0 keeps it, the others start from zero); the
        # start value of a max is idempotent and stays on every rank
        init = 3.5
        part = torch.from_numpy(o.reduce(full[r0:r1], apply=1, init=D._init_for_rank(init, "add", None)))
        D.combine_partials(part, "add")
        ok = ok and np.allclose(part.numpy(), o.reduce(full, apply=1, init=init), rtol=1e-12)
        ok = ok and D._init_for_rank(init, "max", None) == init
        # several partials at once: tensors of one type as a group, other types by themselves
        a, b = torch.full((5,), float(rank + 1)), torch.full((3,), rank + 1, dtype=torch.int64)
        c = torch.full((2,), float(10 * (rank + 1)))
        D.combine_partials_grouped([a, None, b, c], "add")
        tot = sum(range(1, world + 1))
        ok = ok and bool((a == tot).all() and (b == tot).all() and (c == 10 * tot).all())
        # column Linf: MAX
        part = torch.from_numpy(o.reduce(full[r0:r1], apply=1, main_op="abs", reduce_op="max"))
        D.combine_partials(part, "max")
        ok = ok and np.array_equal(part.numpy(), o.reduce(full, apply=1, main_op="abs", reduce_op="max"))
        # keyed sums + counts
        s, c = o.rows_by_key(full[r0:r1], keys[r0:r1], nkeys)
        ts, tc = torch.from_numpy(s), torch.from_numpy(c)
        D.combine_partials(ts, "add")
        D.combine_partials(tc, "add")
        es, ec = o.rows_by_key(full, keys, nkeys)
        ok = ok and np.allclose(ts.numpy(), es, rtol=1e-12) and np.array_equal(tc.numpy(), ec)
        # row-wise outputs are disjoint slices: concatenating the ranks' slices gives the full result
        mine = torch.from_numpy(o.reduce(full[r0:r1], main_op="sq"))
        sizes = [D.shard_rows(n, r, world) for r in range(world)]
        longest = max(b - a for a, b in sizes)
        padded = torch.zeros(longest, dtype=torch.float64)
        padded[:mine.numel()] = mine
        gathered = [torch.empty(longest, dtype=torch.float64) for _ in sizes]
        dist.all_gather(gathered, padded)
        whole = torch.cat([g[:b - a] for g, (a, b) in zip(gathered, sizes)])
        ok = ok and np.array_equal(whole.numpy(), o.reduce(full, main_op="sq"))
        try:
            D.combine_partials(part, "argmin")
            ok = False
        except ValueError:
            pass
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_combine_partials_world_size_2():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=5) for _ in range(world))
    assert results == {0: True, 1: True}
