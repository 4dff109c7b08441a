"""Multi-GPU check of raft_b200.distributed, launched by torchrun (one rank per GPU):
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29511 tests/mg_check.py
Every rank builds its shard of the same seeded matrix with the counter-based generator, runs the
sharded reductions, and rank 0 compares with the single-GPU result on the whole matrix."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from raft_b200 import distributed as D  # noqa: E402
from raft_b200 import linalg  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    n, d, nkeys = 400_003, 64, 300
    r0, r1 = D.shard_rows(n, rank, world)
    shard = torch.empty((r1 - r0, d), dtype=torch.float32, device=dev)
    linalg.synth_fill(shard, 2, "normal", first_index=r0 * d)
    keys = torch.empty((r1 - r0,), dtype=torch.int32, device=dev)
    linalg.synth_fill(keys, 5, "int", 0, nkeys, first_index=r0)

    mean = D.reduce_columns(shard, n, final_op="div_const", final_scalar=float(n))
    linf = D.reduce_columns(shard, n, main_op="abs", reduce_op="max", init=0.0)
    sums, counts = D.reduce_rows_by_key(shard, keys, nkeys)
    norms = D.reduce_rows(shard, main_op="sq", final_op="sqrt")
    # the same through the one-kernel all-reduce over peer memory, three times (both data sets of the area)
    peer = D.PeerExchange(nkeys * d * 4 + nkeys * 8 + 64)
    for _ in range(3):
        p_mean = D.reduce_columns(shard, n, final_op="div_const", final_scalar=float(n), peer=peer)
        p_sums, p_counts = D.reduce_rows_by_key(shard, keys, nkeys, peer=peer)
    peer_ok = peer.status()
    peer.close()

    sizes = [D.shard_rows(n, r, world) for r in range(world)]
    longest = max(b - a for a, b in sizes)
    padded = torch.zeros(longest, dtype=torch.float32, device=dev)
    padded[:norms.numel()] = norms
    gathered = [torch.empty(longest, dtype=torch.float32, device=dev) for _ in sizes]
    dist.all_gather(gathered, padded)
    ok = True
    if rank == 0:
        full = torch.empty((n, d), dtype=torch.float32, device=dev)
        linalg.synth_fill(full, 2, "normal")
        fkeys = torch.empty((n,), dtype=torch.int32, device=dev)
        linalg.synth_fill(fkeys, 5, "int", 0, nkeys)
        e_mean = linalg.reduce(full, linalg.ALONG_COLUMNS, final_op="div_const", final_scalar=float(n))
        e_linf = linalg.reduce(full, linalg.ALONG_COLUMNS, main_op="abs", reduce_op="max")
        e_counts = torch.zeros(nkeys, dtype=torch.int64, device=dev)
        e_sums = linalg.reduce_rows_by_key(full, fkeys, nkeys, counts=e_counts)
        e_norms = linalg.reduce(full, linalg.ALONG_ROWS, main_op="sq", final_op="sqrt")
        whole = torch.cat([g[:b - a] for g, (a, b) in zip(gathered, sizes)])
        checks = {
            "column mean": torch.allclose(mean, e_mean, rtol=1e-5, atol=1e-5),
            "column Linf": torch.equal(linf, e_linf),
            "keyed sums": torch.allclose(sums, e_sums, rtol=1e-5, atol=1e-5),
            "key counts": torch.equal(counts, e_counts),
            "row norms (disjoint slices)": torch.equal(whole, e_norms),
            "peer exchange: no wait ran out": peer_ok == 0,
            "peer exchange: column mean": torch.allclose(p_mean, e_mean, rtol=1e-5, atol=1e-5),
            "peer exchange: keyed sums": torch.allclose(p_sums, e_sums, rtol=1e-5, atol=1e-5),
            "peer exchange: key counts": torch.equal(p_counts, e_counts),
        }
        for k, v in checks.items():
            print(("ok   " if v else "FAIL ") + k, flush=True)
        ok = all(checks.values())
        print("MG ALL PASSED" if ok else "MG FAILED", flush=True)
    dist.barrier(device_ids=[local])
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
