"""raft_b200 - B200 (sm_100a) kernels for RAFT's dense reductions behind a C ABI.

`raft_b200.linalg` mirrors the raft::linalg entry points of the path (reduce,
coalesced_reduction, strided_reduction, norm, reduce_rows_by_key, reduce_cols_by_key) on
torch CUDA tensors; `raft_b200.distributed` shards them by rows over the GPUs of one node.
"""
from . import _lib  # noqa: F401
from . import linalg  # noqa: F401

__all__ = ["linalg", "_lib"]
