"""Helpers shared by the GPU parity tests: seeded inputs present on both sides."""
import numpy as np
import torch

from raft_b200 import linalg

_TORCH_OF = {np.dtype(np.float32): torch.float32, np.dtype(np.float64): torch.float64,
             np.dtype(np.float16): torch.float16, np.dtype(np.int32): torch.int32, np.dtype(np.int16): torch.int16,
             np.dtype(np.int64): torch.int64}


def device_synth(shape, np_dtype, seed, kind, lo, hi, device):
    """Generates on the device with b2r_synth_fill and returns (device tensor, host copy)."""
    t = torch.empty(shape, dtype=_TORCH_OF[np.dtype(np_dtype)], device=device)
    linalg.synth_fill(t, seed, kind, lo, hi)
    return t, t.cpu().numpy()


def as_layout(t, layout):
    """A [r, c] device tensor whose memory is row-major (0) or column-major (1), same values."""
    if layout == 0:
        return t.contiguous()
    return t.t().contiguous().t()
