"""Writes tests/golden/synth_v1.npz: the first 64 values of each synthetic stream the
benchmark configs use, from the host generator in oracle/oracle.c. Run from the repo root:
    python tests/golden/make_synth_golden.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from oracle import oracle as o  # noqa: E402

out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "synth_v1.npz")
np.savez(out,
         uniform_f32=o.synth((64,), np.float32, 0, "uniform", -1, 1),
         normal_f32=o.synth((64,), np.float32, 1, "normal"),
         int_f32=o.synth((64,), np.float32, 3, "int", 0, 16),
         keys_i32=o.synth((64,), np.int32, 5, "int", 0, 1024),
         uniform_f64=o.synth((64,), np.float64, 2, "uniform", 0, 1))
print("wrote", out)
