"""Shared helpers for the tests: golden-fixture loading and the parity metric."""
import glob
import os

import numpy as np
import torch

import haste_oracle as oracle

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# parity bars (max|a-b| / max|b|): fp32 storage and bf16 storage with fp32 accumulate
TOL_F32 = 1e-4
TOL_BF16 = 2e-2


def golden_files(cell=None):
    files = sorted(glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))
    if cell is not None:
        files = [f for f in files if os.path.basename(f).startswith(cell + "_T")]
    return files


def load_golden(path, dtype=torch.float64):
    z = np.load(path)
    name = os.path.basename(path)
    cell = name[:name.index("_T")]
    T, N, C, H = (int(v) for v in z["meta"])
    d = {k[3:]: torch.from_numpy(z[k]).to(dtype) for k in z.files if k.startswith("in_")}
    d.setdefault("mask", None)
    out = {k[4:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("out_")}
    grads = {k[5:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("grad_")}
    return cell, (T, N, C, H), float(z["zoneout"]), d, out, grads


max_rel_err = oracle.max_rel_err
