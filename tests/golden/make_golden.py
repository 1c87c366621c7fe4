"""Generates the golden fixtures in this folder from the REFERENCE implementation.

Run once, on a machine where the reference checkout is present:

    python tests/golden/make_golden.py /path/to/haste

It imports the reference's `haste_pytorch` Python package from
`<checkout>/frameworks/pytorch` (with an empty stand-in for its compiled
`haste_pytorch_lib` module and for the generated `_version` module, neither of
which the CPU path uses), runs each cell's own CPU function
(`LSTMScript`, `GRUScript`, ... ) in float64 on seeded inputs, takes every
gradient with autograd, and stores inputs, outputs and gradients as `.npz`.

The fixtures pin the oracle (`oracle/haste_oracle.py`) and, through it, the CUDA
kernels.  The tests never import the reference; they only read the `.npz` files.
"""

import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import haste_oracle as oracle  # noqa: E402  (input generator only)


def import_reference(root):
    pkg_dir = os.path.join(root, "frameworks", "pytorch")
    sys.modules["haste_pytorch_lib"] = types.ModuleType("haste_pytorch_lib")
    spec = importlib.util.spec_from_file_location(
        "haste_pytorch", os.path.join(pkg_dir, "__init__.py"),
        submodule_search_locations=[pkg_dir])
    ver = types.ModuleType("haste_pytorch._version")
    ver.__version__ = "reference"
    sys.modules["haste_pytorch._version"] = ver
    mod = importlib.util.module_from_spec(spec)
    sys.modules["haste_pytorch"] = mod
    spec.loader.exec_module(mod)
    return mod


# (cell, T, N, C, H, zoneout, seed)
CASES = [
    ("lstm", 5, 3, 4, 6, 0.0, 11),
    ("lstm", 7, 2, 5, 8, 0.3, 12),
    ("gru", 5, 3, 4, 6, 0.0, 21),
    ("gru", 7, 2, 5, 8, 0.3, 22),
    ("indrnn", 6, 3, 4, 6, 0.0, 31),
    ("indrnn", 6, 2, 5, 8, 0.3, 32),
    ("layer_norm_lstm", 5, 3, 4, 6, 0.0, 41),
    ("layer_norm_lstm", 6, 2, 5, 8, 0.3, 42),
    ("layer_norm_gru", 5, 3, 4, 6, 0.0, 51),
    ("layer_norm_gru", 6, 2, 5, 8, 0.3, 52),
    ("layer_norm_indrnn", 6, 3, 4, 6, 0.0, 61),
    ("layer_norm_indrnn", 6, 2, 5, 8, 0.3, 62),
    # a mid-sized case per cell family for the GPU parity tests
    ("lstm", 20, 16, 24, 32, 0.2, 13),
    ("gru", 20, 16, 24, 32, 0.2, 23),
    ("layer_norm_lstm", 12, 8, 24, 32, 0.2, 43),
]


def main():
    # the reference checkout: argument, else $HASTE_REFERENCE_ROOT, else a `reference` directory
    # beside this repository
    here = os.path.dirname(os.path.abspath(__file__))
    sibling = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(here))), "reference")
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("HASTE_REFERENCE_ROOT", sibling)
    if not os.path.isdir(root):
        sys.exit("usage: make_golden.py /path/to/haste   (or HASTE_REFERENCE_ROOT=/path/to/haste)")
    ref = import_reference(root)
    script = {
        "lstm": ref.lstm.LSTMScript,
        "gru": ref.gru.GRUScript,
        "indrnn": ref.indrnn.IndRNNScript,
        "layer_norm_lstm": ref.layer_norm_lstm.LayerNormLSTMScript,
        "layer_norm_gru": ref.layer_norm_gru.LayerNormGRUScript,
        "layer_norm_indrnn": ref.layer_norm_indrnn.LayerNormIndRNNScript,
    }
    for cell, T, N, C, H, zo, seed in CASES:
        d = oracle.make_inputs(cell, T, N, C, H, seed=seed, dtype=torch.float64, zoneout=zo)
        _, names, has_c = oracle.CELLS[cell]
        leaves = {k: d[k].clone().requires_grad_(True) for k in names}
        mask = d["mask"] if d["mask"] is not None else torch.empty(0, 0, 0, dtype=torch.float64)
        out = script[cell](True, zo, *[leaves[k] for k in names], mask)
        if has_c:
            h, c = out
            loss = (h[1:] * d["dh"][1:]).sum() + (c[1:] * d["dc"][1:]).sum()
        else:
            h, c = out, None
            loss = (h[1:] * d["dh"][1:]).sum()
        grads = torch.autograd.grad(loss, [leaves[k] for k in names])
        # inference-mode output as well (expectation form of zoneout)
        with torch.no_grad():
            out_inf = script[cell](False, zo, *[d[k] for k in names], mask)
        h_inf = out_inf[0] if has_c else out_inf
        blob = {"meta": np.array([T, N, C, H], dtype=np.int64), "zoneout": np.array(zo)}
        for k in names:
            blob["in_" + k] = d[k].numpy()
        if d["mask"] is not None:
            blob["in_mask"] = d["mask"].numpy()
        blob["in_dh"] = d["dh"].numpy()
        if has_c:
            blob["in_dc"] = d["dc"].numpy()
            blob["out_c"] = c.detach().numpy()
        blob["out_h"] = h.detach().numpy()
        blob["out_h_inference"] = h_inf.numpy()
        for k, g in zip(names, grads):
            blob["grad_" + k] = g.numpy()
        name = f"{cell}_T{T}_N{N}_C{C}_H{H}_z{int(zo * 10)}.npz"
        np.savez_compressed(os.path.join(HERE, name), **blob)
        print("wrote", name)


if __name__ == "__main__":
    main()
