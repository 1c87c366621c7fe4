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
# float16 storage (GRU only): the stored values are used exactly and accumulated in fp32, so
# what remains is the rounding of stored results to 11 significant bits along the recurrence
TOL_F16 = 5e-3
# LayerNormLSTM in the C ABI's all-bf16 mode (HASTE_B200_BF16: the caller's act_Wx,
# act_Wx_norm and h buffers are bf16, as a C++ caller with __nv_bfloat16 buffers passes them):
# those interface tensors are rounded whatever the arithmetic and three LayerNorms per step
# amplify the rounding.  Exact float64 arithmetic that rounds nothing but them is already
# 2e-2 .. 1e-1 from the unrounded oracle (test_bf16_storage_floor.py), so that mode alone has
# this bar.  The Python layers use HASTE_B200_BF16_WIDE and meet TOL_BF16.
TOL_BF16_ALL_STORAGE_LN_LSTM = 1e-1


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


# ---------------------------------------------------------------------------
# CUDA side: run one layer through the haste_b200 ops (C ABI) with the oracle's
# input dictionary, returning outputs and gradients under the oracle's names.
# ---------------------------------------------------------------------------
def run_cuda(cell, d, zoneout=0.0, dtype=torch.float32, transposed=False, training=True,
             backward=True, device="cuda", grads=None, fwd_kwargs=None, lib=None):
    """Runs one layer through the twelve tensor-level ops: those of `haste_b200.ops`, or of
    `lib` - the compiled `haste_pytorch_lib` module, which has the reference's exact
    signatures (pre-transposed backward inputs, no keyword arguments)."""
    from haste_b200 import ops
    compiled = lib is not None
    if compiled:
        ops, transposed = lib, True
    _, names, has_c = oracle.CELLS[cell]
    t = {k: (v.to(device=device, dtype=dtype).contiguous() if v is not None else None)
         for k, v in d.items()}
    mask = t["mask"] if t.get("mask") is not None else torch.empty(0, 0, 0, device=device, dtype=dtype)
    x = t["x"]
    if cell == "lstm":
        ins = (x, t["h0"], t["c0"], t["W"], t["R"], t["b"], mask)
    elif cell == "gru":
        ins = (x, t["h0"], t["W"], t["R"], t["bx"], t["br"], mask)
    elif cell == "indrnn":
        ins = (x, t["h0"], t["W"], t["u"], t["b"], mask)
    elif cell == "layer_norm_lstm":
        ins = (x, t["h0"], t["c0"], t["W"], t["R"], t["b"], t["gamma"], t["gamma_h"], t["beta_h"], mask)
    elif cell == "layer_norm_gru":
        ins = (x, t["h0"], t["W"], t["R"], t["bx"], t["br"], t["gamma"], mask)
    else:
        ins = (x, t["h0"], t["W"], t["u"], t["b"], t["gamma"], mask)
    fwd = getattr(ops, cell + "_forward")(training, zoneout, *ins, **(fwd_kwargs or {}))
    fwd = fwd if isinstance(fwd, (list, tuple)) else [fwd]
    out = {"h": fwd[0]}
    if has_c:
        out["c"] = fwd[1]
    if not backward:
        return out, {}
    xx = x.permute(2, 0, 1).contiguous() if transposed else x
    W = t["W"].t().contiguous() if transposed else t["W"]
    saved = list(fwd[2:]) if has_c else list(fwd[1:])
    if "indrnn" in cell:
        rec = t["u"]
    else:
        rec = t["R"].t().contiguous() if transposed else t["R"]
    if cell == "lstm":
        args = (xx, W, rec, t["b"], mask, fwd[0], fwd[1], *saved, t["dh"], t["dc"])
        gn = ["x", "h0", "c0", "W", "R", "b"]
    elif cell == "gru":
        args = (xx, W, rec, t["bx"], t["br"], mask, fwd[0], *saved, t["dh"])
        gn = ["x", "h0", "W", "R", "bx", "br"]
    elif cell == "indrnn":
        args = (xx, W, rec, t["b"], mask, fwd[0], t["dh"])
        gn = ["x", "h0", "W", "u", "b"]
    elif cell == "layer_norm_lstm":
        args = (xx, W, rec, t["b"], t["gamma"], t["gamma_h"], t["beta_h"], mask, fwd[0], fwd[1],
                *saved, t["dh"], t["dc"])
        gn = ["x", "h0", "c0", "W", "R", "b", "gamma", "gamma_h", "beta_h"]
    elif cell == "layer_norm_gru":
        args = (xx, W, rec, t["bx"], t["br"], t["gamma"], mask, fwd[0], *saved, t["dh"])
        gn = ["x", "h0", "W", "R", "bx", "br", "gamma"]
    else:
        args = (xx, W, rec, t["b"], t["gamma"], mask, fwd[0], *saved, t["dh"])
        gn = ["x", "h0", "W", "u", "b", "gamma"]
    if compiled:
        got = getattr(ops, cell + "_backward")(*args)
    else:
        got = getattr(ops, cell + "_backward")(*args, transposed=transposed, grads=grads)
    return out, dict(zip(gn, got))


def assert_close(got, want, tol, what=""):
    err = max_rel_err(got, want)
    assert err < tol, f"{what}: max rel err {err:.3e} >= {tol:.1e}"
    return err


# ---------------------------------------------------------------------------
# Stacked / bidirectional networks built from oracle layers (the reference's PyTorch API has
# single layers only; composition follows frameworks/tf/base_rnn.py:115-121: the backward
# direction runs on the time-reversed input and its output is reversed back, the next level
# sees cat([fw, bw], -1)).
# ---------------------------------------------------------------------------
class _RoundForward(torch.autograd.Function):
    """A tensor stored in bf16: rounded on the way forward, gradient passed through."""

    @staticmethod
    def forward(ctx, a):
        return a.to(torch.bfloat16).to(a.dtype)

    @staticmethod
    def backward(ctx, g):
        return g


class _RoundBackward(torch.autograd.Function):
    """A gradient stored in bf16: identity forward, rounded on the way back."""

    @staticmethod
    def forward(ctx, a):
        return a.view_as(a)

    @staticmethod
    def backward(ctx, g):
        return g.to(torch.bfloat16).to(g.dtype)


def seeded_masks(num_layers, dirs, T, N, H, gates, zoneout, dropconnect, base_seed=1234):
    """Zoneout keep-masks [T,N,H] and DropConnect keep-masks [H,gates*H] per layer and
    direction, each pair drawn on the CPU from torch.Generator(base_seed + layer*2 + dir)."""
    masks = []
    for l in range(num_layers):
        level = []
        for d_ in range(dirs):
            g = torch.Generator().manual_seed(base_seed + l * 2 + d_)
            m = {}
            if zoneout:
                m["zoneout_mask"] = torch.bernoulli(torch.full((T, N, H), 1.0 - zoneout), generator=g)
            if dropconnect:
                m["dropconnect_mask"] = torch.bernoulli(torch.full((H, gates * H), 1.0 - dropconnect),
                                                        generator=g)
            level.append(m)
        masks.append(level)
    return masks


def oracle_stack(net, cell, x, dy, masks=None, dropconnect=0.0, zoneout=0.0, bf16=False,
                 dtype=torch.float64):
    """Runs the haste_b200.Stack `net` (cells of kind `cell`) as a composition of oracle
    layers on the CPU with the network's own parameters; returns (y, dx, [per layer and
    direction {parameter name: gradient}]) for the loss sum(y * dy).

    bf16=True restates what bf16 storage means for a stack: every tensor that crosses a
    layer's interface in bf16 is rounded there - the layer's output sequence, the gradient
    handed to the layer below, and the DropConnect-masked recurrent kernel - while each
    layer's own arithmetic stays exact.
    """
    fn, names, has_c = oracle.CELLS[cell]
    pname = {"W": "kernel", "R": "recurrent_kernel", "b": "bias", "bx": "bias",
             "br": "recurrent_bias", "u": "recurrent_scale", "gamma": "gamma",
             "gamma_h": "gamma_h", "beta_h": "beta_h"}
    xo = x.detach().to("cpu", dtype).requires_grad_(True)
    inp, leaves = xo, []
    for l, level in enumerate(net.layers):
        outs = []
        for d_, layer in enumerate(level):
            p = {k: v.detach().to("cpu", dtype).requires_grad_(True)
                 for k, v in layer.named_parameters()}
            leaves.append(p)
            m = masks[l][d_] if masks is not None else {}
            xi = torch.flip(inp, [0]) if d_ == 1 else inp
            if bf16:
                xi = _RoundBackward.apply(xi)
            N, H = xi.shape[1], layer.hidden_size
            args = {"x": xi, "h0": torch.zeros(N, H, dtype=dtype), "c0": torch.zeros(N, H, dtype=dtype)}
            for k in names:
                if k in pname and pname[k] in p and k not in args:
                    args[k] = p[pname[k]]
            if "R" in args and dropconnect and "dropconnect_mask" in m:
                if bf16:
                    scale = (m["dropconnect_mask"].to(torch.bfloat16) / (1.0 - dropconnect)).to(dtype)
                    args["R"] = _RoundForward.apply(args["R"] * scale)
                else:
                    scale = (m["dropconnect_mask"].float() / (1.0 - dropconnect)).to(dtype)
                    args["R"] = args["R"] * scale
            zm = m.get("zoneout_mask")
            out = fn(True, zoneout if zm is not None else 0.0, *[args[k] for k in names],
                     zm.to(dtype) if zm is not None else None)
            h = out[0] if has_c else out
            yo = h[1:]
            if bf16:
                yo = _RoundForward.apply(yo)
            outs.append(torch.flip(yo, [0]) if d_ == 1 else yo)
        inp = torch.cat(outs, -1) if len(outs) > 1 else outs[0]
    (inp * dy.detach().to("cpu", dtype)).sum().backward()
    dx = xo.grad
    if bf16:
        dx = dx.to(torch.bfloat16).to(dtype)
    return inp.detach(), dx, [{k: v.grad for k, v in p.items()} for p in leaves]


def oracle_stack_forward(net, cell, x, masks, dropconnect, zoneout, dtype):
    """Forward pass only of `oracle_stack` (no autograd graph: long sequences stay cheap)."""
    fn, names, has_c = oracle.CELLS[cell]
    pname = {"W": "kernel", "R": "recurrent_kernel", "b": "bias", "bx": "bias",
             "br": "recurrent_bias", "u": "recurrent_scale", "gamma": "gamma",
             "gamma_h": "gamma_h", "beta_h": "beta_h"}
    inp = x.detach().to("cpu", dtype)
    for l, level in enumerate(net.layers):
        outs = []
        for d_, layer in enumerate(level):
            p = {k: v.detach().to("cpu", dtype) for k, v in layer.named_parameters()}
            m = masks[l][d_] if masks is not None else {}
            xi = torch.flip(inp, [0]) if d_ == 1 else inp
            N, H = xi.shape[1], layer.hidden_size
            args = {"x": xi, "h0": torch.zeros(N, H, dtype=dtype), "c0": torch.zeros(N, H, dtype=dtype)}
            for k in names:
                if k in pname and pname[k] in p and k not in args:
                    args[k] = p[pname[k]]
            if "R" in args and dropconnect and "dropconnect_mask" in m:
                args["R"] = args["R"] * (m["dropconnect_mask"].float() / (1.0 - dropconnect)).to(dtype)
            zm = m.get("zoneout_mask")
            out = fn(True, zoneout if zm is not None else 0.0, *[args[k] for k in names],
                     zm.to(dtype) if zm is not None else None)
            yo = (out[0] if has_c else out)[1:]
            outs.append(torch.flip(yo, [0]) if d_ == 1 else yo)
        inp = torch.cat(outs, -1) if len(outs) > 1 else outs[0]
    return inp


def compare_stack(net, y, dx, ref, tol, what, ref_native=None):
    """Outputs, input gradient and EVERY parameter gradient of every layer and direction of a
    Stack against `oracle_stack`'s result; returns the worst error.

    `ref_native`, if given, is the same oracle evaluated in the reference's own working
    precision (float32).  A deep normalised stack amplifies float32 rounding: where the
    reference's own float32 path is itself a multiple of `tol` from the float64 result, no
    float32 implementation can be within `tol`, and the bar for that tensor becomes `tol`
    plus twice the reference path's own distance (the rule the comparison with the
    reference's CUDA build uses)."""
    ref_y, ref_dx, ref_grads = ref

    def bar(native, exact):
        return tol if native is None else tol + 2.0 * max_rel_err(native, exact)

    worst = assert_close(y, ref_y, bar(ref_native and ref_native[0], ref_y), f"{what} y")
    worst = max(worst, assert_close(dx, ref_dx, bar(ref_native and ref_native[1], ref_dx), f"{what} dx"))
    i = 0
    for l, level in enumerate(net.layers):
        for d_, layer in enumerate(level):
            for k, v in layer.named_parameters():
                got, want = v.grad, ref_grads[i][k]
                nat = ref_native[2][i][k] if ref_native else None
                if k == "gamma" and type(layer).__name__ == "LayerNormIndRNN":
                    got, want = got[0], want[0]  # row 1 of gamma is unused by this cell
                    nat = nat[0] if nat is not None else None
                worst = max(worst, assert_close(got, want, bar(nat, want),
                                                f"{what} layer {l} dir {d_} d{k}"))
            i += 1
    return worst
