"""Generates tests/golden/lce_golden.npz by running the REFERENCE's own torch statement of the path.

Run once, in a container where the reference checkout is importable:

    python tests/golden/make_golden.py /path/to/reference_checkout

It imports ``reference_torch`` from ``linear_cross_entropy/ops.py`` of the reference (lines 9-17),
evaluates it on small seeded inputs on the CPU in float32 (its own precision: it casts the logits
to float32), takes gradients with autograd, and stores inputs and outputs. The inputs are multiples
of 1/64 in [-4, 4] (x) and of 1/512 in [-1/8, 1/8] (W), i.e. exactly representable in fp16, bf16
and fp32, so every dtype path of the CUDA library can be fed the identical numbers.
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

CASES = [
    # name, input seed, N,   H,   V, ignore_index, z_reg, scale, frac_ignored
    ("plain", 0, 128, 256, 512, -100, 0.0, 1.0, 0.0),
    ("ignore", 0, 128, 256, 512, -1, 0.0, 1.0, 0.1),
    ("all_options", 0, 128, 256, 512, 5, 1e-2, 0.5, 0.1),
    ("big_scale", 1, 256, 256, 768, -100, 1e-4, 4.0, 0.05),
]


def load_reference(ref_root: Path):
    spec = importlib.util.spec_from_file_location("ref_ops", ref_root / "linear_cross_entropy" / "ops.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.reference_torch


def make_inputs(seed, N, H, V, ignore_index, frac_ignored):
    g = torch.Generator().manual_seed(seed)
    xq = torch.clamp(torch.round(torch.randn(N, H, generator=g) * 64), -256, 256).to(torch.int16)
    wq = torch.clamp(torch.round(torch.randn(H, V, generator=g) / H ** 0.5 * 512), -64, 64).to(torch.int8)
    g = torch.Generator().manual_seed(1000 + seed + 17 * (ignore_index % 1000))
    y = torch.randint(0, V, (N,), generator=g)
    if frac_ignored > 0:
        y[torch.rand(N, generator=g) < frac_ignored] = ignore_index
    return xq, wq, y


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of the reference checkout>")
    ref_root = Path(sys.argv[1])
    reference_torch = load_reference(ref_root)
    torch.set_num_threads(1)  # fixed summation order
    out = {}
    for name, seed, N, H, V, ign, zreg, scale, frac in CASES:
        xq, wq, y = make_inputs(seed, N, H, V, ign, frac)
        x = (xq.float() / 64).requires_grad_(True)
        W = (wq.float() / 512).requires_grad_(True)
        # reference_torch takes the weight as (V, H) like F.linear
        loss, z_value, logit_max, logit_ent, logit_norm = reference_torch(
            x, y, W.t(), ignore_index=ign, z_regularization=zreg, logit_scale=scale
        )
        loss.backward()
        out[f"{name}/meta"] = np.array([N, H, V, ign], dtype=np.int64)
        out[f"{name}/opts"] = np.array([zreg, scale], dtype=np.float64)
        out[f"{name}/inputs"] = np.array([seed], dtype=np.int64)  # x, W are stored once per input seed
        out[f"inputs{seed}/xq"] = xq.numpy()
        out[f"inputs{seed}/wq"] = wq.numpy()
        out[f"{name}/y"] = y.numpy()
        out[f"{name}/scalars"] = np.array(
            [loss.item(), z_value.item(), logit_max.item(), logit_ent.item(), logit_norm.item()], dtype=np.float64
        )
        out[f"{name}/dx"] = x.grad.numpy().astype(np.float32)
        dW = W.grad.numpy()
        out[f"{name}/dW_rows"] = dW[::16].astype(np.float32)  # every 16th row in full
        out[f"{name}/dW_rowsum"] = dW.astype(np.float64).sum(axis=1)
        out[f"{name}/dW_colsum"] = dW.astype(np.float64).sum(axis=0)
        print(name, out[f"{name}/scalars"])
    path = Path(__file__).resolve().parent / "lce_golden.npz"
    np.savez_compressed(path, **out)
    print("wrote", path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
