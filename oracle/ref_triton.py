"""Loader and timing helper for the reference's own Triton implementation.  TEST INFRASTRUCTURE ONLY.

The unmodified reference package is installed into ``oracle/_ref/`` by ``oracle/make_ref.py``; this module imports
it from there (never from the shipped package) so that

* ``tests/test_gpu_vs_triton.py`` can compare the CUDA path with the reference's Triton path on the same inputs, and
* ``bench.py`` can time the reference's Triton op beside its own numbers (a baseline leg, outside the timed
  region of the CUDA path).

Two properties of the reference that every caller here has to respect:

* The first call for a new (V, N, H, monitoring) key autotunes, and Triton's autotuner zeroes the buffers named in
  ``reset_to_zero`` (linear_cross_entropy/ops.py:117) after benchmarking. That wipes the ``-10e5`` initialisation of
  ``lse_local`` (ops.py:697), whose unwritten columns then add ``exp(0)`` terms to the row sums (ops.py:755). Results
  are only right from the SECOND call for a key on. ``call`` below always warms a key up first.
* It asserts N % 512 == 0, V % 4096 == 0, H % 256 == 0 (ops.py:689-691) and N % N_chunk_size == 0 implicitly.
"""
from __future__ import annotations

import importlib
import sys
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"

_module = None
_error = None
_warm = set()


def load():
    """The reference's ``linear_cross_entropy`` package, or raises RuntimeError with the reason it is unavailable."""
    global _module, _error
    if _module is not None:
        return _module
    if _error is not None:
        raise RuntimeError(_error)
    if not (REF_DIR / "linear_cross_entropy" / "ops.py").exists():
        _error = "reference package not installed under oracle/_ref (run oracle/make_ref.py where the checkout exists)"
        raise RuntimeError(_error)
    sys.path.insert(0, str(REF_DIR))
    try:
        _module = importlib.import_module("linear_cross_entropy")
    except Exception as err:  # Triton missing or not importable on this machine
        _error = f"reference package failed to import: {type(err).__name__}: {err}"
        raise RuntimeError(_error) from err
    finally:
        sys.path.remove(str(REF_DIR))
    return _module


def trim_configs(fwd_keep=(0, 9, 12), bwd_keep=(0, 2, 3)) -> None:
    """Shortens the autotune lists IN PLACE, the way the reference's README tells users to (README.md:37-38):
    the autotuners hold the very list objects the package exports. The kept backward entries have SPLIT_N = SPLIT_V
    = 1, the only ones the reference accepts for bf16 (ops.py:35-41)."""
    ref = load()
    for lst, keep in ((ref.fwd_configs, fwd_keep), (ref.bwd_configs, bwd_keep)):
        if len(lst) > len(keep):
            kept = [lst[i] for i in keep]
            del lst[:]
            lst.extend(kept)


def call(x, y, At, ignore_index=-100, z_regularization=0.0, logit_scale=1.0, N_chunk_size=4096, monitoring=False):
    """One forward+backward through the reference's functional API on CUDA tensors, on a warmed-up key.
    Returns (five output scalars as floats, x.grad, At.grad) with the gradients in the dtypes autograd delivers."""
    import torch

    ref = load()
    N = x.numel() // x.shape[-1]
    key = (N, x.shape[-1], At.shape[1], str(x.dtype), bool(monitoring), min(N, int(N_chunk_size)))

    def once():
        xx = x.detach().clone().requires_grad_(True)
        AA = At.detach().clone().requires_grad_(True)
        out = ref.linear_cross_entropy(xx, y, AA, ignore_index, z_regularization, logit_scale, N_chunk_size, monitoring)
        out[0].backward()
        torch.cuda.synchronize()
        return out, xx.grad, AA.grad

    if key not in _warm:
        once()  # autotunes; its results are the unreliable first-call ones
        _warm.add(key)
    out, gx, gA = once()
    return [float(v) for v in out], gx, gA


def time_fwd_bwd(x, y, At, ignore_index, z_regularization, logit_scale, N_chunk_size, monitoring, steps=10, warmup=3):
    """Milliseconds per forward+backward of the reference's op (CUDA events, after the autotune call and ``warmup``
    further calls), plus the autotuner's chosen configurations as text."""
    import torch

    ref = load()
    xx = x.detach().clone().requires_grad_(True)
    AA = At.detach().clone().requires_grad_(True)

    def step():
        loss = ref.linear_cross_entropy(xx, y, AA, ignore_index, z_regularization, logit_scale, N_chunk_size,
                                        monitoring)[0]
        loss.backward()
        xx.grad = None
        AA.grad = None
        return loss

    step()  # autotune
    for _ in range(max(1, warmup)):
        loss = step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    chosen = {}
    for name in ("linear_xent_fwd_prep_bwd_kernel_matmul_t", "linear_xent_bwd_dispatcher"):
        tuner = getattr(ref.ops, name, None)
        best = getattr(tuner, "best_config", None)
        if best is not None:
            chosen[name] = str(best)
    return e0.elapsed_time(e1) / steps, float(loss), chosen
