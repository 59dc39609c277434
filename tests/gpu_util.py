"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from linear_cross_entropy_loss_b200 import linear_cross_entropy
from oracle import oracle

# Tolerances of the GPU path against the float64 oracle (loss relative error, gradient cosine, gradient L2 error
# relative to the gradient norm). The path keeps logits, log-sum-exp and all reductions in fp32; only dZ and the
# MMA inputs are rounded to the input type, so 16-bit gradients are good to a few 1e-3 relative.
TOL = {
    torch.float32: dict(loss=2e-4, cos=0.99999, rel=5e-3),   # TF32 products: 10-bit mantissa
    torch.float16: dict(loss=2e-5, cos=0.999995, rel=2e-3),
    torch.bfloat16: dict(loss=2e-5, cos=0.99999, rel=6e-3),
}


def cosine(a, b):
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def rel_err(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-300))


def random_problem(N, H, V, dtype, seed=0, ignore=-1, frac=0.05, w_std=None):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, H, generator=g).to(dtype)
    W = (torch.randn(H, V, generator=g) * (w_std if w_std is not None else H ** -0.5)).to(dtype)
    y = torch.randint(0, V, (N,), generator=g)
    if frac > 0:
        y[torch.rand(N, generator=g) < frac] = ignore
    return x, y, W


def run_gpu(x, y, W, ignore=-100, zreg=0.0, scale=1.0, chunk=4096, monitoring=True, grad_scale=None):
    xd = x.cuda().requires_grad_(True)
    Wd = W.cuda().requires_grad_(True)
    out = linear_cross_entropy(xd, y.cuda(), Wd, ignore, zreg, scale, chunk, monitoring)
    (out[0] if grad_scale is None else out[0] * grad_scale).backward()
    torch.cuda.synchronize()
    return [v.item() for v in out], xd.grad, Wd.grad


def check_against_oracle(x, y, W, dtype, ignore=-100, zreg=0.0, scale=1.0, chunk=4096, monitoring=True,
                         loss_tol=None):
    """The pass as a user gets it (slab mode chosen by the library) against the float64 oracle; for bf16 / fp32 also
    with one base per row forced, the mode of large problems, which the library does not pick for small chunks."""
    import os

    result = _check_against_oracle(x, y, W, dtype, ignore, zreg, scale, chunk, monitoring, loss_tol)
    if dtype != torch.float16 and "LCE_SLAB_MODE" not in os.environ:
        os.environ["LCE_SLAB_MODE"] = "row"
        try:
            _check_against_oracle(x, y, W, dtype, ignore, zreg, scale, chunk, monitoring, loss_tol)
        finally:
            del os.environ["LCE_SLAB_MODE"]
    return result


def _check_against_oracle(x, y, W, dtype, ignore, zreg, scale, chunk, monitoring, loss_tol):
    got, dx, dW = run_gpu(x, y, W, ignore, zreg, scale, chunk, monitoring)
    ref = oracle.forward_backward(x, y, W, ignore, zreg, scale)
    tol = dict(TOL[dtype])
    if loss_tol is not None:
        tol["loss"] = loss_tol
    assert abs(got[0] - ref.loss) <= tol["loss"] * abs(ref.loss), (got[0], ref.loss)
    assert abs(got[1] - ref.z_value) <= 2 * tol["loss"] * abs(ref.z_value), (got[1], ref.z_value)
    if monitoring:
        assert abs(got[2] - ref.logit_max) <= 2e-3 * abs(ref.logit_max) + 1e-5, (got[2], ref.logit_max)
        assert abs(got[3] - ref.logit_entropy) <= 1e-3 * abs(ref.logit_entropy) + 1e-5, (got[3], ref.logit_entropy)
        assert abs(got[4] - ref.logit_norm) <= 1e-3 * abs(ref.logit_norm), (got[4], ref.logit_norm)
    assert dx.dtype == x.dtype and dW.dtype == W.dtype
    dxn, dWn = dx.double().cpu().numpy(), dW.double().cpu().numpy()
    assert cosine(dxn, ref.dx) >= tol["cos"], cosine(dxn, ref.dx)
    assert cosine(dWn, ref.dW) >= tol["cos"], cosine(dWn, ref.dW)
    # output rounding of a 16-bit gradient adds half an ulp: 2^-9 (bf16) / 2^-12 (fp16) relative
    out_round = {torch.float32: 0.0, torch.float16: 2.5e-4, torch.bfloat16: 2e-3}[dtype]
    assert rel_err(dxn, ref.dx) <= tol["rel"] + out_round, rel_err(dxn, ref.dx)
    assert rel_err(dWn, ref.dW) <= tol["rel"] + out_round, rel_err(dWn, ref.dW)
    return got, dxn, dWn, ref
