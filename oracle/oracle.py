"""CPU oracle of the fused linear + cross-entropy path.  TEST INFRASTRUCTURE ONLY.

This file restates, in float64 numpy, what the reference computes on this path. It is the checker
for the CUDA kernels; nothing in the shipped package imports it. Only ``tests/``,
``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may
call into it.

Parity pin: ``tests/golden/lce_golden.npz`` holds outputs of the reference's own torch statement of
the path, ``reference_torch`` (linear_cross_entropy/ops.py:9-17 of the reference project), produced
by importing the reference (``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks every
function below against those vectors.

Semantics restated (reference file:line):
  z      = logit_scale * (x @ W)                       ops.py:11 and ops.py:200   (W is (H, V))
  lse_i  = logsumexp_j z_ij                            ops.py:13, ops.py:205-206,755
  loss   = mean_valid(lse_i - z_{i,y_i})               ops.py:12 (F.cross_entropy, ignore_index)
           + z_regularization * mean_valid(lse_i^2)    ops.py:13-14, ops.py:756-761
  dZ_ij  = valid_i * (softmax_ij * (1 + 2 z_reg lse_i) - [j == y_i])      ops.py:309-314
  dx     = dZ @ W^T * logit_scale / n_valid            ops.py:317,332
  dW     = x^T @ dZ * logit_scale / n_valid            ops.py:424,443
  z_value        = mean_valid(lse^2)                   ops.py:13
  logit_max      = max over ALL rows, columns of z     ops.py:17
  logit_entropy  = mean_valid(-sum_j p log p)          ops.py:15-16
  logit_norm     = mean over ALL rows of ||z_i||_2     ops.py:17
where "valid" rows are those with y_i != ignore_index and n_valid is their number.
``reference_torch`` casts the logits to float32 (ops.py:11); the oracle keeps float64 throughout.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class OracleResult:
    loss: float
    z_value: float
    logit_max: float
    logit_entropy: float
    logit_norm: float
    dx: np.ndarray | None  # (N, H) float64
    dW: np.ndarray | None  # (H, V) float64
    lse: np.ndarray  # (N,) float64


def _as64(a) -> np.ndarray:
    """numpy view of a numpy array or torch tensor; floating data is widened to float64."""
    if hasattr(a, "detach"):  # torch tensor (any device, any float type incl. bfloat16)
        a = a.detach().to("cpu")
        return a.double().numpy() if a.is_floating_point() else a.numpy()
    a = np.asarray(a)
    return a.astype(np.float64) if a.dtype.kind == "f" else a


def logits64(x, W, logit_scale: float = 1.0) -> np.ndarray:
    """z = logit_scale * (x @ W) in float64 (ops.py:11 without the float32 cast; ops.py:200)."""
    return (_as64(x) @ _as64(W)) * float(logit_scale)


def row_lse(z: np.ndarray) -> np.ndarray:
    """Numerically stable log-sum-exp per row (ops.py:205-206 per tile, ops.py:755 across tiles)."""
    m = z.max(axis=1)
    return m + np.log(np.exp(z - m[:, None]).sum(axis=1))


def forward_backward(x, y, W, ignore_index: int = -100, z_regularization: float = 0.0, logit_scale: float = 1.0,
                     want_grad: bool = True, chunk_rows: int | None = None) -> OracleResult:
    """Loss, the four monitoring values and both gradients, in float64.

    Rows are processed ``chunk_rows`` at a time like the reference's N_chunk loop (ops.py:721); the
    result does not depend on the chunking.
    """
    x = _as64(x)
    W = _as64(W)
    y = np.asarray(_as64(y)).astype(np.int64).reshape(-1)
    x = x.reshape(-1, x.shape[-1])
    N, H = x.shape
    V = W.shape[1]
    assert W.shape[0] == H and y.shape == (N,)
    valid = y != ignore_index
    R = np.float64(valid.sum())  # numpy scalar: 0/0 gives nan instead of raising
    chunk = N if chunk_rows is None else int(chunk_rows)

    sum_nll = sum_lse2 = sum_ent = sum_norm = 0.0
    zmax = -np.inf
    lse_all = np.empty(N)
    dx = np.zeros((N, H)) if want_grad else None
    dW = np.zeros((H, V)) if want_grad else None
    for r0 in range(0, N, chunk):
        sl = slice(r0, min(N, r0 + chunk))
        z = (x[sl] @ W) * float(logit_scale)
        lse = row_lse(z)
        lse_all[sl] = lse
        v = valid[sl]
        yy = np.where(v, y[sl], 0)
        tgt = z[np.arange(z.shape[0]), yy]
        sum_nll += float(((lse - tgt) * v).sum())
        sum_lse2 += float((lse * lse * v).sum())
        logp = z - lse[:, None]
        p = np.exp(logp)
        sum_ent += float(((-(p * logp).sum(axis=1)) * v).sum())
        sum_norm += float(np.sqrt((z * z).sum(axis=1)).sum())
        zmax = max(zmax, float(z.max()))
        if want_grad:
            dz = p * (1.0 + 2.0 * float(z_regularization) * lse)[:, None]
            dz[np.arange(z.shape[0]), yy] -= 1.0
            dz *= v[:, None]
            with np.errstate(invalid="ignore", divide="ignore"):
                dx[sl] = dz @ W.T * (float(logit_scale) / R)
                dW += x[sl].T @ dz * (float(logit_scale) / R)
    with np.errstate(invalid="ignore", divide="ignore"):
        loss = float((np.float64(sum_nll) + float(z_regularization) * sum_lse2) / R)  # R == 0 -> nan, like the reference
        z_value = float(np.float64(sum_lse2) / R)
        ent = float(np.float64(sum_ent) / R)
    return OracleResult(loss, z_value, zmax, ent, sum_norm / N, dx, dW, lse_all)


# ------------------------------------------------------------------------------------------------
# Per-row partial statistics and their combination across vocabulary tiles / shards.
# The reference combines per-V-tile log-sum-exps on the host (ops.py:755); a vocabulary-sharded run
# combines per-rank partials the same way. These closed forms are what the CUDA statistics kernels
# must reproduce.
# ------------------------------------------------------------------------------------------------
def row_partials(z_slab: np.ndarray, y: np.ndarray, vocab_offset: int, ignore_index: int) -> np.ndarray:
    """(6, N) partials of one column slab z[:, offset:offset+Vs], relative to a per-row base b (here b = max_j z;
    any finite base describes the same quantities):
    b, s = sum_j exp(z - b), t = z[i, y_i] if the slab owns column y_i else 0,
    u = sum_j exp(z - b) z, q = sum_j z^2, max_j z."""
    n, vs = z_slab.shape
    m = z_slab.max(axis=1)
    e = np.exp(z_slab - m[:, None])
    s = e.sum(axis=1)
    u = (e * z_slab).sum(axis=1)
    q = (z_slab * z_slab).sum(axis=1)
    yl = y - vocab_offset
    own = (y != ignore_index) & (yl >= 0) & (yl < vs)
    t = np.where(own, z_slab[np.arange(n), np.where(own, yl, 0)], 0.0)
    return np.stack([m, s, t, u, q, m])


def combine_partials(parts: np.ndarray):
    """parts: (G, 6, N) -> (lse, target_logit, entropy, sq_norm, row_max), each (N,).
    B = max_g b_g; S = sum_g s_g e^{b_g - B}; lse = B + log S; entropy = lse - (sum_g u_g e^{b_g - B}) / S."""
    m, s, t, u, q, zmax = (parts[:, k, :] for k in range(6))
    M = m.max(axis=0)
    w = np.exp(m - M[None, :])
    S = (s * w).sum(axis=0)
    lse = M + np.log(S)
    ent = lse - (u * w).sum(axis=0) / S
    return lse, t.sum(axis=0), ent, q.sum(axis=0), zmax.max(axis=0)


# ------------------------------------------------------------------------------------------------
# The reference's torch path as a timed CPU baseline (float32, all host threads).
# ------------------------------------------------------------------------------------------------
def cpu_baseline_step(x, y, W, ignore_index: int = -100, z_regularization: float = 0.0, logit_scale: float = 1.0,
                      chunk_rows: int = 4096):
    """One forward+backward of the path the way the reference states it in torch on the CPU
    (``reference_torch``, ops.py:9-17: F.linear -> float32 logits * scale -> F.cross_entropy + z-reg,
    then autograd), chunked over rows with recomputation-free accumulation like the reference's own
    ground-truth helper ``torch_checkpoint`` (bench_fusions.py:71-83) so that the logits of only one
    chunk are alive. x: (N, H) float32 tensor, W: (H, V) float32 tensor, y: (N,) int64 tensor.
    Returns (loss, dx, dW) as torch tensors.
    """
    import torch
    import torch.nn.functional as F

    N = x.shape[0]
    n_valid = (y != ignore_index).sum().clamp_min(1).to(torch.float32)
    xg = x.detach().requires_grad_(True)
    Wg = W.detach().requires_grad_(True)
    total = torch.zeros((), dtype=torch.float32)
    for r0 in range(0, N, chunk_rows):
        xs = xg[r0:r0 + chunk_rows]
        ys = y[r0:r0 + chunk_rows]
        logits = F.linear(xs, Wg.t()).float() * logit_scale
        part = F.cross_entropy(logits, ys, ignore_index=ignore_index, reduction="sum")
        if z_regularization > 0:
            part = part + z_regularization * logits.logsumexp(dim=-1)[ys != ignore_index].pow(2).sum()
        part = part / n_valid
        part.backward()
        total += part.detach()
    return total, xg.grad, Wg.grad
