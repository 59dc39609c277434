"""Full-size configurations (the default 16384 x 2048 x 131072 point in fp16 and bf16, the 65536 x 4096 x 131072
LM-head case and the 131072 x 8192 x 262144 large-vocabulary case): the float64 oracle cannot redo 26 to 1700 TFLOP
in seconds, so parity is checked through size-independent properties plus float64 checks of row and column subsets:

* dx of row i depends only on row i of x and on W -> the oracle recomputes a random subset of rows exactly;
* dW[:, j] depends on column j of W, on x and on every row's log-sum-exp -> 64 columns are recomputed in float64;
* <dx, x> == <dW, W> (both equal sum dZ * z / n_valid): ties the rest of dW to the verified dx;
* row sums of dW vanish when z_regularization == 0 (softmax - onehot sums to 0 over the vocabulary);
* results do not depend on N_chunk_size, are bitwise reproducible and are linear in grad_output."""
import numpy as np
import pytest
import torch

from gpu_util import cosine
from linear_cross_entropy_loss_b200 import linear_cross_entropy, synthetic
from oracle import oracle

pytestmark = pytest.mark.gpu


def run(cfg, x, y, W, chunk=None, mon=None):
    xd = x.detach().requires_grad_(True)
    Wd = W.detach().requires_grad_(True)
    out = linear_cross_entropy(xd, y, Wd, cfg.ignore_index, cfg.z_regularization, cfg.logit_scale,
                               cfg.N_chunk_size if chunk is None else chunk, cfg.monitoring if mon is None else mon)
    out[0].backward()
    torch.cuda.synchronize()
    return [v.item() for v in out], xd.grad, Wd.grad


def oracle_rows(cfg, x, y, W, rows):
    """float64 log-sum-exp and dx (still to be divided by n_valid) for a subset of rows. The products run on the GPU
    in float64, one block of vocabulary columns at a time, so that W is never widened whole; the log-sum-exp is the
    CPU oracle's."""
    xs = x[rows].double()
    ys = y[rows].cpu().numpy()
    V = W.shape[1]
    z = np.empty((len(rows), V))
    for v0 in range(0, V, 16384):
        z[:, v0:v0 + 16384] = (xs @ W[:, v0:v0 + 16384].double()).cpu().numpy()
    z *= cfg.logit_scale
    lse = oracle.row_lse(z)
    valid = ys != cfg.ignore_index
    dz = np.exp(z - lse[:, None]) * (1 + 2 * cfg.z_regularization * lse)[:, None]
    dz[np.arange(len(rows)), np.where(valid, ys, 0)] -= 1
    dz *= valid[:, None]
    dx = torch.zeros((len(rows), x.shape[1]), dtype=torch.float64, device=x.device)
    for v0 in range(0, V, 16384):
        dx += torch.from_numpy(dz[:, v0:v0 + 16384]).to(x.device) @ W[:, v0:v0 + 16384].double().T
    return lse, dx.cpu().numpy() * cfg.logit_scale


def dW_columns64(cfg, x, y, W, lse_all, cols, n_valid):
    """float64 dW[:, cols] = x^T dZ[:, cols] * logit_scale / n_valid (reference ops.py:424, 443) with
    dZ = valid * (exp(z - lse)(1 + 2 z_reg lse) - onehot) (ops.py:309-314). lse_all: float64 log-sum-exp of every row."""
    Wc = W[:, cols].double()
    out = torch.zeros((x.shape[1], len(cols)), dtype=torch.float64, device=x.device)
    for r0 in range(0, cfg.N, 8192):
        xb = x[r0:r0 + 8192].double()
        yb = y[r0:r0 + 8192]
        l = lse_all[r0:r0 + 8192]
        z = (xb @ Wc) * cfg.logit_scale
        dz = torch.exp(z - l[:, None]) * (1 + 2 * cfg.z_regularization * l)[:, None]
        dz -= (yb[:, None] == cols[None, :]).double()
        dz *= (yb != cfg.ignore_index).double()[:, None]
        out += xb.T @ dz
    return out * (cfg.logit_scale / n_valid)


# name, oracle rows for dx, whether the two extra full passes (chunk-size invariance) run
FULL_SIZE_CASES = [("c2_default_fp16", 48, True), ("c3_default_bf16_all", 48, True), ("c4_llama8b_bf16", 24, True),
                   ("c5_large_vocab_bf16", 16, False)]


@pytest.mark.parametrize("name,n_rows,invariance", FULL_SIZE_CASES, ids=[c[0] for c in FULL_SIZE_CASES])
def test_full_size_properties(name, n_rows, invariance):
    cfg = synthetic.CONFIGS[name]
    need = 6 * (cfg.N * cfg.H + cfg.H * cfg.V) * 2 + 3 * cfg.N_chunk_size * cfg.V * 4 + 3 * cfg.H * cfg.V * 4
    if torch.cuda.mem_get_info()[0] < need:
        pytest.skip(f"{name} needs about {need >> 30} GiB of free device memory")
    x, y, W = synthetic.make_inputs(cfg, device="cuda")
    got, dx, dW = run(cfg, x, y, W)
    n_valid = int((y != cfg.ignore_index).sum())
    assert np.isfinite(got[0])

    # (1) oracle on random rows: per-row dx and the log-sum-exp
    rows = torch.randperm(cfg.N, generator=torch.Generator().manual_seed(1))[:n_rows].cuda()
    lse_rows, dx_rows = oracle_rows(cfg, x, y, W, rows)
    dx_rows /= n_valid
    got_rows = dx[rows].double().cpu().numpy()
    assert cosine(got_rows, dx_rows) > 0.9999, cosine(got_rows, dx_rows)

    # (2) loss, z_value and every row's log-sum-exp recomputed by torch in float32 products / float64 reductions
    total = 0.0
    tot_lse2 = 0.0
    lse_all = torch.empty(cfg.N, dtype=torch.float64, device="cuda")
    Wf = W.float()
    for r0 in range(0, cfg.N, 1024):
        z = (x[r0:r0 + 1024].float() @ Wf) * cfg.logit_scale
        l = torch.logsumexp(z.double(), dim=-1)
        lse_all[r0:r0 + 1024] = l
        yy = y[r0:r0 + 1024]
        v = yy != cfg.ignore_index
        t = z.gather(1, torch.where(v, yy, torch.zeros_like(yy))[:, None])[:, 0].double()
        total += ((l - t) * v).sum().item()
        tot_lse2 += (l * l * v).sum().item()
        del z
    del Wf
    want = (total + cfg.z_regularization * tot_lse2) / n_valid
    assert abs(got[0] - want) <= 1e-4 * abs(want), (got[0], want)
    assert abs(got[1] - tot_lse2 / n_valid) <= 1e-4 * tot_lse2 / n_valid
    assert np.allclose(lse_all[rows].cpu().numpy(), lse_rows, rtol=0, atol=2e-5)  # ties the fp32 pass to the oracle

    # (3) dW, element by element, on 64 columns (the most frequent labels among them) against float64
    g = torch.Generator().manual_seed(2)
    cols = torch.cat([torch.arange(4), torch.randperm(cfg.V - 4, generator=g)[:60] + 4]).cuda()
    want_cols = dW_columns64(cfg, x, y, W, lse_all, cols, n_valid).cpu().numpy()
    got_cols = dW[:, cols].double().cpu().numpy()
    rel = np.linalg.norm(got_cols - want_cols) / np.linalg.norm(want_cols)
    dtype_tol = {torch.float16: 2e-3 + 2.5e-4, torch.bfloat16: 6e-3 + 2e-3}[cfg.dtype]
    assert cosine(got_cols, want_cols) > 0.9999 and rel <= dtype_tol, (cosine(got_cols, want_cols), rel)

    # (4) trace identity <dx, x> == <dW, W> (both equal sum dZ * z / n_valid): ties ALL of dW to the verified dx
    a = sum((dx[r:r + 8192].double() * x[r:r + 8192].double()).sum().item() for r in range(0, cfg.N, 8192))
    b = sum((dW[h:h + 256].double() * W[h:h + 256].double()).sum().item() for h in range(0, cfg.H, 256))
    scale_ab = sum((dx[r:r + 8192].double().abs() * x[r:r + 8192].double().abs()).sum().item()
                   for r in range(0, cfg.N, 8192))
    assert abs(a - b) <= 2e-3 * scale_ab, (a, b, scale_ab)

    # (5) row sums of dW vanish without z-regularisation (softmax - onehot sums to 0 over the vocabulary)
    if cfg.z_regularization == 0:
        rowsum = torch.stack([dW[h:h + 256].double().sum(dim=1) for h in range(0, cfg.H, 256)]).flatten()
        mass = max(dW[h:h + 256].double().abs().sum(dim=1).max().item() for h in range(0, cfg.H, 256))
        assert rowsum.abs().max().item() <= 3e-3 * mass

    # (6) bitwise reproducibility (no atomics anywhere)
    got3, dx3, dW3 = run(cfg, x, y, W)
    assert got3 == got and torch.equal(dx3, dx) and torch.equal(dW3, dW)
    del dx3, dW3

    # (7) chunk-size invariance (half the rows per chunk)
    if invariance:
        got2, dx2, dW2 = run(cfg, x, y, W, chunk=cfg.N_chunk_size // 2)
        assert abs(got2[0] - got[0]) <= 1e-6 * abs(got[0])
        assert cosine(dx2[:2048].double().cpu().numpy(), dx[:2048].double().cpu().numpy()) > 0.999999
        dots = [(dW2[h:h + 256].double() * dW[h:h + 256].double()).sum().item() for h in range(0, cfg.H, 256)]
        n2 = [(dW2[h:h + 256].double() ** 2).sum().item() for h in range(0, cfg.H, 256)]
        n1 = [(dW[h:h + 256].double() ** 2).sum().item() for h in range(0, cfg.H, 256)]
        assert sum(dots) / (sum(n1) ** 0.5 * sum(n2) ** 0.5) > 0.99999


def test_peak_extra_memory_stays_below_one_fp32_chunk_of_logits():
    cfg = synthetic.CONFIGS["headline_bf16"]
    x, y, W = synthetic.make_inputs(cfg, device="cuda")
    x.requires_grad_(True)
    W.requires_grad_(True)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    before = torch.cuda.memory_allocated()
    loss = linear_cross_entropy(x, y, W, cfg.ignore_index, 0.0, 1.0, cfg.N_chunk_size, False)[0]
    loss.backward()
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - before
    budget = cfg.N_chunk_size * cfg.V * 4               # one fp32 chunk of logits: the reference's stated peak
    # Everything the call allocates, gradients included (the reference's own figure for bf16 is 3.39 GiB, BASELINE:
    # bench-mem). Alive at the peak: workspace (slab N_chunk x V x 2 bytes, statistics, split-K partials of dx) + dW
    # and its residual (H x V x 2 bytes each: the sum over the chunks is carried as a pair of bf16 arrays) + dx.
    expected = cfg.N_chunk_size * cfg.V * 2 + cfg.H * cfg.V * 4 + cfg.N * cfg.H * 2
    assert peak <= expected + (224 << 20), (peak, expected)
    assert peak <= 1.13 * budget, (peak, budget)        # 2.24 GiB against the 2 GiB figure, all inclusive
    excl = peak - cfg.H * cfg.V * 4 - cfg.N * cfg.H * 2  # without dW + residual and dx (the reference keeps fp32 dW, dx)
    assert excl <= 0.6 * budget, (excl, budget)


def test_slab_modes_agree_at_the_default_point(monkeypatch):
    """bf16 at full size: one base per row and per-tile slabs are two routes to the same dZ."""
    cfg = synthetic.CONFIGS["headline_bf16"]
    x, y, W = synthetic.make_inputs(cfg, device="cuda")
    monkeypatch.setenv("LCE_SLAB_MODE", "row")
    got_r, dx_r, dW_r = run(cfg, x, y, W)
    monkeypatch.setenv("LCE_SLAB_MODE", "tile")
    got_t, dx_t, dW_t = run(cfg, x, y, W)
    assert abs(got_r[0] - got_t[0]) <= 2e-6 * abs(got_r[0]), (got_r[0], got_t[0])
    cos = torch.nn.functional.cosine_similarity
    assert cos(dx_r.double().flatten(), dx_t.double().flatten(), dim=0).item() > 0.99999
    assert cos(dW_r.double().flatten(), dW_t.double().flatten(), dim=0).item() > 0.99999
