"""The CPU oracle against the golden vectors made by the reference's own torch statement of the path
(tests/golden/make_golden.py), plus its internal identities. No GPU needed."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN_CASES, golden_case
from oracle import oracle


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_oracle_matches_reference_golden(golden, name):
    c = golden_case(golden, name)
    r = oracle.forward_backward(c["x"], c["y"], c["W"], c["ignore_index"], c["z_regularization"], c["logit_scale"])
    got = np.array([r.loss, r.z_value, r.logit_max, r.logit_entropy, r.logit_norm])
    # the golden values went through float32 logits (reference ops.py:11): tolerance 2e-6 relative
    np.testing.assert_allclose(got, c["scalars"], rtol=2e-6, atol=1e-6)
    scale = np.abs(c["dx"]).max()
    np.testing.assert_allclose(r.dx, c["dx"], rtol=0, atol=2e-6 * scale + 1e-9)
    scale = np.abs(c["dW_rows"]).max()
    np.testing.assert_allclose(r.dW[::16], c["dW_rows"], rtol=0, atol=2e-6 * scale + 1e-9)
    # sums of float32 gradients: tolerance relative to the mass that was summed (row sums cancel to 0 exactly
    # when z_regularization == 0)
    np.testing.assert_allclose(r.dW.sum(axis=1), c["dW_rowsum"], rtol=0, atol=2e-6 * np.abs(r.dW).sum(axis=1).max())
    np.testing.assert_allclose(r.dW.sum(axis=0), c["dW_colsum"], rtol=0, atol=2e-6 * np.abs(r.dW).sum(axis=0).max())


def _random_case(seed, N=96, H=24, V=80, ignore=-1, frac=0.2):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((N, H))
    W = rng.standard_normal((H, V)) / np.sqrt(H)
    y = rng.integers(0, V, N)
    y[rng.random(N) < frac] = ignore
    return x, y, W


@pytest.mark.parametrize("zreg,scale", [(0.0, 1.0), (1e-2, 0.5), (1e-3, 3.0)])
def test_closed_form_gradients_match_autograd_fp64(zreg, scale):
    x, y, W = _random_case(1)
    r = oracle.forward_backward(x, y, W, -1, zreg, scale)
    xt = torch.tensor(x, requires_grad=True)
    Wt = torch.tensor(W, requires_grad=True)
    yt = torch.tensor(y)
    z = (xt @ Wt) * scale
    loss = torch.nn.functional.cross_entropy(z, yt, ignore_index=-1)
    loss = loss + zreg * torch.logsumexp(z, -1)[yt != -1].pow(2).mean()
    loss.backward()
    assert abs(r.loss - loss.item()) < 1e-12
    np.testing.assert_allclose(r.dx, xt.grad.numpy(), atol=1e-14)
    np.testing.assert_allclose(r.dW, Wt.grad.numpy(), atol=1e-14)


def test_chunking_does_not_change_the_result():
    x, y, W = _random_case(2)
    a = oracle.forward_backward(x, y, W, -1, 1e-3, 0.7)
    b = oracle.forward_backward(x, y, W, -1, 1e-3, 0.7, chunk_rows=32)
    assert abs(a.loss - b.loss) < 1e-13
    np.testing.assert_allclose(a.dW, b.dW, atol=1e-14)
    np.testing.assert_allclose(a.dx, b.dx, atol=1e-14)


@pytest.mark.parametrize("shards", [1, 2, 4, 5])
def test_shard_partials_combine_to_the_full_row_statistics(shards):
    x, y, W = _random_case(3, V=80)
    z = oracle.logits64(x, W, 0.9)
    vs = 80 // shards
    parts = np.stack([oracle.row_partials(z[:, g * vs:(g + 1) * vs], y, g * vs, -1) for g in range(shards)])
    lse, t, ent, q, m = oracle.combine_partials(parts)
    assert parts.shape[1] == 6
    full = oracle.forward_backward(x, y, W, -1, 0.0, 0.9, want_grad=False)
    np.testing.assert_allclose(lse, full.lse, atol=1e-13)
    valid = y != -1
    np.testing.assert_allclose(t[valid], z[np.arange(len(y)), np.where(valid, y, 0)][valid], atol=1e-14)
    assert np.all(t[~valid] == 0)
    assert abs(ent[valid].mean() - full.logit_entropy) < 1e-12
    assert abs(np.sqrt(q).mean() - full.logit_norm) < 1e-12
    assert abs(m.max() - full.logit_max) < 1e-14


def test_no_valid_rows_gives_nan_like_the_reference():
    x, y, W = _random_case(4)
    y[:] = -1
    r = oracle.forward_backward(x, y, W, -1, 0.0, 1.0, want_grad=False)
    assert np.isnan(r.loss)


def test_ignore_index_that_is_a_real_class_id():
    x, y, W = _random_case(5, ignore=7, frac=0.0)
    y[:10] = 7
    r = oracle.forward_backward(x, y, W, 7, 0.0, 1.0)
    assert np.all(r.dx[:10] == 0)
    assert np.isfinite(r.loss)


def test_cpu_baseline_step_agrees_with_oracle():
    x, y, W = _random_case(6, N=64, H=32, V=128)
    r = oracle.forward_backward(x, y, W, -1, 1e-3, 0.8)
    loss, dx, dW = oracle.cpu_baseline_step(torch.tensor(x, dtype=torch.float32), torch.tensor(y),
                                           torch.tensor(W, dtype=torch.float32), -1, 1e-3, 0.8, chunk_rows=16)
    assert abs(loss.item() - r.loss) < 1e-5
    np.testing.assert_allclose(dx.numpy(), r.dx, atol=1e-6)
    np.testing.assert_allclose(dW.numpy(), r.dW, atol=1e-6)
