"""Parity of the CUDA path (called through the C ABI via the Python surface) against the float64 oracle and the
golden vectors of the reference's torch statement, at sizes the oracle handles in seconds."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN_CASES, golden_case
from gpu_util import TOL, check_against_oracle, cosine, random_problem, rel_err, run_gpu
from linear_cross_entropy_loss_b200 import LinearCrossEntropyLoss, linear_cross_entropy, synthetic
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", GOLDEN_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_golden_vectors_of_the_reference(golden, name, dtype):
    c = golden_case(golden, name)
    x = torch.tensor(c["x"]).to(dtype)      # multiples of 1/64 and 1/512: exact in every dtype
    W = torch.tensor(c["W"]).to(dtype)
    y = torch.tensor(c["y"])
    got, dx, dW = run_gpu(x, y, W, c["ignore_index"], c["z_regularization"], c["logit_scale"], chunk=128)
    tol = TOL[dtype]
    want = c["scalars"]
    assert abs(got[0] - want[0]) <= tol["loss"] * abs(want[0])
    assert abs(got[1] - want[1]) <= 2 * tol["loss"] * abs(want[1])
    assert abs(got[2] - want[2]) <= 2e-3 * abs(want[2])
    assert abs(got[3] - want[3]) <= 1e-3 * abs(want[3])
    assert abs(got[4] - want[4]) <= 1e-3 * abs(want[4])
    dxn, dWn = dx.double().cpu().numpy(), dW.double().cpu().numpy()
    assert cosine(dxn, c["dx"]) >= tol["cos"]
    assert cosine(dWn[::16], c["dW_rows"]) >= tol["cos"]
    mass = np.abs(dWn).sum(axis=0).max()
    assert np.abs(dWn.sum(axis=0) - c["dW_colsum"]).max() <= 4e-3 * mass


def test_config_c1_small_fp32_case():
    cfg = synthetic.CONFIGS["c1_small_fp32"]
    x, y, W = synthetic.make_inputs(cfg, device="cpu")
    check_against_oracle(x, y, W, cfg.dtype, cfg.ignore_index, cfg.z_regularization, cfg.logit_scale, cfg.N_chunk_size)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_reduced_default_configs_with_all_options(dtype):
    # C2 / C3 options at a size the oracle finishes in seconds
    x, y, W = random_problem(2048, 512, 8192, dtype, seed=3, ignore=-1, frac=0.02)
    check_against_oracle(x, y, W, dtype, ignore=-1, zreg=1e-4, scale=0.5, chunk=512)
    check_against_oracle(x, y, W, dtype, ignore=-1, zreg=0.0, scale=1.0, chunk=1024, monitoring=False)


@pytest.mark.parametrize("H,N,V", [(512, 1024, 4096), (1024, 512, 4096), (256, 2048, 16384), (2048, 256, 2048)])
def test_accuracy_sweep_bf16(H, N, V):
    x, y, W = random_problem(N, H, V, torch.bfloat16, seed=H + N)
    check_against_oracle(x, y, W, torch.bfloat16, ignore=-1, zreg=1e-4, scale=0.5, chunk=512)


def test_low_loss_recipe_of_the_reference_benchmarks():
    # the reference's accuracy benchmark plants the label direction into x (bench_fusions.py:480-486)
    g = torch.Generator().manual_seed(0)
    N, H, V = 1024, 256, 4096
    A = torch.randn(V, H, generator=g)
    y = torch.randint(0, V, (N,), generator=g)
    x = (0.1 * A[y] + torch.randn(N, H, generator=g)).half()
    W = A.t().contiguous().half()
    got, dxn, dWn, ref = check_against_oracle(x, y, W, torch.float16, chunk=256)
    # in the reference's own units (torch.dist): the published fp16 figures are 7e-5 (loss) and 1.4e-4 (grads)
    assert abs(got[0] - ref.loss) < 1e-4
    assert 0.5 * (np.linalg.norm(dxn - ref.dx) + np.linalg.norm(dWn - ref.dW)) < 5e-4


@pytest.mark.parametrize("chunk,N", [(128, 384), (256, 640), (512, 512), (4096, 256)])
def test_ragged_last_chunk_and_single_chunk(chunk, N):
    x, y, W = random_problem(N, 256, 1024, torch.bfloat16, seed=N)
    check_against_oracle(x, y, W, torch.bfloat16, ignore=-1, chunk=chunk)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("N,H,V,chunk", [
    (200, 264, 1000, 128),     # everything ragged; bf16 dW rows are only 16-byte aligned -> element-wise epilogue
    (1000, 768, 50264, 512),   # GPT-2 vocabulary padded to a multiple of 8, ragged last chunk
    (72, 64, 1056, 4096),      # fewer rows than one tile, single chunk, aligned rows with a partial last tile
    (640, 320, 151936 // 8, 256),
])
def test_shapes_that_are_not_multiples_of_the_tiles(dtype, N, H, V, chunk):
    x, y, W = random_problem(N, H, V, torch.bfloat16, seed=N + V)
    x, W = x.to(dtype), W.to(dtype)            # bf16-representable values: exact TF32 operands too
    y[-1] = V - 1                              # a label in the last, partial vocabulary tile
    check_against_oracle(x, y, W, dtype, ignore=-1, zreg=1e-4, scale=0.75, chunk=chunk)


@pytest.mark.parametrize("dtype,N,H,V,chunk", [(torch.bfloat16, 300, 250, 2048, 256), (torch.float16, 384, 100, 1001, 128),
                                                (torch.float32, 256, 65, 777, 128)])
def test_hidden_sizes_that_are_not_multiples_of_8(dtype, N, H, V, chunk):
    """Rows of x must start on 16-byte boundaries for TMA: other hidden sizes run on copies padded with zero columns
    of x and zero rows of W, and the gradients come back with the shapes of the inputs."""
    x, y, W = random_problem(N, H, V, torch.bfloat16, seed=H)
    x, W = x.to(dtype), W.to(dtype)
    got, dx, dW, ref = check_against_oracle(x, y, W, dtype, ignore=-1, zreg=1e-4, scale=0.75, chunk=chunk)
    assert dx.shape == (N, H) and dW.shape == (H, V)


@pytest.mark.parametrize("dtype,N,H,V,chunk", [(torch.bfloat16, 300, 264, 1001, 256), (torch.float16, 512, 256, 4099, 256),
                                                (torch.float32, 200, 64, 777, 128), (torch.bfloat16, 130, 128, 3, 128),
                                                (torch.bfloat16, 1024, 256, 50257 // 8, 512)])
def test_vocabulary_sizes_that_are_not_multiples_of_8(dtype, N, H, V, chunk):
    """Tokenizer vocabularies (50257, 32001, ...) are odd: W and dW then live in buffers whose rows are padded to
    16 bytes, the vocabulary itself is not padded (columns past V are masked in the kernels)."""
    x, y, W = random_problem(N, H, V, dtype, seed=V)
    got, dxn, dWn, ref = check_against_oracle(x, y, W, dtype, ignore=-1, zreg=1e-4, scale=0.5, chunk=chunk)
    assert dWn.shape == (H, V)
    # grad_output != 1 scales through the padded rows as well
    xd = x.cuda().requires_grad_(True)
    Wd = W.cuda().requires_grad_(True)
    (linear_cross_entropy(xd, y.cuda(), Wd, -1, 1e-4, 0.5, chunk)[0] * 3.0).backward()
    assert Wd.grad.shape == (H, V)
    assert cosine(Wd.grad.double().cpu().numpy(), 3.0 * ref.dW) > TOL[dtype]["cos"]


def test_labels_on_tile_boundaries_and_repeated_labels():
    x, y, W = random_problem(256, 256, 1024, torch.float16, seed=5, frac=0.0)
    y[:8] = torch.tensor([0, 255, 256, 511, 512, 767, 768, 1023])
    y[8:64] = 300
    check_against_oracle(x, y, W, torch.float16)


def test_ignore_index_that_is_a_class_id():
    x, y, W = random_problem(256, 256, 512, torch.bfloat16, seed=6, frac=0.0)
    y[:100] = 5
    got, dxn, dWn, ref = check_against_oracle(x, y, W, torch.bfloat16, ignore=5)
    assert np.all(dxn[:100] == 0)


def test_all_rows_ignored_gives_nan_loss_like_the_reference():
    x, y, W = random_problem(128, 256, 512, torch.bfloat16, seed=7, frac=0.0)
    y[:] = -100
    got, dx, dW = run_gpu(x, y, W)
    assert np.isnan(got[0])


def test_one_valid_row():
    x, y, W = random_problem(128, 256, 512, torch.float16, seed=8, frac=0.0)
    y[:] = -100
    y[77] = 3
    got, dxn, dWn, ref = check_against_oracle(x, y, W, torch.float16)
    assert np.count_nonzero(np.abs(dxn).sum(axis=1)) == 1


def test_peaked_softmax_large_logit_scale():
    x, y, W = random_problem(256, 256, 1024, torch.bfloat16, seed=9)
    check_against_oracle(x, y, W, torch.bfloat16, ignore=-1, scale=16.0, zreg=1e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_conditional_rerun_when_logits_leave_the_reference_range(dtype):
    # bf16 / fp32 slabs hold exp(z - 0) first; rows whose max logit is beyond +-60 make the chunk run again with
    # reference = row max. scale = 32 puts the row maxima near 100 in the first chunk's rows only.
    x, y, W = random_problem(512, 256, 1024, torch.bfloat16, seed=21)
    x, W = x.to(dtype), W.to(dtype)     # bf16-representable values: exact as TF32 operands too
    x[256:] *= 0.25                     # second chunk stays inside the range: no re-run there
    check_against_oracle(x, y, W, dtype, ignore=-1, scale=32.0, zreg=1e-4, chunk=256)


def test_wide_logits_with_probe_reference_and_outlier_column():
    # V > 1024: the first forward takes its per-row reference from a probe of the first 512 columns. Logits of
    # spread ~40 stay inside the window; a column far above everything the probe saw forces the re-run.
    x, y, W = random_problem(256, 256, 4096, torch.bfloat16, seed=23)
    check_against_oracle(x, y, W, torch.bfloat16, ignore=-1, scale=40.0, chunk=128)
    x2, W2 = x.clone(), W.clone()
    x2[:128, 0] = 8.0
    W2[0, 3000] = 4.0                     # rows 0..127 get a logit near 8 * 4 * 8 = 256 in column 3000
    got, dxn, dWn, ref = check_against_oracle(x2, y, W2, torch.bfloat16, ignore=-1, scale=8.0, chunk=128)
    assert ref.logit_max > 200


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rerun_touches_only_the_row_groups_that_need_it(dtype):
    # 1024-row chunks = four 256-row groups; only rows 300..309 (group 1) and 1900 (second chunk, group 3) carry
    # a logit far above what the probe of the first 512 columns sees
    x, y, W = random_problem(2048, 256, 4096, torch.bfloat16, seed=24)
    x[300:310, 1] = 16.0
    x[1900, 1] = 16.0
    W[1, 2500] = 8.0
    x, W = x.to(dtype), W.to(dtype)
    got, dxn, dWn, ref = check_against_oracle(x, y, W, dtype, ignore=-1, scale=2.0, zreg=1e-4, chunk=1024)
    assert ref.logit_max > 200


def test_conditional_rerun_on_the_underflow_side():
    g = torch.Generator().manual_seed(22)
    x = (torch.rand(256, 256, generator=g) + 0.5).bfloat16()
    W = (-(torch.rand(256, 512, generator=g)) * 0.8).bfloat16()      # every logit is near -100
    y = torch.randint(0, 512, (256,), generator=g)
    got, dxn, dWn, ref = check_against_oracle(x, y, W, torch.bfloat16, chunk=128)
    assert ref.logit_max < -60


def test_strided_rows_of_x_and_w_are_read_in_place():
    x, y, W = random_problem(256, 512, 1024, torch.float16, seed=10)
    xd = x.cuda()[:, :256]            # row stride 512, 256 columns used
    Wd = W.cuda()[:256, :512]         # row stride 1024
    xd.requires_grad_(True)
    Wd.requires_grad_(True)
    out = linear_cross_entropy(xd, (y % 512).cuda(), Wd, -1)
    out[0].backward()
    ref = oracle.forward_backward(x[:, :256], y % 512, W[:256, :512], -1)
    assert abs(out[0].item() - ref.loss) < 2e-5 * ref.loss
    assert cosine(xd.grad.double().cpu().numpy(), ref.dx) > 0.999999


def test_grad_output_factor_and_dtypes():
    x, y, W = random_problem(256, 256, 512, torch.bfloat16, seed=11)
    _, dx1, dW1 = run_gpu(x, y, W, -1)
    _, dx3, dW3 = run_gpu(x, y, W, -1, grad_scale=3.0)
    assert dx1.dtype == torch.bfloat16 and dW1.dtype == torch.bfloat16
    assert rel_err(dx3.double().cpu().numpy(), 3 * dx1.double().cpu().numpy()) < 4e-3
    assert rel_err(dW3.double().cpu().numpy(), 3 * dW1.double().cpu().numpy()) < 4e-3


def test_forward_only_skips_the_gradient_kernels():
    from linear_cross_entropy_loss_b200 import _native
    x, y, W = random_problem(256, 256, 512, torch.bfloat16, seed=12)
    xd, yd, Wd = x.cuda(), y.cuda(), W.cuda()
    before = _native.launch_count()
    out = linear_cross_entropy(xd, yd, Wd, -1)
    fwd_only = _native.launch_count() - before
    torch.cuda.synchronize()
    ref = oracle.forward_backward(x, y, W, -1, want_grad=False)
    assert abs(out[0].item() - ref.loss) < 2e-5 * ref.loss
    before = _native.launch_count()
    out = linear_cross_entropy(xd.requires_grad_(True), yd, Wd, -1)
    assert _native.launch_count() - before > fwd_only


def test_frozen_head_or_frozen_features_skip_one_contraction():
    from linear_cross_entropy_loss_b200 import _native

    x, y, W = random_problem(512, 256, 2048, torch.bfloat16, seed=41)
    ref = oracle.forward_backward(x, y, W, -1)
    xd = x.cuda().requires_grad_(True)
    before = _native.launch_count()
    linear_cross_entropy(xd, y.cuda(), W.cuda(), -1, 0.0, 1.0, 256)[0].backward()
    only_dx = _native.launch_count() - before
    assert cosine(xd.grad.double().cpu().numpy(), ref.dx) > TOL[torch.bfloat16]["cos"]
    Wd = W.cuda().requires_grad_(True)
    before = _native.launch_count()
    linear_cross_entropy(x.cuda(), y.cuda(), Wd, -1, 0.0, 1.0, 256)[0].backward()
    only_dw = _native.launch_count() - before
    assert cosine(Wd.grad.double().cpu().numpy(), ref.dW) > TOL[torch.bfloat16]["cos"]
    xd2 = x.cuda().requires_grad_(True)
    before = _native.launch_count()
    linear_cross_entropy(xd2, y.cuda(), Wd, -1, 0.0, 1.0, 256)[0].backward()
    both = _native.launch_count() - before
    assert only_dx < both and only_dw < both


def test_module_forward_backward_and_metrics():
    torch.manual_seed(0)
    m = LinearCrossEntropyLoss(512, 4096, ignore_index=-1, logit_scale=0.5, z_regularization=1e-4,
                               N_chunk_size=512).cuda().to(torch.bfloat16)
    m.monitoring = True
    x, y, _ = random_problem(1024, 512, 4096, torch.bfloat16, seed=13)
    xd = x.cuda().view(2, 512, 512).requires_grad_(True)
    loss = m(xd, y.cuda().view(2, 512))
    loss.backward()
    ref = oracle.forward_backward(x, y, m.weight, -1, 1e-4, 0.5)
    assert abs(loss.item() - ref.loss) < 2e-5 * ref.loss
    assert set(m.latest_metrics) == {"logit_norm", "logit_max", "logit_entropy", "z_value"}
    assert abs(m.latest_metrics["logit_entropy"].item() - ref.logit_entropy) < 1e-3 * ref.logit_entropy
    assert xd.grad.shape == (2, 512, 512)
    assert cosine(m.weight.grad.double().cpu().numpy(), ref.dW) > 0.99999


def test_autocast_casts_inputs_to_fp16_like_the_reference():
    x, y, W = random_problem(256, 256, 512, torch.float32, seed=14)
    xd = x.cuda().requires_grad_(True)
    Wd = W.cuda().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = linear_cross_entropy(xd, y.cuda(), Wd, -1)[0]
    loss.backward()
    assert xd.grad.dtype == torch.float32 and Wd.grad.dtype == torch.float32
    ref = oracle.forward_backward(x.half(), y, W.half(), -1)
    assert abs(loss.item() - ref.loss) < 2e-5 * ref.loss
    assert cosine(xd.grad.double().cpu().numpy(), ref.dx) > 0.999999


def test_autocast_policy_follow_uses_the_autocast_dtype():
    import linear_cross_entropy_loss_b200 as pkg

    x, y, W = random_problem(256, 256, 512, torch.float32, seed=15)
    xd = x.cuda().requires_grad_(True)
    Wd = W.cuda().requires_grad_(True)
    pkg.set_autocast_policy("follow")
    try:
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = linear_cross_entropy(xd, y.cuda(), Wd, -1)[0]
        loss.backward()
    finally:
        pkg.set_autocast_policy("reference")
    assert xd.grad.dtype == torch.float32 and Wd.grad.dtype == torch.float32
    ref = oracle.forward_backward(x.bfloat16(), y, W.bfloat16(), -1)  # bf16-rounded inputs, not fp16-rounded ones
    assert abs(loss.item() - ref.loss) < 2e-5 * ref.loss
    assert cosine(xd.grad.double().cpu().numpy(), ref.dx) > 0.99999
    ref16 = oracle.forward_backward(x.half(), y, W.half(), -1)
    assert abs(loss.item() - ref16.loss) > abs(loss.item() - ref.loss)


def test_traced_by_torch_compile_without_a_graph_break():
    """The pass is registered as one torch.library operator, so a compiled model contains it as a single node."""
    torch.manual_seed(0)
    head = LinearCrossEntropyLoss(256, 1024, ignore_index=-1, N_chunk_size=256).cuda().bfloat16()
    h = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = torch.randint(0, 1024, (512,), device="cuda")
    eager = head(h, y)
    eager.backward()
    g_h, g_w = h.grad.clone(), head.weight.grad.clone()
    h.grad = head.weight.grad = None
    compiled = torch.compile(lambda a, b: head(torch.tanh(a) + a, b) * 3.0, backend="aot_eager", fullgraph=True)
    plain = head(torch.tanh(h) + h, y) * 3.0
    plain.backward()
    want_h, want_w = h.grad.clone(), head.weight.grad.clone()
    h.grad = head.weight.grad = None
    out = compiled(h, y)
    out.backward()
    assert abs(out.item() - plain.item()) < 1e-6 * abs(plain.item())
    assert torch.allclose(h.grad.float(), want_h.float(), rtol=2e-2, atol=1e-6)
    assert torch.allclose(head.weight.grad.float(), want_w.float(), rtol=2e-2, atol=1e-6)
    assert g_h is not None and g_w is not None


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_per_tile_slab_mode_for_bf16_and_fp32(dtype, monkeypatch):
    """LCE_SLAB_PER_TILE (exp(z - tile max) + one in-place slab pass) gives the same results as the default
    one-base-per-row mode, including sub-chunks on two streams, ragged shapes, and logits far outside the window
    of the default mode (where it never recomputes)."""
    monkeypatch.setenv("LCE_SLAB_MODE", "tile")
    x, y, W = random_problem(2048, 256, 2048, dtype, seed=31)
    check_against_oracle(x, y, W, dtype, ignore=-1, zreg=1e-4, scale=0.5, chunk=1024)        # two sub-chunks per chunk
    x, y, W = random_problem(600, 264, 1000, dtype, seed=32)
    check_against_oracle(x, y, W, dtype, ignore=-1, chunk=256)                               # ragged everything
    x, y, W = random_problem(512, 256, 4096, torch.bfloat16, seed=33)
    check_against_oracle(x.to(dtype), y, W.to(dtype), dtype, ignore=-1, scale=64.0, chunk=256)  # logit spread ~ 64


def test_slab_mode_policy_switches_after_passes_that_recompute(monkeypatch):
    """auto: a shape whose passes recompute most row groups moves to the per-tile mode once the counters of a
    finished pass have arrived (polled, never waited for), and narrow logits of the same shape stay in the default
    mode. Results are right in either mode."""
    from linear_cross_entropy_loss_b200 import _native, ops

    monkeypatch.delenv("LCE_SLAB_MODE", raising=False)
    monkeypatch.setattr(ops.SlabModePolicy, "small_slab_elems", 0)  # small chunks would always use per-tile slabs
    policy = ops.slab_mode_policy
    policy.history.clear()
    x, y, W = random_problem(1024, 256, 4096, torch.bfloat16, seed=34)
    key = (torch.cuda.current_device(), torch.bfloat16, 256, 4096, 512, 1)
    # wide logits (spread ~ 100): every row group leaves the window
    check_against_oracle(x, y, W, torch.bfloat16, ignore=-1, scale=100.0, chunk=512)
    torch.cuda.synchronize()
    assert policy.choose(key, torch.bfloat16) == _native.SLAB_PER_TILE
    assert policy.history[key]["fraction"] > 0.9
    check_against_oracle(x, y, W, torch.bfloat16, ignore=-1, scale=100.0, chunk=512)    # this one ran per tile
    # another shape with LM-like logits: stays in the default mode
    x2, y2, W2 = random_problem(1024, 256, 2048, torch.bfloat16, seed=35)
    key2 = (torch.cuda.current_device(), torch.bfloat16, 256, 2048, 512, 1)
    check_against_oracle(x2, y2, W2, torch.bfloat16, ignore=-1, chunk=512)
    torch.cuda.synchronize()
    assert policy.choose(key2, torch.bfloat16) == _native.SLAB_DEFAULT
    assert policy.history[key2]["fraction"] == 0.0
    policy.history.clear()


@pytest.mark.parametrize("seed", range(12))
def test_randomised_shapes_options_and_modes(seed, monkeypatch):
    """Seeded random draws of shape, chunking, options, dtype and slab mode against the oracle."""
    rng = np.random.default_rng(1000 + seed)
    dtype = [torch.bfloat16, torch.float16, torch.float32][seed % 3]
    monkeypatch.setenv("LCE_SLAB_MODE", ["row", "tile", "auto"][(seed // 3) % 3])
    N = int(rng.integers(1, 1400))
    H = 8 * int(rng.integers(1, 80))
    V = 8 * int(rng.integers(1, 700))
    chunk = int(rng.choice([128, 200, 256, 512, 1024, 4096]))
    scale = float(rng.choice([0.25, 1.0, 3.0]))
    zreg = float(rng.choice([0.0, 1e-4, 1e-2]))
    ignore = int(rng.choice([-100, -1, 5]))
    x, y, W = random_problem(N, H, V, dtype, seed=2000 + seed, ignore=ignore, frac=float(rng.choice([0.0, 0.1, 0.6])))
    y[0] = (5 % V) if ignore != 5 else 6 % V  # at least one valid row
    # The tensor core truncates fp32 operands to TF32 (it does not round them), which shrinks every logit by up to
    # 2^-10 relative: a bias of the loss that grows with the logit scale (measured 5e-4 at scale 3).
    loss_tol = 1e-3 if dtype == torch.float32 else None
    check_against_oracle(x, y, W, dtype, ignore=ignore, zreg=zreg, scale=scale, chunk=chunk,
                         monitoring=bool(seed % 2), loss_tol=loss_tol)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_half_chunks_on_two_streams_at_a_small_size(monkeypatch, dtype):
    """Per-tile slabs run a chunk as two halves, the slab pass of one half on a second stream under the contractions of
    the other. The library only does that from 2^25 slab elements and 8192 rows per chunk on; here both limits are lifted so that
    the two-stream path is checked against the oracle at a size the oracle can do, and against the one-stream pass."""
    from linear_cross_entropy_loss_b200 import ops
    monkeypatch.setenv("LCE_SLAB_MODE", "tile")
    x, y, W = random_problem(2048, 256, 4096, dtype, seed=31)
    whole = run_gpu(x, y, W, -1, 1e-4, 0.5, 1024, True)
    monkeypatch.setattr(ops, "MIN_SPLIT_ELEMS", 0)
    monkeypatch.setattr(ops, "MIN_HALF_ROWS", 512)
    check_against_oracle(x, y, W, dtype, ignore=-1, zreg=1e-4, scale=0.5, chunk=1024)
    halves = run_gpu(x, y, W, -1, 1e-4, 0.5, 1024, True)
    assert abs(halves[0][0] - whole[0][0]) <= 1e-6 * abs(whole[0][0])
    assert cosine(halves[1].double().cpu().numpy(), whole[1].double().cpu().numpy()) > 0.999999
    assert cosine(halves[2].double().cpu().numpy(), whole[2].double().cpu().numpy()) > 0.999999


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_one_call_pass_equals_the_step_by_step_pass_bit_for_bit(monkeypatch, dtype):
    """Unsharded passes are issued as ONE library call (lce_fused_pass); LCE_FUSED_PASS=0 issues the same steps one
    by one from Python. Same kernels in the same order: the results must be identical bit for bit."""
    x, y, W = random_problem(640, 256, 2048, dtype, seed=21)
    monkeypatch.setenv("LCE_FUSED_PASS", "1")
    one = run_gpu(x, y, W, -1, 1e-4, 0.5, 256, True)
    monkeypatch.setenv("LCE_FUSED_PASS", "0")
    steps = run_gpu(x, y, W, -1, 1e-4, 0.5, 256, True)
    assert one[0] == steps[0] and torch.equal(one[1], steps[1]) and torch.equal(one[2], steps[2])


def test_device_status_is_clean_after_a_pass():
    from linear_cross_entropy_loss_b200 import ops
    x, y, W = random_problem(256, 256, 512, torch.bfloat16, seed=15)
    out5, dx, dA, ws = ops.run_pass(x.cuda(), y.cuda(), W.cuda(), -1, 0.0, 1.0, 128, False, True)
    assert ops.get_backend().read_status(ws) == 0
