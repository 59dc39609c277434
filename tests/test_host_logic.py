"""Host-side logic on the CPU: the chunk loop, the autograd plumbing and the module surface, driven through a
stand-in backend that answers each per-chunk call with the float64 oracle (tests/fake_backend.py).
The product path itself has no CPU fallback -- that is tested here too."""
import numpy as np
import pytest
import torch

from fake_backend import FakeBackend
from linear_cross_entropy_loss_b200 import LinearCrossEntropyLoss, linear_cross_entropy, ops
from oracle import oracle


@pytest.fixture
def fake():
    backend = FakeBackend()
    ops.set_backend(backend)
    yield backend
    ops.set_backend(None)


def make(N=512, H=256, V=768, ignore=-1, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, H, generator=g).to(dtype)
    W = (torch.randn(H, V, generator=g) / H ** 0.5).to(dtype)
    y = torch.randint(0, V, (N,), generator=g)
    y[torch.rand(N, generator=g) < 0.1] = ignore
    return x, y, W


def test_product_path_refuses_cpu_tensors():
    ops.set_backend(None)
    x, y, W = make()
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        linear_cross_entropy(x.requires_grad_(True), y, W)


@pytest.mark.parametrize("chunk", [128, 256, 4096])
def test_chunk_loop_matches_oracle(fake, chunk):
    x, y, W = make()
    x.requires_grad_(True)
    W.requires_grad_(True)
    out = linear_cross_entropy(x, y, W, ignore_index=-1, z_regularization=1e-3, logit_scale=0.7, N_chunk_size=chunk,
                               monitoring=True)
    out[0].backward()
    ref = oracle.forward_backward(x, y, W, -1, 1e-3, 0.7)
    got = [v.item() for v in out]
    np.testing.assert_allclose(got, [ref.loss, ref.z_value, ref.logit_max, ref.logit_entropy, ref.logit_norm], rtol=2e-6)
    np.testing.assert_allclose(x.grad.numpy(), ref.dx, atol=1e-7)
    np.testing.assert_allclose(W.grad.numpy(), ref.dW, atol=1e-7)
    n_chunks = -(-512 // min(512, chunk))
    assert fake.calls.count("dw_chunk") == n_chunks and fake.calls.count("forward_chunk") == fake.calls.count("dx_chunk") >= n_chunks
    assert fake.calls[0] == "begin" and "finalize" in fake.calls


def test_grad_output_scales_both_gradients(fake):
    x, y, W = make(seed=1)
    x.requires_grad_(True)
    W.requires_grad_(True)
    loss = linear_cross_entropy(x, y, W, ignore_index=-1)[0]
    (3.0 * loss).backward()
    ref = oracle.forward_backward(x, y, W, -1)
    np.testing.assert_allclose(x.grad.numpy(), 3 * ref.dx, atol=3e-7)
    np.testing.assert_allclose(W.grad.numpy(), 3 * ref.dW, atol=3e-7)


def test_no_gradient_work_without_requires_grad(fake):
    x, y, W = make(seed=2)
    out = linear_cross_entropy(x, y, W, ignore_index=-1)
    assert "dx_chunk" not in fake.calls and "dw_chunk" not in fake.calls
    assert not out[0].requires_grad
    assert abs(out[0].item() - oracle.forward_backward(x, y, W, -1, want_grad=False).loss) < 1e-5
    # evaluation under torch.no_grad() with tensors that do require grad (a trainable weight): forward only as well
    fake.calls.clear()
    xr, Wr = x.clone().requires_grad_(True), W.clone().requires_grad_(True)
    with torch.no_grad():
        out2 = linear_cross_entropy(xr, y, Wr, ignore_index=-1)
        m = LinearCrossEntropyLoss(256, 768, ignore_index=-1)
        m(x, y)
    assert "dx_chunk" not in fake.calls and "dw_chunk" not in fake.calls and "dz_chunk" not in fake.calls
    assert abs(out2[0].item() - out[0].item()) < 1e-7


def test_only_the_requested_gradient_is_computed(fake):
    """A frozen head (only x requires grad) skips the dW contraction, frozen features skip dx."""
    x, y, W = make(seed=4)
    want = oracle.forward_backward(x, y, W, -1)
    xr = x.clone().requires_grad_(True)
    linear_cross_entropy(xr, y, W, ignore_index=-1)[0].backward()
    assert "dx_chunk" in fake.calls and "dw_chunk" not in fake.calls
    assert np.allclose(xr.grad.numpy(), want.dx, atol=2e-7)
    fake.calls.clear()
    Wr = W.clone().requires_grad_(True)
    (linear_cross_entropy(x, y, Wr, ignore_index=-1)[0] * 2).backward()
    assert "dw_chunk" in fake.calls and "dx_chunk" not in fake.calls
    assert np.allclose(Wr.grad.numpy(), 2 * want.dW, atol=4e-7)


def test_leading_dimensions_are_flattened_and_grad_keeps_the_input_shape(fake):
    x, y, W = make(N=512)
    x3 = x.view(4, 128, 256).clone().requires_grad_(True)
    loss = linear_cross_entropy(x3, y.view(4, 128), W.requires_grad_(True), ignore_index=-1)[0]
    loss.backward()
    assert x3.grad.shape == (4, 128, 256)


def test_non_contiguous_inputs_are_accepted(fake):
    x, y, W = make()
    xs = torch.randn(512, 512)[:, ::2]  # inner stride 2 -> copied
    Wt = W.t().contiguous().t()          # (H, V) view with V stride != 1 -> copied
    out = linear_cross_entropy(xs.requires_grad_(True), y, Wt.requires_grad_(True), ignore_index=-1)
    ref = oracle.forward_backward(xs, y, Wt, -1, want_grad=False)
    assert abs(out[0].item() - ref.loss) < 1e-5


def test_shape_and_dtype_checks(fake):
    x, y, W = make()
    # a hidden size that is not a multiple of 8 runs on zero-padded copies and returns gradients of the given shapes
    x100, W100 = x[:, :100].clone().requires_grad_(True), W[:100].clone().requires_grad_(True)
    out = linear_cross_entropy(x100, y, W100, -1)
    out[0].backward()
    ref = oracle.forward_backward(x[:, :100], y, W[:100], -1)
    assert abs(out[0].item() - ref.loss) < 1e-5
    assert x100.grad.shape == (512, 100) and W100.grad.shape == (100, 768)
    assert np.allclose(x100.grad.numpy(), ref.dx, atol=2e-7) and np.allclose(W100.grad.numpy(), ref.dW, atol=2e-7)
    y100 = y.clamp(max=99)
    out = linear_cross_entropy(x, y100, W[:, :100].clone().requires_grad_(True), -1)  # any vocabulary size is taken
    assert abs(out[0].item() - oracle.forward_backward(x, y100, W[:, :100], -1, want_grad=False).loss) < 1e-5
    with pytest.raises(AssertionError):
        linear_cross_entropy(x, y.int(), W)
    with pytest.raises(AssertionError):
        linear_cross_entropy(x, y, W.half())


def test_ragged_row_count_and_chunk_size_are_rounded_to_tiles(fake):
    x, y, W = make(N=300, H=64, V=200)
    x.requires_grad_(True)
    out = linear_cross_entropy(x, y, W.requires_grad_(True), ignore_index=-1, N_chunk_size=100)
    out[0].backward()
    ref = oracle.forward_backward(x, y, W, -1)
    assert abs(out[0].item() - ref.loss) < 1e-5
    np.testing.assert_allclose(x.grad.numpy(), ref.dx, atol=1e-7)
    assert fake.calls.count("forward_chunk") == 3     # chunks of 128, 128 and 44 rows


def test_module_surface_matches_the_reference(fake):
    m = LinearCrossEntropyLoss(256, 768, ignore_index=-1, logit_scale=0.5, z_regularization=1e-4, N_chunk_size=256)
    assert isinstance(m, torch.nn.Linear)
    assert list(m.state_dict().keys()) == ["weight"]
    assert m.weight.shape == (256, 768)          # transposed with respect to nn.Linear
    assert not hasattr(m, "bias") or m.__dict__.get("bias") is None
    assert m.monitoring is False and m.latest_metrics == {}
    assert m.weight.abs().max().item() <= 3 / 256 ** 0.5 + 1e-6
    assert "bias=False" in repr(m)
    x, y, _ = make()
    loss = m(x, y)
    assert loss.dim() == 0 and loss.dtype == torch.float32
    assert m.latest_metrics == {}
    m.monitoring = True
    loss = m(x, y)
    assert set(m.latest_metrics) == {"logit_norm", "logit_max", "logit_entropy", "z_value"}
    loss.backward()
    ref = oracle.forward_backward(x, y, m.weight, -1, 1e-4, 0.5)
    np.testing.assert_allclose(m.weight.grad.numpy(), ref.dW, atol=1e-7)


def test_module_constructor_asserts():
    assert LinearCrossEntropyLoss(256, 1001).weight.shape == (256, 1001)  # any vocabulary size
    assert LinearCrossEntropyLoss(100, 512).weight.shape == (100, 512)    # any hidden size
    for bad in [dict(in_features=0), dict(out_features=0), dict(N_chunk_size=0), dict(logit_scale=0.0),
                dict(z_regularization=-1.0)]:
        kw = dict(in_features=256, out_features=512)
        kw.update(bad)
        with pytest.raises(AssertionError):
            LinearCrossEntropyLoss(**kw)


def test_custom_init_method_is_used():
    m = LinearCrossEntropyLoss(256, 512, init_method=lambda w: torch.nn.init.constant_(w, 0.25))
    assert torch.all(m.weight == 0.25)


def test_module_inside_torch_compile(fake):
    class Head(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.proj = torch.nn.Linear(64, 64)
            self.loss = LinearCrossEntropyLoss(64, 200, ignore_index=-1, N_chunk_size=128)

        def forward(self, h, y):
            return self.loss(torch.tanh(self.proj(h)), y)

    torch.manual_seed(0)
    head = Head()
    h = torch.randn(256, 64)
    y = torch.randint(0, 200, (256,))
    eager = head(h, y)
    eager.backward()
    want = [head.proj.weight.grad.clone(), head.loss.weight.grad.clone()]
    head.zero_grad()
    # fullgraph: the pass is one torch.library operator (lce_b200::fused_pass), so tracing meets no graph break
    compiled = torch.compile(head, backend="aot_eager", fullgraph=True)(h, y)
    assert abs(eager.item() - compiled.item()) < 1e-6
    (compiled * 2).backward()
    assert torch.allclose(head.proj.weight.grad, 2 * want[0], atol=1e-7)
    assert torch.allclose(head.loss.weight.grad, 2 * want[1], atol=1e-7)
    with torch.no_grad():  # traced without gradients: the gradient kernels are not part of the graph
        before = len(fake.calls)
        again = torch.compile(head, backend="aot_eager", fullgraph=True)(h, y)
        assert abs(again.item() - eager.item()) < 1e-6
        assert "dx_chunk" not in fake.calls[before:]


def test_peer_exchange_sequencing_in_the_chunk_loop(fake):
    """With a peer exchange in the shard description the loop calls scatter / reduce / finish per chunk with
    consecutive epochs (continuing over passes) instead of dx_chunk + reduce_dx, and gives the same gradients."""
    class Table:
        scattered, reduced = {}, {}

    class Exchange:
        table, wait_ms, overlap, epoch = Table(), 0, False, 40

        def next_epoch(self):
            self.epoch += 1
            return self.epoch

    ex = Exchange()
    reduce_calls = []
    x, y, W = make(N=640, H=256, V=512)
    want = oracle.forward_backward(x, y, W, -1)
    for n_pass in range(2):
        shard = ops.ShardSpec(rank=0, world=1, vocab_offset=0, gather_row_parts=lambda t: t,
                              reduce_dx=reduce_calls.append, peer_exchange=lambda prob, dt: ex)
        out5, dx, dW, _ = ops.run_pass(x, y, W, -1, 0.0, 1.0, 256, False, True, shard=shard)
        assert np.allclose(dx.numpy(), want.dx, atol=2e-7) and np.allclose(dW.numpy(), want.dW, atol=2e-7)
    assert reduce_calls == [] and "dx_chunk" not in fake.calls
    peer_calls = [c for c in fake.calls if isinstance(c, tuple)]
    assert peer_calls == [(name, e) for e in range(41, 47)
                          for name in ("dx_chunk_peer", "dx_reduce_peer", "dx_finish_peer")]
    # without gradients the exchange is not even asked for
    asked = []
    shard = ops.ShardSpec(rank=0, world=1, vocab_offset=0, gather_row_parts=lambda t: t, reduce_dx=reduce_calls.append,
                          peer_exchange=lambda prob, dt: asked.append(1))
    ops.run_pass(x, y, W, -1, 0.0, 1.0, 256, False, False, shard=shard)
    assert asked == []


def test_pipelined_chunks_with_the_row_partials_exchange(fake):
    """With a row-partials exchange in the shard description the loop runs the chunks software-pipelined -- the
    forward and push of chunk c + 1 before the combine and backward of chunk c, two sets of per-chunk buffers --
    never calls gather_row_parts, reduces dx once at the end when asked to, and gives the same results."""
    class Table:
        slots = {}

    class Exchange:
        table, wait_ms, epoch = Table(), 0, 7

        def next_epoch(self):
            self.epoch += 1
            return self.epoch

    ex = Exchange()
    gathers, reduces, probs = [], [], []
    x, y, W = make(N=640, H=256, V=512)
    want = oracle.forward_backward(x, y, W, -1)
    shard = ops.ShardSpec(rank=0, world=1, vocab_offset=0, gather_row_parts=gathers.append,
                          reduce_dx=lambda rows: reduces.append(tuple(rows.shape)),
                          parts_exchange=lambda prob: (probs.append(prob), ex)[1], reduce_dx_once=True)
    out5, dx, dW, _ = ops.run_pass(x, y, W, -1, 0.0, 1.0, 256, False, True, shard=shard)
    assert abs(out5[0].item() - want.loss) < 1e-5
    assert np.allclose(dx.numpy(), want.dx, atol=2e-7) and np.allclose(dW.numpy(), want.dW, atol=2e-7)
    assert gathers == [] and reduces == [(640, 256)] and probs[0].chunk_buffers == 2
    order = [c if isinstance(c, str) else c[0] + str(c[1]) for c in fake.calls
             if c in ("forward_chunk", "dx_chunk") or isinstance(c, tuple)]
    assert order == ["forward_chunk", "parts_push8", "forward_chunk", "parts_push9", "combine_chunk_peer8", "dx_chunk",
                     "forward_chunk", "parts_push10", "combine_chunk_peer9", "dx_chunk", "combine_chunk_peer10",
                     "dx_chunk"]
    # forward only: same order without the backward steps; one chunk: nothing to pipeline, one set of buffers
    fake.calls.clear()
    ops.run_pass(x, y, W, -1, 0.0, 1.0, 256, False, False, shard=shard)
    assert [c[0] for c in fake.calls if isinstance(c, tuple)] == ["parts_push", "parts_push", "combine_chunk_peer",
                                                                  "parts_push", "combine_chunk_peer",
                                                                  "combine_chunk_peer"]
    ops.run_pass(x[:256], y[:256], W, -1, 0.0, 1.0, 256, False, True, shard=shard)
    assert probs[-1].chunk_buffers == 0 and reduces[-1] == (256, 256)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_collective_sequence_of_a_sharded_pass_does_not_depend_on_the_slab_mode(fake, monkeypatch, dtype):
    """Each rank of a sharded run picks its slab mode by itself (own re-run counters, a polled event), so ranks can
    be in different modes in the same pass. The sequence and sizes of the collectives (and the epochs of the peer
    exchange) must then still be the same on all of them, or NCCL would pair up different calls."""
    from linear_cross_entropy_loss_b200 import _native

    x, y, W = make(N=2048, H=256, V=512)
    x, W = x.to(dtype), W.to(dtype)
    monkeypatch.setattr(ops, "MIN_SPLIT_ELEMS", 0)  # halve chunks even at this toy size
    monkeypatch.setattr(ops, "MIN_HALF_ROWS", 512)

    def sequence(mode):
        monkeypatch.setattr(ops.slab_mode_policy, "choose",
                            lambda key, dt: _native.SLAB_PER_TILE if dt == torch.float16 else mode)
        seq = []

        def gather(t):
            seq.append(("all_gather", t.numel()))
            return t

        shard = ops.ShardSpec(rank=0, world=1, vocab_offset=0, gather_row_parts=gather,
                              reduce_dx=lambda rows: seq.append(("all_reduce", tuple(rows.shape))))
        ops.run_pass(x, y, W, -1, 0.0, 1.0, 1024, False, True, shard=shard)
        return seq

    by_row, by_tile = sequence(_native.SLAB_DEFAULT), sequence(_native.SLAB_PER_TILE)
    assert by_row == by_tile and len(by_row) >= 4
    # fp16 (always per tile, on every rank) keeps its half chunks; the other types run whole chunks when sharded
    halves = dtype == torch.float16
    assert by_row.count(("all_reduce", (512 if halves else 1024, 256))) == (4 if halves else 2)


@pytest.mark.parametrize("V", [768, 1003])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_multi_chunk_dW_is_carried_as_sum_and_residual(fake, dtype, V):
    """More than one chunk: 16-bit gradients get a residual buffer of their own type beside dW (no fp32 buffer the
    size of W), fp32 accumulates in place; the first / last flags frame the pass; dW comes back tightly packed."""
    x, y, W = make(N=640, H=256, V=V, dtype=dtype)
    seen = []
    real = fake.dw_chunk

    def spy(prob, x_, row0, rows, ws, dW, dW_res, first, last):
        seen.append((first, last, None if dW_res is None else (dW_res.dtype, tuple(dW_res.shape))))
        return real(prob, x_, row0, rows, ws, dW, dW_res, first, last)

    fake.dw_chunk = spy
    out5, dx, dW, ws = ops.run_pass(x, y, W, -1, 0.0, 1.0, 256, False, True)
    res = None if dtype == torch.float32 else (dtype, (256, V))
    assert seen == [(True, False, res), (False, False, res), (False, True, res)]
    assert dW.dtype == dtype and dW.shape == (256, V) and dW.stride(1) == 1
    want = oracle.forward_backward(x, y, W, -1).dW
    tol = {torch.float32: 2e-7, torch.float16: 1e-3, torch.bfloat16: 8e-3}[dtype]
    assert np.abs(dW.double().numpy() - want).max() <= tol * np.abs(want).max()
    # one chunk: no residual at all
    seen.clear()
    ops.run_pass(x[:256], y[:256], W, -1, 0.0, 1.0, 256, False, True)
    assert seen == [(True, True, None)]


def test_slab_mode_policy_decisions(monkeypatch):
    """The mode picker on its own: fp16 always per tile; bf16 per row until a finished pass reported that more
    than a quarter of its row groups were recomputed; a retry of the default mode every 64th pass; env overrides."""
    from linear_cross_entropy_loss_b200 import _native

    class DoneEvent:
        def query(self):
            return True

    class PendingEvent:
        def query(self):
            return False

    monkeypatch.delenv("LCE_SLAB_MODE", raising=False)
    pol = ops.SlabModePolicy()
    key = (0, torch.bfloat16, 2048, 131072, 4096, 1)
    assert pol.choose(key, torch.float16) == _native.SLAB_PER_TILE
    assert pol.choose(key, torch.bfloat16) == _native.SLAB_DEFAULT            # nothing known yet
    small = (0, torch.bfloat16, 256, 4096, 256, 1)                              # a chunk of 2^20 slab elements
    assert pol.choose(small, torch.bfloat16) == pol.choose(small, torch.float32) == _native.SLAB_PER_TILE
    pol.history[key] = {"host": torch.tensor([12, 16], dtype=torch.int32), "event": PendingEvent(), "fraction": 0.0,
                        "tile_passes": 0}
    assert pol.choose(key, torch.bfloat16) == _native.SLAB_DEFAULT            # counters not there yet: no waiting
    pol.history[key]["event"] = DoneEvent()
    assert pol.choose(key, torch.bfloat16) == _native.SLAB_PER_TILE           # 12 of 16 groups recomputed
    assert pol.history[key]["fraction"] == 0.75 and pol.history[key]["event"] is None
    modes = [pol.choose(key, torch.bfloat16) for _ in range(130)]
    assert modes.count(_native.SLAB_DEFAULT) == 2                               # passes 64 and 128 probe the default mode
    pol.history[key].update(host=torch.tensor([1, 16], dtype=torch.int32), event=DoneEvent())
    assert pol.choose(key, torch.float32) == _native.SLAB_DEFAULT              # 1 of 16: back to one base per row
    monkeypatch.setenv("LCE_SLAB_MODE", "tile")
    assert pol.choose(key, torch.bfloat16) == _native.SLAB_PER_TILE
    monkeypatch.setenv("LCE_SLAB_MODE", "row")
    pol.history[key]["fraction"] = 1.0
    assert pol.choose(key, torch.bfloat16) == _native.SLAB_DEFAULT
    assert pol.choose(key, torch.float16) == _native.SLAB_PER_TILE


def test_autocast_policy_switch():
    ops.set_autocast_policy("follow")
    ops.set_autocast_policy("reference")
    with pytest.raises(AssertionError):
        ops.set_autocast_policy("bf16")


def test_export_names_of_the_reference_package():
    import linear_cross_entropy_loss_b200 as pkg

    for name in ["fwd_configs", "bwd_configs", "LinearCrossEntropyLoss", "linear_cross_entropy"]:
        assert hasattr(pkg, name)


def test_sharded_fp16_pass_sums_dx_in_fp32_and_hands_back_fp16(fake):
    """Every rank's dx of a sharded pass is a partial sum that an all-reduce adds up. For fp16 these travel as fp32
    (values around 1 / n_valid sit in fp16's subnormal range, and one rounding per rank would add up); backward
    converts while it applies grad_output. bf16 keeps its type."""
    from types import SimpleNamespace

    for dtype, carried in ((torch.float16, torch.float32), (torch.bfloat16, torch.bfloat16)):
        x, y, W = make(N=512, H=256, V=512, dtype=dtype)
        reduced = []
        shard = ops.ShardSpec(rank=0, world=1, vocab_offset=0, gather_row_parts=lambda t: t,
                              reduce_dx=lambda rows: reduced.append((rows.dtype, tuple(rows.shape))), reduce_dx_once=True)
        out5, dx, dW, _ = ops.run_pass(x, y, W, -1, 0.0, 1.0, 256, False, True, shard=shard)
        assert dx.dtype == carried and reduced == [(carried, (512, 256))]
        assert dW.dtype == dtype
        ctx = SimpleNamespace(lce_grads=(dx.clone(), None), lce_x_shape=(2, 256, 256), lce_x_dtype=dtype)
        gx, gW = ops._scaled_grads(ctx, torch.tensor(2.0))
        assert gW is None and gx.dtype == dtype and gx.shape == (2, 256, 256)
        assert torch.allclose(gx.double().reshape(512, 256), 2.0 * dx.double(), rtol=1e-2, atol=1e-7)
    # without sharding nothing changes: fp16 in, fp16 out of run_pass
    x, y, W = make(N=512, H=256, V=512, dtype=torch.float16)
    assert ops.run_pass(x, y, W, -1, 0.0, 1.0, 256, False, True)[1].dtype == torch.float16
