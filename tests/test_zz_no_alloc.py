"""lce_eval_loss_static: the entry point for callers that cannot allocate device memory (loops that must not pay
cudaMalloc's device synchronisation, server plugins that only receive input/output buffers, hooks that run after a
framework's pool has claimed the GPU).
Its scratch is a fixed array inside the library, so this test checks what such a caller relies on: the result equals
that of the workspace-based entry points, on two calls in a row (the second call finds the first call's leftovers in
the shared scratch), and sizes beyond the fixed scratch are refused with a status code.
Collected last on purpose (file name), so that a run that stops at the first failure has run everything else."""
import ctypes

import pytest
import torch

from linear_cross_entropy_loss_b200 import _native, ops
from oracle import oracle

pytestmark = pytest.mark.gpu


def static_loss(x, y, W, ignore_index, zreg, scale, monitoring):
    lib = _native.load()
    prob = _native.Problem(n_rows_total=x.shape[0], chunk_rows=128, hidden=x.shape[1], vocab_local=W.shape[1],
                           vocab_offset=0, ignore_index=ignore_index, world=1, dtype=ops._DTYPE_CODE[x.dtype],
                           monitoring=int(monitoring), want_grad=0, logit_scale=scale, z_regularization=zreg)
    out5 = torch.full((5,), float("nan"), dtype=torch.float32, device=x.device)
    rc = lib.lce_eval_loss_static(ctypes.byref(prob), x.data_ptr(), x.stride(0), W.data_ptr(), W.stride(0),
                                  y.data_ptr(), out5.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, out5


def workspace_loss(x, y, W, ignore_index, zreg, scale, monitoring, chunk):
    out5, _, _, _ = ops.run_pass(x, y, W, ignore_index, zreg, scale, chunk, monitoring, False)
    return out5


def problem(seed, N, H, V, dtype):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, H, generator=g).to(dtype).cuda()
    W = (torch.randn(H, V, generator=g) / H ** 0.5).to(dtype).cuda()
    y = torch.randint(0, V, (N,), generator=g)
    y[torch.rand(N, generator=g) < 0.1] = -1
    return x, y.cuda(), W


def test_static_scratch_entry_matches_the_workspace_path_twice_in_a_row():
    # first call: 4096 rows x 16384 columns in bf16 -> several chunks inside the 8 MiB scratch
    x, y, W = problem(0, 4096, 512, 16384, torch.bfloat16)
    rc, got = static_loss(x, y, W, -1, 1e-4, 0.5, True)
    assert rc == 0, _native.status_string(rc)
    want = workspace_loss(x, y, W, -1, 1e-4, 0.5, True, 1024)
    torch.cuda.synchronize()
    assert torch.allclose(got, want, rtol=2e-5, atol=1e-6), (got, want)
    # and against the float64 oracle directly, so that this file stands on its own
    ref = oracle.forward_backward(x, y, W, -1, 1e-4, 0.5, want_grad=False)
    assert abs(got[0].item() - ref.loss) <= 2e-5 * abs(ref.loss), (got[0].item(), ref.loss)
    assert abs(got[1].item() - ref.z_value) <= 4e-5 * abs(ref.z_value)
    assert abs(got[3].item() - ref.logit_entropy) <= 1e-3 * abs(ref.logit_entropy)

    # second call, different shape, dtype and options: must not see anything of the first call
    x2, y2, W2 = problem(1, 640, 256, 4096, torch.float16)
    rc, got2 = static_loss(x2, y2, W2, -1, 0.0, 1.0, False)
    assert rc == 0, _native.status_string(rc)
    want2 = workspace_loss(x2, y2, W2, -1, 0.0, 1.0, False, 256)
    torch.cuda.synchronize()
    assert torch.allclose(got2[:2], want2[:2], rtol=2e-5, atol=1e-6), (got2, want2)

    # and the first problem again gives the first answer again
    rc, got3 = static_loss(x, y, W, -1, 1e-4, 0.5, True)
    torch.cuda.synchronize()
    assert rc == 0 and torch.equal(got3, got)


def test_sizes_beyond_the_fixed_scratch_are_refused():
    lib = _native.load()
    x = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(128, dtype=torch.int64, device="cuda")
    out5 = torch.zeros(5, dtype=torch.float32, device="cuda")
    too_wide = _native.Problem(n_rows_total=128, chunk_rows=128, hidden=256, vocab_local=256 * 16384, vocab_offset=0,
                               ignore_index=-1, world=1, dtype=1, monitoring=0, want_grad=0, logit_scale=1.0,
                               z_regularization=0.0)
    rc = lib.lce_eval_loss_static(ctypes.byref(too_wide), x.data_ptr(), 256, x.data_ptr(), 256 * 16384, y.data_ptr(),
                                  out5.data_ptr(), None)
    assert rc == -8 and "maximum" in _native.status_string(rc)
    bad_shape = _native.Problem(n_rows_total=128, chunk_rows=128, hidden=252, vocab_local=512, vocab_offset=0,
                                ignore_index=-1, world=1, dtype=1, monitoring=0, want_grad=0, logit_scale=1.0,
                                z_regularization=0.0)
    assert lib.lce_eval_loss_static(ctypes.byref(bad_shape), x.data_ptr(), 256, x.data_ptr(), 512, y.data_ptr(),
                                    out5.data_ptr(), None) == -2
    assert lib.lce_eval_loss_static(None, None, 0, None, 0, None, None, None) == -1
