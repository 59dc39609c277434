"""Vocabulary sharding through the C ABI. On one GPU the G ranks are emulated one after the other (each with its own
workspace and weight slab); with two or more GPUs the real NCCL path runs in child processes."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import TOL, cosine, random_problem
from linear_cross_entropy_loss_b200 import _native, ops
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("world", [2, 4, 8])
def test_emulated_shards_on_one_gpu(world):
    dtype = torch.bfloat16
    N, H, V, chunk = 512, 256, 4096, 256
    x, y, W = random_problem(N, H, V, dtype, seed=world)
    xd, yd = x.cuda(), y.cuda()
    vl = V // world
    slabs = [W[:, g * vl:(g + 1) * vl].contiguous().cuda() for g in range(world)]
    be = ops.get_backend()
    probs = [_native.Problem(n_rows_total=N, chunk_rows=chunk, hidden=H, vocab_local=vl, vocab_offset=g * vl,
                             ignore_index=-1, world=world, dtype=_native.DTYPE_BF16, monitoring=1, want_grad=1,
                             logit_scale=0.5, z_regularization=1e-3) for g in range(world)]
    ws = [torch.empty(be.workspace_bytes(p), dtype=torch.uint8, device="cuda") for p in probs]
    parts = torch.empty(world, 6 * chunk, dtype=torch.float32, device="cuda")
    dxs = [torch.zeros(N, H, dtype=torch.float32, device="cuda") for _ in range(world)]
    dWs = [torch.empty(H, vl, dtype=torch.float32, device="cuda") for _ in range(world)]
    outs = [torch.empty(5, dtype=torch.float32, device="cuda") for _ in range(world)]
    for g in range(world):
        be.begin(probs[g], yd, ws[g])
    for row0 in range(0, N, chunk):
        for g in range(world):
            be.forward_chunk(probs[g], xd, slabs[g], yd, row0, chunk, ws[g], parts[g])
        for g in range(world):
            be.combine_chunk(probs[g], parts, yd, row0, chunk, ws[g])
            be.dz_chunk(probs[g], xd, yd, row0, chunk, ws[g])
            be.dx_chunk(probs[g], slabs[g], row0, chunk, ws[g], dxs[g])
            be.dw_chunk(probs[g], xd, row0, chunk, ws[g], dWs[g], row0 == 0, None)
    for g in range(world):
        be.finalize(probs[g], ws[g], outs[g])
    torch.cuda.synchronize()
    ref = oracle.forward_backward(x, y, W, -1, 1e-3, 0.5)
    for g in range(1, world):
        assert torch.equal(outs[g], outs[0]), "every rank must compute bitwise the same scalars"
    got = outs[0].cpu().numpy()
    want = np.array([ref.loss, ref.z_value, ref.logit_max, ref.logit_entropy, ref.logit_norm])
    np.testing.assert_allclose(got, want, rtol=1e-3)
    assert abs(got[0] - ref.loss) < TOL[dtype]["loss"] * ref.loss
    dx = sum(d.double() for d in dxs).cpu().numpy()
    dW = torch.cat(dWs, dim=1).double().cpu().numpy()
    assert cosine(dx, ref.dx) > TOL[dtype]["cos"]
    assert cosine(dW, ref.dW) > TOL[dtype]["cos"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_nccl_vocab_sharding_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300), str(ROOT / "tests" / "nccl_worker.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "SHARDED_OK" in proc.stdout
