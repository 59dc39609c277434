"""Vocabulary sharding over a real process group (gloo, world size 2 and 4, CPU): the all-gather of row
partials, the dx all-reduce and the rank-ordered combine, with the kernels answered by the oracle stand-in."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, results):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fake_backend import FakeBackend
        from linear_cross_entropy_loss_b200 import ops
        from linear_cross_entropy_loss_b200.sharded import VocabShardedLinearCrossEntropyLoss, linear_cross_entropy_sharded
        from oracle import oracle

        ops.set_backend(FakeBackend())
        g = torch.Generator().manual_seed(0)
        N, H, V = 512, 256, 1024
        x = torch.randn(N, H, generator=g)
        W = torch.randn(H, V, generator=g) / H ** 0.5
        y = torch.randint(0, V, (N,), generator=g)
        y[torch.rand(N, generator=g) < 0.1] = -1
        vl = V // world
        Ws = W[:, rank * vl:(rank + 1) * vl].contiguous().requires_grad_(True)
        xr = x.clone().requires_grad_(True)
        out = linear_cross_entropy_sharded(xr, y, Ws, None, -1, 1e-3, 0.8, 256, True)
        out[0].backward()
        ref = oracle.forward_backward(x, y, W, -1, 1e-3, 0.8)
        got = np.array([v.item() for v in out])
        want = np.array([ref.loss, ref.z_value, ref.logit_max, ref.logit_entropy, ref.logit_norm])
        ok = np.allclose(got, want, rtol=3e-6)
        ok &= np.allclose(xr.grad.numpy(), ref.dx, atol=2e-7)
        ok &= np.allclose(Ws.grad.numpy(), ref.dW[:, rank * vl:(rank + 1) * vl], atol=2e-7)
        # every rank must hold bitwise the same scalars
        gathered = [torch.zeros(5, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(gathered, torch.tensor(got))
        ok &= all(torch.equal(gathered[0], t) for t in gathered)

        # module: same start as one unsharded draw with the same seed
        m = VocabShardedLinearCrossEntropyLoss(256, 1024, ignore_index=-1, N_chunk_size=256, init_seed=3)
        full = torch.empty(256, 1024)
        gen = torch.Generator().manual_seed(3)
        for h0 in range(0, 256, 64):
            torch.nn.init.trunc_normal_(full[h0:h0 + 64], std=1 / 16, a=-3 / 16, b=3 / 16, generator=gen)
        ok &= torch.equal(m.weight.detach(), full[:, rank * vl:(rank + 1) * vl])
        loss = m(x, y)
        ok &= abs(loss.item() - oracle.forward_backward(x, y, full, -1, want_grad=False).loss) < 1e-5
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_vocab_sharded_pass_over_gloo(world):
    import socket

    with socket.socket() as sock:  # a port that is free right now (a fixed one can still be in TIME_WAIT from an earlier run)
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {r: True for r in range(world)}
