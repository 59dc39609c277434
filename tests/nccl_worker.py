"""Child process of tests/test_gpu_sharded.py: one rank of a vocabulary-sharded pass over NCCL."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from gpu_util import cosine, random_problem  # noqa: E402
from linear_cross_entropy_loss_b200.sharded import linear_cross_entropy_sharded  # noqa: E402
from oracle import oracle  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    from linear_cross_entropy_loss_b200 import ops
    ops.MIN_SPLIT_ELEMS = 0  # the fp16 case below must exercise half chunks on two streams at this small size
    ops.MIN_HALF_ROWS = 512
    N, H, V = 1024, 512, 8192
    vl = V // world
    ok = True
    # bf16: one base per row; fp16: per-tile slabs, each 1024-row chunk as two sub-chunks on two streams
    for dtype, chunk, cos_min in ((torch.bfloat16, 256, 0.99999), (torch.float16, 1024, 0.999995)):
        x, y, W = random_problem(N, H, V, dtype, seed=0)
        ref = oracle.forward_backward(x, y, W, -1, 1e-4, 0.5)
        # four data paths: dx summed by the contraction's own stores into peer-mapped memory; row partials pushed
        # over peer memory with pipelined chunks and ONE all-reduce of dx per pass; the default (all-gather of the
        # partials per chunk, one all-reduce of dx per pass); all-gather and all-reduce per chunk
        for peer_dx, peer_parts, dx_reduce in (("1", "0", "pass"), ("0", "1", "pass"), ("0", "0", "pass"),
                                               ("0", "0", "chunk")):
            os.environ["LCE_PEER_DX"] = peer_dx
            os.environ["LCE_PEER_PARTS"] = peer_parts
            os.environ["LCE_DX_REDUCE"] = dx_reduce
            xd = x.cuda().requires_grad_(True)
            Ws = W[:, rank * vl:(rank + 1) * vl].contiguous().cuda().requires_grad_(True)
            for _ in range(2):  # twice: the second pass reuses the exchange buffers with later epochs
                xd.grad = Ws.grad = None
                out = linear_cross_entropy_sharded(xd, y.cuda(), Ws, None, -1, 1e-4, 0.5, chunk, True)
                out[0].backward()
            torch.cuda.synchronize()
            good = abs(out[0].item() - ref.loss) < 2e-5 * ref.loss
            good &= cosine(xd.grad.double().cpu().numpy(), ref.dx) > cos_min
            good &= cosine(Ws.grad.double().cpu().numpy(), ref.dW[:, rank * vl:(rank + 1) * vl]) > cos_min
            if peer_dx == "1":
                from linear_cross_entropy_loss_b200.sharded import PeerExchange
                good &= len(PeerExchange._cache) >= 1  # the peer path really ran
                theirs = xd.grad.clone()
                dist.broadcast(theirs, src=0)
                good &= torch.equal(theirs, xd.grad)  # bitwise the same dx on every rank
            if peer_dx == "0" and peer_parts == "1" and dtype == torch.bfloat16:
                from linear_cross_entropy_loss_b200.sharded import PartsExchange
                good &= len(PartsExchange._cache) >= 1  # the pipelined path with pushed partials really ran
            if not good:
                print(f"rank {rank}: mismatch with {dtype}, LCE_PEER_DX={peer_dx} LCE_PEER_PARTS={peer_parts} "
                      f"LCE_DX_REDUCE={dx_reduce}: loss {out[0].item()} vs {ref.loss}", flush=True)
            ok &= bool(good)
    flag = torch.tensor([1.0 if ok else 0.0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and flag.item() == 1.0:
        print("SHARDED_OK")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1.0 else 1)


if __name__ == "__main__":
    main()
