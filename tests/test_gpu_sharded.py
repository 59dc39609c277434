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
    dWs = [torch.empty(H, vl, dtype=dtype, device="cuda") for _ in range(world)]
    res = [torch.empty(H, vl, dtype=dtype, device="cuda") for _ in range(world)]
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
            be.dw_chunk(probs[g], xd, row0, chunk, ws[g], dWs[g], res[g], row0 == 0, row0 + chunk >= N)
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


@pytest.mark.parametrize("world,dtype,N,chunk", [(2, torch.bfloat16, 768, 512), (4, torch.float16, 1024, 512),
                                                 (8, torch.float32, 2048, 1024), (2, torch.bfloat16, 300, 256)])
def test_emulated_peer_exchange_of_dx_on_one_gpu(world, dtype, N, chunk):
    """The dx exchange over peer-mapped memory, with the G ranks' buffers all on this GPU. The ranks are run phase
    by phase, so every flag a kernel waits for has been published by an earlier launch on the same stream. The
    result must equal, bit for bit on all ranks, the sum of the per-rank fp32 partials rounded once -- and be at
    least as close to the oracle as the all-reduce of rounded rows."""
    H, V = 256, 2048
    x, y, W = random_problem(N, H, V, dtype, seed=10 + world)
    xd, yd = x.cuda(), y.cuda()
    vl = V // world
    slabs = [W[:, g * vl:(g + 1) * vl].contiguous().cuda() for g in range(world)]
    be = ops.get_backend()
    probs = [_native.Problem(n_rows_total=N, chunk_rows=chunk, hidden=H, vocab_local=vl, vocab_offset=g * vl,
                             ignore_index=-1, world=world, dtype=ops._DTYPE_CODE[dtype], monitoring=0, want_grad=1,
                             logit_scale=1.0, z_regularization=0.0) for g in range(world)]
    ws = [torch.empty(be.workspace_bytes(p), dtype=torch.uint8, device="cuda") for p in probs]
    nbytes = be.peer_bytes(probs[0], dtype)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    tables = []
    for g in range(world):
        t = _native.PeerTable()
        t.world, t.rank = world, g
        for k in range(world):
            t.base[k] = bufs[k].data_ptr()
        tables.append(t)
    parts = torch.empty(world, 6 * chunk, dtype=torch.float32, device="cuda")
    dx_peer = [torch.zeros(N, H, dtype=dtype, device="cuda") for _ in range(world)]
    dx_plain = [torch.zeros(N, H, dtype=torch.float32, device="cuda") for _ in range(world)]
    for g in range(world):
        be.begin(probs[g], yd, ws[g])
    epoch = 0
    for row0 in range(0, N, chunk):
        rows = min(chunk, N - row0)
        epoch += 1
        for g in range(world):
            be.forward_chunk(probs[g], xd, slabs[g], yd, row0, rows, ws[g], parts[g])
        for g in range(world):
            be.combine_chunk(probs[g], parts, yd, row0, rows, ws[g])
            be.dz_chunk(probs[g], xd, yd, row0, rows, ws[g])
            be.dx_chunk(probs[g], slabs[g], row0, rows, ws[g], dx_plain[g])
            be.dx_chunk_peer(probs[g], slabs[g], row0, rows, ws[g], tables[g], dtype, epoch)
        for g in range(world):
            be.dx_reduce_peer(probs[g], row0, rows, ws[g], tables[g], dtype, epoch, 2000)
        for g in range(world):
            be.dx_finish_peer(probs[g], row0, rows, ws[g], tables[g], epoch, dx_peer[g], 2000)
    torch.cuda.synchronize()
    for g in range(world):
        assert be.read_status(ws[g]) == 0
        assert torch.equal(dx_peer[g], dx_peer[0]), "dx must be bitwise identical on all ranks"
    ref = oracle.forward_backward(x, y, W, -1, 0.0, 1.0)
    want = sum(d.double() for d in dx_plain)
    got = dx_peer[0].double()
    assert cosine(got.cpu().numpy(), ref.dx) > TOL[dtype]["cos"]
    # one rounding of the fp32 sum: within one unit in the last place of the output type of the fp32 sum
    eps = {torch.float32: 2.0 ** -22, torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -10}[dtype]
    mass = sum(d.double().abs() for d in dx_plain)  # fp32 accumulation error is relative to the summed magnitudes
    tiny = 6e-8 if dtype == torch.float16 else 1e-12  # fp16 gradients of this size are subnormal: absolute spacing 2^-24
    assert torch.all((got - want).abs() <= eps * want.abs() + 5e-7 * mass + tiny)


def _tables(bufs):
    world = len(bufs)
    tables = []
    for g in range(world):
        t = _native.PeerTable()
        t.world, t.rank = world, g
        for k in range(world):
            t.base[k] = bufs[k].data_ptr()
        tables.append(t)
    return tables


@pytest.mark.parametrize("world,dtype,N,chunk", [(2, torch.bfloat16, 768, 256), (4, torch.float32, 1280, 256),
                                                 (8, torch.bfloat16, 600, 256)])
def test_emulated_pipelined_pass_with_the_row_partials_exchange(world, dtype, N, chunk):
    """The software-pipelined sharded pass through the C ABI, G ranks emulated on this GPU: forward and push of chunk
    c + 1 before combine and backward of chunk c, two sets of per-chunk buffers per workspace, row partials stored
    into every rank's exchange buffer (four slots) instead of an all-gather. Ranks run phase by phase, so every flag
    a kernel waits for was published by an earlier launch. Checked against the oracle; scalars bitwise equal on all
    ranks; two passes in a row (epochs continue, slots are reused)."""
    H, V = 256, 4096
    x, y, W = random_problem(N, H, V, dtype, seed=20 + world)
    xd, yd = x.cuda(), y.cuda()
    vl = V // world
    slabs = [W[:, g * vl:(g + 1) * vl].contiguous().cuda() for g in range(world)]
    be = ops.get_backend()
    probs = [_native.Problem(n_rows_total=N, chunk_rows=chunk, hidden=H, vocab_local=vl, vocab_offset=g * vl,
                             ignore_index=-1, world=world, dtype=ops._DTYPE_CODE[dtype], monitoring=1, want_grad=1,
                             logit_scale=0.5, z_regularization=1e-3, chunk_buffers=2) for g in range(world)]
    one_buffer = _native.Problem(n_rows_total=N, chunk_rows=chunk, hidden=H, vocab_local=vl, vocab_offset=0,
                                 ignore_index=-1, world=world, dtype=ops._DTYPE_CODE[dtype], monitoring=1, want_grad=1,
                                 logit_scale=0.5, z_regularization=1e-3)
    assert be.workspace_bytes(probs[0]) > be.workspace_bytes(one_buffer)  # two sets of per-chunk buffers
    ws = [torch.empty(be.workspace_bytes(p), dtype=torch.uint8, device="cuda") for p in probs]
    bufs = [torch.zeros(be.parts_bytes(probs[0]), dtype=torch.uint8, device="cuda") for _ in range(world)]
    tables = _tables(bufs)
    local = [torch.empty(6 * chunk, dtype=torch.float32, device="cuda") for _ in range(world)]
    chunks = [(r0, min(chunk, N - r0)) for r0 in range(0, N, chunk)]
    epoch = 0
    ref = oracle.forward_backward(x, y, W, -1, 1e-3, 0.5)
    for n_pass in range(2):
        dxs = [torch.zeros(N, H, dtype=torch.float32, device="cuda") for _ in range(world)]
        dWs = [torch.empty(H, vl, dtype=dtype, device="cuda") for _ in range(world)]
        res = [None if dtype == torch.float32 else torch.empty(H, vl, dtype=dtype, device="cuda") for _ in range(world)]
        outs = [torch.empty(5, dtype=torch.float32, device="cuda") for _ in range(world)]
        for g in range(world):
            be.begin(probs[g], yd, ws[g])

        def forward_and_push(ci):
            nonlocal epoch
            epoch += 1
            r0, n = chunks[ci]
            for g in range(world):
                be.forward_chunk(probs[g], xd, slabs[g], yd, r0, n, ws[g], local[g])
                be.parts_push(probs[g], local[g], r0, n, tables[g], epoch, ws[g])
            return epoch

        epochs = {0: forward_and_push(0)}
        for ci, (r0, n) in enumerate(chunks):
            if ci + 1 < len(chunks):
                epochs[ci + 1] = forward_and_push(ci + 1)
            for g in range(world):
                be.combine_chunk_peer(probs[g], tables[g], epochs[ci], yd, r0, n, ws[g], 2000)
                be.dz_chunk(probs[g], xd, yd, r0, n, ws[g])
                be.dx_chunk(probs[g], slabs[g], r0, n, ws[g], dxs[g])
                be.dw_chunk(probs[g], xd, r0, n, ws[g], dWs[g], res[g], ci == 0, ci == len(chunks) - 1)
        for g in range(world):
            be.finalize(probs[g], ws[g], outs[g])
        torch.cuda.synchronize()
        for g in range(world):
            assert be.read_status(ws[g]) == 0
            assert torch.equal(outs[g], outs[0]), "every rank must compute bitwise the same scalars"
        got = outs[0].cpu().numpy()
        want = np.array([ref.loss, ref.z_value, ref.logit_max, ref.logit_entropy, ref.logit_norm])
        np.testing.assert_allclose(got, want, rtol=2e-3)
        assert abs(got[0] - ref.loss) < 10 * TOL[dtype]["loss"] * ref.loss
        dx = sum(d.double() for d in dxs).cpu().numpy()
        dW = torch.cat(dWs, dim=1).double().cpu().numpy()
        assert cosine(dx, ref.dx) > TOL[dtype]["cos"]
        assert cosine(dW, ref.dW) > TOL[dtype]["cos"]


def test_wait_for_row_partials_runs_out_and_reports():
    """Nobody pushes: the combine step's bounded wait gives up after wait_ms, merges nothing, and the status word
    turns the loss of the pass into NaN. The kernel returns normally."""
    be = ops.get_backend()
    N, H = 256, 256
    prob = _native.Problem(n_rows_total=N, chunk_rows=256, hidden=H, vocab_local=512, vocab_offset=0, ignore_index=-1,
                           world=2, dtype=_native.DTYPE_BF16, monitoring=0, want_grad=0, logit_scale=1.0,
                           z_regularization=0.0)
    ws = torch.empty(be.workspace_bytes(prob), dtype=torch.uint8, device="cuda")
    y = torch.zeros(N, dtype=torch.int64, device="cuda")
    be.begin(prob, y, ws)
    bufs = [torch.zeros(be.parts_bytes(prob), dtype=torch.uint8, device="cuda") for _ in range(2)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    be.combine_chunk_peer(prob, _tables(bufs)[0], 1, y, 0, N, ws, 200)
    t1.record()
    torch.cuda.synchronize()
    assert 150 < t0.elapsed_time(t1) < 2000
    assert be.read_status(ws) == -6  # LCE_ERR_DEVICE_TIMEOUT
    # a pass whose status word is set does not wait again: a broken exchange costs one expired wait per pass
    t0.record()
    be.combine_chunk_peer(prob, _tables(bufs)[0], 2, y, 0, N, ws, 200)
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 50
    out5 = torch.zeros(5, dtype=torch.float32, device="cuda")
    be.finalize(prob, ws, out5)
    assert torch.isnan(out5[0])


def test_peer_wait_runs_out_and_reports_instead_of_hanging():
    """A flag that nothing sets: the bounded wait gives up after wait_ms, copies nothing, and the status word turns
    the loss of the pass into NaN. (No fault is provoked: the kernel returns normally.)"""
    be = ops.get_backend()
    N = H = 256
    prob = _native.Problem(n_rows_total=N, chunk_rows=256, hidden=H, vocab_local=512, vocab_offset=0, ignore_index=-1,
                           world=2, dtype=_native.DTYPE_BF16, monitoring=0, want_grad=1, logit_scale=1.0,
                           z_regularization=0.0)
    ws = torch.empty(be.workspace_bytes(prob), dtype=torch.uint8, device="cuda")
    y = torch.zeros(N, dtype=torch.int64, device="cuda")
    be.begin(prob, y, ws)
    bufs = [torch.zeros(be.peer_bytes(prob, torch.bfloat16), dtype=torch.uint8, device="cuda") for _ in range(2)]
    table = _native.PeerTable()
    table.world, table.rank = 2, 0
    table.base[0], table.base[1] = bufs[0].data_ptr(), bufs[1].data_ptr()
    dx = torch.full((N, H), 7.0, dtype=torch.bfloat16, device="cuda")
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    be.dx_finish_peer(prob, 0, N, ws, table, 1, dx, 200)  # nobody ever publishes flag B of epoch 1
    t1.record()
    torch.cuda.synchronize()
    assert 150 < t0.elapsed_time(t1) < 2000
    assert be.read_status(ws) == -6  # LCE_ERR_DEVICE_TIMEOUT
    assert torch.all(dx == 7.0)
    out5 = torch.zeros(5, dtype=torch.float32, device="cuda")
    be.finalize(prob, ws, out5)
    assert torch.isnan(out5[0])


def test_a_rank_whose_wait_ran_out_publishes_nothing_so_its_peers_report_too():
    """Two emulated ranks. Rank 0 never runs its dx contraction, so the owner step of rank 0 runs out of time. It must
    then NOT publish its "rows are staged" flag: rank 1, whose own owner step succeeded, has to run out in its copy
    step as well -- status set, dx untouched -- instead of copying rows that rank 0 never staged. Every wait is
    bounded (200 ms); nothing faults."""
    be = ops.get_backend()
    world, N, H, V, dtype = 2, 256, 256, 1024, torch.bfloat16
    x, y, W = random_problem(N, H, V, dtype, seed=5)
    xd, yd = x.cuda(), y.cuda()
    vl = V // world
    slabs = [W[:, g * vl:(g + 1) * vl].contiguous().cuda() for g in range(world)]
    probs = [_native.Problem(n_rows_total=N, chunk_rows=256, hidden=H, vocab_local=vl, vocab_offset=g * vl,
                             ignore_index=-1, world=world, dtype=_native.DTYPE_BF16, monitoring=0, want_grad=1,
                             logit_scale=1.0, z_regularization=0.0) for g in range(world)]
    ws = [torch.empty(be.workspace_bytes(p), dtype=torch.uint8, device="cuda") for p in probs]
    bufs = [torch.zeros(be.peer_bytes(probs[0], dtype), dtype=torch.uint8, device="cuda") for _ in range(world)]
    tables = []
    for g in range(world):
        t = _native.PeerTable()
        t.world, t.rank = world, g
        for k in range(world):
            t.base[k] = bufs[k].data_ptr()
        tables.append(t)
    parts = torch.empty(world, 6 * 256, dtype=torch.float32, device="cuda")
    dx = [torch.full((N, H), 7.0, dtype=dtype, device="cuda") for _ in range(world)]
    for g in range(world):
        be.begin(probs[g], yd, ws[g])
        be.forward_chunk(probs[g], xd, slabs[g], yd, 0, N, ws[g], parts[g])
    for g in range(world):
        be.combine_chunk(probs[g], parts, yd, 0, N, ws[g])
        be.dz_chunk(probs[g], xd, yd, 0, N, ws[g])
    be.dx_chunk_peer(probs[1], slabs[1], 0, N, ws[1], tables[1], dtype, 1)   # rank 1 scatters and signals; rank 0 never does
    bufs[1][:1024].view(torch.int32)[0] = 1   # as if rank 0's "tiles sent" flag had reached rank 1 only
    for g in range(world):
        be.dx_reduce_peer(probs[g], 0, N, ws[g], tables[g], dtype, 1, 200)   # rank 0 runs out, rank 1 succeeds
    for g in range(world):
        be.dx_finish_peer(probs[g], 0, N, ws[g], tables[g], 1, dx[g], 200)
    torch.cuda.synchronize()
    for g in range(world):
        assert be.read_status(ws[g]) == -6, f"rank {g} must report the timeout"
        assert torch.all(dx[g] == 7.0), f"rank {g} must not have copied anything"


def test_peer_exchange_refuses_what_it_cannot_do():
    be = ops.get_backend()
    prob = _native.Problem(n_rows_total=384, chunk_rows=384, hidden=256, vocab_local=1024, vocab_offset=0,
                           ignore_index=-1, world=2, dtype=_native.DTYPE_BF16, monitoring=0, want_grad=1,
                           logit_scale=1.0, z_regularization=0.0)
    with pytest.raises(_native.LceError):  # 384 rows cannot be split into two owners of whole 128-row tiles
        be.peer_bytes(prob, torch.bfloat16)
    prob.chunk_rows, prob.world = 512, 9
    with pytest.raises(_native.LceError):
        be.peer_bytes(prob, torch.bfloat16)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_nccl_vocab_sharding_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300), str(ROOT / "tests" / "nccl_worker.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "SHARDED_OK" in proc.stdout
