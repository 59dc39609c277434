"""Vocabulary-sharded execution of the fused loss over the GPUs of one node.

Rank g of a process group holds the column slab ``W[:, g*V/G:(g+1)*V/G]`` of the (H, V) weight; ``x``
and ``y`` are replicated. Per row chunk:

1. every rank runs the forward GEMM on its slab and produces six per-row partials
   (base, sum exp, target logit, sum exp*z, sum z^2, max);
2. ONE small all-gather (``6 * chunk_rows`` floats per rank) makes all partials visible everywhere and a
   local kernel merges them in rank order into the global log-sum-exp -- bitwise identical on every
   rank, which a max/sum all-reduce pair would not guarantee;
   ``LCE_PEER_PARTS=1`` selects a form without that collective: every rank stores its partials into all ranks'
   peer-mapped buffers and publishes a flag (``PartsExchange``), and the chunks are software-pipelined -- the
   forward of chunk c + 1 is enqueued before the combine and backward of chunk c, on two alternating slabs -- so
   the partials of a chunk have a whole backward step to arrive before anyone waits for them (bounded waits).
   Measured on 2 and 4 x B200 it does not beat the all-gather (22.6-22.8 against 22.3 ms per step on 4 GPUs at the
   default shape, 45.9 against 45.2 ms on the 65536 x 4096 x 131072 case), so the all-gather stays the default;
3. every rank forms dZ for its slab, its own dW slab (no communication) and a partial dx, which is
   summed over the ranks with ONE all-reduce of the whole dx at the end of the pass (``LCE_DX_REDUCE=chunk``:
   one all-reduce per chunk, of that chunk's rows, in stream order). ``LCE_PEER_DX=1`` selects the device-side exchange instead (``PeerExchange``): the epilogue of
   the dx contraction stores each fp32 output tile into peer-mapped memory of the rank that owns the
   rows, the owner adds the tiles of all ranks in a fixed order, rounds once and stores the finished rows
   back to everyone, on a second stream underneath the next contractions; dx is then bitwise identical
   on all ranks and rounded once instead of twice. Measured on 8 x B200 it is 1 % faster than the all-reduce
   at the default shape (22.24 against 22.48 ms per step), equal on 2 and 4 GPUs, and 2.5 % slower when the
   slab per rank is small (N=65536, H=4096, 16384 columns per rank: 24.33 against 23.73 ms): NCCL reduces
   inside the NVSwitch, the scatter moves fp32 partials of twice the volume. It needs 0.3 GB of peer-mapped
   memory per rank, so it is opt-in.

The reference has no multi-GPU path; the collectives here are NCCL through ``torch.distributed`` (gloo on
CPU in the unit tests). Loss and metrics come out identical on all ranks.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.distributed as dist

from . import _native, ops
from ._native import ROW_PARTS


class _Collectives:
    """The two per-chunk exchanges of one pass, with their scratch buffer and pending work handles."""

    def __init__(self, group, world: int):
        self.group = group
        self.world = world
        self.gathered: Optional[torch.Tensor] = None
        self.pending = []

    def gather_row_parts(self, local: torch.Tensor) -> torch.Tensor:
        if self.gathered is None:
            self.gathered = torch.empty(self.world * local.numel(), dtype=local.dtype, device=local.device)
        try:
            dist.all_gather_into_tensor(self.gathered, local, group=self.group)
        except (RuntimeError, NotImplementedError):  # backend without a flat all-gather
            dist.all_gather(list(self.gathered.chunk(self.world)), local, group=self.group)
        return self.gathered

    def reduce_dx(self, dx_rows: torch.Tensor) -> None:
        # In stream order by default: measured on 4 x B200, an all-reduce that overlaps the next contraction takes
        # SMs away from that persistent one-CTA-per-SM kernel and costs more (23.10 ms per step) than it hides
        # (22.57 ms in order; 22.32 ms on one GPU). LCE_OVERLAP_DX_REDUCE=1 selects the overlapped form.
        if os.environ.get("LCE_OVERLAP_DX_REDUCE") == "1":
            self.pending.append(dist.all_reduce(dx_rows, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        else:
            dist.all_reduce(dx_rows, op=dist.ReduceOp.SUM, group=self.group)

    def wait_all(self) -> None:
        for work in self.pending:
            work.wait()
        self.pending.clear()


class PeerExchange:
    """Peer-mapped exchange buffers (one per rank, symmetric memory) for the dx partials of one process group.

    Built collectively by all ranks of the group on first use for a given size and kept for the life of the
    process; ``next_epoch`` must advance identically on all ranks, which it does when all ranks run the same
    sequence of passes.
    """

    _cache = {}
    _unavailable = set()

    def __init__(self, group, nbytes: int, device: torch.device):
        import torch.distributed._symmetric_memory as symm

        pg = group if group is not None else dist.group.WORLD
        self.buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, pg)
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        ptrs = list(self.handle.buffer_ptrs)
        assert len(ptrs) == world and ptrs[rank] == self.buf.data_ptr()
        self.table = _native.PeerTable()
        self.table.world, self.table.rank = world, rank
        for g in range(world):
            self.table.base[g] = ptrs[g]
        self.epoch = 0
        self.wait_ms = int(os.environ.get("LCE_PEER_WAIT_MS", "0"))
        self.overlap = os.environ.get("LCE_PEER_OVERLAP", "1") != "0"
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's flags are zero before anyone signals

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    @classmethod
    def for_problem(cls, group, prob, dx_dtype, device) -> Optional["PeerExchange"]:
        """The exchange for this problem, or None when the all-reduce has to be used instead. The decision
        depends only on values that are equal on all ranks."""
        backend = ops.get_backend()
        world = dist.get_world_size(group)
        if (os.environ.get("LCE_PEER_DX", "0") != "1" or not getattr(backend, "requires_cuda", True)
                or device.type != "cuda" or world < 2 or world > _native.MAX_PEERS
                or prob.chunk_rows % (128 * world) != 0):
            return None
        gid = id(group) if group is not None else 0
        if (gid, device.index) in cls._unavailable:
            return None
        nbytes = backend.peer_bytes(prob, dx_dtype)
        key = (gid, device.index, nbytes)
        if key not in cls._cache:
            try:
                cls._cache[key] = cls(group, nbytes, device)
            except (RuntimeError, ImportError, AssertionError) as err:  # no peer mapping between these GPUs
                cls._unavailable.add((gid, device.index))
                print(f"linear_cross_entropy_loss_b200: peer exchange unavailable ({err}); using all-reduce")
                return None
        return cls._cache[key]


class PartsExchange:
    """Peer-mapped buffers (one per rank, symmetric memory) through which the ranks hand each other the per-row
    softmax partials of a chunk: every rank stores its partials into all ranks' buffers and publishes a flag
    (``lce_parts_push``); the combine step waits for the flags with a bounded wait (``lce_combine_chunk_peer``).
    Replaces the per-chunk all-gather, a cross-rank synchronisation in the middle of every chunk.

    Built collectively on first use for a given size and kept for the life of the process. ``next_epoch`` must
    advance identically on all ranks, which it does when all ranks run the same sequence of passes.
    Opt-in (``LCE_PEER_PARTS=1``): measured on 2 and 4 x B200 it ties with or loses 1-2 % to the all-gather, and it
    holds a second slab per rank."""

    _cache = {}
    _unavailable = set()

    def __init__(self, group, nbytes: int, device: torch.device):
        import torch.distributed._symmetric_memory as symm

        pg = group if group is not None else dist.group.WORLD
        self.buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, pg)
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        ptrs = list(self.handle.buffer_ptrs)
        assert len(ptrs) == world and ptrs[rank] == self.buf.data_ptr()
        self.table = _native.PeerTable()
        self.table.world, self.table.rank = world, rank
        for g in range(world):
            self.table.base[g] = ptrs[g]
        self.epoch = 0
        self.wait_ms = int(os.environ.get("LCE_PEER_WAIT_MS", "0"))
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's flags are zero before anyone signals

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    @classmethod
    def for_problem(cls, group, prob, device) -> Optional["PartsExchange"]:
        """The exchange for this problem, or None when the all-gather has to be used. The decision depends only on
        values that are equal on all ranks."""
        backend = ops.get_backend()
        world = dist.get_world_size(group)
        if (os.environ.get("LCE_PEER_PARTS", "0") != "1" or os.environ.get("LCE_PEER_DX", "0") == "1"
                or not getattr(backend, "requires_cuda", True) or device.type != "cuda" or world < 2
                or world > _native.MAX_PEERS):
            return None
        gid = id(group) if group is not None else 0
        if (gid, device.index) in cls._unavailable:
            return None
        nbytes = backend.parts_bytes(prob)
        key = (gid, device.index, nbytes)
        if key not in cls._cache:
            try:
                cls._cache[key] = cls(group, nbytes, device)
            except (RuntimeError, ImportError, AssertionError) as err:  # no peer mapping between these GPUs
                cls._unavailable.add((gid, device.index))
                print(f"linear_cross_entropy_loss_b200: peer exchange of row partials unavailable ({err}); "
                      f"using all-gather")
                return None
        return cls._cache[key]


class VocabShardedLinearXent(torch.autograd.Function):
    """Sharded counterpart of ``ops.LinearXentImplementation``: same outputs, W given as this rank's slab."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, x_in, y, At_shard, group=None, ignore_index=-100, z_regularization: float = 0.0,
                logit_scale: float = 1.0, N_chunk_size: int = 4096, monitoring: bool = False):
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        with ops._device_guard(x_in):
            x, y_flat, A = ops._prepare(x_in, y, At_shard)
            v_local = A.shape[1]
            coll = _Collectives(group, world)
            spec = ops.ShardSpec(rank=rank, world=world, vocab_offset=rank * v_local,
                                 gather_row_parts=coll.gather_row_parts, reduce_dx=coll.reduce_dx,
                                 peer_exchange=lambda prob, dt: PeerExchange.for_problem(group, prob, dt, x.device),
                                 parts_exchange=lambda prob: PartsExchange.for_problem(group, prob, x.device),
                                 reduce_dx_once=os.environ.get("LCE_DX_REDUCE", "pass") != "chunk")
            want = (bool(ctx.needs_input_grad[0]), bool(ctx.needs_input_grad[2]))
            with torch.no_grad():
                out5, dx, dA, _ = ops.run_pass(x, y_flat, A, ignore_index, z_regularization, logit_scale,
                                               N_chunk_size, monitoring, want, shard=spec)
                coll.wait_all()
            ctx.lce_grads = (dx, dA) if any(want) else None
            ctx.lce_x_shape = x_in.shape
            ctx.lce_x_dtype = x.dtype
            loss, z_value, logit_max, logit_ent, logit_norm = out5.unbind(0)
            ctx.mark_non_differentiable(z_value, logit_max, logit_ent, logit_norm)
            return loss, z_value, logit_max, logit_ent, logit_norm

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_output, void0, void1, void2, void3):
        if ctx.lce_grads is None:
            raise RuntimeError("backward called twice, or forward ran without any input requiring grad")
        with ops._device_guard(grad_output), torch.no_grad():
            gx, gA = ops._scaled_grads(ctx, grad_output)
        return gx, None, gA, None, None, None, None, None, None


def linear_cross_entropy_sharded(x, y, At_shard, group=None, ignore_index=-100, z_regularization: float = 0.0,
                                 logit_scale: float = 1.0, N_chunk_size: int = 4096, monitoring: bool = False):
    """``linear_cross_entropy`` with W sharded by columns over ``group``. x and y must be equal on all ranks.

    Returns the same 5-tuple on every rank. ``x.grad`` is the full gradient (summed over the shards),
    ``At_shard.grad`` is the gradient of this rank's slab.
    """
    if not torch.is_grad_enabled():  # evaluation under torch.no_grad(): forward-only pass (see ops._apply)
        x, At_shard = x.detach(), At_shard.detach()
    return VocabShardedLinearXent.apply(x, y, At_shard, group, ignore_index, z_regularization, logit_scale,
                                        N_chunk_size, monitoring)


class VocabShardedLinearCrossEntropyLoss(torch.nn.Module):
    """``LinearCrossEntropyLoss`` whose weight is this rank's ``(in_features, out_features / world)`` slab.

    ``full_weight_init`` (default) draws the whole ``(in_features, out_features)`` matrix from one seeded
    generator on every rank and keeps the local columns, so the sharded module starts from the same
    weights as an unsharded one built with the same ``init_seed``.
    """

    def __init__(self, in_features: int, out_features: int, group=None, device=None, dtype=None,
                 ignore_index: int = -100, logit_scale: float = 1.0, z_regularization: float = 0.0,
                 N_chunk_size: int = 4096, init_seed: int = 0):
        super().__init__()
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        assert in_features >= 1
        assert out_features % (8 * world) == 0, "every rank's slab must be a multiple of 8 columns"
        assert N_chunk_size >= 1
        assert logit_scale > 0 and z_regularization >= 0
        self.group = group
        self.in_features, self.out_features = in_features, out_features
        self.local_features = out_features // world
        self.vocab_offset = rank * self.local_features
        self.ignore_index, self.logit_scale = ignore_index, logit_scale
        self.z_regularization, self.N_chunk_size = z_regularization, N_chunk_size
        self.monitoring = False
        self.latest_metrics = {}
        self.weight = torch.nn.Parameter(torch.empty((in_features, self.local_features), device=device, dtype=dtype))
        self.reset_parameters(init_seed)

    def reset_parameters(self, seed: int = 0) -> None:
        std = math.sqrt(1 / self.in_features)
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for h0 in range(0, self.in_features, 64):
                h1 = min(self.in_features, h0 + 64)
                blk = torch.empty((h1 - h0, self.out_features))
                torch.nn.init.trunc_normal_(blk, mean=0.0, std=std, a=-3 * std, b=3 * std, generator=g)
                self.weight[h0:h1] = blk[:, self.vocab_offset:self.vocab_offset + self.local_features].to(
                    device=self.weight.device, dtype=self.weight.dtype)

    def forward(self, x, y):
        loss, z_reg, logit_max, logit_ent, logit_norm = linear_cross_entropy_sharded(
            x, y, self.weight, self.group, self.ignore_index, self.z_regularization, self.logit_scale,
            self.N_chunk_size, self.monitoring)
        if self.monitoring:
            self.latest_metrics = {"logit_norm": logit_norm, "logit_max": logit_max, "logit_entropy": logit_ent,
                                   "z_value": z_reg}
        return loss

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"local_features={self.local_features}, bias=False")
