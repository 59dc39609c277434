"""Fused linear + cross-entropy loss on B200: the reference's Python surface over the C ABI.

Mirrors ``linear_cross_entropy/ops.py`` of JonasGeiping/linear_cross_entropy_loss:

* ``LinearXentImplementation`` (ops.py:661-810 there): an ``autograd.Function`` that computes the loss
  AND both gradients during ``forward`` -- chunk by chunk over the rows, so that at most one
  ``N_chunk_size x V`` slab is live -- and only rescales them by ``grad_output`` in ``backward``.
* ``linear_cross_entropy`` (ops.py:814-826): functional form returning the 5-tuple
  ``(loss, z_value, logit_max, logit_entropy, logit_norm)``.
* ``LinearCrossEntropyLoss`` (ops.py:830-955): ``nn.Linear`` subclass whose weight is stored
  transposed, ``(in_features, out_features)``.

Everything numeric happens in ``liblce_b200.so`` (hand-written sm_100a kernels); this file only owns
device memory, streams and the chunk loop. There is no CPU or eager fallback.
"""
from __future__ import annotations

import contextlib
import ctypes
import math
import os
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from . import _native
from ._native import DTYPE_BF16, DTYPE_F16, DTYPE_F32, ROW_PARTS, Problem

# The reference exports its Triton autotune lists under these names (linear_cross_entropy/__init__.py:1)
# so that users can trim them. There is nothing to autotune here; the names stay importable.
fwd_configs: list = []
bwd_configs: list = []

_DTYPE_CODE = {torch.float16: DTYPE_F16, torch.bfloat16: DTYPE_BF16, torch.float32: DTYPE_F32}


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class NativeBackend:
    """Calls into liblce_b200.so on the current CUDA stream of the tensors' device."""

    name = "liblce_b200"
    requires_cuda = True

    def __init__(self):
        self.lib = _native.load()

    @staticmethod
    def _stream(t: torch.Tensor) -> int:
        return torch.cuda.current_stream(t.device).cuda_stream

    def workspace_bytes(self, prob: Problem) -> int:
        out = ctypes.c_size_t(0)
        _native.check(self.lib.lce_workspace_bytes(ctypes.byref(prob), ctypes.byref(out)), "lce_workspace_bytes")
        return int(out.value)

    def begin(self, prob, y, workspace):
        _native.check(
            self.lib.lce_begin(ctypes.byref(prob), _ptr(y), _ptr(workspace), self._stream(workspace)), "lce_begin"
        )

    def forward_chunk(self, prob, x, At, y, row0, rows, workspace, row_parts):
        _native.check(
            self.lib.lce_forward_chunk(
                ctypes.byref(prob), _ptr(x), x.stride(0), _ptr(At), At.stride(0), _ptr(y), row0, rows,
                _ptr(workspace), _ptr(row_parts), self._stream(workspace),
            ),
            "lce_forward_chunk",
        )

    def combine_chunk(self, prob, row_parts_all, y, row0, rows, workspace):
        _native.check(
            self.lib.lce_combine_chunk(
                ctypes.byref(prob), _ptr(row_parts_all), _ptr(y), row0, rows, _ptr(workspace), self._stream(workspace)
            ),
            "lce_combine_chunk",
        )

    def parts_bytes(self, prob) -> int:
        out = ctypes.c_size_t(0)
        _native.check(self.lib.lce_parts_bytes(ctypes.byref(prob), ctypes.byref(out)), "lce_parts_bytes")
        return int(out.value)

    def parts_push(self, prob, row_parts, row0, rows, table, epoch, stream_of):
        _native.check(
            self.lib.lce_parts_push(ctypes.byref(prob), _ptr(row_parts), row0, rows, ctypes.byref(table), epoch,
                                    self._stream(stream_of)),
            "lce_parts_push",
        )

    def combine_chunk_peer(self, prob, table, epoch, y, row0, rows, workspace, wait_ms=0):
        _native.check(
            self.lib.lce_combine_chunk_peer(ctypes.byref(prob), ctypes.byref(table), epoch, _ptr(y), row0, rows,
                                            _ptr(workspace), wait_ms, self._stream(workspace)),
            "lce_combine_chunk_peer",
        )

    def dz_chunk(self, prob, x, y, row0, rows, workspace):
        _native.check(
            self.lib.lce_dz_chunk(ctypes.byref(prob), _ptr(x), x.stride(0), _ptr(y), row0, rows, _ptr(workspace),
                                  self._stream(workspace)),
            "lce_dz_chunk",
        )

    def dx_chunk(self, prob, At, row0, rows, workspace, dx):
        _native.check(
            self.lib.lce_dx_chunk(
                ctypes.byref(prob), _ptr(At), At.stride(0), row0, rows, _ptr(workspace), _ptr(dx), dx.stride(0),
                _DTYPE_CODE[dx.dtype], self._stream(workspace),
            ),
            "lce_dx_chunk",
        )

    def peer_bytes(self, prob, dx_dtype) -> int:
        out = ctypes.c_size_t(0)
        _native.check(self.lib.lce_peer_bytes(ctypes.byref(prob), _DTYPE_CODE[dx_dtype], ctypes.byref(out)),
                      "lce_peer_bytes")
        return int(out.value)

    def dx_chunk_peer(self, prob, At, row0, rows, workspace, table, dx_dtype, epoch):
        _native.check(
            self.lib.lce_dx_chunk_peer(
                ctypes.byref(prob), _ptr(At), At.stride(0), row0, rows, _ptr(workspace), ctypes.byref(table),
                _DTYPE_CODE[dx_dtype], epoch, self._stream(workspace),
            ),
            "lce_dx_chunk_peer",
        )

    def dx_reduce_peer(self, prob, row0, rows, workspace, table, dx_dtype, epoch, wait_ms=0):
        _native.check(
            self.lib.lce_dx_reduce_peer(
                ctypes.byref(prob), row0, rows, _ptr(workspace), ctypes.byref(table), _DTYPE_CODE[dx_dtype], epoch,
                wait_ms, self._stream(workspace),
            ),
            "lce_dx_reduce_peer",
        )

    def dx_finish_peer(self, prob, row0, rows, workspace, table, epoch, dx, wait_ms=0):
        _native.check(
            self.lib.lce_dx_finish_peer(
                ctypes.byref(prob), row0, rows, _ptr(workspace), ctypes.byref(table), epoch, _ptr(dx), dx.stride(0),
                _DTYPE_CODE[dx.dtype], wait_ms, self._stream(workspace),
            ),
            "lce_dx_finish_peer",
        )

    def dw_chunk(self, prob, x, row0, rows, workspace, dW, dW_res, first, last):
        _native.check(
            self.lib.lce_dw_chunk(
                ctypes.byref(prob), _ptr(x), x.stride(0), row0, rows, _ptr(workspace), _ptr(dW), dW.stride(0),
                _ptr(dW_res), 0 if dW_res is None else dW_res.stride(0), 1 if first else 0, 1 if last else 0,
                self._stream(workspace),
            ),
            "lce_dw_chunk",
        )

    def fused_pass(self, prob, x, At, y, workspace, row_parts, dx, dW, dW_res, out5):
        _native.check(
            self.lib.lce_fused_pass(
                ctypes.byref(prob), _ptr(x), x.stride(0), _ptr(At), At.stride(0), _ptr(y), _ptr(workspace),
                _ptr(row_parts), _ptr(dx), 0 if dx is None else dx.stride(0), _DTYPE_CODE[x.dtype], _ptr(dW),
                0 if dW is None else dW.stride(0), _ptr(dW_res), 0 if dW_res is None else dW_res.stride(0),
                _ptr(out5), self._stream(workspace),
            ),
            "lce_fused_pass",
        )

    def finalize(self, prob, workspace, out5):
        _native.check(
            self.lib.lce_finalize(ctypes.byref(prob), _ptr(workspace), _ptr(out5), self._stream(workspace)),
            "lce_finalize",
        )

    def grad_scale_cast(self, src, dst, factor):
        cols = -(-src.shape[1] // 8) * 8  # whole groups of 8: the padding columns of an aligned-rows buffer go along
        assert cols <= src.stride(0) and cols <= dst.stride(0)
        _native.check(
            self.lib.lce_grad_scale_cast(
                _ptr(src), _DTYPE_CODE[src.dtype], src.stride(0), _ptr(dst), _DTYPE_CODE[dst.dtype], dst.stride(0),
                src.shape[0], cols, _ptr(factor), self._stream(src),
            ),
            "lce_grad_scale_cast",
        )

    def rerun_stats_async(self, workspace, host_int32x2) -> None:
        _native.check(self.lib.lce_rerun_stats_async(_ptr(workspace), host_int32x2.data_ptr(),
                                                     self._stream(workspace)), "lce_rerun_stats_async")

    def read_status(self, workspace) -> int:
        return int(self.lib.lce_read_status(_ptr(workspace), self._stream(workspace)))


_backend = None


def get_backend():
    """The object the chunk loop drives. Always the native library outside of unit tests."""
    global _backend
    if _backend is None:
        _backend = NativeBackend()
    return _backend


def set_backend(backend) -> None:
    """Test hook: substitute the object that receives the per-chunk calls (None restores the library)."""
    global _backend
    _backend = backend


@dataclass
class ShardSpec:
    """Vocabulary sharding of W over the ranks of a process group (None = the whole W is local).

    gather_row_parts(local[ROW_PARTS * chunk_rows]) -> all[world * ROW_PARTS * chunk_rows] (rank-major)
    reduce_dx(dx_rows) sums the chunk's dx rows over the ranks, in place.
    peer_exchange(prob, dx_dtype) -> None or an object with ``table`` (a ``_native.PeerTable``), ``next_epoch()``
    and ``wait_ms``: when given, dx is exchanged by the contraction's own stores into peer-mapped memory
    (``lce_dx_chunk_peer`` and friends) and reduce_dx is not called.
    parts_exchange(prob) -> None or an object with ``table``, ``next_epoch()`` and ``wait_ms``: when given, the row
    partials travel by stores into peer-mapped memory (``lce_parts_push`` / ``lce_combine_chunk_peer``) instead of
    gather_row_parts, and the chunks are software-pipelined: the forward of chunk c + 1 is enqueued before the combine
    and backward steps of chunk c, so nobody waits for partials that have not had a whole backward step to arrive.
    reduce_dx_once: reduce_dx is called once, with the whole dx, after the last chunk (one collective and one
    cross-rank synchronisation point per pass) instead of once per chunk with that chunk's rows.
    """

    rank: int
    world: int
    vocab_offset: int
    gather_row_parts: Callable[[torch.Tensor], torch.Tensor]
    reduce_dx: Callable[[torch.Tensor], None]
    peer_exchange: Optional[Callable] = None
    parts_exchange: Optional[Callable] = None
    reduce_dx_once: bool = False


# A chunk whose row count allows it is processed as this many sub-chunks, so that the memory-bound slab transform
# of one sub-chunk runs on a second stream underneath the tensor-core kernels of the other.
SUBCHUNKS = 2
MIN_SPLIT_ELEMS = 1 << 25  # slab elements of a chunk from which halving pays (equal on all ranks of a sharded run)
# Rows a half must keep. Measured inside the power-capped step (fp16, per-tile slabs, A/B inside one call): chunks
# of 8192 rows as two halves 193.4 ms per step against 196.0 whole (N=65536, H=4096, V=131072); chunks of 4096 rows
# as two halves between 2 % slower and 1 % faster than whole over four calls at the default shape (a half of 2048
# rows streams the weight a second time), with 56 instead of 32 launches per step and no single-call pass.
MIN_HALF_ROWS = 4096
_side_streams: dict = {}


def _side_stream(device: torch.device, role: str = "slab"):
    key = (device.type, device.index, role)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]


def _split_rows(row0: int, rows: int, split: bool):
    """Sub-chunks of a chunk: halves when each half keeps the 256-row granularity of the CTA-pair kernels.
    Only the per-tile slab mode has a slab-wide transform worth hiding; the default mode of bf16 / fp32 runs a
    chunk as one piece."""
    if split and SUBCHUNKS == 2 and rows >= 2 * MIN_HALF_ROWS and rows % 512 == 0:
        return [(row0, rows // 2), (row0 + rows // 2, rows // 2)]
    return [(row0, rows)]


def _wants_subchunks(per_tile: bool, want_grad: bool, dtype, sharded: bool) -> bool:
    """Whether chunks are processed as two halves. Every half issues its own collectives in a sharded run, so there
    the answer may only depend on values that are equal on all ranks: the slab mode is not one of them (each rank
    picks it from its own re-run counters and a polled event), the dtype is. The row partials a rank exports are
    the same in both modes (base, sums), so ranks in different modes still combine correctly."""
    if not want_grad:
        return False
    return dtype == torch.float16 if sharded else per_tile


class SlabModePolicy:
    """Picks ``lce_problem.slab_mode`` for bf16 / fp32 passes (fp16 always normalises per tile).

    The default mode keeps one base per row and recomputes the row groups whose logits leave the window around
    it; with very wide logits (standard deviation of a row's logits beyond about 50, e.g. the reference's
    ``A~randn`` benchmark inputs at H >= 4096) that happens in most chunks and the per-tile mode is faster.
    ``LCE_SLAB_MODE=row|tile`` fixes the mode; ``auto`` (default) uses per-tile slabs for small chunks (below 2^24
    slab elements, where launches count and the slab pass does not) and otherwise starts in the default mode, reads -- without
    ever synchronising: a pinned-memory copy plus an event that is only polled -- how many row groups the last
    finished pass of the same shape recomputed, switches to per-tile above ``threshold`` and tries the default
    mode again every ``retry_every`` passes. Polling an event is not allowed while a stream is being captured
    into a CUDA graph: fix the mode with ``LCE_SLAB_MODE`` when capturing passes.
    """

    threshold = 0.25
    retry_every = 64
    # chunks whose slab has fewer elements than this always use per-tile slabs: the in-place pass over such a slab
    # takes microseconds, and the mode needs fewer launches per chunk (no conditional re-run pair, no probe)
    small_slab_elems = 1 << 24

    def __init__(self):
        self.history = {}

    def choose(self, key, dtype) -> int:
        if dtype == torch.float16:
            return _native.SLAB_PER_TILE
        forced = os.environ.get("LCE_SLAB_MODE", "auto")
        if forced == "row":
            return _native.SLAB_DEFAULT
        if forced == "tile":
            return _native.SLAB_PER_TILE
        if key[3] * key[4] < self.small_slab_elems:  # key = (device, dtype, H, V, rows per chunk, world)
            return _native.SLAB_PER_TILE
        h = self.history.get(key)
        if h is None:
            return _native.SLAB_DEFAULT
        self._poll(h)
        if h["fraction"] <= self.threshold:
            return _native.SLAB_DEFAULT
        h["tile_passes"] += 1
        if h["tile_passes"] % self.retry_every == 0:
            return _native.SLAB_DEFAULT
        return _native.SLAB_PER_TILE

    @staticmethod
    def _poll(h) -> None:
        if h["event"] is not None and h["event"].query():
            rerun, seen = h["host"].tolist()
            h["event"] = None
            if seen > 0:
                h["fraction"] = rerun / seen

    def record(self, key, backend, workspace) -> None:
        """After a default-mode pass: start the copy of its re-run counters (no synchronisation)."""
        h = self.history.get(key)
        if h is None:
            h = self.history[key] = {"host": torch.zeros(2, dtype=torch.int32).pin_memory(), "event": None,
                                     "fraction": 0.0, "tile_passes": 0}
        if h["event"] is not None:  # the previous copy has not been seen to finish: leave it alone
            self._poll(h)
            if h["event"] is not None:
                return
        backend.rerun_stats_async(workspace, h["host"])
        h["event"] = torch.cuda.Event()
        h["event"].record(torch.cuda.current_stream(workspace.device))


slab_mode_policy = SlabModePolicy()


def run_pass(x, y, At, ignore_index, z_regularization, logit_scale, N_chunk_size, monitoring, want_grad,
             shard: Optional[ShardSpec] = None):
    """One forward(+gradient) pass over all row chunks.

    x: (N, H) with unit inner stride, y: (N,) int64 contiguous, At: (H, V_local) with unit inner stride.
    Returns (out5, dx, dW, workspace): out5 = float32[5] (loss, z_value, logit_max, logit_entropy,
    logit_norm); dx (N, H) and dW (H, V_local) in the dtype of x / At, or None without want_grad.
    Follows the chunk loop of the reference (ops.py:721-791): per chunk forward, [all-gather of the row
    partials,] log-sum-exp combine, dZ preparation, dx, dW accumulation. For fp16 -- whose dZ preparation is a
    pass over the whole slab -- a chunk runs as two sub-chunks and the combine + slab pass of one sub-chunk go
    to a second stream, underneath the tensor-core kernels of the other.
    """
    backend = get_backend()
    # want_grad: a bool, or (gradient for x wanted, gradient for the weight wanted) -- a frozen head or frozen
    # features skip the contraction whose result nobody asks for (a third of the pass each)
    want_dx, want_dW = (want_grad, want_grad) if isinstance(want_grad, bool) else (bool(want_grad[0]), bool(want_grad[1]))
    want_grad = want_dx or want_dW
    native = getattr(backend, "requires_cuda", True)
    if native and not (x.is_cuda and y.is_cuda and At.is_cuda):
        raise RuntimeError("linear_cross_entropy_loss_b200 runs on CUDA tensors only; there is no CPU fallback")
    N, H = x.shape
    H_A, V = At.shape
    assert H_A == H, "x and the weight disagree on the hidden size"
    assert y.shape == (N,), "labels must have one entry per row of x"
    assert x.dtype == At.dtype, "x and the weight must have the same dtype"
    assert x.dtype in _DTYPE_CODE, f"unsupported dtype {x.dtype}"
    assert y.dtype == torch.int64, "labels must be int64"
    assert N >= 1, "x must have at least one row"
    assert logit_scale > 0 and z_regularization >= 0
    assert int(N_chunk_size) >= 1
    if H % 8 != 0:
        # The kernels move rows of x in 16-byte units. A hidden size that is not a multiple of 8 runs on copies
        # padded with zero columns of x and zero rows of the weight: the logits do not change, and the gradients of
        # the padding are dropped again (they are zero columns of dx and unused rows of dW).
        H8 = -(-H // 8) * 8
        x_pad = x.new_zeros((N, H8))
        x_pad[:, :H] = x
        A_pad = _aligned_rows_like((H8, V), At.dtype, At.device)
        A_pad[:H] = At
        A_pad[H:] = 0
        out5, dx, dW, workspace = run_pass(x_pad, y, A_pad, ignore_index, z_regularization, logit_scale, N_chunk_size,
                                           monitoring, (want_dx, want_dW), shard)
        # dx stays a view of the padded buffer: its rows keep the 16-byte alignment the rescaling kernel of backward needs
        return out5, (None if dx is None else dx[:, :H]), (None if dW is None else dW[:H]), workspace
    # rows per chunk as in the reference (ops.py:687), rounded up to the 128-row tile of the kernels
    N_group = -(-min(N, int(N_chunk_size)) // 128) * 128

    world = 1 if shard is None else shard.world
    policy_key = (x.device.index, x.dtype, H, V, N_group, world)
    slab_mode = slab_mode_policy.choose(policy_key, x.dtype)
    per_tile = slab_mode == _native.SLAB_PER_TILE
    # chunks too small to halve, or whose slab pass is too short to be worth hiding (the per-step calls from Python
    # then cost more than the overlap gains), run whole on one stream -- unsharded as one library call
    split = (_wants_subchunks(per_tile, want_grad, x.dtype, shard is not None)
             and len(_split_rows(0, N_group, True)) > 1 and N_group * V >= MIN_SPLIT_ELEMS)
    prob = Problem(
        n_rows_total=N, chunk_rows=N_group, hidden=H, vocab_local=V,
        vocab_offset=0 if shard is None else shard.vocab_offset, ignore_index=int(ignore_index), world=world,
        dtype=_DTYPE_CODE[x.dtype], monitoring=1 if monitoring else 0, want_grad=1 if want_grad else 0,
        logit_scale=float(logit_scale), z_regularization=float(z_regularization), slab_mode=slab_mode,
    )
    dev = x.device
    n_chunks = -(-N // N_group)
    # Row partials over peer memory (sharded runs): whether it is used depends only on values that are equal on all
    # ranks. It comes with software pipelining of the chunks, which needs a second set of per-chunk buffers.
    parts = None
    if shard is not None and shard.parts_exchange is not None and not split:
        parts = shard.parts_exchange(prob)
        if parts is not None and n_chunks > 1:
            prob.chunk_buffers = 2
    workspace = torch.empty(backend.workspace_bytes(prob), dtype=torch.uint8, device=dev)
    row_parts = torch.empty(ROW_PARTS * N_group, dtype=torch.float32, device=dev)
    out5 = torch.empty(5, dtype=torch.float32, device=dev)
    dx = dW = dW_res = None
    if want_dW:
        dW = _aligned_rows_like((H, V), At.dtype, dev)
        if n_chunks > 1 and At.dtype != torch.float32:
            # Across chunks the 16-bit gradient is carried as dW + dW_res (the rounding error of dW, in the same
            # type): about 16 significant bits, no fp32 buffer the size of W, and dW is complete after the last chunk.
            dW_res = _aligned_rows_like((H, V), At.dtype, dev)

    # second stream only where sub-chunks exist (per-tile slabs); everything else runs in order on the caller's stream
    use_side = native and dev.type == "cuda" and split and SUBCHUNKS == 2
    main = torch.cuda.current_stream(dev) if use_side else None
    side = _side_stream(dev) if use_side else None

    def on_side(after_event):
        if side is None:
            return contextlib.nullcontext()
        side.wait_event(after_event)
        return torch.cuda.stream(side)

    peer = None
    if shard is not None and want_dx and shard.peer_exchange is not None and parts is None:
        peer = shard.peer_exchange(prob, x.dtype)
    dx_once = shard is not None and shard.reduce_dx_once and peer is None
    if want_dx:
        # fp16 partial sums that an all-reduce adds up travel as fp32: with dx around 1e-6 (1 / n_valid) every rank's
        # partial would otherwise be rounded to fp16's absolute spacing of 6e-8 before the sum (measured on 2 GPUs at
        # the default shape: cosine to the float64 dx 0.99986, against 0.99991 for the one rounding an fp16 result
        # needs anyway). The caller's backward converts while it applies grad_output (_scaled_grads). bf16 has the
        # exponent range of fp32 and the peer exchange sums in fp32 itself, so both keep the input type.
        wide = shard is not None and peer is None and x.dtype == torch.float16
        dx = torch.empty((N, H), dtype=torch.float32 if wide else x.dtype, device=dev)

    peer_done = []
    xstream = None
    if peer is not None and getattr(peer, "overlap", False):
        xstream = _side_stream(dev, "exchange")

    if (shard is None and not use_side and hasattr(backend, "fused_pass")
            and os.environ.get("LCE_FUSED_PASS", "1") != "0"):
        # unsharded, one stream: the whole pass is ONE call into the library (same kernels, same order as the loop
        # below; what it saves is host time per call, which is all that small problems cost)
        backend.fused_pass(prob, x, At, y, workspace, row_parts, dx, dW, dW_res, out5)
        if native and not per_tile and x.dtype != torch.float16 and os.environ.get("LCE_SLAB_MODE", "auto") == "auto":
            slab_mode_policy.record(policy_key, backend, workspace)
        return out5, dx, dW, workspace
    backend.begin(prob, y, workspace)
    chunks = [] if parts is None else [(ci, r0, min(N_group, N - r0)) for ci, r0 in enumerate(range(0, N, N_group))]
    if parts is not None:
        # Pipelined order:  F0 P0 | F1 P1 C0 B0 | F2 P2 C1 B1 | ... | C(n-1) B(n-1)   (F forward, P push of the row
        # partials to all ranks, C wait + combine, B backward). Consecutive chunks use alternate slabs.
        def forward_and_push(ci, r0, n):
            backend.forward_chunk(prob, x, At, y, r0, n, workspace, row_parts)
            epoch = parts.next_epoch()
            backend.parts_push(prob, row_parts, r0, n, parts.table, epoch, workspace)
            return epoch

        epochs = {0: forward_and_push(*chunks[0])}
    for ci, row0, rows in chunks:
        if ci + 1 < n_chunks:
            epochs[ci + 1] = forward_and_push(*chunks[ci + 1])
        backend.combine_chunk_peer(prob, parts.table, epochs.pop(ci), y, row0, rows, workspace, parts.wait_ms)
        if want_grad:
            backend.dz_chunk(prob, x, y, row0, rows, workspace)
            if want_dx:
                backend.dx_chunk(prob, At, row0, rows, workspace, dx)
                if not dx_once:
                    shard.reduce_dx(dx[row0:row0 + rows])
            if want_dW:
                backend.dw_chunk(prob, x, row0, rows, workspace, dW, dW_res, ci == 0, ci == n_chunks - 1)
    for ci, row0 in enumerate(range(0, N, N_group) if parts is None else ()):
        rows = min(N_group, N - row0)
        subs = _split_rows(row0, rows, split)
        ready = []
        for r0, n in subs:
            backend.forward_chunk(prob, x, At, y, r0, n, workspace, row_parts)
            fwd_done = None
            if side is not None:
                fwd_done = torch.cuda.Event()
                fwd_done.record(main)
            with on_side(fwd_done):
                parts_all = row_parts if shard is None else shard.gather_row_parts(row_parts)
                backend.combine_chunk(prob, parts_all, y, r0, n, workspace)
                if want_grad:
                    backend.dz_chunk(prob, x, y, r0, n, workspace)
                if side is not None:
                    done = torch.cuda.Event()
                    done.record(side)
                    ready.append(done)
        if want_grad:
            for i, (r0, n) in enumerate(subs):
                if side is not None:
                    main.wait_event(ready[i])
                if not want_dx:
                    continue
                if peer is not None:
                    # The contraction scatters its tiles to the owning ranks; the owners' sum, the broadcast and the
                    # copy into dx follow on a second stream, underneath the next contractions (they wait for other
                    # ranks, this stream never does). Two epochs may be in flight: one per half of the buffers.
                    epoch = peer.next_epoch()
                    if xstream is None:  # everything in order on one stream
                        backend.dx_chunk_peer(prob, At, r0, n, workspace, peer.table, dx.dtype, epoch)
                        backend.dx_reduce_peer(prob, r0, n, workspace, peer.table, dx.dtype, epoch, peer.wait_ms)
                        backend.dx_finish_peer(prob, r0, n, workspace, peer.table, epoch, dx, peer.wait_ms)
                        continue
                    cur = torch.cuda.current_stream(dev)
                    if len(peer_done) >= 2:
                        cur.wait_event(peer_done[-2])
                    backend.dx_chunk_peer(prob, At, r0, n, workspace, peer.table, dx.dtype, epoch)
                    scattered = torch.cuda.Event()
                    scattered.record(cur)
                    xstream.wait_event(scattered)
                    with torch.cuda.stream(xstream):
                        backend.dx_reduce_peer(prob, r0, n, workspace, peer.table, dx.dtype, epoch, peer.wait_ms)
                        backend.dx_finish_peer(prob, r0, n, workspace, peer.table, epoch, dx, peer.wait_ms)
                        done = torch.cuda.Event()
                        done.record(xstream)
                    peer_done.append(done)
                    continue
                backend.dx_chunk(prob, At, r0, n, workspace, dx)
                if shard is not None and not dx_once:
                    shard.reduce_dx(dx[r0:r0 + n])
            if want_dW:
                backend.dw_chunk(prob, x, row0, rows, workspace, dW, dW_res, ci == 0, ci == n_chunks - 1)
    if side is not None:
        main.wait_stream(side)
    if xstream is not None:
        torch.cuda.current_stream(dev).wait_stream(xstream)
    if dx_once and want_dx:
        shard.reduce_dx(dx)
    backend.finalize(prob, workspace, out5)
    if native and not per_tile and x.dtype != torch.float16 and os.environ.get("LCE_SLAB_MODE", "auto") == "auto":
        slab_mode_policy.record(policy_key, backend, workspace)
    return out5, dx, dW, workspace


def _device_guard(t: torch.Tensor):
    """Makes the tensor's GPU current (needed for devices other than 0, as in reference ops.py:680)."""
    return torch.cuda.device(t.device) if t.is_cuda else contextlib.nullcontext()


def _aligned_rows_like(shape, dtype, device):
    """An uninitialised (rows, cols) tensor whose rows start on 16-byte boundaries: a view of a buffer that is a few
    columns wider when cols is not a multiple of 8 (vocabulary sizes such as 50257)."""
    rows, cols = shape
    ld = -(-cols // 8) * 8  # whole groups of 8 elements: 16 bytes for 16-bit types, 32 for fp32 (vector accesses)
    buf = torch.empty((rows, ld), dtype=dtype, device=device)
    return buf if ld == cols else buf[:, :cols]


def _tma_ready(t):
    return t.stride(-1) == 1 and (t.stride(0) * t.element_size()) % 16 == 0 and t.data_ptr() % 16 == 0


def _prepare(x_in, y, At):
    x = x_in.reshape(-1, x_in.shape[-1])
    if not _tma_ready(x):
        x = x.contiguous()
    y = y.reshape(-1)
    if not y.is_contiguous():
        y = y.contiguous()
    if not _tma_ready(At):  # e.g. a vocabulary size that is not a multiple of 8: copy into 16-byte aligned rows
        copy = _aligned_rows_like(At.shape, At.dtype, At.device)
        copy.copy_(At)
        At = copy
    return x, y, At


def _scaled_grads(ctx, grad_output):
    """grad * grad_output, in place (reference ops.py:804-810). The gradients already have the dtype of their
    inputs; when grad_output is exactly 1 -- a plain loss.backward() -- the kernels leave them untouched."""
    backend = get_backend()
    dx, dW = ctx.lce_grads  # either may be None: the input did not require grad, so its contraction never ran
    ctx.lce_grads = None
    dev = dx.device if dx is not None else dW.device
    factor = grad_output.detach().reshape(1).to(device=dev, dtype=torch.float32).contiguous()
    if dx is not None:
        dx_dtype = getattr(ctx, "lce_x_dtype", dx.dtype)
        if dx.dtype != dx_dtype:  # fp32 sums of a sharded fp16 pass (run_pass): scale and convert in one kernel
            narrow = _aligned_rows_like(tuple(dx.shape), dx_dtype, dev)
            backend.grad_scale_cast(dx, narrow, factor)
            dx = narrow
        else:
            backend.grad_scale_cast(dx, dx, factor)
        dx = dx.reshape(ctx.lce_x_shape)
    if dW is not None:
        backend.grad_scale_cast(dW, dW, factor)
    return dx, dW


class LinearXentImplementation(torch.autograd.Function):
    """Same call signature and outputs as the reference's autograd function (ops.py:661-810)."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, x_in, y, At, ignore_index=-100, z_regularization: float = 0.0, logit_scale: float = 1.0,
                N_chunk_size: int = 4096, monitoring: bool = True):
        # Under CUDA autocast the decorator casts floating inputs to fp16 and disables autocast
        # inside, exactly as the reference does (ops.py:665-667).
        with _device_guard(x_in):
            x, y_flat, A = _prepare(x_in, y, At)
            want = (bool(ctx.needs_input_grad[0]), bool(ctx.needs_input_grad[2]))
            with torch.no_grad():
                out5, dx, dA, _ = run_pass(x, y_flat, A, ignore_index, z_regularization, logit_scale, N_chunk_size,
                                           monitoring, want)
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
        with _device_guard(grad_output), torch.no_grad():
            gx, gA = _scaled_grads(ctx, grad_output)
        return gx, None, gA, None, None, None, None, None


# ------------------------------------------------------------------------------------------------
# torch.library registration: the same pass as ONE opaque operator, so that torch.compile / export can
# trace through a model that contains the loss without a graph break (the reference cannot be traced:
# its author lists this as open, reference ops.py:706 and README). Eager calls keep using the
# autograd.Function above; the operator is picked while a compiler is tracing.
# ------------------------------------------------------------------------------------------------
@torch.library.custom_op("lce_b200::fused_pass", mutates_args=())
def fused_pass_op(x: torch.Tensor, y: torch.Tensor, At: torch.Tensor, ignore_index: int, z_regularization: float,
                  logit_scale: float, N_chunk_size: int, monitoring: bool,
                  want_grad: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(out5, dx, dW): out5 = float32[5] (loss, z_value, logit_max, logit_entropy, logit_norm); the gradients of the
    loss with respect to x and At (empty tensors without want_grad)."""
    with _device_guard(x):
        x2, y_flat, A = _prepare(x, y, At)
        out5, dx, dA, _ = run_pass(x2, y_flat, A, ignore_index, z_regularization, logit_scale, N_chunk_size,
                                   monitoring, want_grad)
    if not want_grad:
        return out5, x.new_empty(0), At.new_empty(0)
    return out5, dx.reshape(x.shape), dA


@fused_pass_op.register_fake
def _fused_pass_fake(x, y, At, ignore_index, z_regularization, logit_scale, N_chunk_size, monitoring, want_grad):
    out5 = x.new_empty(5, dtype=torch.float32)
    if not want_grad:
        return out5, x.new_empty(0), At.new_empty(0)
    return out5, x.new_empty(x.shape), At.new_empty(At.shape)


def _fused_pass_setup(ctx, inputs, output):
    ctx.lce_want_grad = inputs[-1]
    ctx.save_for_backward(output[1], output[2])


def _fused_pass_backward(ctx, grad_out5, grad_dx, grad_dW):
    if not ctx.lce_want_grad:
        raise RuntimeError("the fused loss was traced without gradients")
    dx, dW = ctx.saved_tensors
    g = grad_out5[0]  # only the loss is differentiable (reference ops.py:804-810)
    return (dx * g).to(dx.dtype), None, (dW * g).to(dW.dtype), None, None, None, None, None, None


fused_pass_op.register_autograd(_fused_pass_backward, setup_context=_fused_pass_setup)

# What CUDA autocast does to the inputs: "reference" = cast to fp16 whatever the autocast dtype is, as the
# reference does (ops.py:665-667); "follow" = cast to the autocast dtype (bf16 autocast -> bf16 kernels).
_AUTOCAST_POLICY = "reference"


def set_autocast_policy(policy: str) -> None:
    global _AUTOCAST_POLICY
    assert policy in ("reference", "follow")
    _AUTOCAST_POLICY = policy


def _autocast_target(x) -> Optional[torch.dtype]:
    if not x.is_cuda or not torch.is_autocast_enabled("cuda"):
        return None
    return torch.float16 if _AUTOCAST_POLICY == "reference" else torch.get_autocast_dtype("cuda")


def _apply(x, y, At, ignore_index, z_regularization, logit_scale, N_chunk_size, monitoring):
    """The 5-tuple of the reference's autograd function, through the operator that fits the calling context."""
    if not torch.is_grad_enabled():
        # Evaluation under torch.no_grad() with a trainable weight: inside autograd.Function.forward the inputs still
        # look as if they needed gradients, so the gradient kernels would run for nothing (as they do in the
        # reference, which always computes them). Detached inputs select the forward-only pass.
        x, At = x.detach(), At.detach()
    if torch.compiler.is_compiling():
        target = _autocast_target(x)
        if target is not None:
            x, At = x.to(target), At.to(target)
        want_grad = torch.is_grad_enabled() and (x.requires_grad or At.requires_grad)
        out5, _, _ = fused_pass_op(x, y, At, int(ignore_index), float(z_regularization), float(logit_scale),
                                   int(N_chunk_size), bool(monitoring), want_grad)
        return out5[0], out5[1].detach(), out5[2].detach(), out5[3].detach(), out5[4].detach()
    if _AUTOCAST_POLICY == "follow" and _autocast_target(x) is not None:
        target = _autocast_target(x)
        with torch.autocast(device_type="cuda", enabled=False):
            return LinearXentImplementation.apply(x.to(target), y, At.to(target), ignore_index, z_regularization,
                                                  logit_scale, N_chunk_size, monitoring)
    return LinearXentImplementation.apply(x, y, At, ignore_index, z_regularization, logit_scale, N_chunk_size,
                                          monitoring)


def linear_cross_entropy(
    x,
    y,
    At,
    ignore_index=-100,
    z_regularization: float = 0.0,
    logit_scale: float = 1.0,
    N_chunk_size: int = 4096,
    monitoring: bool = False,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Functional form (reference ops.py:814-826): returns (loss, z_value, logit_max, logit_entropy, logit_norm)."""
    return _apply(x, y, At, ignore_index, z_regularization, logit_scale, N_chunk_size, monitoring)  # type: ignore


class LinearCrossEntropyLoss(torch.nn.Linear):
    r"""``z = x @ weight`` followed at once by the cross-entropy of ``z`` with labels ``y``; returns the scalar loss.

    Drop-in for the reference module (ops.py:830-955): same constructor, attributes and ``state_dict``
    (one key, ``weight``, of shape ``(in_features, out_features)`` -- transposed with respect to
    ``nn.Linear``; there is no bias). It subclasses ``nn.Linear`` so that code which looks for linear
    layers (initialisation, weight decay groups) finds it.

    Setting ``module.monitoring = True`` makes ``forward`` also fill ``module.latest_metrics`` with
    ``logit_norm``, ``logit_max``, ``logit_entropy`` and ``z_value``, defined as in the reference's
    ``reference_torch`` (ops.py:9-17).

    Differences from the reference, all of them relaxations: any number of rows, any H and any V (the
    reference needs N % 512, H % 256, V % 4096; sizes that are not multiples of 8 run on padded copies), there is no autotuning on the first call, and gradients are
    only computed when an input requires them.
    """

    def __init__(
        self,
        in_features: int,
        out_features: int,
        device=None,
        dtype=None,
        ignore_index: int = -100,
        logit_scale: float = 1.0,
        z_regularization: float = 0.0,
        N_chunk_size: int = 4096,
        init_method=None,
    ):
        factory_kwargs = {"device": device, "dtype": dtype}
        torch.nn.Module.__init__(self)  # not nn.Linear.__init__: no bias, transposed weight

        assert in_features >= 1
        assert out_features >= 1
        assert N_chunk_size >= 1
        assert logit_scale > 0
        assert z_regularization >= 0

        self.in_features = in_features
        self.out_features = out_features
        self.weight = torch.nn.Parameter(torch.empty((in_features, out_features), **factory_kwargs))

        self.logit_scale = logit_scale
        self.ignore_index = ignore_index
        self.z_regularization = z_regularization
        self.N_chunk_size = N_chunk_size

        self.monitoring = False
        self.latest_metrics = {}
        self.init_method = init_method

        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.init_method is not None:
            self.init_method(self.weight)
        else:
            std = math.sqrt(1 / self.in_features)
            torch.nn.init.trunc_normal_(self.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)

    def forward(self, x, y):
        loss, z_reg, logit_max, logit_ent, logit_norm = _apply(
            x, y, self.weight, self.ignore_index, self.z_regularization, self.logit_scale, self.N_chunk_size,
            self.monitoring,
        )  # type: ignore
        if self.monitoring:
            self.latest_metrics = {
                "logit_norm": logit_norm,
                "logit_max": logit_max,
                "logit_entropy": logit_ent,
                "z_value": z_reg,
            }
        return loss

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias=False"
