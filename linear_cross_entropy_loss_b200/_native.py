"""ctypes binding of ``liblce_b200.so`` (the C ABI declared in ``include/lce_b200.h``).

The shared library is built in-tree by :func:`build` (``nvcc`` for sm_100a) and loaded with
``ctypes``; there is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import threading
from pathlib import Path

_PKG_DIR = Path(__file__).resolve().parent
_CSRC = _PKG_DIR / "csrc"
_INCLUDE = _PKG_DIR.parent / "include"
# LCE_B200_LIB points at an alternative build of the library (A/B measurements); it is used as it is, never rebuilt.
_OVERRIDE = os.environ.get("LCE_B200_LIB")
LIB_PATH = Path(_OVERRIDE) if _OVERRIDE else _PKG_DIR / "liblce_b200.so"

LCE_OK = 0
DTYPE_F16, DTYPE_BF16, DTYPE_F32 = 0, 1, 2
ROW_PARTS = 6

_lock = threading.Lock()
_lib = None


class LceError(RuntimeError):
    """A call into liblce_b200 returned a non-zero status."""

    def __init__(self, status: int, message: str, where: str):
        super().__init__(f"{where}: {message} (status {status})")
        self.status = status


class Problem(ctypes.Structure):
    """Mirror of ``lce_problem`` (include/lce_b200.h)."""

    _fields_ = [
        ("n_rows_total", ctypes.c_int64),
        ("chunk_rows", ctypes.c_int64),
        ("hidden", ctypes.c_int64),
        ("vocab_local", ctypes.c_int64),
        ("vocab_offset", ctypes.c_int64),
        ("ignore_index", ctypes.c_int64),
        ("world", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
        ("monitoring", ctypes.c_int32),
        ("want_grad", ctypes.c_int32),
        ("logit_scale", ctypes.c_float),
        ("z_regularization", ctypes.c_float),
        ("slab_mode", ctypes.c_int32),
        ("chunk_buffers", ctypes.c_int32),
    ]


def _sources():
    return sorted(list(_CSRC.glob("*.cu")) + list(_CSRC.glob("*.cuh")) + list(_INCLUDE.glob("*.h")))


def needs_build() -> bool:
    if _OVERRIDE:
        return False
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(src.stat().st_mtime > built for src in _sources())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA sources for sm_100a into ``liblce_b200.so`` next to this file."""
    if not force and not needs_build():
        return LIB_PATH
    # One build at a time across PROCESSES too: under torchrun every rank may find the library stale at once.
    # The file lock serialises them; whoever gets it second finds the library fresh and returns.
    import fcntl

    with open(_PKG_DIR / ".build.lock", "w") as lock_file:
        fcntl.flock(lock_file, fcntl.LOCK_EX)
        try:
            if not force and not needs_build():
                return LIB_PATH
            return _build_locked(verbose)
        finally:
            fcntl.flock(lock_file, fcntl.LOCK_UN)


def _build_locked(verbose: bool) -> Path:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: liblce_b200.so cannot be built")
    tmp = LIB_PATH.parent / f"{LIB_PATH.name}.{os.getpid()}.tmp"
    cmd = [
        nvcc,
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-O3", "-lineinfo", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC",
        "-I", str(_INCLUDE),
        "-o", str(tmp),
        str(_CSRC / "lce_api.cu"),
    ]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    os.replace(tmp, LIB_PATH)
    if verbose:
        print(proc.stderr)
    return LIB_PATH


_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_i32 = ctypes.c_int32
_u32 = ctypes.c_uint32

MAX_PEERS = 8
SLAB_DEFAULT, SLAB_PER_TILE = 0, 1


class PeerTable(ctypes.Structure):
    """Mirror of ``lce_peer_table``: every rank's exchange buffer as addressed from this GPU."""

    _fields_ = [("world", ctypes.c_int32), ("rank", ctypes.c_int32), ("base", ctypes.c_void_p * MAX_PEERS)]


# name -> (restype, argtypes); kept in one table so that a test can check it against the header.
SIGNATURES = {
    "lce_version": (ctypes.c_int, []),
    "lce_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "lce_launch_count": (ctypes.c_longlong, []),
    "lce_workspace_bytes": (ctypes.c_int, [ctypes.POINTER(Problem), ctypes.POINTER(ctypes.c_size_t)]),
    "lce_begin": (ctypes.c_int, [ctypes.POINTER(Problem), _vp, _vp, _vp]),
    "lce_forward_chunk": (ctypes.c_int, [ctypes.POINTER(Problem), _vp, _i64, _vp, _i64, _vp, _i64, _i64, _vp, _vp, _vp]),
    "lce_combine_chunk": (ctypes.c_int, [ctypes.POINTER(Problem), _vp, _vp, _i64, _i64, _vp, _vp]),
    "lce_parts_bytes": (ctypes.c_int, [ctypes.POINTER(Problem), ctypes.POINTER(ctypes.c_size_t)]),
    "lce_parts_push": (ctypes.c_int, [ctypes.POINTER(Problem), _vp, _i64, _i64, ctypes.POINTER(PeerTable), _u32, _vp]),
    "lce_combine_chunk_peer": (
        ctypes.c_int, [ctypes.POINTER(Problem), ctypes.POINTER(PeerTable), _u32, _vp, _i64, _i64, _vp, _i32, _vp]),
    "lce_dz_chunk": (ctypes.c_int, [ctypes.POINTER(Problem), _vp, _i64, _vp, _i64, _i64, _vp, _vp]),
    "lce_dx_chunk": (ctypes.c_int, [ctypes.POINTER(Problem), _vp, _i64, _i64, _i64, _vp, _vp, _i64, _i32, _vp]),
    "lce_peer_bytes": (ctypes.c_int, [ctypes.POINTER(Problem), _i32, ctypes.POINTER(ctypes.c_size_t)]),
    "lce_dx_chunk_peer": (
        ctypes.c_int, [ctypes.POINTER(Problem), _vp, _i64, _i64, _i64, _vp, ctypes.POINTER(PeerTable), _i32, _u32, _vp]),
    "lce_dx_reduce_peer": (
        ctypes.c_int, [ctypes.POINTER(Problem), _i64, _i64, _vp, ctypes.POINTER(PeerTable), _i32, _u32, _i32, _vp]),
    "lce_dx_finish_peer": (
        ctypes.c_int,
        [ctypes.POINTER(Problem), _i64, _i64, _vp, ctypes.POINTER(PeerTable), _u32, _vp, _i64, _i32, _i32, _vp]),
    "lce_dw_chunk": (
        ctypes.c_int, [ctypes.POINTER(Problem), _vp, _i64, _i64, _i64, _vp, _vp, _i64, _vp, _i64, _i32, _i32, _vp]),
    "lce_backward_chunk": (
        ctypes.c_int,
        [ctypes.POINTER(Problem), _vp, _i64, _vp, _i64, _vp, _i64, _i64, _vp, _vp, _i64, _i32, _vp, _i64, _vp, _i64,
         _i32, _i32, _vp],
    ),
    "lce_fused_pass": (
        ctypes.c_int,
        [ctypes.POINTER(Problem), _vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i32, _vp, _i64, _vp, _i64, _vp, _vp],
    ),
    "lce_finalize": (ctypes.c_int, [ctypes.POINTER(Problem), _vp, _vp, _vp]),
    "lce_grad_scale_cast": (ctypes.c_int, [_vp, _i32, _i64, _vp, _i32, _i64, _i64, _i64, _vp, _vp]),
    "lce_read_status": (ctypes.c_int, [_vp, _vp]),
    "lce_rerun_stats_async": (ctypes.c_int, [_vp, _vp, _vp]),
    "lce_eval_loss_static": (ctypes.c_int, [ctypes.POINTER(Problem), _vp, _i64, _vp, _i64, _vp, _vp, _vp]),
    "lce_profile_enable": (ctypes.c_int, [_i32]),
    "lce_profile_read": (ctypes.c_int, [ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_longlong)]),
    "lce_debug_gemm": (
        ctypes.c_int,
        [_i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _vp, _vp],
    ),
}


def load():
    """Load (building first if the sources are newer) and return the ctypes library handle."""
    global _lib
    with _lock:
        if _lib is None:
            if needs_build():
                build()
            lib = ctypes.CDLL(str(LIB_PATH))
            for name, (restype, argtypes) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = restype
                fn.argtypes = argtypes
            _lib = lib
    return _lib


def status_string(status: int) -> str:
    return load().lce_status_string(status).decode()


def check(status: int, where: str) -> None:
    if status != LCE_OK:
        raise LceError(status, status_string(status), where)


def launch_count() -> int:
    return int(load().lce_launch_count())


def profile_enable(on: bool) -> None:
    check(load().lce_profile_enable(1 if on else 0), "lce_profile_enable")


def profile_read():
    """({"fwd": ms, "dx": ms, "dw": ms}, {"fwd": launches, ...}) since the previous read."""
    ms = (ctypes.c_double * 3)()
    n = (ctypes.c_longlong * 3)()
    check(load().lce_profile_read(ms, n), "lce_profile_read")
    names = ("fwd", "dx", "dw")
    return {k: ms[i] for i, k in enumerate(names)}, {k: int(n[i]) for i, k in enumerate(names)}
