"""The C-ABI shared library without a GPU: it builds, loads, exports every symbol the header declares,
and rejects bad arguments with status codes before touching a device."""
import ctypes
import re
from pathlib import Path

import pytest

from linear_cross_entropy_loss_b200 import _native

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "lce_b200.h").read_text()


@pytest.fixture(scope="module")
def lib():
    return _native.load()


def declared_functions():
    return sorted(set(re.findall(r"^(?:int|long long|const char\*)\s+(lce_\w+)\s*\(", HEADER, flags=re.M)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for required in ["lce_begin", "lce_forward_chunk", "lce_combine_chunk", "lce_backward_chunk", "lce_finalize",
                     "lce_grad_scale_cast", "lce_workspace_bytes", "lce_status_string", "lce_version"]:
        assert required in names


def test_library_exports_every_declared_symbol(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in lce_b200.h but not exported"
    assert set(_native.SIGNATURES) == set(declared_functions())


def test_every_entry_point_cites_the_reference_or_says_it_has_no_counterpart():
    assert HEADER.count("ops.py:") >= 8
    assert "No counterpart in the reference" in HEADER


def test_header_is_plain_c_and_the_ctypes_mirrors_have_its_layout(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 on its own, and the ctypes structures must have the
    size and field offsets the C compiler gives lce_problem and lce_peer_table."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    fields_p = [f[0] for f in _native.Problem._fields_]
    fields_t = [f[0] for f in _native.PeerTable._fields_]
    src = tmp_path / "layout.c"
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{ROOT / "include" / "lce_b200.h"}"', "int main(void) {",
             '  printf("%zu\\n", sizeof(lce_problem));']
    lines += [f'  printf("%zu\\n", offsetof(lce_problem, {f}));' for f in fields_p]
    lines += ['  printf("%zu\\n", sizeof(lce_peer_table));']
    lines += [f'  printf("%zu\\n", offsetof(lce_peer_table, {f}));' for f in fields_t]
    lines += ["  return 0;", "}"]
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-pedantic", "-o", str(exe), str(src)], check=True)
    got = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    want = [ctypes.sizeof(_native.Problem)] + [getattr(_native.Problem, f).offset for f in fields_p]
    want += [ctypes.sizeof(_native.PeerTable)] + [getattr(_native.PeerTable, f).offset for f in fields_t]
    assert got == want


def test_any_vocabulary_size_is_a_valid_problem(lib):
    rc, nbytes = workspace_bytes(lib, problem(vocab_local=4001))
    assert rc == 0 and nbytes > 0


def test_version_and_status_strings(lib):
    assert lib.lce_version() >= 100
    assert _native.status_string(0) == "ok"
    seen = {_native.status_string(code) for code in range(-8, 1)}
    assert len(seen) == 9 and "unknown status" not in seen
    assert _native.status_string(-99) == "unknown status"


def problem(**kw):
    base = dict(n_rows_total=1024, chunk_rows=256, hidden=256, vocab_local=4096, vocab_offset=0, ignore_index=-100,
                world=1, dtype=_native.DTYPE_BF16, monitoring=0, want_grad=1, logit_scale=1.0, z_regularization=0.0)
    base.update(kw)
    return _native.Problem(**base)


def workspace_bytes(lib, p):
    out = ctypes.c_size_t(0)
    return lib.lce_workspace_bytes(ctypes.byref(p), ctypes.byref(out)), out.value


def test_workspace_size_accounts_for_slab_statistics_and_partials(lib):
    rc, nbytes = workspace_bytes(lib, problem())
    assert rc == 0
    slab = 256 * 4096 * 2
    stats = 2 * (4096 // 256) * 256 * 4
    assert nbytes >= slab + stats + 256 * 256 * 4
    assert nbytes < 2 * (slab + stats) + 16 * 256 * 256 * 4
    rc, fwd_only = workspace_bytes(lib, problem(want_grad=0))
    assert rc == 0 and fwd_only < slab
    rc, mon = workspace_bytes(lib, problem(monitoring=1))
    assert rc == 0 and mon == nbytes + stats
    # headline shape: slab + split-K partials stay below N_chunk x V x 4 bytes
    rc, big = workspace_bytes(lib, problem(n_rows_total=16384, chunk_rows=4096, hidden=2048, vocab_local=131072))
    assert rc == 0 and big <= 4096 * 131072 * 4


@pytest.mark.parametrize("kw,code", [
    (dict(dtype=7), -1), (dict(hidden=0), -1), (dict(logit_scale=0.0), -1), (dict(z_regularization=-1.0), -1),
    (dict(world=0), -1), (dict(n_rows_total=0), -1),
    (dict(hidden=100), -2), (dict(chunk_rows=192), -2), (dict(slab_mode=5), -1), (dict(chunk_buffers=3), -1),
    (dict(vocab_local=1 << 31), -8),
])
def test_invalid_problems_are_rejected_without_a_device(lib, kw, code):
    rc, _ = workspace_bytes(lib, problem(**kw))
    assert rc == code
    # the same validation guards the launching entry points (checked before any CUDA call)
    assert lib.lce_begin(ctypes.byref(problem(**kw)), 16, 16, None) == code


def test_null_pointers_are_rejected(lib):
    p = problem()
    assert lib.lce_begin(ctypes.byref(p), None, None, None) == -1
    assert lib.lce_forward_chunk(ctypes.byref(p), None, 256, None, 4096, None, 0, 256, None, None, None) == -1
    assert lib.lce_finalize(ctypes.byref(p), None, None, None) == -1
    assert lib.lce_grad_scale_cast(None, 0, 1, None, 0, 1, 1, 1, None, None) == -1
    assert lib.lce_read_status(None, None) == -1
    assert lib.lce_workspace_bytes(None, None) == -1


def test_one_call_pass_checks_its_arguments_before_touching_a_device(lib):
    p = problem()
    args = lambda prob, **kw: (ctypes.byref(prob), 16, 256, 16, 4096, 16, kw.get("ws", 16), 16, kw.get("dx", 16), 256, 1,
                               kw.get("dw", 16), 4096, 16, 4096, 16, None)
    assert lib.lce_fused_pass(*args(problem(world=2))) == -1          # sharded callers issue the steps themselves
    assert lib.lce_fused_pass(*args(p, ws=None)) == -1
    assert lib.lce_fused_pass(*args(p, dx=None, dw=None)) == -1       # gradients wanted but no output given
    assert lib.lce_fused_pass(*args(problem(want_grad=0))) == -1      # outputs given but no gradient wanted
    assert lib.lce_fused_pass(*args(problem(hidden=100))) == -2


def test_exchange_buffer_sizes_need_no_device(lib):
    out = ctypes.c_size_t(0)
    p = problem(world=4)
    assert lib.lce_parts_bytes(ctypes.byref(p), ctypes.byref(out)) == 0
    assert out.value >= 1024 + 4 * 4 * 6 * 256 * 4                      # flags + 4 slots x world x 6 x chunk rows floats
    assert lib.lce_parts_bytes(ctypes.byref(problem(world=9)), ctypes.byref(out)) == -1
    two = ctypes.c_size_t(0)
    assert lib.lce_workspace_bytes(ctypes.byref(problem(chunk_buffers=2)), ctypes.byref(two)) == 0
    rc, one = workspace_bytes(lib, problem())
    assert one < two.value < 2 * one


def test_chunk_bounds_are_checked(lib):
    p = problem()
    args = (16, 256, 16, 4096, 16)
    assert lib.lce_forward_chunk(ctypes.byref(p), *args, 0, 512, 16, 16, None) == -1    # more rows than a chunk
    assert lib.lce_forward_chunk(ctypes.byref(p), *args, 1024, 256, 16, 16, None) == -1  # past the end
    assert lib.lce_forward_chunk(ctypes.byref(p), *args, 64, 128, 16, 16, None) == -2    # unaligned start
    assert lib.lce_forward_chunk(ctypes.byref(p), *args, 0, 100, 16, 16, None) == -2     # ragged rows not at the end
    assert lib.lce_forward_chunk(ctypes.byref(p), *args, 768, 300, 16, 16, None) == -1   # crosses a chunk boundary


def test_launch_counter_starts_at_zero_without_a_gpu(lib):
    assert lib.lce_launch_count() >= 0
