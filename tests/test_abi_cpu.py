"""The C-ABI library loads without a GPU and exports every function include/flce_b200.h declares.
No compute entry point is called here."""

import ctypes as C
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "flce_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(flce_b200_\w+)\s*\(", text)))


def test_header_symbols_are_exported():
    from liger_kernel_b200 import _lib

    names = _declared_functions()
    assert len(names) >= 15
    raw = C.CDLL(_lib.LIB_PATH)
    missing = [n for n in names if not hasattr(raw, n)]
    assert not missing, missing
    assert set(_lib.EXPORTS) <= set(names)


def test_struct_sizes_match_header_layout():
    from liger_kernel_b200 import _lib

    # 7 int64 + 2 int32 + int64 + 3 float + 2 int32 (+pad) + 5 pointers
    assert C.sizeof(_lib.Problem) == 7 * 8 + 8 + 8 + 12 + 8 + 4 + 6 * 8
    assert C.sizeof(_lib.ForwardOut) == 7 * 8
    assert C.sizeof(_lib.SceProblem) == 5 * 8 + 8 + 8 + 8 + 3 * 8
    assert C.sizeof(_lib.BackwardArgs) == 4 * 8 + 8 + 3 * 8 + 8 + 6 * 8 + 8 + 2 * 8


def test_host_side_argument_errors_without_gpu():
    from liger_kernel_b200 import _lib

    lib = _lib.lib
    assert lib.flce_b200_version().decode().startswith("flce_b200")
    assert lib.flce_b200_status_string(3).decode() == "workspace too small"
    p = _lib.Problem()
    assert lib.flce_b200_workspace_bytes(C.byref(p), 0, 0) == 0          # empty problem is rejected
    assert b"shapes must be positive" in lib.flce_b200_last_error()
    p.n_rows, p.hidden, p.vocab, p.vocab_total, p.ld_x, p.ld_w = 64, 60, 100, 100, 60, 60
    p.x = p.w = p.target = 16
    assert lib.flce_b200_workspace_bytes(C.byref(p), 0, 0) == 0          # hidden not a multiple of 8
    assert b"multiples of 8" in lib.flce_b200_last_error()
    p.hidden = p.ld_x = p.ld_w = 64
    assert lib.flce_b200_workspace_bytes(C.byref(p), 0, 0) > 0
    n_slabs, cols = C.c_int32(), C.c_int64()
    assert lib.flce_b200_backward_plan(C.byref(p), 64 * 2 * 256, C.byref(n_slabs), C.byref(cols)) == 0
    assert (n_slabs.value, cols.value) == (1, 256)
    # token chunks of the default mode: the height that fills whole waves of the few, long grad_input tiles
    # (hidden / 512 tiles per 256 rows on 74 CTA pairs), within the last quarter of what the 2.5 GiB default allows
    n_chunks, rows = C.c_int32(), C.c_int64()
    for (n, h, v), want in (((32768, 4096, 128256), (4, 9472)),     # 37 x 8 = 4 x 74 tiles per chunk
                            ((32768, 3584, 152064), (5, 7936)),     # 31 x 7 = 217 tiles: 3 waves
                            ((65536, 8192, 128256), (7, 9472)),
                            ((4096, 4096, 128256), (1, 4096))):
        q = _lib.Problem()
        q.n_rows, q.hidden, q.vocab, q.vocab_total, q.ld_x, q.ld_w = n, h, v, v, h, h
        q.x = q.w = q.target = 16
        assert lib.flce_b200_forward_backward_plan(C.byref(q), 0, C.byref(n_chunks), C.byref(rows)) == 0
        assert (n_chunks.value, rows.value) == want, (n, h, v, n_chunks.value, rows.value)
    p.dtype = _lib.FLCE_FP32 + 5
    assert lib.flce_b200_workspace_bytes(C.byref(p), 0, 0) == 0
    assert lib.flce_b200_set_option(b"no_such_option", 1) == 1
    with pytest.raises(_lib.FlceError):
        _lib.set_option("raster_group_bytes", -1)


def test_cpu_tensors_are_rejected_not_computed():
    from liger_kernel_b200 import LigerFusedLinearCrossEntropyLoss

    x = torch.randn(8, 16, dtype=torch.bfloat16)
    w = torch.randn(32, 16, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        LigerFusedLinearCrossEntropyLoss()(w, x, torch.zeros(8, dtype=torch.long))


def test_module_argument_checks_follow_the_reference():
    from liger_kernel_b200 import LigerFusedLinearCrossEntropyLoss

    with pytest.raises(AssertionError, match="label_smoothing must be between"):
        LigerFusedLinearCrossEntropyLoss(label_smoothing=1.5)
    with pytest.raises(AssertionError, match="reduction must be"):
        LigerFusedLinearCrossEntropyLoss(reduction="median")
    with pytest.raises(AssertionError, match="softcap must greater than"):
        LigerFusedLinearCrossEntropyLoss(softcap=0.0)


def test_public_header_is_plain_c(tmp_path):
    """include/flce_b200.h must be usable from C (the boundary is a C ABI): compile a translation unit with gcc -std=c99."""
    import shutil
    import subprocess

    if shutil.which("gcc") is None:
        pytest.skip("gcc not available")
    src = tmp_path / "use_header.c"
    src.write_text('#include "flce_b200.h"\nint main(void) { flce_problem_t p; flce_sce_problem_t q; (void)p; (void)q; return 0; }\n')
    include = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
    done = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-I", include, str(src)],
                          capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
