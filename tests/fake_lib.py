"""A stand-in for libflce_b200.so that lets the Python host layer run on CPU tensors.

The compute entry points only record that they were called (outputs stay whatever torch.empty gave them, unless a test
installs a hook), but the small data-movement entry points (row compaction, row scatter) are carried out for real on
host memory, so the bookkeeping built on them can be checked exactly.  Only the tests use this."""

import contextlib
import ctypes as C

import numpy as np
import torch


def _array(addr, ctype, n):
    return np.ctypeslib.as_array((ctype * n).from_address(addr))


def _addr(v):
    if v is None:
        return 0
    return v.value if isinstance(v, C.c_void_p) else int(v)


class FakeLib:
    def __init__(self):
        self.calls = []
        self.hooks = {}
        self.structs = {}

    # ---- entry points with real host-side semantics
    def flce_b200_workspace_bytes(self, p, phase, budget):
        self.calls.append("flce_b200_workspace_bytes")
        return 4096

    def flce_b200_backward_plan(self, p, budget, n_slabs, slab_cols):
        self.calls.append("flce_b200_backward_plan")
        vocab = p._obj.vocab
        n_slabs._obj.value = 3
        slab_cols._obj.value = (vocab + 2) // 3
        return 0

    def flce_b200_compact_rows(self, p, xc, tc, perm, active, stream):
        self.calls.append("flce_b200_compact_rows")
        prob = p._obj
        n, h, ld = prob.n_rows, prob.hidden, prob.ld_x
        tgt = _array(prob.target, C.c_int64, n)
        live = np.nonzero(tgt != prob.ignore_index)[0]
        rest = np.nonzero(tgt == prob.ignore_index)[0]
        order = np.concatenate([live, rest]).astype(np.int32)
        _array(_addr(perm), C.c_int32, n)[:] = order
        _array(_addr(active), C.c_int32, 1)[0] = len(live)
        src = _array(prob.x, C.c_uint16, n * ld).reshape(n, ld)[:, :h]
        _array(_addr(xc), C.c_uint16, n * h).reshape(n, h)[:] = src[order]
        _array(_addr(tc), C.c_int64, n)[:] = tgt[order]
        return 0

    def flce_b200_scatter_rows(self, src, row_bytes, perm, active, n_rows, dst, stream):
        self.calls.append("flce_b200_scatter_rows")
        s = _array(_addr(src), C.c_uint8, n_rows * row_bytes).reshape(n_rows, row_bytes)
        d = _array(_addr(dst), C.c_uint8, n_rows * row_bytes).reshape(n_rows, row_bytes)
        order = _array(_addr(perm), C.c_int32, n_rows)
        live = int(_array(_addr(active), C.c_int32, 1)[0])
        d[order[:live]] = s[:live]
        d[order[live:]] = 0
        return 0

    def flce_b200_last_error(self):
        return b"fake library"

    def flce_b200_status_string(self, status):
        return b"fake status"

    def flce_b200_kernel_launches(self):
        return len(self.calls)

    # ---- everything else: record, run an optional hook, succeed
    def __getattr__(self, name):
        if not name.startswith("flce_b200_"):
            raise AttributeError(name)

        def entry(*args):
            self.calls.append(name)
            for a in args:
                obj = getattr(a, "_obj", None)
                if isinstance(obj, C.Structure):
                    self.structs.setdefault(name, []).append(obj)
            hook = self.hooks.get(name)
            return hook(*args) if hook is not None else 0

        return entry


@contextlib.contextmanager
def installed(monkeypatch):
    """Route the package's host layer to a FakeLib and let it accept CPU tensors."""
    import liger_kernel_b200.ops.cross_entropy as ce
    import liger_kernel_b200.ops.fused_linear_cross_entropy as fl
    import liger_kernel_b200.sharded as sh

    fake = FakeLib()
    for mod in (fl, ce, sh):
        monkeypatch.setattr(mod, "lib", fake)
    monkeypatch.setattr(fl, "_stream", lambda device: None)
    monkeypatch.setattr(fl, "_device_guard", lambda device: contextlib.nullcontext())
    monkeypatch.setattr(fl, "_require_cuda", lambda t: None)
    yield fake


def float_array(addr, n):
    return _array(_addr(addr), C.c_float, n)


def tensor_from(addr, n, dtype=torch.float32):
    ctype = {torch.float32: C.c_float, torch.int64: C.c_int64, torch.int32: C.c_int32}[dtype]
    return torch.from_numpy(_array(_addr(addr), ctype, n))
