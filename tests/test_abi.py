"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header declares, and rejects bad
descriptors without touching a GPU."""
import ctypes
import os
import re

from compactwarprnntloss_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "cwarp_rnnt_b200.h")).read()
    return sorted(set(re.findall(r"CWRNNT_API[^;(]*?\b(cwrnnt_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from compactwarprnntloss_b200 import build
    build.build_library()
    L = capi.lib()
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(L, n), n
    assert sorted(capi.EXPORTS) == names
    assert L.cwrnnt_abi_version() == 2


def test_descriptor_validation_and_workspace_size():
    L = capi.lib()
    p = capi.Problem(n_rows=1000, V=64, B=4, y_stride=9, max_u=9, blank=0, dtype=capi.F32, flags=capi.FUSED_LOG_SOFTMAX)
    n = L.cwrnnt_workspace_bytes(ctypes.byref(p))
    assert n >= 40 * 1000 and n % 256 == 0
    p2 = capi.Problem(n_rows=2000, V=64, B=4, y_stride=9, max_u=9, blank=0, dtype=capi.F32)
    assert L.cwrnnt_workspace_bytes(ctypes.byref(p2)) > n
    for bad in (dict(blank=64), dict(blank=-1), dict(dtype=7), dict(flags=0x100), dict(y_stride=3),
                dict(flags=capi.REDUCE_MEAN | capi.REDUCE_SUM), dict(n_rows=-1), dict(max_u=capi.MAX_COLUMNS)):
        kw = dict(n_rows=10, V=64, B=1, y_stride=9, max_u=9, blank=0, dtype=0, flags=0)
        kw.update(bad)
        if "max_u" in bad:
            kw["y_stride"] = bad["max_u"]
        assert L.cwrnnt_workspace_bytes(ctypes.byref(capi.Problem(**kw))) < 0, bad
    assert L.cwrnnt_status_string(2).decode().startswith("workspace")
    assert L.cwrnnt_scatter_scratch_bytes(10) == 256


def test_null_pointers_are_rejected_before_any_launch():
    L = capi.lib()
    p = capi.Problem(n_rows=10, V=8, B=1, y_stride=1, max_u=1, blank=0, dtype=0, flags=0)
    assert L.cwrnnt_forward(ctypes.byref(p), None, None, None, None, None, 0, None, None, None) == 1
    assert L.cwrnnt_backward(ctypes.byref(p), None, None, None, None, None, None, 0, None, None) == 1
