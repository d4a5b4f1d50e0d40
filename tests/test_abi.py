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
    assert L.cwrnnt_abi_version() == 3


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


def test_pipeline_group_plan_is_host_arithmetic():
    """cwrnnt_pipeline_groups: the number of sequence groups of a pipelined step, from the problem's size alone."""
    def groups(n_rows, V, B, dtype=capi.F32, forced=0):
        p = capi.Problem(n_rows=n_rows, V=V, B=B, y_stride=80, max_u=80, blank=0, dtype=dtype,
                         flags=capi.FUSED_LOG_SOFTMAX)
        return capi.pipeline_groups(p, forced)

    assert groups(314340, 1024, 32) == 4             # 1.29 GB, ordinary batch
    assert groups(1420000, 512, 4) == 8              # a handful of long sequences
    assert groups(40000, 256, 40) == 1               # 41 MB: below 256 MB the step is not cut up
    assert groups(100000, 1024, 32) == 4             # 410 MB
    assert groups(1500, 64, 4) == 1                  # small: no grouping
    assert groups(314340, 1024, 32, forced=3) == 3
    assert groups(300, 1024, 32, forced=8) == 1      # fewer rows than one aligned range
    assert groups(3000, 64, 4, forced=8) == 6        # ranges are multiples of 512 rows
    assert groups(3600000, 128, 256, dtype=capi.F16) == 4
    L = capi.lib()
    p = capi.Problem(n_rows=10, V=8, B=1, y_stride=1, max_u=1, blank=0, dtype=0, flags=0)
    assert L.cwrnnt_pipeline_groups(ctypes.byref(p), 9) < 0
    assert L.cwrnnt_pipeline_groups(ctypes.byref(p), -1) < 0


def test_pipelined_step_rejects_bad_arguments_before_any_launch():
    L = capi.lib()
    p = capi.Problem(n_rows=10, V=8, B=1, y_stride=1, max_u=1, blank=0, dtype=0, flags=capi.COSTS_ONLY)
    args = [None] * 5 + [0, None, None, None, 0, None, None, 0, None, 0, None]
    assert L.cwrnnt_loss_grad(None, ctypes.byref(p), *args) == 1       # costs-only has no gradient
    p.flags = 0
    assert L.cwrnnt_loss_grad(None, ctypes.byref(p), *args) == 1       # null pointers
    args[-2] = 9
    assert L.cwrnnt_loss_grad(None, ctypes.byref(p), *args) == 1       # more groups than supported
    assert L.cwrnnt_scale_grad(ctypes.byref(p), None, None, None) == 1
    out = (ctypes.c_int32 * 4)()
    assert L.cwrnnt_validate(ctypes.byref(p), None, None, None, None, ctypes.byref(out), None) == 1
