"""Tensor-parallel slice planner over the C ABI (mirrors cpp_runtime/tensor_parallel.h:23-118
and tensor_parallel_granularity, cpp_runtime/mfq_decode.cpp:9445-9461)."""

from __future__ import annotations

import ctypes as C

from ._capi import check, lib


def plan_tensor_parallel_slices(extent: int, granularity: int, devices, weights=()):
    """Return ``[(device, begin, end), ...]``; raises ``MfqbError`` where the reference throws."""
    n = len(devices)
    if len(weights) not in (0, n):
        from ._capi import ERR_ARG, MfqbError
        raise MfqbError(ERR_ARG, "tensor-parallel split count must match device count")
    b, e = (C.c_int64 * max(n, 1))(), (C.c_int64 * max(n, 1))()
    w = (C.c_double * n)(*weights) if len(weights) else None
    check(lib.mfqb_tp_plan(extent, granularity, n, w, b, e))
    return [(devices[i], b[i], e[i]) for i in range(n)]


def validate_tensor_parallel_slices(slices, extent: int, granularity: int) -> None:
    n = len(slices)
    b = (C.c_int64 * max(n, 1))(*[s[1] for s in slices])
    e = (C.c_int64 * max(n, 1))(*[s[2] for s in slices])
    check(lib.mfqb_tp_validate(extent, granularity, n, b, e))


def tensor_parallel_granularity(extent: int, preferred: int, n_devices: int) -> int:
    out = C.c_int64()
    check(lib.mfqb_tp_granularity(extent, preferred, n_devices, C.byref(out)))
    return out.value
