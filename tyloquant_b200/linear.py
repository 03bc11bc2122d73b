"""Dense quantized weights on a GPU (mirrors ``NintWeight`` / ``NvqWeight`` with
``nint_matmul`` / ``nvq_matmul`` / ``QuantLinear::forward`` of the reference runtime,
cpp_runtime/mfq_decode.cpp:2102-2165, 4027-4055, 8130-8315, 7884-7932, 9209).

torch is used only for device memory and streams; all arithmetic runs in the library."""

from __future__ import annotations

import ctypes as C

from . import _capi
from ._capi import BF16, F32, WeightInfo, check, lib


def _torch():
    import torch
    return torch


def _stream_ptr(device_index: int) -> int:
    return _torch().cuda.current_stream(device_index).cuda_stream


class QuantWeight:
    """One NINT or NVQ3 tensor, decoded from its MFQ blob into the device layout."""

    def __init__(self, handle: C.c_void_p):
        self._h = handle
        info = WeightInfo()
        check(lib.mfqb_weight_info_get(self._h, C.byref(info)))
        self.info = info
        self.n, self.k, self.device = info.n, info.k, info.device

    @classmethod
    def from_blob(cls, dtype: str, blob, device: int = 0, *, axis: int = 0, begin: int = 0, end: int = -1):
        addr, n, keep = _capi.buffer_address(blob)
        h = C.c_void_p()
        check(lib.mfqb_weight_from_blob_slice(dtype.encode(), addr, n, axis, begin, end, device, C.byref(h)))
        del keep
        return cls(h)

    def clone(self) -> "QuantWeight":
        """A second handle with its own device copy (no host-side re-layout)."""
        h = C.c_void_p()
        check(lib.mfqb_weight_clone(self._h, C.byref(h)))
        return QuantWeight(h)

    @property
    def payload_bytes(self) -> int:
        return self.info.payload_bytes

    @property
    def device_bytes(self) -> int:
        return self.info.device_bytes

    def dequantize(self, dtype="float32"):
        """[n, k] tensor: float32 is bit-identical to the reference decoder."""
        torch = _torch()
        tdt = torch.float32 if str(dtype).endswith("float32") else torch.bfloat16
        out = torch.empty((self.n, self.k), dtype=tdt, device=f"cuda:{self.device}")
        check(lib.mfqb_dequant(self._h, out.data_ptr(), F32 if tdt == torch.float32 else BF16, _stream_ptr(self.device)))
        return out

    def matmul(self, x, out_dtype=None, out=None):
        """``y = x @ W.T`` for a bf16 CUDA tensor ``x`` of shape [m, k] (or [k]); ``out``: an
        existing [m, n] float32 or bfloat16 tensor to write (graph capture wants fixed buffers)."""
        torch = _torch()
        squeeze = x.dim() == 1
        x2 = x.reshape(1, -1) if squeeze else x
        if x2.dtype != torch.bfloat16 or not x2.is_cuda or x2.device.index != self.device:
            raise ValueError(f"x must be a bfloat16 tensor on cuda:{self.device}")
        if x2.shape[-1] != self.k:
            raise ValueError(f"x has {x2.shape[-1]} columns, the weight has k={self.k}")
        x2 = x2.contiguous()
        tdt = out.dtype if out is not None else (out_dtype or torch.bfloat16)
        y = out if out is not None else torch.empty((x2.shape[0], self.n), dtype=tdt, device=x2.device)
        if y.shape != (x2.shape[0], self.n) or not y.is_contiguous():
            raise ValueError("out must be a contiguous [m, n] tensor")
        check(lib.mfqb_mul_mat(self._h, x2.data_ptr(), x2.shape[0], y.data_ptr(),
                               F32 if tdt == torch.float32 else BF16, _stream_ptr(self.device)))
        return y[0] if squeeze else y

    def matmul_rmsnorm(self, h, gamma, delta=None, eps: float = 1e-5, gated: bool = False, out_dtype=None, return_residual: bool = False):
        """One float32 residual row ``h`` [k]: ``W @ ((h + delta) / rms(h + delta) * gamma)`` (or its gated form) in one
        launch; with ``return_residual`` also ``h + delta``."""
        torch = _torch()
        h1 = h.reshape(-1).contiguous()
        tdt = out_dtype or torch.bfloat16
        y = torch.empty((self.n // 2 if gated else self.n,), dtype=tdt, device=h1.device)
        h_out = torch.empty_like(h1) if return_residual else None
        check(lib.mfqb_mul_mat_rmsnorm(self._h, h1.data_ptr(), None if delta is None else delta.contiguous().data_ptr(), gamma.contiguous().data_ptr(),
                                       eps, None if h_out is None else h_out.data_ptr(), y.data_ptr(),
                                       F32 if tdt == torch.float32 else BF16, int(gated), _stream_ptr(self.device)))
        return (y, h_out) if return_residual else y

    def matmul_glu(self, x, out_dtype=None):
        """Gated product for a weight whose 16-row blocks alternate gate and up rows:
        ``up * silu(gate)`` of ``x @ W.T``, shape [m, n / 2]."""
        torch = _torch()
        x2 = x.reshape(-1, self.k).contiguous()
        if x2.dtype != torch.bfloat16 or not x2.is_cuda or x2.device.index != self.device:
            raise ValueError(f"x must be a bfloat16 tensor on cuda:{self.device}")
        tdt = out_dtype or torch.bfloat16
        y = torch.empty((x2.shape[0], self.n // 2), dtype=tdt, device=x2.device)
        check(lib.mfqb_mul_mat_glu(self._h, x2.data_ptr(), x2.shape[0], y.data_ptr(),
                                   F32 if tdt == torch.float32 else BF16, _stream_ptr(self.device)))
        return y

    def matmul_swiglu(self, gate_up, out_dtype=None):
        """``(up * silu(gate)) @ W.T`` for a float32 CUDA tensor ``gate_up`` [m, 2k] (gate columns first)."""
        torch = _torch()
        gu = gate_up.reshape(-1, 2 * self.k).contiguous()
        if gu.dtype != torch.float32 or not gu.is_cuda or gu.device.index != self.device:
            raise ValueError(f"gate_up must be a float32 tensor on cuda:{self.device}")
        tdt = out_dtype or torch.bfloat16
        y = torch.empty((gu.shape[0], self.n), dtype=tdt, device=gu.device)
        check(lib.mfqb_mul_mat_swiglu(self._h, gu.data_ptr(), gu.shape[0], y.data_ptr(),
                                      F32 if tdt == torch.float32 else BF16, _stream_ptr(self.device)))
        return y

    @staticmethod
    def matmul_multi(weights, x, out_dtype=None):
        """One bf16 row ``x`` [k] against up to 8 NINT weights of one shape class in a single launch
        (q|k|v, gate|up): returns the list of ``x @ W_i.T``."""
        torch = _torch()
        dev = weights[0].device
        x1 = x.reshape(-1).contiguous()
        if x1.dtype != torch.bfloat16 or not x1.is_cuda or x1.device.index != dev:
            raise ValueError(f"x must be a bfloat16 tensor on cuda:{dev}")
        tdt = out_dtype or torch.bfloat16
        ys = [torch.empty((w.n,), dtype=tdt, device=x1.device) for w in weights]
        hs = (C.c_void_p * len(weights))(*[w._h for w in weights])
        ps = (C.c_void_p * len(weights))(*[y.data_ptr() for y in ys])
        check(lib.mfqb_mul_mat_multi(hs, len(weights), x1.data_ptr(), ps,
                                     F32 if tdt == torch.float32 else BF16, _stream_ptr(dev)))
        return ys

    def matmul_host(self, x_bits, out_f32: bool = False):
        """Host-buffer product: ``x_bits`` is a uint16 numpy array of bf16 bit patterns [m, k];
        returns a numpy array (uint16 bf16 bits, or float32)."""
        import numpy as np
        x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16).reshape(-1, self.k)
        m = x_bits.shape[0]
        y = np.empty((m, self.n), dtype=np.float32 if out_f32 else np.uint16)
        check(lib.mfqb_mul_mat_host(self._h, x_bits.ctypes.data, m, y.ctypes.data, F32 if out_f32 else BF16))
        return y

    def free(self) -> None:
        if self._h:
            lib.mfqb_weight_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
