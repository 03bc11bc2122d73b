"""Mixture-of-experts operators over the C ABI: router, route plan, expert-wise mixed-precision
weights and the routed expert matmul / FFN (mirrors ``moe_topk``, ``MoeRoutePlan.build``,
``NintMoeWeight`` and ``nint_moe_ffn_forward`` of the reference, mfq/kernels/cuda/moe.py:301-384,
cpp_runtime/mfq_decode.cpp:2681-3071, 3394-3416)."""

from __future__ import annotations

import ctypes as C

from . import _capi
from ._capi import BF16, F32, MoeInfo, check, lib

SOFTMAX, SIGMOID, SQRT_SOFTPLUS, DELAYED_SOFTMAX = 0, 1, 2, 3


def _torch():
    import torch
    return torch


def _stream(t) -> int:
    return _torch().cuda.current_stream(t.device.index).cuda_stream


def moe_topk(logits, k: int, mode: int = DELAYED_SOFTMAX, bias=None, normalize: bool = False, norm_floor: float = 0.0,
             scale: float = 1.0):
    """logits: float32 CUDA tensor [tokens, experts] -> (ids int32 [tokens, k], weights float32 [tokens, k])."""
    torch = _torch()
    z = logits.contiguous()
    if z.dtype != torch.float32 or not z.is_cuda or z.dim() != 2:
        raise ValueError("logits must be a float32 CUDA tensor [tokens, experts]")
    t, e = z.shape
    ids = torch.empty((t, k), dtype=torch.int32, device=z.device)
    w = torch.empty((t, k), dtype=torch.float32, device=z.device)
    b = None if bias is None else bias.contiguous().float()
    with torch.cuda.device(z.device):
        check(lib.mfqb_moe_topk(z.data_ptr(), t, e, k, mode, None if b is None else b.data_ptr(), int(normalize),
                                norm_floor, scale, ids.data_ptr(), w.data_ptr(), _stream(z)))
    return ids, w


def route_plan(ids, n_experts: int, tile_m: int = 8):
    """-> (expert_bounds [E+1], tile_bounds [E+1], pair_order [tokens*k]) int32 CUDA tensors."""
    torch = _torch()
    ids = ids.contiguous()
    t, k = ids.shape
    eb = torch.empty(n_experts + 1, dtype=torch.int32, device=ids.device)
    tb = torch.empty(n_experts + 1, dtype=torch.int32, device=ids.device)
    order = torch.empty(t * k, dtype=torch.int32, device=ids.device)
    with torch.cuda.device(ids.device):
        check(lib.mfqb_moe_route_plan(ids.data_ptr(), t, k, n_experts, tile_m, eb.data_ptr(), tb.data_ptr(), order.data_ptr(),
                                      _stream(ids)))
    return eb, tb, order


class MoeWeight:
    """One ``NINTM`` record [experts, out, k] on a GPU (optionally only an expert range)."""

    def __init__(self, blob, device: int = 0, expert_begin: int = 0, expert_end: int = -1):
        addr, n, keep = _capi.buffer_address(blob)
        self._h = C.c_void_p()
        check(lib.mfqb_nintm_from_blob(addr, n, expert_begin, expert_end, device, C.byref(self._h)))
        info = MoeInfo()
        check(lib.mfqb_moe_info_get(self._h, C.byref(info)))
        self.info = info
        self.device = device

    def expert_bytes(self, expert: int) -> int:
        v = C.c_uint64()
        check(lib.mfqb_moe_expert_bytes(self._h, expert, C.byref(v)))
        return v.value

    def dequantize_expert(self, expert: int, dtype="float32"):
        torch = _torch()
        tdt = torch.float32 if str(dtype).endswith("float32") else torch.bfloat16
        out = torch.empty((self.info.out_per_expert, self.info.k), dtype=tdt, device=f"cuda:{self.device}")
        check(lib.mfqb_moe_dequant_expert(self._h, expert, out.data_ptr(), F32 if tdt == torch.float32 else BF16, _stream(out)))
        return out

    def matmul_id(self, x, ids, out_dtype=None):
        """x: bf16 [tokens, k] (shared by a token's routes) or [tokens, routes, k]; ids int32 [tokens, routes]."""
        torch = _torch()
        ids = ids.contiguous()
        t, r = ids.shape
        x = x.contiguous()
        per_pair = x.dim() == 3
        if x.dtype != torch.bfloat16 or x.shape[-1] != self.info.k:
            raise ValueError("x must be bfloat16 with k columns")
        tdt = out_dtype or torch.bfloat16
        out = torch.empty((t, r, self.info.out_per_expert), dtype=tdt, device=x.device)
        check(lib.mfqb_mul_mat_id(self._h, x.data_ptr(), int(per_pair), ids.data_ptr(), t, r, out.data_ptr(),
                                  F32 if tdt == torch.float32 else BF16, _stream(x)))
        return out

    def free(self) -> None:
        if self._h:
            lib.mfqb_moe_weight_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def swiglu(gate_up):
    torch = _torch()
    g = gate_up.contiguous()
    rows, f2 = g.reshape(-1, g.shape[-1]).shape
    out = torch.empty(g.shape[:-1] + (f2 // 2,), dtype=torch.bfloat16, device=g.device)
    check(lib.mfqb_moe_swiglu(g.data_ptr(), F32 if g.dtype == torch.float32 else BF16, rows, f2 // 2, out.data_ptr(), _stream(g)))
    return out


def weighted_reduce(expert_out, weights, out_dtype=None):
    torch = _torch()
    e = expert_out.contiguous()
    t, r, h = e.shape
    tdt = out_dtype or torch.float32
    y = torch.empty((t, h), dtype=tdt, device=e.device)
    check(lib.mfqb_moe_weighted_reduce(e.data_ptr(), F32 if e.dtype == torch.float32 else BF16, weights.contiguous().data_ptr(),
                                       t, r, h, y.data_ptr(), F32 if tdt == torch.float32 else BF16, _stream(e)))
    return y


def moe_ffn(gate_up: MoeWeight, down: MoeWeight, x, ids, weights, out_dtype=None):
    """y[t] = sum_r weights[t, r] * down_e(silu(gate_e x[t]) * up_e x[t]), e = ids[t, r]."""
    torch = _torch()
    x = x.contiguous()
    ids = ids.contiguous()
    weights = weights.contiguous()
    t, r = ids.shape
    tdt = out_dtype or torch.float32
    y = torch.empty((t, down.info.out_per_expert), dtype=tdt, device=x.device)
    check(lib.mfqb_moe_ffn(gate_up._h, down._h, x.data_ptr(), ids.data_ptr(), weights.data_ptr(), t, r, y.data_ptr(),
                           F32 if tdt == torch.float32 else BF16, _stream(x)))
    return y
