"""ctypes binding of ``libmfqb200.so`` (the C ABI declared in ``include/mfqb200.h``).

The library is built in-tree by :mod:`tyloquant_b200.build`.  There is no fallback: if the
shared library is missing, importing this module raises.
"""

from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libmfqb200.so")

OK, ERR_ARG, ERR_FORMAT, ERR_UNSUPPORTED, ERR_CUDA, ERR_IO, ERR_TIMEOUT = range(7)
F32, BF16 = 0, 1
FAMILY_NINT, FAMILY_NVQ = 1, 2


class MfqbError(RuntimeError):
    """Raised when a library call returns a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[mfqb status {code}] {message}")
        self.code = code
        self.message = message


class WeightInfo(C.Structure):
    _fields_ = [("family", C.c_int), ("bits", C.c_int), ("groupsize", C.c_int), ("sub_bits", C.c_int),
                ("n", C.c_int64), ("k", C.c_int64), ("device", C.c_int), ("jsc_banks", C.c_int),
                ("payload_bytes", C.c_uint64), ("device_bytes", C.c_uint64)]


class DecoderConfig(C.Structure):
    _fields_ = [("hidden", C.c_int), ("n_q_heads", C.c_int), ("n_kv_heads", C.c_int), ("head_dim", C.c_int),
                ("ffn", C.c_int), ("vocab", C.c_int), ("layers", C.c_int), ("max_ctx", C.c_int), ("max_batch", C.c_int),
                ("rope_theta", C.c_float), ("rms_eps", C.c_float)]


class MoeInfo(C.Structure):
    _fields_ = [("n_experts", C.c_int), ("out_per_expert", C.c_int), ("k", C.c_int), ("expert_begin", C.c_int),
                ("expert_end", C.c_int), ("n_pools", C.c_int), ("device", C.c_int), ("payload_bytes", C.c_uint64),
                ("device_bytes", C.c_uint64)]


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python tyloquant_b200/build.py` "
        "(there is no CPU or pure-Python execution path)")

lib = C.CDLL(LIB_PATH)

_vp, _i, _i64, _u64, _cp = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_char_p
_P = C.POINTER

_SIGNATURES = {
    "mfqb_last_error": (_cp, []),
    "mfqb_version": (_i, []),
    "mfqb_file_open": (_i, [_cp, _P(_vp)]),
    "mfqb_file_open_memory": (_i, [_vp, _u64, _P(_vp)]),
    "mfqb_file_close": (_i, [_vp]),
    "mfqb_file_header": (_i, [_vp, _P(C.c_uint32), _P(_cp), _P(_i), _P(_i)]),
    "mfqb_file_extra": (_i, [_vp, _i, _P(_cp), _P(_cp)]),
    "mfqb_file_record": (_i, [_vp, _i, _P(_cp), _P(_cp), _P(_u64)]),
    "mfqb_file_find": (_i, [_vp, _cp, _P(_i)]),
    "mfqb_file_blob": (_i, [_vp, _i, _P(_vp), _P(_u64)]),
    "mfqb_weight_from_blob": (_i, [_cp, _vp, _u64, _i, _P(_vp)]),
    "mfqb_weight_from_blob_slice": (_i, [_cp, _vp, _u64, _i, _i64, _i64, _i, _P(_vp)]),
    "mfqb_weight_info_get": (_i, [_vp, _P(WeightInfo)]),
    "mfqb_weight_free": (_i, [_vp]),
    "mfqb_dequant": (_i, [_vp, _vp, _i, _vp]),
    "mfqb_mul_mat": (_i, [_vp, _vp, _i, _vp, _i, _vp]),
    "mfqb_device_status": (_i, [_i, _P(_i)]),
    "mfqb_tune": (_i, [_cp, _i]),
    "mfqb_mul_mat_rmsnorm": (_i, [_vp, _vp, _vp, _vp, C.c_float, _vp, _vp, _i, _i, _vp]),
    "mfqb_mul_mat_glu": (_i, [_vp, _vp, _i, _vp, _i, _vp]),
    "mfqb_mul_mat_swiglu": (_i, [_vp, _vp, _i, _vp, _i, _vp]),
    "mfqb_mul_mat_multi": (_i, [_P(_vp), _i, _vp, _P(_vp), _i, _vp]),
    "mfqb_weight_clone": (_i, [_vp, _P(_vp)]),
    "mfqb_decoder_create": (_i, [_vp, _i, _i, _vp, _i, _P(_vp)]),
    "mfqb_decoder_set_layer": (_i, [_vp, _i, _vp, _vp, _vp, _vp]),
    "mfqb_decoder_vocab_shard": (_i, [_vp, _P(_i), _P(_i)]),
    "mfqb_decoder_set_head": (_i, [_vp, _vp, _vp]),
    "mfqb_decoder_fill_cache": (_i, [_vp, _i, C.c_uint, _vp]),
    "mfqb_decoder_step": (_i, [_vp, _vp, _i, _vp, _vp]),
    "mfqb_decoder_layer": (_i, [_vp, _i, _vp, _i, _vp, _vp]),
    "mfqb_decoder_read_cache": (_i, [_vp, _i, _i, _i, _i, _vp, _vp]),
    "mfqb_decoder_read_logits": (_i, [_vp, _i, _vp, _vp]),
    "mfqb_decoder_free": (_i, [_vp]),
    "mfqb_mul_mat_host": (_i, [_vp, _vp, _i, _vp, _i]),
    "mfqb_mul_mat_host_multi": (_i, [_P(_vp), _i, _P(_vp), _i, _P(_vp), _i]),
    "mfqb_tp_plan": (_i, [_i64, _i64, _i, _P(C.c_double), _P(_i64), _P(_i64)]),
    "mfqb_tp_validate": (_i, [_i64, _i64, _i, _P(_i64), _P(_i64)]),
    "mfqb_tp_granularity": (_i, [_i64, _i64, _i, _P(_i64)]),
    "mfqb_selfcheck_layout": (_i, [_cp, _vp, _u64, _P(_u64)]),
    "mfqb_moe_topk": (_i, [_vp, _i, _i, _i, _i, _vp, _i, C.c_float, C.c_float, _vp, _vp, _vp]),
    "mfqb_moe_route_plan": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "mfqb_nintm_from_blob": (_i, [_vp, _u64, _i, _i, _i, _P(_vp)]),
    "mfqb_moe_info_get": (_i, [_vp, _P(MoeInfo)]),
    "mfqb_moe_expert_bytes": (_i, [_vp, _i, _P(_u64)]),
    "mfqb_moe_weight_free": (_i, [_vp]),
    "mfqb_moe_dequant_expert": (_i, [_vp, _i, _vp, _i, _vp]),
    "mfqb_mul_mat_id": (_i, [_vp, _vp, _i, _vp, _i, _i, _vp, _i, _vp]),
    "mfqb_moe_swiglu": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "mfqb_moe_weighted_reduce": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _i, _vp]),
    "mfqb_moe_ffn": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _i, _vp]),
    "mfqb_comm_create": (_i, [_i, _i, _u64, _i, _P(_vp)]),
    "mfqb_comm_handle": (_i, [_vp, _vp]),
    "mfqb_comm_attach": (_i, [_vp, _i, _vp]),
    "mfqb_comm_set_timeout_ms": (_i, [_vp, _i]),
    "mfqb_allreduce_f32": (_i, [_vp, _vp, _vp, _u64, _vp]),
    "mfqb_mul_mat_allreduce": (_i, [_vp, _vp, _i, _vp, _vp, _i, _vp]),
    "mfqb_comm_reset": (_i, [_vp]),
    "mfqb_comm_debug_set_seq": (_i, [_vp, C.c_uint]),
    "mfqb_comm_status": (_i, [_vp, _P(_i)]),
    "mfqb_comm_destroy": (_i, [_vp]),
    "mfqb_moe_ffn_static": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _i, _vp]),
}

for _name, (_res, _args) in _SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def check(status: int) -> None:
    if status != OK:
        raise MfqbError(status, lib.mfqb_last_error().decode("utf-8", "replace"))


def buffer_address(data) -> tuple[int, int, object]:
    """(address, nbytes, keepalive) of a bytes-like object, without copying when possible."""
    mv = memoryview(data)
    if mv.readonly:
        keep = (C.c_char * mv.nbytes).from_buffer_copy(mv)
    else:
        keep = (C.c_char * mv.nbytes).from_buffer(mv)
    return C.addressof(keep), mv.nbytes, keep
