"""The allocation-free expert FFN entry point against the regular one.

Some callers of this library cannot allocate device memory where they call it (inside a stream
capture, or in a server that has given all spare HBM to its KV cache), so
``mfqb_moe_ffn_static`` keeps its intermediates in a fixed array inside the library.  This file
is collected last on purpose: a run that stops at the first failure has then already run every
other test.  It calls both entry points through the C ABI, twice in a row with different batch
sizes (the array keeps the previous call's contents), and checks the size limit's error.
"""

import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from tyloquant_b200 import _capi, encode, moe  # noqa: E402
from tyloquant_b200._capi import F32, lib  # noqa: E402


def _ffn(entry, gu, dn, x, ids, wts, check_no_alloc=False):
    t, r = ids.shape
    y = torch.empty((t, dn.info.out_per_expert), dtype=torch.float32, device=x.device)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = entry(gu._h, dn._h, x.data_ptr(), ids.data_ptr(), wts.data_ptr(), t, r, y.data_ptr(), F32,
               torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    if check_no_alloc:   # the entry point's contract: the device's free memory is the same after the call
        free_after = torch.cuda.mem_get_info()[0]
        assert free_after == free_before, (free_before, free_after)
    return rc, y


def test_static_scratch_ffn_matches_allocating_ffn_twice_in_a_row():
    e_count, h, f, k = 16, 256, 96, 4
    bits = np.random.default_rng(7).choice([2, 3, 4, 6], e_count)
    rng = np.random.default_rng(11)
    wgu = encode.bf16_round(rng.standard_normal((e_count, 2 * f, h), dtype=np.float32) * np.float32(0.02))
    wdn = encode.bf16_round(rng.standard_normal((e_count, h, f), dtype=np.float32) * np.float32(0.02))
    gu = moe.MoeWeight(encode.quantize_expertwise(wgu, bits, device="cuda"))
    dn = moe.MoeWeight(encode.quantize_expertwise(wdn, bits, device="cuda"))
    for tokens in (9, 40, 2):   # later calls run over the earlier calls' leftovers; 40 tokens take the tiled path
        x = torch.from_numpy(encode.bf16_round(rng.standard_normal((tokens, h), dtype=np.float32))).cuda().to(torch.bfloat16)
        z = torch.from_numpy(rng.standard_normal((tokens, e_count)).astype(np.float32)).cuda()
        ids, wts = moe.moe_topk(z, k)
        rc_a, y_a = _ffn(lib.mfqb_moe_ffn, gu, dn, x, ids, wts)
        # the first launch of a kernel makes the driver load its code (device memory the library does not
        # own): one call of this shape first, then the call that is checked
        rc_w, _ = _ffn(lib.mfqb_moe_ffn_static, gu, dn, x, ids, wts)
        rc_b, y_b = _ffn(lib.mfqb_moe_ffn_static, gu, dn, x, ids, wts, check_no_alloc=True)
        assert rc_a == 0 and rc_w == 0 and rc_b == 0, lib.mfqb_last_error()
        torch.cuda.synchronize()
        a, b = y_a.cpu().numpy().astype(np.float64), y_b.cpu().numpy().astype(np.float64)
        assert np.isfinite(b).all()
        # same kernels on the same inputs; partial sums meet in shared memory in arbitrary order
        assert np.linalg.norm(a - b) / np.linalg.norm(a) < 1e-5
        # the same call recorded into a CUDA graph (after the warm-up above) and replayed
        y_g = torch.zeros_like(y_b)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            rc_g = lib.mfqb_moe_ffn_static(gu._h, dn._h, x.data_ptr(), ids.data_ptr(), wts.data_ptr(), tokens, k, y_g.data_ptr(), F32,
                                           torch.cuda.current_stream().cuda_stream)
        assert rc_g == 0, lib.mfqb_last_error()
        y_g.zero_()
        graph.replay()
        torch.cuda.synchronize()
        c = y_g.cpu().numpy().astype(np.float64)
        assert np.linalg.norm(a - c) / np.linalg.norm(a) < 1e-5
    # beyond the built-in array: a clear refusal, nothing launched
    per_pair = 2 * f * 4 + f * 4 + h * 4
    too_many = (8 << 20) // (per_pair * k) + 8
    x = torch.zeros((too_many, h), dtype=torch.bfloat16, device="cuda")
    ids = torch.zeros((too_many, k), dtype=torch.int32, device="cuda")
    wts = torch.zeros((too_many, k), dtype=torch.float32, device="cuda")
    rc, _ = _ffn(lib.mfqb_moe_ffn_static, gu, dn, x, ids, wts)
    assert rc == _capi.ERR_ARG
    msg = lib.mfqb_last_error().decode()
    assert "scratch" in msg and str(8 << 20) in msg
    gu.free()
    dn.free()
