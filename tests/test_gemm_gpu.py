"""GPU parity for the tcgen05 prefill GEMM (more than 16 activation rows), through the C ABI."""

import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import mfq_oracle as O  # noqa: E402
from tyloquant_b200 import QuantWeight, encode  # noqa: E402
from tyloquant_b200._capi import lib  # noqa: E402
from test_nint_gpu import rel_l2, bf16_tensor, REL_L2, MAX_ABS_BF16  # noqa: E402


def _status():
    s = C.c_int(-1)
    assert lib.mfqb_device_status(0, C.byref(s)) == 0
    return s.value


@pytest.mark.parametrize("profile", [(4, 24, 6), (4, 32, 6), (8, 32, 7), (3, 24, 5), (2, 16, 5), (6, 24, 7), (5, 24, 7), (8, 48, 7), (6, 40, 7),
                                     (5, 64, 7)])
def test_tile_gemm_matches_oracle(profile):
    bits, gs, sb = profile
    for (n, k, ms) in [(256, 1000, (17, 64, 200)), (130, 4096, (33,))]:
        blob = encode.random_nint_blob(n, k, bits, gs, sb, seed=n + k + bits)
        ref = O.dequant_nint(O.unpack_nint(blob))
        w = QuantWeight.from_blob(f"NINT{bits}", blob)
        for m in ms:
            x = encode.bf16_round(np.random.default_rng(m).standard_normal((m, k), dtype=np.float32))
            y_ref = O.linear(x, ref)
            y32 = w.matmul(bf16_tensor(x), out_dtype=torch.float32).cpu().numpy()
            assert _status() == 0
            assert rel_l2(y32, y_ref) <= REL_L2, (profile, n, k, m)
            y16 = w.matmul(bf16_tensor(x)).float().cpu().numpy()
            assert rel_l2(y16, O.bf16_round(y_ref)) <= REL_L2
            assert np.abs(y16 - y_ref).max() <= MAX_ABS_BF16
        w.free()


def test_config2_shape_nint4_gs32():
    """BASELINE config 2 at reduced N (the full 14336 rows only change the tile count): M = 512, K = 4096."""
    blob = encode.random_nint_blob(1024, 4096, 4, 32, 6, seed=2001, device="cuda")
    ref = O.dequant_nint(O.unpack_nint(blob))
    w = QuantWeight.from_blob("NINT4", blob)
    x = encode.bf16_round(np.random.default_rng(2002).standard_normal((512, 4096), dtype=np.float32))
    y = w.matmul(bf16_tensor(x), out_dtype=torch.float32).cpu().numpy()
    assert _status() == 0
    assert rel_l2(y, O.linear(x, ref)) <= REL_L2
    w.free()
