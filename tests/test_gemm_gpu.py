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
            # bf16 output: the same criterion as for the batched GEMV -- per element one bf16 step of the oracle value
            # plus the accuracy bound (weights rounded to f16 once: a few 1e-4 relative L2, single elements a few times
            # that), and the L2 distance that rounding an exact result to bf16 allows
            step = np.exp2(np.floor(np.log2(np.maximum(np.abs(y_ref), 1e-30))) - 7)
            rms = float(np.sqrt(np.mean(np.square(y_ref, dtype=np.float64))))
            assert np.all(np.abs(y16 - O.bf16_round(y_ref)) <= step + 2 * REL_L2 * rms)
            assert rel_l2(y16, y_ref) <= 3e-3
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


def test_nonfinite_inputs_stay_nonfinite_on_the_tile_kernel():
    """An infinity or a NaN in a row of x makes that row of the output NaN on every path: the
    integer kernels (m <= 16) and the f16 tile kernel (m > 16) must agree on that."""
    blob = encode.random_nint_blob(256, 1024, 4, 32, 6, seed=77)
    w = QuantWeight.from_blob("NINT4", blob)
    x = torch.randn(32, 1024, device="cuda", generator=torch.Generator("cuda").manual_seed(3)).to(torch.bfloat16)
    x[5, 100] = float("inf")
    x[9, 7] = float("-inf")
    x[20, 512] = float("nan")
    x[30, 3] = 3.0e38   # finite, beyond the f16 range: saturates, stays finite
    y = w.matmul(x, out_dtype=torch.float32)
    assert _status() == 0
    for r in (5, 9, 20):
        assert torch.isnan(y[r]).all(), r
    finite_rows = [r for r in range(32) if r not in (5, 9, 20)]
    assert torch.isfinite(y[finite_rows]).all()
    w.free()


def test_library_scratch_survives_growth_under_a_captured_graph():
    """A graph captured at m = 4 keeps working after a later, larger call made the per-device
    scratch grow (the old block must stay alive), and growth inside a capture is refused."""
    from tyloquant_b200 import MfqbError
    blob = encode.random_nint_blob(512, 2048, 3, 24, 5, seed=5)
    ref = O.dequant_nint(O.unpack_nint(blob))
    w = QuantWeight.from_blob("NINT3", blob)
    rng = np.random.default_rng(11)
    x4 = bf16_tensor(encode.bf16_round(rng.standard_normal((4, 2048), dtype=np.float32)))
    y4 = torch.empty((4, 512), dtype=torch.float32, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        w.matmul(x4, out=y4)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            w.matmul(x4, out=y4)
        # a much larger batched call on the same device: the planes buffer has to grow
        big = QuantWeight.from_blob("NINT3", encode.random_nint_blob(64, 65536, 3, 24, 5, seed=6, device="cuda"))
        big.matmul(torch.randn(8, 65536, device="cuda").to(torch.bfloat16))
        y4.zero_()
        g.replay()
        stream.synchronize()
    assert rel_l2(y4.cpu().numpy(), O.linear(x4.float().cpu().numpy(), ref)) <= REL_L2
    # growth while capturing: refused with a message, the capture survives being abandoned
    huge = QuantWeight.from_blob("NINT3", encode.random_nint_blob(64, 262144, 3, 24, 5, seed=7, device="cuda"))
    xh = torch.randn(8, 262144, device="cuda").to(torch.bfloat16)
    s2 = torch.cuda.Stream()
    with torch.cuda.stream(s2):
        g2 = torch.cuda.CUDAGraph()
        try:
            with pytest.raises(MfqbError):
                with torch.cuda.graph(g2, stream=s2):
                    huge.matmul(xh)
        except RuntimeError:
            pass   # torch may complain about the abandoned capture; the library call itself must have raised MfqbError
    torch.cuda.synchronize()
    for t in (w, big, huge):
        t.free()
