"""Activation edge cases of the integer pipeline, through the C ABI, against the CPU oracle.

The streaming kernels quantise every activation group to 16-bit integers with a power-of-two
scale taken from the group's largest magnitude.  These cases aim at that step: one huge outlier
per group, all-zero groups, magnitudes next to the bf16 maximum, subnormal inputs, negative
zeros, and row lengths that end inside a group -- on the single-row kernel (m = 1), the batched
kernel (m = 4, 8) and the routed expert kernels.  The bound is the one stated for the path:
relative L2 <= 1e-3 against dequantize-then-matmul (accumulated here in float64 so that the
reference itself does not overflow or cancel).
"""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import mfq_oracle as O  # noqa: E402
from tyloquant_b200 import QuantWeight, encode, moe  # noqa: E402
from test_nint_gpu import REL_L2, bf16_tensor, rel_l2  # noqa: E402


def _cases(rng, m, k, gs):
    ng = -(-k // gs)
    base = encode.bf16_round(rng.standard_normal((m, k), dtype=np.float32))
    out = {}
    x = base.copy()                       # one 2^12 outlier in every group
    for g in range(ng):
        j = g * gs + int(rng.integers(0, min(gs, k - g * gs)))
        x[:, j] *= np.float32(4096.0)
    out["outlier_per_group"] = x
    x = base.copy()                       # a single 2^12 outlier in the whole row
    x[:, k // 3] = np.float32(3000.0)
    out["one_outlier"] = x
    x = base.copy()                       # all-zero groups (every third) and negative zeros
    for g in range(0, ng, 3):
        x[:, g * gs:(g + 1) * gs] = 0.0
    x[:, 1::7] = np.float32(-0.0)
    out["zero_groups_and_negative_zero"] = x
    out["all_zero"] = np.zeros((m, k), dtype=np.float32)
    x = np.zeros((m, k), dtype=np.float32)   # a few magnitudes next to the bf16 maximum, the rest small
    x[:, ::97] = encode.bf16_round(np.full((m, len(range(0, k, 97))), 3.0e38, dtype=np.float32)) * np.sign(base[:, ::97])
    x[:, 5::97] = base[:, 5::97]
    out["near_bf16_max"] = x
    x = base.copy()                       # subnormal bf16 values among ordinary ones
    x[:, ::5] = np.float32(1e-40)
    x[:, 2::5] = np.float32(-3e-39)
    out["subnormals_mixed"] = encode.bf16_round(x)
    # everything tiny but normal: groups keep all 16 bits down to a largest magnitude of 2^-88
    # (below that the fixed 2^-24 head-room of the group scales eats into them)
    x = encode.bf16_round(base * np.float32(2.0 ** -80))
    out["tiny_normals"] = x
    # the oracle and the device must see the same values: everything on the bf16 grid
    return {name: encode.bf16_round(v) for name, v in out.items()}


def _check(y, x, w_ref, name):
    y_ref = x.astype(np.float64) @ w_ref.astype(np.float64).T
    assert np.isfinite(y).all(), name
    if not np.any(y_ref):
        assert not np.any(y), name
        return
    assert rel_l2(y, y_ref) <= REL_L2, (name, rel_l2(y, y_ref))


@pytest.mark.parametrize("profile", [(3, 24, 5), (4, 32, 6), (2, 16, 5), (8, 48, 7), (5, 28, 7)])
@pytest.mark.parametrize("m", [1, 4, 8])
def test_dense_products_on_hard_activations(profile, m):
    bits, gs, sb = profile
    n, k = 160, 1000 + gs // 2          # the row ends inside a group
    blob = encode.random_nint_blob(n, k, bits, gs, sb, seed=bits * 100 + m)
    w_ref = O.dequant_nint(O.unpack_nint(blob))
    w = QuantWeight.from_blob(f"NINT{bits}", blob)
    rng = np.random.default_rng(900 + bits + m)
    for name, x in _cases(rng, m, k, gs).items():
        y = w.matmul(bf16_tensor(x), out_dtype=torch.float32).cpu().numpy().astype(np.float64)
        _check(y, x, w_ref, (profile, m, name))
    # only subnormal inputs: below the smallest scale the integer grid has (2^-126 per unit), they
    # count as zero -- the result must be finite and no larger than the true product's bound
    x = np.full((m, k), 1e-40, dtype=np.float32)
    y = w.matmul(bf16_tensor(x), out_dtype=torch.float32).cpu().numpy()
    assert np.isfinite(y).all() and np.abs(y).max() <= 1e-40 * np.abs(w_ref).sum(axis=1).max() * 1.01 + 1e-45
    w.free()


def test_full_width_row_on_hard_activations():
    """4096 columns (the headline shape's row length, 170 groups and a 16-column tail), m = 1 and 8."""
    blob = encode.random_nint_blob(256, 4096, 3, 24, 5, seed=77, device="cuda")
    w_ref = O.dequant_nint(O.unpack_nint(blob))
    w = QuantWeight.from_blob("NINT3", blob)
    for m in (1, 8):
        for name, x in _cases(np.random.default_rng(50 + m), m, 4096, 24).items():
            y = w.matmul(bf16_tensor(x), out_dtype=torch.float32).cpu().numpy().astype(np.float64)
            _check(y, x, w_ref, (m, name))
    w.free()


@pytest.mark.parametrize("tokens", [1, 3, 40])
def test_routed_expert_products_on_hard_activations(tokens):
    """Routed matmul (single-pair kernel for 1 and 3 tokens, route-plan tiles for 40)."""
    e_count, h, f, k_top = 16, 264, 40, 4       # 264 = 11 groups of 24: the last chunk is partial
    bits = np.random.default_rng(6003).choice([2, 3, 4, 6], e_count)
    rng = np.random.default_rng(6001)
    wgu = encode.bf16_round(rng.standard_normal((e_count, 2 * f, h), dtype=np.float32) * np.float32(0.02))
    blob = encode.quantize_expertwise(wgu, bits, device="cuda")
    ref = O.dequant_nintm(O.unpack_nintm(blob))
    w = moe.MoeWeight(blob)
    ids = np.stack([rng.choice(e_count, k_top, replace=False) for _ in range(tokens)]).astype(np.int32)
    ids_t = torch.from_numpy(ids).cuda()
    for name, x in _cases(rng, tokens, h, 24).items():
        out = w.matmul_id(bf16_tensor(x), ids_t, out_dtype=torch.float32).cpu().numpy().astype(np.float64)
        want = np.stack([[ref[ids[t, r]].astype(np.float64) @ x[t].astype(np.float64) for r in range(k_top)] for t in range(tokens)])
        assert np.isfinite(out).all(), name
        if np.any(want):
            assert rel_l2(out, want) <= REL_L2, (tokens, name, rel_l2(out, want))
        else:
            assert not np.any(out)
    w.free()
