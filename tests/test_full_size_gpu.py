"""Parity at the sizes the benchmark runs (configs 2, 3 and 4 of the baseline), through the C ABI.

The CPU oracle would need minutes to unpack these tensors whole, so it decodes seeded samples of
rows (ranges that start on multiples of 8, where every file stream is byte-aligned) and the
products are compared on those rows; a weighted checksum over *all* output rows, compared with the
same checksum taken on the GPU-decoded weights in float64, covers the rows in between (the decoder
itself is bit-exact against the oracle on the sampled rows).  Tolerance: relative L2 <= 1e-3."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import mfq_oracle as O  # noqa: E402
from tyloquant_b200 import QuantWeight, encode, moe  # noqa: E402
from test_nint_gpu import REL_L2, bf16_tensor, rel_l2  # noqa: E402


def _row_samples(n, count, width, seed):
    starts = np.random.default_rng(seed).choice(n // 8 - width // 8, count, replace=False) * 8
    return [(int(s), int(s) + width) for s in sorted(starts)]


def _check_sampled(w, unpack, dequant, blob, xs, n, samples):
    """xs: list of (x float32 on the bf16 grid [m, k]); compares rows of y with the oracle."""
    wd = w.dequantize()   # float32 [n, k] on the device
    refs = []
    for r0, r1 in samples:
        ref = dequant(unpack(blob, rows=(r0, r1)))
        assert np.array_equal(wd[r0:r1].cpu().numpy().view(np.uint32), ref.view(np.uint32)), (r0, r1)
        refs.append(ref)
    for x in xs:
        y = w.matmul(bf16_tensor(x), out_dtype=torch.float32)
        for (r0, r1), ref in zip(samples, refs):
            assert rel_l2(y[:, r0:r1].cpu().numpy(), O.linear(x, ref)) <= REL_L2, (x.shape, r0)
        # every row: against the float64 product with the decoded weights, on the device
        y64 = torch.from_numpy(x).cuda().double() @ wd.double().T
        err = float((y.double() - y64).norm() / y64.norm())
        assert err <= REL_L2, (x.shape, err)
    del wd


@pytest.mark.parametrize("profile", [(4, 32, 6), (8, 48, 7)])
def test_config2_prefill_gemm_full_shape(profile):
    """M = 512, N = 14336, K = 4096: NINT4 groupsize 32 and NINT8 groupsize 48 (the 256-token-tile plan)."""
    bits, gs, sb = profile
    n, k = 14336, 4096
    blob = encode.random_nint_blob(n, k, bits, gs, sb, seed=2001, device="cuda")
    w = QuantWeight.from_blob(f"NINT{bits}", blob)
    x = encode.bf16_round(np.random.default_rng(2002).standard_normal((512, k), dtype=np.float32))
    _check_sampled(w, O.unpack_nint, O.dequant_nint, blob, [x], n, _row_samples(n, 6, 128, seed=bits))
    w.free()


@pytest.mark.parametrize("jsc", [False, True])
def test_config3_lattice_gemv_full_shape(jsc):
    """17408 x 5120, NVQ3 (256-entry D4) and NVQ3J-512 (two 512-entry banks), batch 1, 4 and 8."""
    n, k = 17408, 5120
    rng = np.random.default_rng(3001)
    wf = encode.bf16_round(rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    banks = encode.synthetic_d4_banks(512, 2, seed=9) if jsc else encode.d4_256_codebook()[None]
    blob = encode.nvq_blob(encode.quantize_nvq3(wf, banks, jsc=jsc, device="cuda"))
    del wf
    w = QuantWeight.from_blob("NVQ3J-512" if jsc else "NVQ3", blob)
    xs = [encode.bf16_round(np.random.default_rng(3002 + m).standard_normal((m, k), dtype=np.float32)) for m in (1, 4, 8)]
    _check_sampled(w, O.unpack_nvq, O.dequant_nvq, blob, xs, n, _row_samples(n, 6, 64, seed=7 + jsc))
    w.free()


def test_config1_headline_shape_every_width():
    """4096 x 4096 and the decoder's FFN shape 14336 x 4096, single row, every canonical width."""
    for bits, (b, gs, sb) in encode.CANONICAL_NINT.items():
        for n in (4096, 14336):
            blob = encode.random_nint_blob(n, 4096, b, gs, sb, seed=1010 + bits, device="cuda")
            w = QuantWeight.from_blob(f"NINT{b}", blob)
            x = encode.bf16_round(np.random.default_rng(1002).standard_normal((1, 4096), dtype=np.float32))
            _check_sampled(w, O.unpack_nint, O.dequant_nint, blob, [x], n, _row_samples(n, 3, 64, seed=bits + n))
            w.free()


@pytest.mark.parametrize("tokens", [1, 32, 256])
def test_config4_expert_layer_full_shape(tokens):
    """Hidden 2048, 128 experts, top-8, FFN width 768, per-expert bits drawn from {2, 3, 4, 6} with
    seed 4003.  Routing ids exact; the routed gate|up products and the whole FFN against the oracle on
    a seeded sample of tokens (the oracle dequantizes only the experts those tokens use)."""
    h, e_count, f, k_top = 2048, 128, 768, 8
    bits = np.random.default_rng(4003).choice([2, 3, 4, 6], e_count)
    gen = torch.Generator("cuda").manual_seed(4001)
    wgu = (torch.randn((e_count, 2 * f, h), device="cuda", generator=gen) * 0.02).to(torch.bfloat16).float()
    wdn = (torch.randn((e_count, h, f), device="cuda", generator=gen) * 0.02).to(torch.bfloat16).float()
    gu_blob = encode.quantize_expertwise(wgu, bits, device="cuda")
    dn_blob = encode.quantize_expertwise(wdn, bits, device="cuda")
    del wgu, wdn
    gu, dn = moe.MoeWeight(gu_blob), moe.MoeWeight(dn_blob)
    rng = np.random.default_rng(4002)
    x = encode.bf16_round(rng.standard_normal((tokens, h), dtype=np.float32))
    z = np.random.default_rng(4004).standard_normal((tokens, e_count)).astype(np.float32)
    ids, wts = moe.moe_topk(torch.from_numpy(z).cuda(), k_top)
    rid, rw = O.moe_topk(z, k_top)
    assert np.array_equal(ids.cpu().numpy(), rid)
    np.testing.assert_allclose(wts.cpu().numpy(), rw, rtol=2e-6, atol=1e-7)
    out = gu.matmul_id(bf16_tensor(x), ids, out_dtype=torch.float32).cpu().numpy()
    y = moe.moe_ffn(gu, dn, bf16_tensor(x), ids, wts, out_dtype=torch.float32).cpu().numpy()
    sample = sorted(np.random.default_rng(5).choice(tokens, min(tokens, 6), replace=False).tolist())
    experts = sorted({int(e) for t in sample for e in rid[t]})
    gu_ref = {e: gu.dequantize_expert(e).cpu().numpy() for e in experts}   # bit-exact vs the oracle: checked on two of them
    dn_ref = {e: dn.dequantize_expert(e).cpu().numpy() for e in experts}
    tgu, tdn = O.unpack_nintm(gu_blob), O.unpack_nintm(dn_blob)
    full_gu, full_dn = None, None
    for e in experts[:2]:
        if full_gu is None:
            full_gu, full_dn = O.dequant_nintm_experts(tgu, experts[:2]), O.dequant_nintm_experts(tdn, experts[:2])
        assert np.array_equal(gu_ref[e].view(np.uint32), full_gu[e].view(np.uint32))
        assert np.array_equal(dn_ref[e].view(np.uint32), full_dn[e].view(np.uint32))
    for t in sample:
        want = np.stack([gu_ref[int(e)] @ x[t] for e in rid[t]])
        assert rel_l2(out[t], want) <= REL_L2, (t, rel_l2(out[t], want))
        acc = np.zeros(h, dtype=np.float32)
        for r, e in enumerate(rid[t]):
            g = gu_ref[int(e)] @ x[t]
            acc += rw[t, r] * (dn_ref[int(e)] @ O.swiglu(g[:f], g[f:]))
        assert rel_l2(y[t], acc) <= REL_L2, (t, rel_l2(y[t], acc))
    gu.free()
    dn.free()
