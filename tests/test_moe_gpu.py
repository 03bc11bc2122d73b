"""GPU parity for the mixture-of-experts rows of the path: router, route plan, NINTM weights,
routed expert matmul, expert FFN and expert-range shards, against the CPU oracle."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import mfq_oracle as O  # noqa: E402
from tyloquant_b200 import encode, moe  # noqa: E402
from test_nint_gpu import rel_l2, bf16_tensor, REL_L2  # noqa: E402


@pytest.mark.parametrize("tokens,experts,k", [(1, 128, 8), (33, 128, 8), (7, 256, 6), (5, 16, 16), (9, 384, 12), (3, 100, 8), (64, 4096, 4)])
def test_router_ids_are_bit_exact(tokens, experts, k):
    rng = np.random.default_rng(tokens + experts)
    z = rng.standard_normal((tokens, experts)).astype(np.float32)
    z[0, :4] = z[0, 4]          # ties resolve to the smaller expert id
    if tokens > 1:
        z[1, 3] = np.nan        # NaN ranks last
    zt = torch.from_numpy(z).cuda()
    for mode in (O.ROUTER_DELAYED_SOFTMAX, O.ROUTER_SOFTMAX, O.ROUTER_SIGMOID, O.ROUTER_SQRT_SOFTPLUS):
        ids, w = moe.moe_topk(zt, k, mode=mode, normalize=(mode != O.ROUTER_DELAYED_SOFTMAX), norm_floor=1e-20, scale=1.5)
        rid, rw = O.moe_topk(z, k, mode=mode, normalize=(mode != O.ROUTER_DELAYED_SOFTMAX), norm_floor=1e-20, scale=1.5)
        if mode in (O.ROUTER_DELAYED_SOFTMAX, O.ROUTER_SIGMOID):
            # selection on monotone functions of the raw logits: exact
            assert np.array_equal(ids.cpu().numpy(), rid), mode
            np.testing.assert_allclose(w.cpu().numpy(), rw, rtol=2e-6, atol=1e-7)
        else:
            # scores pass through expf / log1pf, whose last bits may differ between the device and
            # numpy: an id may differ from the oracle's only where the two scores involved are
            # within 2 float32 units of each other (a numerical tie)
            got = ids.cpu().numpy()
            scores = O.router_scores(z, mode)
            for t, r in zip(*np.nonzero(got != rid)):
                a, b = scores[t, got[t, r]], scores[t, rid[t, r]]
                assert abs(a - b) <= 2 * np.spacing(max(abs(a), abs(b)).astype(np.float32)), (mode, t, r, a, b)
    bias = torch.from_numpy(rng.standard_normal(experts).astype(np.float32)).cuda()
    ids, w = moe.moe_topk(zt, k, bias=bias)
    rid, rw = O.moe_topk(z, k, bias=bias.cpu().numpy())
    assert np.array_equal(ids.cpu().numpy(), rid)
    np.testing.assert_allclose(w.cpu().numpy(), rw, rtol=2e-6, atol=1e-7)


def test_router_matches_torch_topk():
    z = torch.randn(256, 128, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    ids, w = moe.moe_topk(z, 8)
    tv, ti = torch.topk(z, 8, dim=1)
    assert torch.equal(ids.long(), ti)
    assert torch.allclose(w, torch.softmax(tv, dim=1), rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("tokens,experts,k", [(1, 128, 8), (40, 128, 8), (300, 64, 4), (3, 7, 2), (700, 128, 8)])
def test_route_plan_matches_oracle(tokens, experts, k):
    rng = np.random.default_rng(tokens)
    ids = np.stack([rng.choice(experts, k, replace=False) for _ in range(tokens)]).astype(np.int32)
    eb, tb, order = moe.route_plan(torch.from_numpy(ids).cuda(), experts, tile_m=8)
    reb, rtb, _, rorder = O.route_plan(ids, experts, 8)
    assert np.array_equal(eb.cpu().numpy(), reb)
    assert np.array_equal(tb.cpu().numpy(), rtb)
    assert np.array_equal(order.cpu().numpy(), rorder)   # ascending pair index inside every expert segment


def _moe_case(e_count, h, f, bits, seed):
    rng = np.random.default_rng(seed)
    wgu = encode.bf16_round(rng.standard_normal((e_count, 2 * f, h), dtype=np.float32) * np.float32(0.02))
    wdn = encode.bf16_round(rng.standard_normal((e_count, h, f), dtype=np.float32) * np.float32(0.02))
    return encode.quantize_expertwise(wgu, bits, device="cuda"), encode.quantize_expertwise(wdn, bits, device="cuda")


def test_golden_nintm_experts_decode_bit_exact(golden):
    for key in ("nintm_gate_up", "nintm_down"):
        blob = golden[key + "__blob"].tobytes()
        ref = golden[key + "__w"]
        w = moe.MoeWeight(blob)
        assert (w.info.n_experts, w.info.out_per_expert, w.info.k) == ref.shape
        for e in range(ref.shape[0]):
            got = w.dequantize_expert(e).cpu().numpy()
            assert np.array_equal(got.view(np.uint32), ref[e].view(np.uint32)), (key, e)
        w.free()


def test_golden_nintm_ffn_matches_oracle(golden):
    gu_ref, dn_ref = golden["nintm_gate_up__w"], golden["nintm_down__w"]
    gu = moe.MoeWeight(golden["nintm_gate_up__blob"].tobytes())
    dn = moe.MoeWeight(golden["nintm_down__blob"].tobytes())
    e_count, _, h = gu_ref.shape
    rng = np.random.default_rng(8)
    for tokens in (1, 5):
        x = encode.bf16_round(rng.standard_normal((tokens, h), dtype=np.float32))
        z = rng.standard_normal((tokens, e_count)).astype(np.float32)
        ids, wts = moe.moe_topk(torch.from_numpy(z).cuda(), 2)
        rid, rw = O.moe_topk(z, 2)
        assert np.array_equal(ids.cpu().numpy(), rid)
        out = gu.matmul_id(bf16_tensor(x), ids, out_dtype=torch.float32).cpu().numpy()
        want = np.stack([[gu_ref[rid[t, r]] @ x[t] for r in range(2)] for t in range(tokens)])
        assert rel_l2(out, want) <= REL_L2
        y = moe.moe_ffn(gu, dn, bf16_tensor(x), ids, wts).cpu().numpy()
        y_ref = O.moe_ffn(x, gu_ref, dn_ref, rid, rw)
        # nothing is rounded between the two matmuls (the activation stays float32, or is never
        # stored at all at decode sizes): the stated bound holds against the all-float32 oracle
        assert rel_l2(y, y_ref) <= REL_L2
    gu.free()
    dn.free()


@pytest.mark.parametrize("tokens", [1, 32, 101])
def test_mixed_precision_layer_and_expert_shards(tokens):
    """A scaled-down config-4 layer: 16 experts, bits drawn from {2,3,4,6}, top-4."""
    e_count, h, f, k = 16, 256, 96, 4
    bits = np.random.default_rng(4003).choice([2, 3, 4, 6], e_count)
    gu_blob, dn_blob = _moe_case(e_count, h, f, bits, seed=4001)
    gu_ref = O.dequant_nintm(O.unpack_nintm(gu_blob))
    dn_ref = O.dequant_nintm(O.unpack_nintm(dn_blob))
    gu, dn = moe.MoeWeight(gu_blob), moe.MoeWeight(dn_blob)
    rng = np.random.default_rng(4002)
    x = encode.bf16_round(rng.standard_normal((tokens, h), dtype=np.float32))
    z = rng.standard_normal((tokens, e_count)).astype(np.float32)
    ids, wts = moe.moe_topk(torch.from_numpy(z).cuda(), k)
    rid, rw = O.moe_topk(z, k)
    assert np.array_equal(ids.cpu().numpy(), rid)
    y = moe.moe_ffn(gu, dn, bf16_tensor(x), ids, wts).cpu().numpy()
    assert rel_l2(y, O.moe_ffn(x, gu_ref, dn_ref, rid, rw)) <= REL_L2
    assert sum(gu.expert_bytes(e) for e in range(e_count)) == gu.info.payload_bytes
    # expert-parallel shards: each holds a contiguous expert range; their outputs add up
    parts = []
    for b, e in ((0, 6), (6, 16)):
        sgu, sdn = moe.MoeWeight(gu_blob, expert_begin=b, expert_end=e), moe.MoeWeight(dn_blob, expert_begin=b, expert_end=e)
        parts.append(moe.moe_ffn(sgu, sdn, bf16_tensor(x), ids, wts))
        sgu.free()
        sdn.free()
    assert rel_l2((parts[0] + parts[1]).cpu().numpy(), y) <= 1e-5
    gu.free()
    dn.free()


@pytest.mark.parametrize("tokens", [16, 40, 400])
def test_route_plan_tiles_and_grouped_tile_kernel(tokens):
    """48 experts, top-4: 16 tokens give tiles of two pairs, 40 tokens tiles of four (with the four
    canonical precisions every cohort then runs in the same launch), 400 tokens (33 pairs per expert)
    go to the tensor-core tile kernel grouped by expert.  Also through an expert shard."""
    e_count, h, f, k = 48, 256, 96, 4
    bits = np.random.default_rng(5003).choice([2, 3, 4, 6], e_count)
    gu_blob, dn_blob = _moe_case(e_count, h, f, bits, seed=5001)
    gu_ref = O.dequant_nintm(O.unpack_nintm(gu_blob))
    dn_ref = O.dequant_nintm(O.unpack_nintm(dn_blob))
    gu, dn = moe.MoeWeight(gu_blob), moe.MoeWeight(dn_blob)
    rng = np.random.default_rng(5002 + tokens)
    x = encode.bf16_round(rng.standard_normal((tokens, h), dtype=np.float32))
    z = rng.standard_normal((tokens, e_count)).astype(np.float32)
    ids, wts = moe.moe_topk(torch.from_numpy(z).cuda(), k)
    rid, rw = O.moe_topk(z, k)
    out = gu.matmul_id(bf16_tensor(x), ids, out_dtype=torch.float32).cpu().numpy()
    want = np.stack([[gu_ref[rid[t, r]] @ x[t] for r in range(k)] for t in range(tokens)])
    assert rel_l2(out, want) <= REL_L2
    y = moe.moe_ffn(gu, dn, bf16_tensor(x), ids, wts).cpu().numpy()
    assert rel_l2(y, O.moe_ffn(x, gu_ref, dn_ref, rid, rw)) <= REL_L2
    parts = []
    for b, e in ((0, 20), (20, 48)):
        sgu, sdn = moe.MoeWeight(gu_blob, expert_begin=b, expert_end=e), moe.MoeWeight(dn_blob, expert_begin=b, expert_end=e)
        parts.append(moe.moe_ffn(sgu, sdn, bf16_tensor(x), ids, wts))
        sgu.free()
        sdn.free()
    assert rel_l2((parts[0] + parts[1]).cpu().numpy(), y) <= 1e-5
    gu.free()
    dn.free()
