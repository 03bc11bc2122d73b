"""Pin the CPU oracle against blobs and decoded tensors produced by the reference itself.

The fixtures come from ``tests/golden/make_golden.py``; every comparison here is exact.
"""

import numpy as np
import pytest

from oracle import mfq_oracle as O


def _blob(g, key):
    return g[key + "__blob"].tobytes()


def test_nint_decoder_matches_reference_bit_for_bit(golden):
    keys = [str(k) for k in golden["nint_keys"]]
    assert len(keys) >= 12
    for key in keys:
        t = O.unpack_nint(_blob(golden, key))
        w = O.dequant_nint(t)
        ref = golden[key + "__w"]
        assert w.dtype == np.float32 and w.shape == ref.shape
        assert np.array_equal(w.view(np.uint32), ref.view(np.uint32)), key
        assert str(golden[key + "__dtype"]) == f"NINT{t.bits}"
        assert len(_blob(golden, key)) - (14 + 4 + 16 + 8) == O.nint_payload_nbytes(
            t.out, t.neuron_len, t.bits, t.gs, t.sub_bits)


def test_nint_legacy_tail(golden):
    w = O.dequant_nint(O.unpack_nint(_blob(golden, "nint_legacy")))
    assert np.array_equal(w.view(np.uint32), golden["nint_legacy__w"].view(np.uint32))


def test_nint_linear_matches_reference_runtime(golden):
    key = "nint_b3_g24_s5"
    w = O.dequant_nint(O.unpack_nint(_blob(golden, key)))
    y = O.linear(golden[key + "__x"], w)
    np.testing.assert_allclose(y, golden[key + "__y"], rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("key", ["nvq3_a", "nvq3_b", "nvq3_custom", "nvq3j512_a", "nvq3j512_b"])
def test_nvq_decoder_matches_reference_bit_for_bit(golden, key):
    t = O.unpack_nvq(_blob(golden, key))
    w = O.dequant_nvq(t)
    ref = golden[key + "__w"]
    assert w.shape == ref.shape
    assert np.array_equal(w.view(np.uint32), ref.view(np.uint32))
    banks = t.codebooks.shape[0] if t.jsc else 0
    custom = 2 * (1 << t.index_bits) if key == "nvq3_custom" else 0
    assert len(_blob(golden, key)) - (20 + 16 + 4) - custom == O.nvq_payload_nbytes(
        t.out, t.neuron_len, t.index_bits, t.vec, t.gs, t.sub_bits, banks)
    if key.startswith("nvq3j512"):
        assert t.index_bits == 9 and t.codebooks.shape == (2, 512, 4)
        assert int(t.indices.max()) > 255


def test_d4_table_checksum():
    cb = O.d4_256_codebook()
    assert cb.shape == (256, 4) and cb.min() == 1 and cb.max() == 15 and np.all(cb % 2 == 1)


@pytest.mark.parametrize("key", ["nintm_gate_up", "nintm_down"])
def test_nintm_decoder_matches_reference(golden, key):
    t = O.unpack_nintm(_blob(golden, key))
    w = O.dequant_nintm(t)
    assert np.array_equal(w.view(np.uint32), golden[key + "__w"].view(np.uint32))
    bits = golden["nintm_bits"]
    for p in t.pools:
        assert all(int(bits[e]) == int(p.dtype[4:]) for e in p.expert_ids)


def test_container_matches_reference(golden):
    f = O.parse_mfq(golden["file__image"].tobytes())
    assert f.version == 2 and f.arch == "llama"
    assert f.extra == {"general.name": "golden", "n": 3}
    assert [r.name for r in f.records] == [str(n) for n in golden["file__names"]]
    assert [r.dtype for r in f.records] == ["NINT4", "NVQ3", "F32", "BLOB"]
    w0 = O.dequant_record("NINT4", f.blob(f.records[0].name))
    w1 = O.dequant_record("NVQ3", f.blob(f.records[1].name))
    assert np.array_equal(w0, golden["file__w0"]) and np.array_equal(w1, golden["file__w1"])
    assert f.blob("__mfq_asset__/tokenizer.json") == b'{"k": 1}'
    with pytest.raises(ValueError):
        O.parse_mfq(golden["file__image"].tobytes() + b"\0")
    with pytest.raises(ValueError):
        O.parse_mfq(golden["file__image"].tobytes()[:-1])


def test_bit_packer_round_trip():
    rng = np.random.default_rng(7)
    for bits in (1, 2, 3, 4, 5, 6, 7, 8, 9):
        v = rng.integers(0, 1 << bits, size=1001)
        raw = O.pack_bits(v, bits)
        assert len(raw) == (1001 * bits + 7) // 8
        back, off = O.unpack_bits(raw, 0, 1001, bits)
        assert off == len(raw) and np.array_equal(back, v)


def test_router_matches_topk_semantics():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(11)
    z = rng.standard_normal((64, 128)).astype(np.float32)
    ids, w = O.moe_topk(z, 8)
    tv, ti = torch.topk(torch.from_numpy(z), 8, dim=1)
    assert np.array_equal(ids, ti.numpy().astype(np.int32))
    np.testing.assert_allclose(w, torch.softmax(tv, dim=1).numpy(), rtol=1e-6)
    # ties resolve to the smaller expert id; NaN ranks last
    z2 = np.zeros((1, 16), dtype=np.float32)
    z2[0, 5] = np.nan
    ids2, _ = O.moe_topk(z2, 4)
    assert ids2.tolist() == [[0, 1, 2, 3]]
    ids3, w3 = O.moe_topk(z, 8, mode=O.ROUTER_SOFTMAX, normalize=True)
    assert np.array_equal(ids3, ids)
    np.testing.assert_allclose(w3.sum(axis=1), 1.0, rtol=1e-5)


def test_tp_planner_reference_cases():
    # the cases of the reference's own planner test
    s = O.tp_plan(5120, 128, [0, 1])
    O.tp_validate(s, 5120, 128)
    assert [(e - b) for _, b, e in s] == [2560, 2560]
    s = O.tp_plan(5120, 128, [0, 2], [1.0, 3.0])
    O.tp_validate(s, 5120, 128)
    assert [(d, e - b) for d, b, e in s] == [(0, 1280), (2, 3840)]
    s = O.tp_plan(17408, 128, [0, 1, 2])
    O.tp_validate(s, 17408, 128)
    assert sum(e - b for _, b, e in s) == 17408
    with pytest.raises(ValueError):
        O.tp_plan(128, 128, [0, 1])
    assert O.tp_granularity(128, 128, 8) == 16
