"""GPU parity for NVQ3 / NVQ3J-512 weights, through the C ABI, against the CPU oracle."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import mfq_oracle as O  # noqa: E402
from tyloquant_b200 import QuantWeight, encode  # noqa: E402
from test_nint_gpu import check_products, rel_l2, bf16_tensor, REL_L2  # noqa: E402

GOLDEN = [("nvq3_a", "NVQ3"), ("nvq3_b", "NVQ3"), ("nvq3_custom", "NVQ3"), ("nvq3j512_a", "NVQ3J-512"),
          ("nvq3j512_b", "NVQ3J-512")]


@pytest.mark.parametrize("key,dtype", GOLDEN)
def test_golden_blobs_decode_bit_exact_and_multiply(golden, key, dtype):
    blob = golden[key + "__blob"].tobytes()
    ref = golden[key + "__w"]
    w = QuantWeight.from_blob(dtype, blob)
    got = w.dequantize().cpu().numpy()
    assert got.shape == ref.shape
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    got16 = w.dequantize("bfloat16").view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got16, O.bf16_bits(ref))
    for m in (1, 3):
        check_products(w, ref, m, seed=m)
    w.free()


def test_dtype_label_must_match_blob(golden):
    from tyloquant_b200 import MfqbError
    with pytest.raises(MfqbError):
        QuantWeight.from_blob("NVQ3", golden["nvq3j512_a__blob"].tobytes())
    with pytest.raises(MfqbError):
        QuantWeight.from_blob("NVQ3J-512", golden["nvq3_a__blob"].tobytes())


@pytest.mark.parametrize("jsc", [False, True])
def test_synthetic_shapes_and_slices(jsc):
    dtype = "NVQ3J-512" if jsc else "NVQ3"
    banks = encode.synthetic_d4_banks(512, 2, seed=5) if jsc else O.d4_256_codebook()[None]
    for (n, k) in [(1, 24), (19, 100), (130, 1000), (64, 5120)]:
        rng = np.random.default_rng(n + k)
        wt = encode.bf16_round(rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
        blob = encode.nvq_blob(encode.quantize_nvq3(wt, banks, jsc=jsc, device="cuda"))
        t = O.unpack_nvq(blob)
        ref = O.dequant_nvq(t)
        w = QuantWeight.from_blob(dtype, blob)
        assert w.payload_bytes == O.nvq_payload_nbytes(n, k, t.index_bits, 4, 24, 4, 2 if jsc else 0)
        assert np.array_equal(w.dequantize().cpu().numpy().view(np.uint32), ref.view(np.uint32))
        for m in (1, 2, 4):
            check_products(w, ref, m, seed=m + n)
        w.free()
    # row slice and a column slice on a multiple of 24
    rows = QuantWeight.from_blob(dtype, blob, axis=0, begin=16, end=48)
    assert np.array_equal(rows.dequantize().cpu().numpy(), ref[16:48])
    cols = QuantWeight.from_blob(dtype, blob, axis=1, begin=2400, end=5120)
    assert np.array_equal(cols.dequantize().cpu().numpy(), ref[:, 2400:5120])
    x = encode.bf16_round(np.random.default_rng(3).standard_normal((1, 5120), dtype=np.float32))
    head = QuantWeight.from_blob(dtype, blob, axis=1, begin=0, end=2400)
    y = head.matmul(bf16_tensor(x[:, :2400]), out_dtype=torch.float32) + cols.matmul(bf16_tensor(x[:, 2400:]), out_dtype=torch.float32)
    assert rel_l2(y.cpu().numpy(), O.linear(x, ref)) <= REL_L2
