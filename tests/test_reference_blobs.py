"""Two checks that tie the package's blob writers and the oracle to the reference itself.

* ``golden_cfg1.npz`` (written by ``tests/golden/make_golden.py --cfg1`` with the reference's own
  encoder, decoder and runtime): a 1024 x 4096 NINT3 (3, 24, 5) record of the headline
  configuration.  The oracle must decode it to the tensor the reference decoded (SHA-256 of all
  of it, a sample of rows element by element) and reproduce the reference runtime's products.
* Where the reference tree is present (the container the fixtures are made in), the reference's
  reader must accept the blobs ``tyloquant_b200/encode.py`` writes -- every canonical NINT
  profile, NVQ3, NVQ3J-512, NINTM and a whole file image -- and decode them to what the oracle
  gives.  Elsewhere this part is skipped: nothing here needs the reference at run time.
"""

import hashlib
import os
import sys
import tempfile

import numpy as np
import pytest

from oracle import mfq_oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE_ROOT = os.environ.get("MFQ_REFERENCE_ROOT", "/root/reference")


def test_oracle_decodes_the_reference_encoded_headline_record():
    g = np.load(os.path.join(HERE, "golden", "golden_cfg1.npz"))
    assert str(g["dtype"]) == "NINT3"
    w = O.dequant_nint(O.unpack_nint(g["blob"].tobytes()))
    assert w.shape == (1024, 4096) and w.dtype == np.float32
    assert hashlib.sha256(np.ascontiguousarray(w).tobytes()).hexdigest() == str(g["w_sha256"])
    assert np.array_equal(w[g["rows"]], g["w_rows"])
    # the reference runtime's product (cached float32 W, x @ W.T): same arithmetic, same order
    y = O.linear(g["x"], w)
    assert np.allclose(y, g["y"], rtol=1e-5, atol=1e-6 * float(np.abs(g["y"]).max()))


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE_ROOT, "mfq")), reason="the reference tree is not present here")
def test_reference_reader_accepts_the_package_writers_blobs():
    encode = pytest.importorskip("tyloquant_b200.encode")
    sys.path.insert(0, REFERENCE_ROOT)
    sys.dont_write_bytecode = True
    try:
        from mfq.formats import io as mio
        from mfq.quantize import nint_quant, nvq_quant
        from mfq.quantize.expert_nint import dequantize_expertwise
        from mfq.quantize.nvq_jsc import dequantize_nvq_jsc
    finally:
        sys.path.remove(REFERENCE_ROOT)
    for bits, (b, gs, sb) in encode.CANONICAL_NINT.items():
        blob = encode.random_nint_blob(50, 200, b, gs, sb, seed=bits)
        ref = nint_quant.dequantize(mio._unpack_tensor(f"NINT{b}", blob))
        assert np.array_equal(ref, O.dequant_nint(O.unpack_nint(blob))), bits
    rng = np.random.default_rng(1)
    w = encode.bf16_round(rng.standard_normal((30, 200), dtype=np.float32) * np.float32(0.02))
    blob = encode.nvq_blob(encode.quantize_nvq3(w, O.d4_256_codebook()[None]))
    assert np.array_equal(nvq_quant.dequantize(mio._unpack_tensor("NVQ3", blob)), O.dequant_nvq(O.unpack_nvq(blob)))
    blob = encode.nvq_blob(encode.quantize_nvq3(w, encode.synthetic_d4_banks(512, 2, 7), jsc=True))
    assert np.array_equal(dequantize_nvq_jsc(mio._unpack_tensor("NVQ3J-512", blob)), O.dequant_nvq(O.unpack_nvq(blob)))
    wm = encode.bf16_round(rng.standard_normal((6, 32, 100), dtype=np.float32) * np.float32(0.02))
    blob = encode.quantize_expertwise(wm, [2, 3, 4, 6, 3, 4])
    assert np.array_equal(dequantize_expertwise(mio._unpack_tensor("NINTM", blob)), O.dequant_nintm(O.unpack_nintm(blob)))
    image = encode.mfq_file_image("llama", [("a", "NINT3", encode.random_nint_blob(16, 48, 3, 24, 5, 1))], {"x": 1})
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "t.mfq")
        with open(path, "wb") as f:
            f.write(image)
        header, tensors = mio.load(path)
        assert header.model_arch == "llama" and list(tensors) == ["a"]
