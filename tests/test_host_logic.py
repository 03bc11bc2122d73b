"""Host-side logic of the library, checked on CPU against the oracle and the golden files."""

import ctypes as C
import os

import numpy as np
import pytest

import tyloquant_b200 as T
from oracle import mfq_oracle as O
from tyloquant_b200 import _capi, encode
from tyloquant_b200._capi import MfqbError, lib


def _selfcheck(dtype, blob):
    addr, n, keep = _capi.buffer_address(blob)
    bad = C.c_uint64(1 << 40)
    _capi.check(lib.mfqb_selfcheck_layout(dtype.encode(), addr, n, C.byref(bad)))
    return bad.value


def test_container_reader_matches_reference_file(golden, tmp_path):
    image = golden["file__image"].tobytes()
    ref = O.parse_mfq(image)
    for f in (T.MfqFile(image=image), None):
        if f is None:
            p = tmp_path / "g.mfq"
            p.write_bytes(image)
            f = T.MfqFile(str(p))
        assert (f.version, f.arch, f.extra) == (ref.version, ref.arch, ref.extra)
        assert [(n, d, b) for n, d, b in f.records] == [(r.name, r.dtype, r.nbytes) for r in ref.records]
        for r in ref.records:
            assert f.blob(r.name) == ref.blob(r.name)
        assert f.find("nope") == -1
        f.close()


def test_container_rejects_damaged_files(golden):
    image = golden["file__image"].tobytes()
    for bad in (image + b"\0", image[:-1], b"MFQ2" + image[4:], image[:10]):
        with pytest.raises(MfqbError) as e:
            T.MfqFile(image=bad)
        assert e.value.code == _capi.ERR_FORMAT
    with pytest.raises(MfqbError) as e:
        T.MfqFile("/nonexistent/x.mfq")
    assert e.value.code == _capi.ERR_IO


def test_sharded_file_set(tmp_path):
    blobs = [encode.random_nint_blob(16, 48, 4, 24, 6, seed=s) for s in range(3)]
    for i in range(3):
        extra = {"split.no": i, "split.count": 3, "split.records.count": 3, "split.tensors.count": 3}
        img = encode.mfq_file_image("llama", [(f"w{i}", "NINT4", blobs[i])], extra)
        (tmp_path / f"m-{i + 1:05d}-of-00003.mfq").write_bytes(img)
    f = T.MfqFile(str(tmp_path / "m-00001-of-00003.mfq"))
    assert f.names() == ["w0", "w1", "w2"]
    assert [f.blob(n) for n in f.names()] == blobs
    f.close()
    # opening a later shard finds the same set
    f = T.MfqFile(str(tmp_path / "m-00002-of-00003.mfq"))
    assert f.names() == ["w0", "w1", "w2"]
    f.close()
    os.remove(tmp_path / "m-00003-of-00003.mfq")
    with pytest.raises(MfqbError):
        T.MfqFile(str(tmp_path / "m-00001-of-00003.mfq"))


def test_device_layout_round_trips_every_golden_nint_profile(golden):
    for key in [str(k) for k in golden["nint_keys"]] + ["nint_legacy"]:
        blob = golden[key + "__blob"].tobytes()
        dtype = f"NINT{blob[0]}"
        assert _selfcheck(dtype, blob) == 0, key


def test_device_layout_round_trips_every_golden_nvq_profile(golden):
    for key, dtype in [("nvq3_a", "NVQ3"), ("nvq3_b", "NVQ3"), ("nvq3_custom", "NVQ3"), ("nvq3j512_a", "NVQ3J-512"),
                       ("nvq3j512_b", "NVQ3J-512")]:
        assert _selfcheck(dtype, golden[key + "__blob"].tobytes()) == 0, key
    banks = encode.synthetic_d4_banks(512, 2, seed=1)
    w = encode.bf16_round(np.random.default_rng(0).standard_normal((21, 250), dtype=np.float32) * np.float32(0.02))
    assert _selfcheck("NVQ3J-512", encode.nvq_blob(encode.quantize_nvq3(w, banks, jsc=True))) == 0
    assert _selfcheck("NVQ3", encode.nvq_blob(encode.quantize_nvq3(w, O.d4_256_codebook()[None]))) == 0


def test_device_layout_round_trips_ragged_shapes():
    for (n, k, bits, gs, sb) in [(1, 24, 3, 24, 5), (17, 25, 4, 24, 6), (33, 4096, 2, 16, 5), (16, 769, 5, 28, 7),
                                 (5, 100, 8, 48, 7), (40, 500, 6, 30, 7), (9, 64, 4, 32, 4), (9, 64, 4, 32, 8)]:
        assert _selfcheck(f"NINT{bits}", encode.random_nint_blob(n, k, bits, gs, sb, seed=n + k)) == 0


def test_bad_blobs_are_rejected_with_a_status():
    blob = encode.random_nint_blob(16, 48, 3, 24, 5, seed=1)
    addr, n, keep = _capi.buffer_address(blob[:-3])
    bad = C.c_uint64()
    assert lib.mfqb_selfcheck_layout(b"NINT3", addr, n - 0, C.byref(bad)) == _capi.ERR_FORMAT
    assert b"tail" in lib.mfqb_last_error()
    addr, n, keep = _capi.buffer_address(blob)
    assert lib.mfqb_selfcheck_layout(b"NEPQ0-S", addr, n, C.byref(bad)) == _capi.ERR_UNSUPPORTED
    assert lib.mfqb_selfcheck_layout(None, addr, n, C.byref(bad)) == _capi.ERR_ARG
    seven = bytearray(blob)
    seven[0] = 7
    addr, n, keep = _capi.buffer_address(bytes(seven))
    assert lib.mfqb_selfcheck_layout(b"NINT7", addr, n, C.byref(bad)) in (_capi.ERR_FORMAT, _capi.ERR_UNSUPPORTED)


def test_tp_planner_matches_oracle_and_reference_cases():
    assert [(e - b) for _, b, e in T.plan_tensor_parallel_slices(5120, 128, [0, 1])] == [2560, 2560]
    assert T.plan_tensor_parallel_slices(5120, 128, [0, 2], [1.0, 3.0]) == [(0, 0, 1280), (2, 1280, 5120)]
    s = T.plan_tensor_parallel_slices(17408, 128, [0, 1, 2])
    T.validate_tensor_parallel_slices(s, 17408, 128)
    assert sum(e - b for _, b, e in s) == 17408
    with pytest.raises(MfqbError):
        T.plan_tensor_parallel_slices(128, 128, [0, 1])
    rng = np.random.default_rng(3)
    for _ in range(300):
        n = int(rng.integers(1, 9))
        gran = int(rng.choice([1, 8, 24, 128, 384]))
        extent = int(rng.integers(n * gran, n * gran * 40 + 1))
        weights = [] if rng.random() < 0.5 else [float(x) for x in rng.uniform(0.1, 4.0, n)]
        devs = list(range(n))
        mine = T.plan_tensor_parallel_slices(extent, gran, devs, weights)
        assert mine == O.tp_plan(extent, gran, devs, weights)
        try:  # a clamped boundary can be misaligned when extent % gran != 0: both must agree
            O.tp_validate(mine, extent, gran)
            valid = True
        except ValueError:
            valid = False
        if valid:
            T.validate_tensor_parallel_slices(mine, extent, gran)
        else:
            with pytest.raises(MfqbError):
                T.validate_tensor_parallel_slices(mine, extent, gran)
        pref = int(rng.choice([16, 128]))
        assert T.tensor_parallel_granularity(extent, pref, n) == O.tp_granularity(extent, pref, n)
    with pytest.raises(MfqbError):
        T.validate_tensor_parallel_slices([(0, 0, 100), (1, 100, 256)], 256, 128)
    with pytest.raises(MfqbError):
        T.plan_tensor_parallel_slices(1024, 128, [0, 1], [1.0, -1.0])


def test_package_encoders_produce_blobs_the_oracle_reads():
    for bits, (b, gs, sb) in encode.CANONICAL_NINT.items():
        t = O.unpack_nint(encode.random_nint_blob(20, 100, b, gs, sb, seed=bits))
        assert (t.bits, t.gs, t.sub_bits, t.out, t.neuron_len) == (b, gs, sb, 20, 100)
        w = O.dequant_nint(t)
        ref = encode.bf16_round(np.random.default_rng(bits).standard_normal((20, 100), dtype=np.float32) * np.float32(0.02))
        snr = 10 * np.log10((ref ** 2).sum() / ((w - ref) ** 2).sum())
        assert snr > 5 * b - 2, (b, snr)


def test_header_sizes_are_checked_before_anything_is_allocated_for_them():
    """A few dozen bytes that claim gigabytes: the NINT reader compares the tail length with the header
    before it sizes its arrays, the container reader bounds the record count by the bytes that are left."""
    import struct
    out, ng, gs = 2, 50_000_000, 24
    head = struct.pack("<BBiii", 3, 5, gs, 0, ng * gs) + struct.pack("<I", 2) + struct.pack("<qq", out, ng * gs)
    head += struct.pack("<II", out, ng) + b"\0" * (4 * out)
    addr, n, keep = _capi.buffer_address(head)
    bad = C.c_uint64()
    assert lib.mfqb_selfcheck_layout(b"NINT3", addr, n, C.byref(bad)) == _capi.ERR_FORMAT
    assert b"tail" in lib.mfqb_last_error()
    image = b"MFQ1" + struct.pack("<I", 1) + struct.pack("<I", 0) + struct.pack("<I", 0xFFFFFFF0)
    with pytest.raises(MfqbError) as e:
        T.MfqFile(image=image)
    assert e.value.code == _capi.ERR_FORMAT and "record count" in str(e.value)


def test_tune_switch_checks_key_and_range():
    """Execution-plan switches need no device; an unknown key or a value outside the key's range is an
    argument error and leaves the plan as it was."""
    assert lib.mfqb_tune(b"gemv1_kernel", 0) == 0
    assert lib.mfqb_tune(b"gemm_plan", 0) == 0
    assert lib.mfqb_tune(b"moe_f16_tiles_from_x2", 4) == 0
    for key, value in ((b"gemv1_kernel", 3), (b"gemm_plan", -1), (b"moe_f16_tiles_from_x2", 1), (b"no_such_key", 0)):
        assert lib.mfqb_tune(key, value) == _capi.ERR_ARG
        assert b"mfqb_tune" in lib.mfqb_last_error()
    assert lib.mfqb_tune(None, 0) == _capi.ERR_ARG
