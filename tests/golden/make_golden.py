"""Generate the golden fixtures in this directory from the reference implementation.

Run once, in a container that has the reference project checked out:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

It imports the reference's own encoder, serializer and decoder (Python, CPU), encodes
small seeded tensors in every profile on the packed-weight execution path, and stores

* the serialized blob exactly as the reference wrote it, and
* the float32 tensor the reference's decoder returned for it,

in ``golden.npz`` (compressed), plus one complete ``.mfq`` file image.  With ``--cfg1`` it
writes ``golden_cfg1.npz`` instead: a 1024 x 4096 slice of the headline configuration (N(0, 0.02)
weights rounded to bf16, NINT3 groupsize 24 sub-bits 5) encoded by the reference encoder, with the
SHA-256 of the reference decoder's float32 output, a sample of its rows, and the reference
runtime's products for seeded activations.  The tests never import the reference; they only read
these files.
"""

from __future__ import annotations

import io as _io
import os
import struct
import sys
import tempfile

import numpy as np


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.dont_write_bytecode = True
    from mfq.calibration.artifact import ExpertPrecision
    from mfq.formats import io as mio
    from mfq.formats.header import FileHeader
    from mfq.formats.nint import NintSpec
    from mfq.formats.nvq import NVQ3_D4, NVQ3_D4_512, D4_256, NvqTensor
    from mfq.quantize import nint_quant, nvq_quant
    from mfq.quantize.expert_nint import dequantize_expertwise, quantize_expertwise
    from mfq.quantize.nvq_jsc import (NvqJscConfig, dequantize_nvq_jsc, initial_jsc_tables,
                                      quantize_nvq_jsc_fixed)
    from mfq.runtime.linear import NintLinear

    out = {}

    def bf16(x):
        u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
        r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
        return r.astype(np.uint32).view(np.float32).reshape(x.shape)

    # ---- NINT: canonical profiles, the config profiles and odd catalog members ----------
    nint_profiles = [(2, 16, 5), (3, 24, 5), (4, 24, 6), (4, 32, 6), (5, 28, 7), (5, 24, 7),
                     (6, 24, 7), (6, 22, 7), (6, 40, 7), (8, 48, 7), (8, 32, 7), (8, 24, 7),
                     (4, 16, 6), (4, 48, 6), (5, 64, 7), (6, 64, 7)]
    names = []
    for i, (bits, gs, sb) in enumerate(nint_profiles):
        rng = np.random.default_rng(100 + i)
        n, k = 40, 200 + 8 * (i % 3)  # tails: 200, 208, 216 are not multiples of most gs
        w = bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        t = nint_quant.quantize(w, NintSpec(bits=bits, groupsize=gs, sub_bits=sb))
        dtype, blob = mio._pack_tensor(t)
        back = mio._unpack_tensor(dtype, blob)
        ref = nint_quant.dequantize(back)
        key = f"nint_b{bits}_g{gs}_s{sb}"
        names.append(key)
        out[key + "__blob"] = np.frombuffer(blob, dtype=np.uint8)
        out[key + "__w"] = ref.astype(np.float32)
        out[key + "__dtype"] = np.array(dtype)
        if i == 1:
            x = bf16(rng.standard_normal((3, k)).astype(np.float32))
            out[key + "__x"] = x
            out[key + "__y"] = NintLinear(back).forward(x).astype(np.float32)
    out["nint_keys"] = np.array(names)

    # legacy NINT tail (whole-uint storage) built from a reference tensor by hand
    rng = np.random.default_rng(150)
    w = (rng.standard_normal((8, 50)) * 0.02).astype(np.float32)
    t = nint_quant.quantize(w, NintSpec(bits=3, groupsize=24, sub_bits=5))
    s = t.spec
    parts = [struct.pack("<BBiii", s.bits, s.sub_bits, s.groupsize, t.axis, t.neuron_len),
             struct.pack("<I", 2), struct.pack("<2q", *t.shape),
             struct.pack("<II", t.q.shape[0], t.q.shape[1]),
             t.neuron_scale.astype(np.float16).tobytes(), t.neuron_min.astype(np.float16).tobytes(),
             t.sub_scale.astype(np.uint8).tobytes(), t.sub_min.astype(np.uint8).tobytes(),
             t.q.astype(np.uint8).tobytes()]
    legacy = b"".join(parts)
    out["nint_legacy__blob"] = np.frombuffer(legacy, dtype=np.uint8)
    out["nint_legacy__w"] = nint_quant.dequantize(mio.unpack_nint(legacy)).astype(np.float32)

    # ---- NVQ3 (256-entry D4, built-in table), also with an explicit custom table -------
    for key, (n, k), seed, custom in [("nvq3_a", (24, 200), 200, False),
                                      ("nvq3_b", (17, 196), 201, False),
                                      ("nvq3_custom", (9, 96), 202, True)]:
        rng = np.random.default_rng(seed)
        w = bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        cb = None
        if custom:
            cb = D4_256[::-1].copy()
        t = nvq_quant.quantize(w, NVQ3_D4, codebook=cb)
        dtype, blob = mio._pack_tensor(t)
        back = mio._unpack_tensor(dtype, blob)
        out[key + "__blob"] = np.frombuffer(blob, dtype=np.uint8)
        out[key + "__w"] = nvq_quant.dequantize(back).astype(np.float32)
        out[key + "__dtype"] = np.array(dtype)

    # ---- NVQ3J-512 (two int8 banks of the 512-entry D4 lattice inside the blob) ---------
    import torch

    for key, (n, k), seed in [("nvq3j512_a", (20, 200), 300), ("nvq3j512_b", (12, 192), 301)]:
        rng = np.random.default_rng(seed)
        w = bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        tables = initial_jsc_tables(NvqJscConfig(banks=2, spec=NVQ3_D4_512))
        t = quantize_nvq_jsc_fixed(torch.from_numpy(w), tables, device="cpu")
        dtype, blob = mio._pack_tensor(t)
        back = mio._unpack_tensor(dtype, blob)
        out[key + "__blob"] = np.frombuffer(blob, dtype=np.uint8)
        out[key + "__w"] = dequantize_nvq_jsc(back).astype(np.float32)
        out[key + "__dtype"] = np.array(dtype)

    # ---- NINTM: per-expert mixed precision, gate_up [E, 2F, H] and down [E, H, F] ------
    e_count, hdim, fdim = 6, 96, 40
    rng = np.random.default_rng(400)
    bits = np.array([2, 3, 4, 6, 3, 4])
    spec_of = {2: NintSpec(2, 16, 5), 3: NintSpec(3, 24, 5), 4: NintSpec(4, 24, 6), 6: NintSpec(6, 24, 7)}
    profiles = [ExpertPrecision(family=f"NINT{b}", nint_spec=spec_of[int(b)]) for b in bits]
    wgu = bf16((rng.standard_normal((e_count, 2 * fdim, hdim)) * 0.02).astype(np.float32))
    wdn = bf16((rng.standard_normal((e_count, hdim, fdim)) * 0.02).astype(np.float32))
    for key, w in [("nintm_gate_up", wgu), ("nintm_down", wdn)]:
        t = quantize_expertwise(w, profiles, device="cpu")
        dtype, blob = mio._pack_tensor(t)
        back = mio._unpack_tensor(dtype, blob)
        out[key + "__blob"] = np.frombuffer(blob, dtype=np.uint8)
        out[key + "__w"] = dequantize_expertwise(back).astype(np.float32)
        out[key + "__dtype"] = np.array(dtype)
    out["nintm_bits"] = bits

    # ---- a complete .mfq file (version 2 with extra metadata, dense and asset records) -
    rng = np.random.default_rng(500)
    w1 = (rng.standard_normal((16, 72)) * 0.02).astype(np.float32)
    w2 = (rng.standard_normal((8, 48)) * 0.02).astype(np.float32)
    tensors = {
        "model.layers.0.self_attn.q_proj.weight": nint_quant.quantize(w1, NintSpec(4, 24, 6)),
        "model.layers.0.mlp.down_proj.weight": nvq_quant.quantize(w2, NVQ3_D4),
        "model.norm.weight": np.arange(16, dtype=np.float32),
        "__mfq_asset__/tokenizer.json": b'{"k": 1}',
    }
    hdr = FileHeader(model_arch="llama", version=2, extra={"general.name": "golden", "n": 3})
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "g.mfq")
        mio.save(path, hdr, tensors)
        raw = open(path, "rb").read()
        with mio.open_mmap(path) as store:
            out["file__names"] = np.array(list(store))
            out["file__w0"] = nint_quant.dequantize(store["model.layers.0.self_attn.q_proj.weight"])
            out["file__w1"] = nvq_quant.dequantize(store["model.layers.0.mlp.down_proj.weight"])
    out["file__image"] = np.frombuffer(raw, dtype=np.uint8)

    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "golden.npz"), **out)
    print("wrote", os.path.join(here, "golden.npz"), "with", len(out), "arrays")


def main_cfg1(ref_root: str) -> None:
    import hashlib

    sys.path.insert(0, ref_root)
    sys.dont_write_bytecode = True
    from mfq.formats import io as mio
    from mfq.formats.nint import NintSpec
    from mfq.quantize import nint_quant
    from mfq.runtime.linear import NintLinear

    def bf16(x):
        u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
        r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
        return r.astype(np.uint32).view(np.float32).reshape(x.shape)

    n, k = 1024, 4096
    w = bf16((np.random.default_rng(1001).standard_normal((n, k)) * 0.02).astype(np.float32))
    t = nint_quant.quantize(w, NintSpec(bits=3, groupsize=24, sub_bits=5))
    dtype, blob = mio._pack_tensor(t)
    back = mio._unpack_tensor(dtype, blob)
    ref = np.ascontiguousarray(nint_quant.dequantize(back), dtype=np.float32)
    x = bf16(np.random.default_rng(1002).standard_normal((4, k)).astype(np.float32))
    rows = np.arange(0, n, 37)
    out = {"blob": np.frombuffer(blob, dtype=np.uint8), "dtype": np.array(dtype),
           "w_sha256": np.array(hashlib.sha256(ref.tobytes()).hexdigest()),
           "rows": rows, "w_rows": ref[rows], "x": x,
           "y": NintLinear(back).forward(x).astype(np.float32)}
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "golden_cfg1.npz"), **out)
    print("wrote golden_cfg1.npz:", len(blob), "blob bytes")


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if a != "--cfg1"]
    (main_cfg1 if "--cfg1" in sys.argv else main)(args[0] if args else "/root/reference")
