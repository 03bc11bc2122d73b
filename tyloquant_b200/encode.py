"""Writers for synthetic MFQ tensors: simple quantizers plus the blob / file serializers.

The execution path only *reads* MFQ data; benchmarks and tests still need packed weights
of the right shapes, and the reference encoder is not available where they run.  The
quantizers here are deliberately plain (min/max affine groups for NINT, nearest lattice
point for NVQ3) -- throughput and decoder parity do not depend on encoder quality -- while
the serializers follow the format exactly (mfq/formats/io.py:144-248, 304-446, 646-685;
mfq/formats/nvq.py:454-490, 603-713), so that the reference reader accepts the output.

Heavy array work uses torch so it can run on the GPU when one is present.
"""

from __future__ import annotations

import json
import struct

import numpy as np

CANONICAL_NINT = {2: (2, 16, 5), 3: (3, 24, 5), 4: (4, 24, 6), 5: (5, 28, 7), 6: (6, 24, 7), 8: (8, 48, 7)}


# ---------------------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------------------

def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bfloat16 -> float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16)."""
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


def pack_bits(values: np.ndarray, bits: int) -> bytes:
    """LSB-first bitstream: value i occupies stream bits [i*bits, (i+1)*bits)."""
    v = np.ascontiguousarray(values).reshape(-1)
    if bits == 8:
        return v.astype(np.uint8).tobytes()
    nbytes = (v.size * bits + 7) // 8
    if bits < 8:
        # eight values fill exactly `bits` bytes: build them as one little-endian uint64 per octet
        pad = (-v.size) % 8
        u = v.astype(np.uint64)
        if pad:
            u = np.concatenate([u, np.zeros(pad, dtype=np.uint64)])
        u = u.reshape(-1, 8)
        word = np.zeros(u.shape[0], dtype=np.uint64)
        for i in range(8):
            word |= u[:, i] << np.uint64(bits * i)
        out = word.view(np.uint8).reshape(-1, 8)[:, :bits]
        return np.ascontiguousarray(out).tobytes()[:nbytes]
    out = bytearray()
    step = 1 << 20  # multiple of 8 values, so every chunk ends on a byte boundary
    for s in range(0, v.size, step):
        c = v[s:s + step].astype(np.uint16)
        stream = ((c[:, None] >> np.arange(bits, dtype=np.uint16)[None, :]) & 1).astype(np.uint8)
        out += np.packbits(stream.reshape(-1), bitorder="little").tobytes()
    return bytes(out)


def _torch():
    import torch
    return torch


def _pack_any(values, bits: int) -> bytes:
    """pack_bits for numpy arrays or torch tensors (the latter packed on their own device)."""
    if isinstance(values, np.ndarray) or bits >= 8:
        return pack_bits(np.asarray(values.cpu()) if not isinstance(values, np.ndarray) else values, bits)
    torch = _torch()
    v = values.reshape(-1).to(torch.int64)
    nbytes = (v.numel() * bits + 7) // 8
    pad = (-v.numel()) % 8
    if pad:
        v = torch.cat([v, torch.zeros(pad, dtype=torch.int64, device=v.device)])
    v = v.reshape(-1, 8)
    word = torch.zeros(v.shape[0], dtype=torch.int64, device=v.device)
    for i in range(8):
        word |= v[:, i] << (bits * i)
    out = word.view(torch.uint8).reshape(-1, 8)[:, :bits].contiguous()
    return out.cpu().numpy().tobytes()[:nbytes]


# ---------------------------------------------------------------------------------------
# NINT
# ---------------------------------------------------------------------------------------

def quantize_nint(weight: np.ndarray, bits: int, gs: int, sub_bits: int, device: str = "cpu") -> dict:
    """Min/max affine groups anchored on per-row f16 scale / min.  ``weight`` is [n, k]."""
    torch = _torch()
    if isinstance(weight, torch.Tensor):
        w = weight.to(device=device, dtype=torch.float32)
    else:
        w = torch.as_tensor(np.ascontiguousarray(weight, dtype=np.float32), device=device)
    n, k = w.shape
    ng = -(-k // gs)
    pad = ng * gs - k
    if pad:
        w = torch.nn.functional.pad(w, (0, pad))
    g = w.reshape(n, ng, gs)
    nmax, kmax = (1 << bits) - 1, (1 << sub_bits) - 1
    lo = torch.clamp(g.amin(-1), max=0.0)
    hi = torch.clamp(g.amax(-1), min=0.0)
    scale = (hi - lo) / nmax
    the_min = -lo
    neu_s, neu_m = scale.amax(-1), the_min.amax(-1)
    neu_d = (neu_s / kmax).to(torch.float16).to(torch.float32)
    neu_dm = (neu_m / kmax).to(torch.float16).to(torch.float32)
    ss = torch.clamp(torch.round(kmax * scale / torch.where(neu_s > 0, neu_s, torch.ones_like(neu_s))[:, None]), 0, kmax)
    sm = torch.clamp(torch.round(kmax * the_min / torch.where(neu_m > 0, neu_m, torch.ones_like(neu_m))[:, None]), 0, kmax)
    d_eff = neu_d[:, None] * ss
    m_eff = neu_dm[:, None] * sm
    de = torch.where(d_eff > 0, d_eff, torch.ones_like(d_eff))
    q = torch.clamp(torch.round((g + m_eff[..., None]) / de[..., None]), 0, nmax)
    return dict(bits=bits, gs=gs, sub_bits=sub_bits, n=n, k=k, ng=ng,
                neuron_scale=neu_d.cpu().numpy().astype(np.float16),
                neuron_min=neu_dm.cpu().numpy().astype(np.float16),
                sub_scale=ss.to(torch.uint8), sub_min=sm.to(torch.uint8), q=q.to(torch.uint8))


def nint_blob(t: dict) -> bytes:
    """mfq/formats/io.py:191-203."""
    parts = [struct.pack("<BBiii", t["bits"], t["sub_bits"], t["gs"], 0, t["k"]),
             struct.pack("<I", 2), struct.pack("<2q", t["n"], t["k"]), struct.pack("<II", t["n"], t["ng"]),
             np.ascontiguousarray(t["neuron_scale"], dtype="<f2").tobytes(),
             np.ascontiguousarray(t["neuron_min"], dtype="<f2").tobytes(),
             _pack_any(t["sub_scale"], t["sub_bits"]), _pack_any(t["sub_min"], t["sub_bits"]),
             _pack_any(t["q"], t["bits"])]
    return b"".join(parts)


def random_nint_blob(n: int, k: int, bits: int, gs: int, sub_bits: int, seed: int, std: float = 0.02,
                     device: str = "cpu") -> bytes:
    """Seeded N(0, std) bf16 weights, quantized and serialized as an ``NINT<bits>`` blob."""
    rng = np.random.default_rng(seed)
    w = bf16_round((rng.standard_normal((n, k), dtype=np.float32) * np.float32(std)))
    return nint_blob(quantize_nint(w, bits, gs, sub_bits, device=device))


# ---------------------------------------------------------------------------------------
# NVQ3 / NVQ3J-512
# ---------------------------------------------------------------------------------------

def _nearest_code(target, table, chunk: int = 1 << 18):
    """Index of the nearest codebook row for every 4-vector of ``target`` ([m, 4])."""
    torch = _torch()
    t2 = (table * table).sum(-1)
    out = torch.empty(target.shape[0], dtype=torch.int64, device=target.device)
    for s in range(0, target.shape[0], chunk):
        x = target[s:s + chunk]
        out[s:s + chunk] = (t2[None, :] - 2.0 * (x @ table.T)).argmin(-1)
    return out


def quantize_nvq3(weight: np.ndarray, codebooks: np.ndarray, *, jsc: bool = False, device: str = "cpu") -> dict:
    """Nearest-lattice-point NVQ3 encoder.  ``codebooks`` is int8 [banks, entries, 4].

    Plain profile: one bank, integer sub-scale 1..15.  JSC profile: analytic state tables for
    two D4 banks (scale = state // banks + 1, bank = state % banks); the bank of a group
    alternates with the group index.  The eighth sign of each block is forced to the
    parity of the first seven, as the format stores only seven.
    """
    torch = _torch()
    w = torch.as_tensor(np.ascontiguousarray(weight, dtype=np.float32), device=device)
    n, k = w.shape
    gs = 24
    ng = -(-k // gs)
    pad = ng * gs - k
    if pad:
        w = torch.nn.functional.pad(w, (0, pad))
    g = w.reshape(n, ng, gs)
    banks, entries, _ = codebooks.shape
    levels = 16 // banks if jsc else 15                    # distinct scale values
    amax = g.abs().amax(-1)                                # [n, ng]
    t = amax / 11.0
    anchor = (t.amax(-1) / levels).to(torch.float16).to(torch.float32)
    safe = torch.where(anchor > 0, anchor, torch.ones_like(anchor))
    sval = torch.clamp(torch.round(t / safe[:, None]), 1, levels)      # scale multiplier
    if jsc:
        bank = (torch.arange(ng, device=w.device)[None, :] + torch.arange(n, device=w.device)[:, None]) % banks
        state = ((sval - 1) * banks + bank).to(torch.int64)
    else:
        bank = torch.zeros((n, ng), dtype=torch.int64, device=w.device)
        state = sval.to(torch.int64)
    mag = g.abs() / (safe[:, None] * sval)[..., None]
    cb = torch.as_tensor(codebooks.astype(np.float32), device=w.device)
    idx = torch.empty((n, ng, 6), dtype=torch.int64, device=w.device)
    vec = mag.reshape(n, ng, 6, 4)
    for b in range(banks):
        sel = bank == b
        if sel.any():
            idx[sel] = _nearest_code(vec[sel].reshape(-1, 4), cb[b]).reshape(-1, 6)
    neg = (g < 0).reshape(n, ng * 3, 8)[:, :, :7].to(torch.int64)
    masks = (neg << torch.arange(7, device=w.device)).sum(-1)
    nvec, nsign = -(-k // 4), -(-k // 8)
    return dict(n=n, k=k, ng=ng, jsc=jsc, banks=banks, index_bits=int(np.log2(entries)),
                anchors=anchor.cpu().numpy().astype(np.float16),
                sub=state.to(torch.uint8).cpu().numpy(),
                indices=idx.reshape(n, ng * 6)[:, :nvec].to(torch.int16).cpu().numpy().astype(np.uint16),
                signs=masks[:, :nsign].to(torch.uint8).cpu().numpy(),
                codebooks=np.ascontiguousarray(codebooks, dtype=np.int8))


def nvq_blob(t: dict) -> bytes:
    """mfq/formats/nvq.py:603-713 (plain profile with the built-in table, or NVQ-JSC)."""
    cid = {8: 2, 9: 3, 10: 6}[t["index_bits"]]
    hdr = struct.pack("<4sBBHiiI", b"NVQ1", cid | (0x20 if t["jsc"] else 0), 4, 24, 0, t["k"], 2)
    parts = [hdr, struct.pack("<2q", t["n"], t["k"]), struct.pack("<I", t["n"])]
    if t["jsc"]:
        banks = t["banks"]
        meta = bytearray(64)
        meta[0], meta[1], meta[2], meta[3] = 1, banks, 16, 1
        state = np.arange(16)
        meta[4:36] = ((state // banks) + 1).astype("<f2").tobytes() if banks > 1 else state.astype("<f2").tobytes()
        meta[36:52] = (state % banks).astype(np.uint8).tobytes()
        parts += [bytes(meta), t["codebooks"].tobytes()]
    parts += [np.ascontiguousarray(t["anchors"], dtype="<f2").tobytes(), pack_bits(t["sub"], 4),
              pack_bits(t["indices"], t["index_bits"]), pack_bits(t["signs"], 7)]
    return b"".join(parts)


# Packed 256-entry D4 magnitude grid of plain NVQ3 (format constant, see csrc/nvq_d4_256.h):
# 256 little-endian uint16, four 3-bit digits each, magnitude = 2*digit + 1.
_D4_256_HEX = (
    "00000200040009000b000f0010001200190022003b003d004100430048004a005100550058005a0061006c00780080008200840089009000920099009b009f00"
    "a900af00bd00c100c700c800ca00d500f8000b011f0124012f013b013d01410147015a016a019d01b401c801cc01ce01e301f1010102030208020a0211021302"
    "18021a021c0227022802400242024902500252028102830288028a0291029802ba02c002c202d002d902e602f60201030503280350035403660379038503d203"
    "e0030004020409040b041004120416041904220441044304450448044a04510458047304770478048004820489048f04900492049f04a004ad04c104c804cc04"
    "f804fc041d052b054305570561057c05c105c305ce05e505010608060a0611061306280635063a064006420650065906640666068106830688069506aa06ba06"
    "c906db06180727073a074007460752076d078c079e07b307db07f00704080f081d081f082b082f087c0890089f08a008b008b608c708e5080409290934095509"
    "63097809c509c809ca09d8090a0a210a380a400a460a560a6d0a8c0a9a0aba0ac20aeb0a080b130b170b3a0b420b590ba80bd40be20b140c240c260c340c510c"
    "710c8f0cb40cd80cde0c240d450d6a0d9b0dc30dd10d030e050e070e080e1a0e2a0e560e600e8a0ea50eaa0ec00ecd0edb0ef00e110f210f400f420f540f980f"
)


def d4_256_codebook() -> np.ndarray:
    """The built-in 256-entry D4 grid of plain NVQ3 as int8 [256, 4] (odd magnitudes 1..15)."""
    enc = np.frombuffer(bytes.fromhex(_D4_256_HEX), dtype="<u2")
    digits = (enc[:, None] >> (3 * np.arange(4, dtype=np.uint16))[None, :]) & 7
    return np.ascontiguousarray(2 * digits + 1, dtype=np.int8)


def synthetic_d4_banks(entries: int, banks: int, seed: int) -> np.ndarray:
    """Seeded stand-in for the learned NVQ-JSC banks: ``entries`` distinct rows of odd
    magnitudes 1..15 per bank.  (Real files carry their banks inside the blob.)"""
    rng = np.random.default_rng(seed)
    digits = np.stack(np.meshgrid(*[np.arange(8)] * 4, indexing="ij"), -1).reshape(-1, 4)
    out = np.empty((banks, entries, 4), dtype=np.int8)
    for b in range(banks):
        out[b] = (2 * digits[rng.choice(digits.shape[0], entries, replace=False)] + 1).astype(np.int8)
    return out


# ---------------------------------------------------------------------------------------
# NINTM and the file container
# ---------------------------------------------------------------------------------------

def nintm_blob(n_experts: int, out_per_expert: int, k: int, pools) -> bytes:
    """``pools`` = [(expert_ids, dtype, payload_blob)].  mfq/formats/io.py:304-347."""
    parts = [struct.pack("<4sIIII", b"NIM2", n_experts, out_per_expert, k, len(pools))]
    for ids, dtype, payload in pools:
        ids = np.ascontiguousarray(ids, dtype="<i4")
        d = dtype.encode("ascii")
        parts += [struct.pack("<IIQQ", ids.size, len(d), len(payload), 0), ids.tobytes(), d, payload]
    return b"".join(parts)


def quantize_expertwise(weight: np.ndarray, bits_per_expert, device: str = "cpu") -> bytes:
    """[E, out, k] float32 + one NINT code width per expert -> ``NINTM`` blob.  Experts of equal
    width form one cohort, in ascending expert order (mfq/quantize/expert_nint.py:507-583)."""
    e_count, out, k = weight.shape
    cohorts: dict[int, list[int]] = {}
    for e, b in enumerate(bits_per_expert):
        cohorts.setdefault(int(b), []).append(e)
    pools = []
    for b, ids in cohorts.items():
        bits, gs, sb = CANONICAL_NINT[b]
        rows = weight[ids].reshape(len(ids) * out, k)   # numpy array or torch tensor
        pools.append((ids, f"NINT{bits}", nint_blob(quantize_nint(rows, bits, gs, sb, device=device))))
    return nintm_blob(e_count, out, k, pools)


def mfq_file_image(arch: str, records, extra: dict | None = None, version: int = 2) -> bytes:
    """``records`` = [(name, dtype, blob)].  mfq/formats/io.py:646-685."""
    def s(x: str) -> bytes:
        b = x.encode("utf-8")
        return struct.pack("<I", len(b)) + b

    extra = extra or {}
    if extra and version < 2:
        version = 2
    parts = [b"MFQ1", struct.pack("<I", version), s(arch)]
    if version >= 2:
        parts.append(struct.pack("<I", len(extra)))
        for k, v in extra.items():
            parts += [s(str(k)), s(json.dumps(v))]
    parts.append(struct.pack("<I", len(records)))
    for name, dtype, blob in records:
        parts += [s(name), s(dtype), struct.pack("<Q", len(blob))]
    parts += [blob for _, _, blob in records]
    return b"".join(parts)
