"""Dense decoder step over the C ABI (mirrors ``QuantLinear`` / ``FFN`` / ``FullBlock::forward`` /
``Model::next_token`` of the reference runtime, cpp_runtime/mfq_decode.cpp:9116-9407, 10456-10602,
12210-12400, 13993-14145, for Llama-shaped blocks).  torch only provides device memory and streams."""

from __future__ import annotations

import ctypes as C

import numpy as np

from ._capi import DecoderConfig, check, lib
from .linear import QuantWeight, _stream_ptr, _torch


class Decoder:
    """One rank's share of a decoder: borrowed weight handles, KV cache, one greedy step per call."""

    def __init__(self, *, hidden, n_q_heads, n_kv_heads, ffn, vocab, layers, max_ctx, max_batch,
                 rope_theta=500000.0, rms_eps=1e-5, rank=0, world=1, comm=None, device=0):
        self.cfg = DecoderConfig(hidden, n_q_heads, n_kv_heads, 128, ffn, vocab, layers, max_ctx, max_batch, rope_theta, rms_eps)
        self.rank, self.world, self.device = rank, world, device
        self._comm = comm
        self._keep = []   # the weights are borrowed by the native object: keep them alive here
        self._h = C.c_void_p()
        check(lib.mfqb_decoder_create(C.byref(self.cfg), rank, world, comm._h if comm is not None else None, device, C.byref(self._h)))

    def set_layer(self, layer: int, qkv: QuantWeight, o: QuantWeight, gate_up: QuantWeight, down: QuantWeight) -> None:
        check(lib.mfqb_decoder_set_layer(self._h, layer, qkv._h, o._h, gate_up._h, down._h))
        self._keep += [qkv, o, gate_up, down]

    def vocab_shard(self):
        b, n = C.c_int(), C.c_int()
        check(lib.mfqb_decoder_vocab_shard(self._h, C.byref(b), C.byref(n)))
        return b.value, n.value

    def set_head(self, lm_head: QuantWeight, embedding) -> None:
        torch = _torch()
        if embedding.dtype != torch.bfloat16 or not embedding.is_cuda or not embedding.is_contiguous():
            raise ValueError("embedding must be a contiguous bfloat16 CUDA tensor [vocab, hidden]")
        check(lib.mfqb_decoder_set_head(self._h, lm_head._h, embedding.data_ptr()))
        self._keep += [lm_head, embedding]

    def fill_cache(self, ctx_len: int, seed: int = 0) -> None:
        check(lib.mfqb_decoder_fill_cache(self._h, ctx_len, seed, _stream_ptr(self.device)))

    def step(self, ids_in, ids_out=None):
        torch = _torch()
        if ids_in.dtype != torch.int32 or not ids_in.is_cuda:
            raise ValueError("ids_in must be an int32 CUDA tensor [batch]")
        ids_out = torch.empty_like(ids_in) if ids_out is None else ids_out
        check(lib.mfqb_decoder_step(self._h, ids_in.data_ptr(), ids_in.numel(), ids_out.data_ptr(), _stream_ptr(self.device)))
        return ids_out

    def layer(self, layer: int, h_in):
        torch = _torch()
        h_in = h_in.contiguous().float()
        out = torch.empty_like(h_in)
        check(lib.mfqb_decoder_layer(self._h, layer, h_in.data_ptr(), h_in.shape[0], out.data_ptr(), _stream_ptr(self.device)))
        return out

    def read_cache(self, layer: int, row: int, which: int, ctx: int):
        torch = _torch()
        nkv = self.cfg.n_kv_heads // self.world
        out = torch.empty((nkv, ctx, 128), dtype=torch.bfloat16, device=f"cuda:{self.device}")
        check(lib.mfqb_decoder_read_cache(self._h, layer, row, which, ctx, out.data_ptr(), _stream_ptr(self.device)))
        return out

    def read_logits(self, rows: int):
        """float32 [rows, vocabulary rows of this rank]: the logits of the last step."""
        torch = _torch()
        begin, n = C.c_int(), C.c_int()
        check(lib.mfqb_decoder_vocab_shard(self._h, C.byref(begin), C.byref(n)))
        out = torch.empty((rows, n.value), dtype=torch.float32, device=f"cuda:{self.device}")
        check(lib.mfqb_decoder_read_logits(self._h, rows, out.data_ptr(), _stream_ptr(self.device)))
        return out

    def free(self) -> None:
        if self._h:
            lib.mfqb_decoder_free(self._h)
            self._h = C.c_void_p()
        self._keep = []

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def random_decoder(*, hidden, n_q_heads, n_kv_heads, ffn, vocab, layers, max_ctx, max_batch, rank=0, world=1, comm=None,
                   device=0, seed=5000, attn_profile=(4, 24, 6), ffn_profile=(6, 24, 7), distinct_layers=2, keep_blobs=False):
    """A random-init decoder in this rank's tensor-parallel shapes: attention projections in
    ``attn_profile``, FFN and lm_head in ``ffn_profile`` (bits, group size, sub-scale bits).
    ``distinct_layers`` layers are packed from their own seeded blobs; the others are device copies of
    those (every layer still streams its own memory).  Returns (decoder, blobs) -- blobs of the packed
    layers when ``keep_blobs`` (for parity checks against the oracle)."""
    from . import encode
    torch = _torch()
    d = f"cuda:{device}"
    dec = Decoder(hidden=hidden, n_q_heads=n_q_heads, n_kv_heads=n_kv_heads, ffn=ffn, vocab=vocab, layers=layers, max_ctx=max_ctx,
                  max_batch=max_batch, rank=rank, world=world, comm=comm, device=device)
    nq, nkv, f = n_q_heads // world, n_kv_heads // world, ffn // world
    shapes = {"qkv": ((nq + 2 * nkv) * 128, hidden, attn_profile), "o": (hidden, nq * 128, attn_profile),
              "gate_up": (2 * f, hidden, ffn_profile), "down": (hidden, f, ffn_profile)}
    base, blobs = [], []
    for li in range(min(distinct_layers, layers)):
        ws, bl = {}, {}
        for j, (name, (n, k, (bits, gs, sb))) in enumerate(shapes.items()):
            blob = encode.random_nint_blob(n, k, bits, gs, sb, seed=seed + 100 * li + 10 * j + rank * 7919, device=d)
            ws[name] = QuantWeight.from_blob(f"NINT{bits}", blob, device=device)
            if keep_blobs:
                bl[name] = blob
        base.append(ws)
        blobs.append(bl)
    for li in range(layers):
        src = base[li % len(base)]
        ws = src if li < len(base) else {k: v.clone() for k, v in src.items()}
        dec.set_layer(li, ws["qkv"], ws["o"], ws["gate_up"], ws["down"])
    vb, vn = dec.vocab_shard()
    bits, gs, sb = ffn_profile
    head_blob = encode.random_nint_blob(vn, hidden, bits, gs, sb, seed=seed + 9000 + rank * 7919, device=d)
    lm_head = QuantWeight.from_blob(f"NINT{bits}", head_blob, device=device)
    gen = torch.Generator(d).manual_seed(seed + 1)   # the embedding is replicated: same seed on every rank
    emb = torch.randn((vocab, hidden), device=d, generator=gen).to(torch.bfloat16)
    dec.set_head(lm_head, emb)
    if keep_blobs:
        blobs.append({"lm_head": head_blob, "embedding": emb})
    return dec, blobs
