"""Multi-GPU: one-shot NVLink all-reduce, the expert-parallel FFN, the row-parallel product that
reduces in its epilogue and the tensor-parallel decoder step, as child processes on 2, 4 and 8 GPUs
(each case is skipped on a box with fewer).  Failures are made on the host: a rank that does not
join makes the peer's bounded wait run out, which must surface as a status, not a hang; the
communicator is then reset and used again."""

import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist

    from oracle import mfq_oracle as O
    from tyloquant_b200 import _capi, comm, encode, moe

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    res = {}
    try:
        c = comm.Communicator(rank, world, 1 << 16, rank).connect()
        # 1. sums, identical on every rank, several sizes back to back
        for n in (1, 2048, 5000, 1 << 16):
            g = torch.Generator("cuda").manual_seed(100 + rank)
            x = torch.randn(n, device="cuda", generator=g)
            y = c.allreduce(x)
            xs = [torch.empty(n) for _ in range(world)]
            dist.all_gather(xs, x.cpu())
            want = sum(xs[1:], xs[0].clone())          # rank order, like the kernel
            res[f"sum{n}"] = bool(torch.equal(y.cpu(), want))
            ys = [torch.empty(n) for _ in range(world)]
            dist.all_gather(ys, y.cpu())
            res[f"same{n}"] = all(torch.equal(ys[0], t) for t in ys)
        torch.cuda.synchronize()
        res["status_ok"] = c.status() == 0

        # 2. expert-parallel FFN: each rank holds an expert range, partial outputs are all-reduced
        e_count, h, f, k, tokens = 16, 256, 96, 4, 5
        bits = np.random.default_rng(1).choice([2, 3, 4, 6], e_count)
        rng = np.random.default_rng(2)
        wgu = encode.bf16_round(rng.standard_normal((e_count, 2 * f, h), dtype=np.float32) * np.float32(0.02))
        wdn = encode.bf16_round(rng.standard_normal((e_count, h, f), dtype=np.float32) * np.float32(0.02))
        gu_blob, dn_blob = encode.quantize_expertwise(wgu, bits), encode.quantize_expertwise(wdn, bits)
        b, e = comm.shard_range(e_count, rank, world, 128)
        gu, dn = moe.MoeWeight(gu_blob, rank, b, e), moe.MoeWeight(dn_blob, rank, b, e)
        x = encode.bf16_round(rng.standard_normal((tokens, h), dtype=np.float32))
        z = rng.standard_normal((tokens, e_count)).astype(np.float32)
        ids, wts = moe.moe_topk(torch.from_numpy(z).cuda(), k)
        part = moe.moe_ffn(gu, dn, torch.from_numpy(x).cuda().to(torch.bfloat16), ids, wts)
        y = c.allreduce(part.reshape(-1)).reshape(tokens, h).cpu().numpy()
        rid, rw = O.moe_topk(z, k)
        y_ref = O.moe_ffn(x, O.dequant_nintm(O.unpack_nintm(gu_blob)), O.dequant_nintm(O.unpack_nintm(dn_blob)), rid, rw)
        res["ep_err"] = float(np.linalg.norm(y - y_ref) / np.linalg.norm(y_ref))

        # 2b. row-parallel linear fused with its reduction: each rank holds a K-slice of the weight
        from tyloquant_b200 import QuantWeight
        for bits_, gs_, sb_, dtype_ in ((3, 24, 5, "NINT3"), (4, 32, 6, "NINT4")):
            n_rows, k_cols = 200, 40 * gs_
            blob = encode.random_nint_blob(n_rows, k_cols, bits_, gs_, sb_, seed=77)
            g0, g1 = comm.shard_range(40, rank, world, 16)   # whole groups, reference granularity rule
            lo, hi = g0 * gs_, g1 * gs_
            shard = QuantWeight.from_blob(dtype_, blob, device=rank, axis=1, begin=lo, end=hi)
            xr = encode.bf16_round(np.random.default_rng(5).standard_normal((3, k_cols), dtype=np.float32))
            y_f = c.matmul_allreduce(shard, torch.from_numpy(xr[:, lo:hi].copy()).cuda().to(torch.bfloat16), out_dtype=torch.float32)
            y_want = O.linear(xr, O.dequant_nint(O.unpack_nint(blob)))
            res[f"rowpar_err_{dtype_}"] = float(np.linalg.norm(y_f.cpu().numpy() - y_want) / np.linalg.norm(y_want))
            ys = [torch.empty(y_f.shape) for _ in range(world)]
            dist.all_gather(ys, y_f.cpu())
            res[f"rowpar_same_{dtype_}"] = all(torch.equal(ys[0], t) for t in ys)
            shard.free()
        torch.cuda.synchronize()
        res["status_ok2"] = c.status() == 0

        # 2c. the call number across its 32-bit wrap: the slot sets must keep alternating
        dist.barrier()
        _capi.check(_capi.lib.mfqb_comm_debug_set_seq(c._h, 0xFFFFFFFD))
        dist.barrier()
        ok = True
        for i in range(6):
            x = torch.full((300,), float(rank + 1 + i), device="cuda")
            ok = ok and bool(torch.equal(c.allreduce(x).cpu(), torch.full((300,), float(sum(r + 1 + i for r in range(world))))))
        torch.cuda.synchronize()
        res["wrap_ok"] = ok and c.status() == 0

        # 2d. tensor-parallel decoder steps: every rank must emit the same tokens
        from tyloquant_b200 import decoder as D
        cd = comm.Communicator(rank, world, 3 * 1024, rank).connect()
        dec, _ = D.random_decoder(hidden=1024, n_q_heads=8, n_kv_heads=8, ffn=512 * world, vocab=3000, layers=2, max_ctx=48, max_batch=3,
                                  rank=rank, world=world, comm=cd, device=rank, seed=31)
        dec.fill_cache(16, seed=4)
        toks = []
        for batch in (1, 3):
            a = torch.arange(1, batch + 1, dtype=torch.int32, device="cuda")
            for _ in range(2):
                a = dec.step(a)
            torch.cuda.synchronize()
            toks.append(a.cpu())
        gathered = [None] * world
        dist.all_gather_object(gathered, [t.tolist() for t in toks])
        res["decoder_same"] = all(g == gathered[0] for g in gathered)
        res["decoder_range"] = all(0 <= v < 3000 for t in toks for v in t.tolist())
        res["decoder_status"] = cd.status() == 0
        dec.free()
        cd.close()

        # 3. a rank that does not join: the other rank's wait runs out and reports it; then the
        # communicator is reset on every rank and works again
        dist.barrier()
        c.set_timeout_ms(200)
        if rank == 0:
            c.allreduce(torch.ones(64, device="cuda"))
            torch.cuda.synchronize()
            res["timeout_status"] = c.status()
            res["context_alive"] = bool((torch.ones(4, device="cuda") * 2).sum().item() == 8.0)
        dist.barrier()
        c.reset()
        c.set_timeout_ms(2000)
        y = c.allreduce(torch.full((128,), float(rank), device="cuda"))
        torch.cuda.synchronize()
        res["after_reset"] = bool(torch.equal(y.cpu(), torch.full((128,), float(sum(range(world)))))) and c.status() == 0
        dist.barrier()
        c.close()
    finally:
        q.put((rank, res))
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_allreduce_expert_parallel_decoder_and_timeout(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    from tyloquant_b200 import _capi
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank in range(world):
        r = results[rank]
        for n in (1, 2048, 5000, 1 << 16):
            assert r[f"sum{n}"] and r[f"same{n}"], (rank, n)
        assert r["status_ok"]
        assert r["ep_err"] <= 1e-3
        for dt in ("NINT3", "NINT4"):
            assert r[f"rowpar_err_{dt}"] <= 1e-3 and r[f"rowpar_same_{dt}"], (rank, dt)
        assert r["status_ok2"]
        assert r["wrap_ok"]
        assert r["decoder_same"] and r["decoder_range"] and r["decoder_status"]
        assert r["after_reset"]
    assert results[0]["timeout_status"] == _capi.ERR_TIMEOUT
    assert results[0]["context_alive"]
