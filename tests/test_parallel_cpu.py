"""Host-side logic of the multi-GPU path on CPU: two gloo ranks agree on expert / slice ownership,
the shards cover the whole extent, and the communicator rejects misuse with a status."""

import ctypes as C
import os
import socket

import numpy as np
import pytest

import tyloquant_b200 as T
from tyloquant_b200 import _capi, comm
from tyloquant_b200._capi import lib


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = {"experts": comm.shard_range(128, rank, world, 128), "rows": comm.shard_range(14336, rank, world, 128),
                "groups": comm.shard_range(171, rank, world, 16)}
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        q.put((rank, gathered))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_ranks_agree_on_contiguous_cover(world):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    views = [g for _, g in results]
    assert all(v == views[0] for v in views)          # every rank sees the same plan
    for key, extent in (("experts", 128), ("rows", 14336), ("groups", 171)):
        spans = [views[0][r][key] for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == extent
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        assert all(e > b for b, e in spans)


def test_communicator_argument_checks():
    h = C.c_void_p()
    assert lib.mfqb_comm_create(2, 2, 1024, 0, C.byref(h)) == _capi.ERR_ARG      # rank out of range
    assert lib.mfqb_comm_create(0, 9, 1024, 0, C.byref(h)) == _capi.ERR_ARG      # world too large
    assert lib.mfqb_comm_create(0, 2, 0, 0, C.byref(h)) == _capi.ERR_ARG         # empty buffer
    assert lib.mfqb_comm_create(0, 2, 1 << 30, 0, C.byref(h)) == _capi.ERR_ARG   # beyond the one-shot limit
    assert b"max_elems" in lib.mfqb_last_error()
    assert lib.mfqb_comm_status(None, None) == _capi.ERR_ARG
