"""One-shot NVLink all-reduce between the one-process-per-GPU ranks of a ``torch.distributed``
group (stands in for ``reduce_tensor_parallel_outputs``, cpp_runtime/mfq_decode.cpp:9009-9114).
``torch.distributed`` only carries the 64-byte IPC handles at set-up; the reduction itself is the
library's kernel over peer memory."""

from __future__ import annotations

import ctypes as C

from ._capi import check, lib


def shard_range(extent: int, rank: int, world: int, granularity: int = 1):
    """Contiguous [begin, end) of ``extent`` owned by ``rank`` under the reference slice planner with
    equal weights (expert ranges, row/column slices)."""
    from .tp import plan_tensor_parallel_slices, tensor_parallel_granularity
    gran = tensor_parallel_granularity(extent, granularity, world)
    _, b, e = plan_tensor_parallel_slices(extent, gran, list(range(world)))[rank]
    return b, e


class Communicator:
    def __init__(self, rank: int, world: int, max_elems: int, device: int):
        self.rank, self.world, self.device = rank, world, device
        self._h = C.c_void_p()
        check(lib.mfqb_comm_create(rank, world, max_elems, device, C.byref(self._h)))

    def handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        check(lib.mfqb_comm_handle(self._h, buf))
        return buf.raw

    def attach(self, peer: int, handle: bytes) -> None:
        check(lib.mfqb_comm_attach(self._h, peer, C.create_string_buffer(handle, 64)))

    def connect(self, group=None) -> "Communicator":
        """Exchange the IPC handles over a ``torch.distributed`` group and attach every peer."""
        import torch.distributed as dist
        handles = [None] * self.world
        dist.all_gather_object(handles, self.handle(), group=group)
        for peer, h in enumerate(handles):
            if peer != self.rank:
                self.attach(peer, h)
        dist.barrier(group=group)
        return self

    def set_timeout_ms(self, ms: int) -> None:
        check(lib.mfqb_comm_set_timeout_ms(self._h, ms))

    def allreduce(self, x, out=None):
        """Sum the float32 CUDA tensor ``x`` over all ranks (same shape on every rank)."""
        import torch
        if x.dtype != torch.float32 or not x.is_cuda:
            raise ValueError("allreduce takes a float32 CUDA tensor")
        x = x.contiguous()
        out = torch.empty_like(x) if out is None else out
        check(lib.mfqb_allreduce_f32(self._h, x.data_ptr(), out.data_ptr(), x.numel(),
                                     torch.cuda.current_stream(self.device).cuda_stream))
        return out

    def matmul_allreduce(self, weight, x, out_dtype=None):
        """Row-parallel linear: ``weight`` is this rank's input-axis slice (``QuantWeight``), ``x`` the
        matching slice ``[m, k_slice]`` in bf16; returns the sum over ranks ``[m, n]`` on every rank.
        The product kernel itself pushes its partial rows to the peers and adds theirs."""
        import torch
        out_dtype = out_dtype or torch.bfloat16
        if x.dtype != torch.bfloat16 or not x.is_cuda:
            raise ValueError("matmul_allreduce takes a bf16 CUDA tensor")
        x = x.contiguous().reshape(-1, weight.k)
        y = torch.empty((x.shape[0], weight.n), dtype=out_dtype, device=x.device)
        from ._capi import BF16, F32
        check(lib.mfqb_mul_mat_allreduce(weight._h, x.data_ptr(), x.shape[0], self._h, y.data_ptr(),
                                         F32 if out_dtype == torch.float32 else BF16,
                                         torch.cuda.current_stream(self.device).cuda_stream))
        return y

    def reset(self, group=None) -> None:
        """After a timeout: clear this rank's slots and call number, then meet the other ranks."""
        import torch.distributed as dist
        check(lib.mfqb_comm_reset(self._h))
        dist.barrier(group=group)

    def status(self) -> int:
        s = C.c_int()
        check(lib.mfqb_comm_status(self._h, C.byref(s)))
        return s.value

    def close(self) -> None:
        if self._h:
            lib.mfqb_comm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
