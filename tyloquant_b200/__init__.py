"""B200-native execution path for MFQ packed weights (NINT / NVQ3 / NINTM).

Host-side mirror of the reference operator surface over the C ABI of ``libmfqb200.so``:

* :class:`MfqFile` -- container reader (the reference ``MfqFile`` / ``open_mmap``),
* :class:`QuantWeight` -- a dense quantized weight on a GPU with ``dequantize`` and
  ``matmul`` (the reference ``NintWeight`` / ``NvqWeight`` + ``nint_matmul`` / ``nvq_matmul``),
* :func:`plan_tensor_parallel_slices` and friends -- the tensor-parallel slice planner,
* :mod:`tyloquant_b200.encode` -- writers for synthetic MFQ tensors (benchmarks, tests).
"""

from ._capi import BF16, F32, MfqbError
from .container import MfqFile
from .linear import QuantWeight
from .tp import plan_tensor_parallel_slices, tensor_parallel_granularity, validate_tensor_parallel_slices

__all__ = ["BF16", "F32", "MfqbError", "MfqFile", "QuantWeight", "plan_tensor_parallel_slices",
           "tensor_parallel_granularity", "validate_tensor_parallel_slices"]
