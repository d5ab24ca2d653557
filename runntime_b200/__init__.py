"""runntime_b200 — the attention hot path of ruNNtime as hand-written sm_100a
CUDA behind the runtime's own operator API.

``sdpa``, ``sdpaPacked``, ``rope``, ``slice``, ``writeRows`` and ``MultiHeadAttention`` keep the
reference's names, options and errors; ``CudaExecutor`` + ``evalValues`` /
``toArray`` stand where its WebGPU executor does.  ``engine`` holds the batched
entry points (padded-batch prefill, batched KV-cache decode, KV-sequence
sharded decode).  Everything computes through librt_attn.so (include/rt_attn.h);
there is no CPU path.
"""
from .errors import RUNNTIME_ERROR_CODES, RunntimeError
from .executor import CudaExecutor, evalValues, gpuExecutor, toArray
from .nn import MultiHeadAttention, Parameter
from .ops import (ACT_CODE, argmaxDot, chunk, localAttention, matmul, rope, sdpa, sdpaPacked,
                  slice, softmax, writeRows)
from .value import DeviceBuffer, Value, ValueMeta, materialized, matrix, pending

__all__ = [
    "RUNNTIME_ERROR_CODES", "RunntimeError", "CudaExecutor", "gpuExecutor", "evalValues",
    "toArray", "MultiHeadAttention", "Parameter", "rope", "sdpa", "sdpaPacked", "writeRows",
    "slice", "chunk", "softmax", "localAttention", "matmul", "argmaxDot", "ACT_CODE",
    "DeviceBuffer", "Value", "ValueMeta", "materialized", "matrix", "pending",
]
