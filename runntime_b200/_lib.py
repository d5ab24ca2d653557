"""ctypes binding of librt_attn.so — the same C ABI a Node N-API addon binds.

There is no CPU fallback: if the library is missing the import of anything that
computes fails with NOT_INITIALIZED and says how to build it.
"""
from __future__ import annotations

import ctypes as C
import os

from .errors import RunntimeError, code_of_status

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librt_attn.so")

RT_F32, RT_F16 = 0, 1
WINDOW_INF = 0x3FFFFFFF
OPT_PREFILL_TC = 1
OPT_WAIT_POLLS = 2
XMEM_HANDLE_BYTES = 64
DTYPE_CODE = {"f32": RT_F32, "f16": RT_F16}


class AttnArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("sinks", C.c_void_p), ("segments", C.c_void_p),
        ("dtype", C.c_int32), ("qkvPacked", C.c_int32),
        ("qLen", C.c_int64), ("kvLen", C.c_int64),
        ("qHeads", C.c_int32), ("kvHeads", C.c_int32), ("headDim", C.c_int32),
        ("windowLeft", C.c_int32), ("windowRight", C.c_int32), ("maxSegment", C.c_int32),
        ("qPosOffset", C.c_int64),
        ("hasKeyBias", C.c_int32), ("biasStart", C.c_int32), ("biasEnd", C.c_int32),
        ("biasValue", C.c_float),
        ("seqStride", C.c_int32), ("seqLens", C.c_void_p),
    ]


MAX_PEERS = 8


class Exchange(C.Structure):
    """rt_exchange: where the ranks sharing a set of sequences trade partials."""
    _fields_ = [
        ("world", C.c_int32), ("rank", C.c_int32),
        ("partials", C.c_void_p * MAX_PEERS), ("flags", C.c_void_p * MAX_PEERS),
        ("step", C.c_void_p), ("stage", C.c_void_p), ("phases", C.c_int32),
    ]


class DecodeSecond(C.Structure):
    """rt_decode_second: a second attention (cross-attention) in the same decode launch."""
    _fields_ = [
        ("q", C.c_void_p), ("out", C.c_void_p), ("kCache", C.c_void_p), ("vCache", C.c_void_p),
        ("kCachePtrs", C.c_void_p), ("vCachePtrs", C.c_void_p), ("kvLens", C.c_void_p),
        ("cacheSeqStride", C.c_int64), ("qRowStride", C.c_int64),
        ("cacheRows", C.c_int32), ("kvLen", C.c_int32), ("windowLeft", C.c_int32),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("out", C.c_void_p), ("kCache", C.c_void_p), ("vCache", C.c_void_p),
        ("kNew", C.c_void_p), ("vNew", C.c_void_p), ("kvLens", C.c_void_p),
        ("sinks", C.c_void_p), ("partialsOut", C.c_void_p),
        ("cacheSeqStride", C.c_int64),
        ("dtype", C.c_int32), ("batch", C.c_int32), ("cacheRows", C.c_int32),
        ("kvLen", C.c_int32), ("qHeads", C.c_int32), ("kvHeads", C.c_int32),
        ("headDim", C.c_int32), ("windowLeft", C.c_int32), ("splits", C.c_int32),
        ("ropeByPosition", C.c_int32), ("ropeCos", C.c_void_p), ("ropeSin", C.c_void_p),
        ("qRowStride", C.c_int64), ("kNewRowStride", C.c_int64), ("vNewRowStride", C.c_int64),
        ("exchange", C.POINTER(Exchange)),
        ("kvSharded", C.c_int32), ("shardStart", C.c_int32),
        ("kCachePtrs", C.c_void_p), ("vCachePtrs", C.c_void_p),
        ("second", C.POINTER(DecodeSecond)),
    ]


# name -> (restype, argtypes); every symbol include/rt_attn.h declares.
SYMBOLS = {
    "rt_ctx_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "rt_ctx_destroy": (C.c_int, [C.c_void_p]),
    "rt_ctx_set_stream": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int]),
    "rt_ctx_set_option": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "rt_last_error": (C.c_char_p, [C.c_void_p]),
    "rt_sync": (C.c_int, [C.c_void_p]),
    "rt_launch_count": (C.c_int64, [C.c_void_p]),
    "rt_buf_alloc": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "rt_buf_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "rt_buf_upload": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]),
    "rt_buf_download": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]),
    "rt_attn": (C.c_int, [C.c_void_p, C.POINTER(AttnArgs)]),
    "rt_attn_route": (C.c_int, [C.c_void_p, C.POINTER(AttnArgs), C.POINTER(C.c_char_p)]),
    "rt_attn_decode": (C.c_int, [C.c_void_p, C.POINTER(DecodeArgs)]),
    "rt_attn_decode_noalloc": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "rt_attn_decode_noalloc_status": (C.c_int, [C.c_void_p]),
    "rt_xmem_create": (C.c_int, [C.c_int, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                 C.POINTER(C.c_void_p)]),
    "rt_xmem_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "rt_xmem_import": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    "rt_xmem_attach": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    "rt_xmem_exchange": (C.c_int, [C.c_void_p, C.POINTER(Exchange)]),
    "rt_xmem_destroy": (C.c_int, [C.c_void_p]),
    "rt_attn_merge_partials": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32,
                                         C.c_void_p, C.c_int32]),
    "rt_rope": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                          C.c_int64, C.c_int32, C.c_int64, C.c_int64, C.c_int32]),
    "rt_matmul": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                            C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int32,
                            C.c_int32]),
    "rt_argmax_dot": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                C.c_int64, C.c_int32]),
    "rt_local_attention": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_float,
                                     C.c_float, C.c_int32]),
    "rt_softmax": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                             C.c_int32, C.c_int32, C.c_int32]),
    "rt_slice": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                           C.c_int64, C.c_int64, C.c_int64, C.c_int32]),
    "rt_kv_append": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                               C.c_int64, C.c_int64, C.c_int32]),
}

_lib = None


def load():
    """The loaded library, or NOT_INITIALIZED if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RunntimeError(
                "NOT_INITIALIZED",
                f"{LIB_PATH} is missing: build it with `python -m runntime_b200.build` "
                "(there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int, ctx=None):
    """Raises RunntimeError for a non-zero rt_status."""
    if status != 0:
        msg = load().rt_last_error(ctx)
        raise RunntimeError(code_of_status(status), (msg or b"").decode("utf-8", "replace"))
