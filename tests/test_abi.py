"""The C-ABI library loads without a GPU and exports exactly what
include/rt_attn.h declares; calls that need no device behave as documented."""
import ctypes as C
import os
import re

import pytest

import runntime_b200._lib as L
from runntime_b200 import RunntimeError
from runntime_b200.errors import RUNNTIME_ERROR_CODES, code_of_status

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    src = open(os.path.join(ROOT, "include", "rt_attn.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(rt_[a-z_]+)\s*\(", src)))


def test_header_and_binding_agree():
    assert _declared() == sorted(L.SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(L.LIB_PATH)
    for name in _declared():
        assert hasattr(lib, name), name


def test_status_codes_follow_reference_order():
    src = open(os.path.join(ROOT, "include", "rt_attn.h")).read()
    for i, code in enumerate(RUNNTIME_ERROR_CODES, start=1):
        assert re.search(rf"RT_{code} = {i}\b", src), code
        assert code_of_status(i) == code


def test_struct_layouts_match_header_field_order():
    src = open(os.path.join(ROOT, "include", "rt_attn.h")).read()
    for struct, cls in (("rt_attn_args", L.AttnArgs), ("rt_decode_args", L.DecodeArgs)):
        body = re.search(r"typedef struct \{([^}]*)\} " + struct + ";", src).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = re.findall(r"(\w+)\s*;", body)
        assert names == [f[0] for f in cls._fields_], struct


def test_calls_without_context_fail_cleanly():
    lib = L.load()
    assert lib.rt_sync(None) == 8  # NOT_INITIALIZED
    assert b"rt_ctx_create" in lib.rt_last_error(None)
    with pytest.raises(RunntimeError) as e:
        L.check(lib.rt_attn(None, None))
    assert e.value.code == "NOT_INITIALIZED"
    assert lib.rt_launch_count(None) == -1


def test_context_creation_needs_a_blackwell_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = L.load()
    ctx = C.c_void_p()
    status = lib.rt_ctx_create(0, C.byref(ctx))
    assert status == 4 and not ctx.value  # UNSUPPORTED_DEVICE
    assert lib.rt_ctx_create(0, None) == 6  # INVALID_ARGUMENT


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RunntimeError) as e:
        L.load()
    assert e.value.code == "NOT_INITIALIZED" and "no CPU fallback" in str(e.value)
