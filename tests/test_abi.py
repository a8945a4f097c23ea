"""The C-ABI library loads without a GPU, exports every symbol include/dsa_v32.h declares, keeps the
frozen struct sizes, and rejects bad arguments before any launch."""
import ctypes as C
import os
import re

import pytest

from opfoundry_b200 import api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "dsa_v32.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dsa_v32_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(built_lib):
    syms = declared_symbols()
    assert len(syms) >= 14
    for s in syms:
        assert hasattr(built_lib, s), s
    assert sorted(api.EXPORTS) == syms
    assert built_lib.dsa_v32_abi_version() == 1


def test_struct_sizes_match_header():
    assert C.sizeof(api.WorkInfo) == 32          # same size as the reference's work_info (defs.h:64-73,173)
    assert C.sizeof(api.Shape) == 40
    assert C.sizeof(api.PlanInfo) == 24
    assert C.sizeof(api.AttnArgs) == 7 * 8 + 7 * 8 + 8 * 4


def test_error_strings(built_lib):
    assert built_lib.dsa_v32_error_string(0) == b"ok"
    assert b"NULL" in built_lib.dsa_v32_error_string(-1)
    assert b"wait" in built_lib.dsa_v32_error_string(1001)


def test_arguments_rejected_before_launch(built_lib):
    a = api.AttnArgs()
    assert built_lib.dsa_v32_decode_bf16(C.byref(a), None) == -1          # null pointers
    assert built_lib.dsa_v32_decode_bf16(None, None) == -1
    buf = (C.c_uint8 * 4096)()
    base = (C.addressof(buf) + 255) & ~255
    a.q = a.kv = a.out = a.indices = a.workspace = base
    a.kv_dtype = api.KV_FP8
    assert built_lib.dsa_v32_decode_bf16(C.byref(a), None) == -5          # dtype mismatch
    a.kv_dtype = api.KV_BF16
    assert built_lib.dsa_v32_decode_bf16(C.byref(a), None) == -2          # zero shape
    a.total_q, a.H, a.topk, a.s_q, a.num_kv_rows = 4, 128, 64, 1, 100
    a.stride_q_head, a.stride_q_row, a.stride_o_head, a.stride_o_row = 576, 128 * 576, 512, 128 * 512
    a.sm_scale = 0.07
    a.q = base + 2
    assert built_lib.dsa_v32_decode_bf16(C.byref(a), None) == -3          # misaligned q
    a.q = base
    a.stride_q_row = 128 * 576 + 4
    assert built_lib.dsa_v32_decode_bf16(C.byref(a), None) == -3          # stride not a multiple of 16 bytes
    a.stride_q_row = 128 * 576
    a.sm_scale = 0.0
    assert built_lib.dsa_v32_decode_bf16(C.byref(a), None) == -2
    a.sm_scale = 0.07
    assert built_lib.dsa_v32_decode_bf16(C.byref(a), None) == -4          # workspace never planned
    assert built_lib.dsa_v32_combine(C.byref(a), None) == -4
    assert built_lib.dsa_v32_pack_fp8_rows(None, None, None, None, 4, None) == -1


def test_missing_library_is_loud(monkeypatch):
    monkeypatch.setattr(api, "_lib", None)
    monkeypatch.setattr(api, "LIB_PATH", "/nonexistent/libdsa_v32.so")
    with pytest.raises(ImportError):
        api.lib()
