"""The C-ABI library builds, loads and exports exactly what include/mdb200.h
declares; the ctypes table agrees with the header.  No GPU calls."""
import ctypes
import os
import re

import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "mdb200.h")


def _declared():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    out = {}
    for m in re.finditer(r"\b(?:const\s+char\s*\*|int64_t|int)\s+(mdb_\w+)\s*\(([^;{]*?)\)\s*;", src, flags=re.S):
        args = m.group(2).strip()
        n = 0 if args in ("", "void") else len([a for a in args.split(",") if a.strip()])
        out[m.group(1)] = n
    return out


@pytest.fixture(scope="module")
def built():
    import __graft_entry__ as entry
    entry.build()
    import importlib
    return importlib.import_module("mineru-diffusion_b200")


def test_header_declares_the_path():
    decl = _declared()
    for name in ("mdb_kv_commit", "mdb_attn_block_paged", "mdb_attn_staircase_varlen", "mdb_gemm_bf16",
                 "mdb_gemm_splitk_partials", "mdb_gemm_gateup_swiglu", "mdb_add_rmsnorm", "mdb_qknorm_rope_commit",
                 "mdb_lmhead_sample", "mdb_unmask_decide", "mdb_last_device_status", "mdb_strerror"):
        assert name in decl


def test_library_exports_every_declared_symbol(built):
    handle = ctypes.CDLL(built._lib.LIB_PATH)
    for name in _declared():
        assert hasattr(handle, name), f"{name} declared in mdb200.h but not exported"


def test_ctypes_table_matches_header(built):
    decl = _declared()
    table = built._lib.SIGNATURES
    assert set(table) == set(decl)
    for name, n in decl.items():
        assert len(table[name][1]) == n, f"{name}: header has {n} parameters, ctypes table {len(table[name][1])}"


def test_host_side_checks_need_no_gpu(built):
    lib = built._lib.lib()
    assert lib.mdb_version() >= 100
    assert lib.mdb_strerror(0) == b"ok"
    assert b"aligned" in lib.mdb_strerror(-2)
    # argument validation happens before any launch
    assert lib.mdb_kv_commit(None, 8, None, 8, None, None, None, 4, 1024, 100, None) == -1
    assert lib.mdb_kv_commit(None, 8, None, 8, None, None, None, 0, 1024, 100, None) == 0    # empty input
    assert lib.mdb_attn_block_paged(None, None, None, None, None, 1, None, 2, 32, 16, 5, 10, 0.1, 1, None, 0, None) == -1
    assert lib.mdb_gemm_splitk_workspace_bytes(32, 4096, 2) == 2 * 32 * 4096 * 4
    assert lib.mdb_attn_paged_workspace_bytes(4, 32, 16, 1) == 0
    assert lib.mdb_attn_paged_workspace_bytes(4, 32, 16, 3) == 4 * 3 * 16 * 32 * 130 * 4
    assert lib.mdb_lmhead_workspace_bytes(32, 151936) > 0


def test_ops_refuse_cpu_tensors(built):
    import torch
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        built.ops.linear(x, x)
    with pytest.raises(RuntimeError):
        built.ops.store_kvcache(x.view(4, 1, 64), x.view(4, 1, 64), x, x, torch.zeros(4, dtype=torch.int32))
