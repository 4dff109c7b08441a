"""The C-ABI library loads and exports exactly the symbols include/raft_b200.h declares, and the
ctypes binding knows every one of them. No compute call is made (runs without a GPU)."""
import ctypes
import os
import re

from raft_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header="raft_b200.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"B2R_API\s+[\w\s\*]+?\b(b2r_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared()
    for must in ("b2r_reduce", "b2r_norm", "b2r_reduce_rows_by_key", "b2r_reduce_cols_by_key",
                 "b2r_reduce_workspace_bytes", "b2r_status_string"):
        assert must in names


def test_library_exports_every_declared_symbol():
    assert os.path.exists(_lib.LIB_PATH), "run __graft_entry__.build() first"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in _declared():
        assert hasattr(lib, name), f"{name} declared in raft_b200.h but not exported"


def test_binding_covers_every_declared_symbol():
    assert sorted(_lib.SIGNATURES) == _declared()
    lib = _lib.load()
    assert lib.b2r_status_string(0).decode() == "ok"
    assert lib.b2r_status_string(4).decode().startswith("size beyond")
    assert b"sm_100a" in lib.b2r_version()


def test_descriptor_layout_matches_the_header():
    # b2r_reduce_desc: 4 x int32, 2 x int64, 4 x int32, double, 2 x int64, double = 80 bytes
    assert ctypes.sizeof(_lib.ReduceDesc) == 80
    assert _lib.ReduceDesc.n_rows.offset == 16 and _lib.ReduceDesc.init.offset == 48
    assert _lib.ReduceDesc.final_scalar.offset == 72


def test_multi_device_library_exports_every_declared_symbol():
    """libraft_b200_mg.so (NCCL layer, include/raft_b200_mg.h). Loading needs NCCL on the loader path;
    no device call is made."""
    path = os.path.join(ROOT, "raft_b200", "libraft_b200_mg.so")
    assert os.path.exists(path), "run __graft_entry__.build() first"
    ctypes.CDLL(_lib.LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    lib = ctypes.CDLL(path)
    names = _declared("raft_b200_mg.h")
    assert "b2r_mg_reduce" in names and "b2r_mg_reduce_rows_by_key" in names and "b2r_mg_comm_create" in names
    for name in names:
        assert hasattr(lib, name), f"{name} declared in raft_b200_mg.h but not exported"
    lib.b2r_mg_comm_size.argtypes = [ctypes.c_void_p]
    assert lib.b2r_mg_comm_size(None) == 0
