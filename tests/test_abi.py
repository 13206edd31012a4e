"""The C-ABI library loads and exports every symbol include/fastlstm_b200.h declares.
No compute calls (runs without a GPU)."""
import ctypes
import os
import re

import pytest

from fastlstm_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "fastlstm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(blstm_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_agree():
    declared = _declared_symbols()
    assert declared, "no declarations found"
    assert sorted(_lib.SIGNATURES) == declared


def test_library_exports_every_declared_symbol():
    if not os.path.exists(_lib.LIB_PATH):
        from fastlstm_b200.build import build
        build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in _declared_symbols():
        assert hasattr(lib, name), name


def test_host_only_entry_points():
    lib = _lib.load()
    assert lib.blstm_abi_version() == _lib.ABI_VERSION
    assert b"ok" == lib.blstm_strerror(0)
    assert b"wait" in lib.blstm_strerror(_lib.E_WAIT_TIMEOUT)
    d = _lib.Desc(_lib.F32, 64, 16, 128, 128, 0, 0, 0)
    fwd = lib.blstm_workspace_bytes(d, _lib.PHASE_FWD)
    bwd = lib.blstm_workspace_bytes(d, _lib.PHASE_BWD)
    assert fwd >= 256 and fwd % 256 == 0 and bwd > fwd and bwd % 256 == 0
    assert lib.blstm_plan_name(d, _lib.PHASE_FWD) == b"generic"
    bad = _lib.Desc(7, 64, 16, 128, 128, 0, 0, 0)
    assert lib.blstm_workspace_bytes(bad, _lib.PHASE_FWD) == 0
    # argument validation happens before any CUDA call
    assert lib.blstm_fwd(bad, *([None] * 11), 0, None) == 1
    assert lib.blstm_fwd(d, *([None] * 11), 0, None) == 1
    # 16-bit tensors move in 16-byte pieces: a misaligned base pointer is refused (fake addresses;
    # the check comes before anything touches them)
    h = _lib.Desc(_lib.BF16, 8, 128, 64, 64, 0, 0, 0)
    ok_ptr, odd_ptr = 0x10000, 0x10002
    assert lib.blstm_fwd_recurrence(h, odd_ptr, ok_ptr, ok_ptr, ok_ptr, None, 0, None) == 1
    assert lib.blstm_fwd_recurrence(h, ok_ptr, ok_ptr, ok_ptr, odd_ptr, None, 0, None) == 1
    assert lib.blstm_fwd_recurrence(h, ok_ptr, ok_ptr, ok_ptr, ok_ptr, None, 0, None) == 3
    assert lib.blstm_fwd_recurrence_static(h, ok_ptr, odd_ptr, ok_ptr, ok_ptr, None) == 1


def test_desc_struct_layout_matches_header():
    assert ctypes.sizeof(_lib.Desc) == 32
