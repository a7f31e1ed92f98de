"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "cache_dit_b200.h")


@pytest.fixture(scope="module")
def library():
  from cache_dit_b200.csrc import build
  from cache_dit_b200 import _native
  build.build()
  return _native.lib()


def declared_functions():
  text = open(HEADER).read()
  return sorted(set(re.findall(r"CDB_API[^;(]*?\b(cdb_\w+)\s*\(", text)))


def test_header_declares_something():
  assert len(declared_functions()) >= 8


def test_every_declared_symbol_is_exported(library):
  for name in declared_functions():
    assert hasattr(library, name), name


def test_binding_table_covers_header(library):
  from cache_dit_b200 import _native
  assert sorted(_native.SIGNATURES) == declared_functions()


def test_metadata_calls_work_without_gpu(library):
  assert library.cdb_abi_version() >= 1
  assert library.cdb_status_string(0) == b"ok"
  assert library.cdb_status_string(6) == b"bounded device-side wait expired"
  assert 16 <= library.cdb_rel_l1_scratch_bytes() <= 4096


def test_argument_validation_needs_no_gpu(library):
  # null pointers / bad sizes are rejected before any CUDA call is made
  assert library.cdb_rel_l1(None, None, None, None, 0, 1, None, None, 0, None) == 1
  assert library.cdb_fp8_quant_rows(None, 1, 8, 8, None, None, None) == 1
  assert library.cdb_fp8_gemm_rowscaled(None, None, None, None, None, None, 1, 8, 16, 8, None, None) == 1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
  from cache_dit_b200 import _native
  monkeypatch.setattr(_native, "_lib", None)
  monkeypatch.setattr(_native, "LIB_PATH", str(tmp_path / "nope.so"))
  with pytest.raises(_native.NativeLibraryError):
    _native.lib()
