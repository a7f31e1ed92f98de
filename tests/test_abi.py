"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
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
  assert 16 <= library.cdb_rel_l1_scratch_bytes() <= 65536


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


C_CONSUMER = r"""
#include <stdio.h>
#include "cache_dit_b200.h"
int main(void) {
  /* metadata and argument validation: no CUDA call is reached */
  if (cdb_abi_version() < 1) return 2;
  if (cdb_rel_l1(NULL, NULL, NULL, NULL, 0, 1, NULL, NULL, 0, NULL) != 1) return 3;
  if (cdb_fp8_gemm_rowscaled(NULL, NULL, NULL, NULL, NULL, NULL, 1, 8, 16, 8, NULL, NULL) != 1) return 4;
  printf("%s|%d\n", cdb_status_string(0), (int)cdb_rel_l1_scratch_bytes());
  return 0;
}
"""


def test_plain_c_program_includes_header_and_links(library, tmp_path):
  """The boundary is C, not C++: a C99 translation unit includes the header with -pedantic, links the shared
  library and calls it (what a cgo / JNI / FFI binding does)."""
  import shutil
  import subprocess
  from cache_dit_b200 import _native
  if shutil.which("gcc") is None:
    pytest.skip("no gcc")
  src = tmp_path / "consumer.c"
  src.write_text(C_CONSUMER)
  exe = tmp_path / "consumer"
  libdir = os.path.dirname(_native.LIB_PATH)
  subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", os.path.dirname(HEADER), str(src),
                  "-o", str(exe), "-L", libdir, "-l:" + os.path.basename(_native.LIB_PATH), "-Wl,-rpath," + libdir],
                 check=True, capture_output=True)
  out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.strip()
  assert out.split("|")[0] == "ok" and int(out.split("|")[1]) >= 16
