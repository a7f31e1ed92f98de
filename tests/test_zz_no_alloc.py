"""The relative-L1 entry point that allocates nothing, called through the C ABI.

Who needs it: code that is not allowed to call cudaMalloc where the cache check runs - a plug-in
that lives inside another framework's memory pool, a process whose device memory was handed out
up front, a serving loop that forbids allocation after warm-up.  Such callers cannot provide the
scratch buffer `cdb_rel_l1` asks for, so `cdb_rel_l1_static` keeps its scratch in a fixed array
inside the library.  This file checks that it returns what the ordinary entry point returns, twice
in a row (the array is shared between calls and keeps the previous call's contents), and that it
refuses sizes beyond its stated maximum.  It is collected last on purpose, and passes both alone
in a fresh process and after the rest of the suite.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ELEMS = 1 << 30  # CDB_REL_L1_STATIC_MAX_ELEMS in include/cache_dit_b200.h
DTYPE_ID = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def _p(t):
  return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
  return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _with_caller_scratch(lib, cur, base, prev, res, means):
  scratch = torch.zeros(lib.cdb_rel_l1_scratch_bytes(), dtype=torch.uint8, device="cuda")
  rc = lib.cdb_rel_l1(_p(cur), _p(base), _p(prev), _p(res), cur.numel(), DTYPE_ID[cur.dtype], _p(means),
                      _p(scratch), scratch.numel(), _stream())
  assert rc == 0, lib.cdb_status_string(rc)
  torch.cuda.synchronize()


def _without_allocation(lib, cur, base, prev, res, means):
  rc = lib.cdb_rel_l1_static(_p(cur), _p(base), _p(prev), _p(res), cur.numel(), DTYPE_ID[cur.dtype], _p(means),
                             _stream())
  assert rc == 0, (lib.cdb_status_string(rc), lib.cdb_last_cuda_error())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 37, 72), (1, 4096, 3072)])
@pytest.mark.parametrize("fused_residual", [False, True])
def test_matches_the_ordinary_entry_point_twice_in_a_row(dtype, shape, fused_residual):
  from cache_dit_b200 import _native
  lib = _native.lib()
  g = torch.Generator().manual_seed(7)
  prev = torch.randn(shape, generator=g).to(dtype).cuda()
  base = torch.randn(shape, generator=g).to(dtype).cuda() if fused_residual else None
  want = torch.zeros(2, dtype=torch.float32, device="cuda")
  got = torch.zeros(2, dtype=torch.float32, device="cuda")
  for call in range(2):
    # different data on the second call: stale scratch contents would show up as a wrong mean
    cur = (prev.float() * (1.0 + 0.03 * (call + 1)) + 0.05 * torch.randn(shape, generator=g).cuda()
           + (base.float() if base is not None else 0.0)).to(dtype)
    res_want = torch.empty_like(cur) if fused_residual else None
    res_got = torch.empty_like(cur) if fused_residual else None
    _with_caller_scratch(lib, cur, base, prev, res_want, want)
    if call == 0:
      # warm-up: the first call on a device loads the kernels and looks up the array's address, which is
      # one-time driver work and not what the no-allocation promise is about
      _without_allocation(lib, cur, base, prev, res_got, got)
      torch.cuda.synchronize()
    # free device memory as the DRIVER sees it: a cudaMalloc inside the library would show here, whereas
    # torch's own counters only see torch's caching allocator
    free_before = torch.cuda.mem_get_info()[0]
    _without_allocation(lib, cur, base, prev, res_got, got)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    w, g_ = want.cpu(), got.cpu()
    # same kernel, same launch shape: the tolerance the kernel tests use (one unit in the last
    # place of the storage dtype) is more than enough; in practice the values are identical
    ulp = 2.0**-8 if dtype == torch.bfloat16 else 1e-6
    assert abs(float(g_[0]) - float(w[0])) <= ulp * abs(float(w[0])), (call, g_, w)
    assert abs(float(g_[1]) - float(w[1])) <= ulp * abs(float(w[1])), (call, g_, w)
    if fused_residual:
      assert torch.equal(res_got, res_want)


def test_sizes_beyond_the_maximum_are_refused_with_a_reason():
  from cache_dit_b200 import _native
  lib = _native.lib()
  small = torch.zeros(8, dtype=torch.bfloat16, device="cuda")
  means = torch.zeros(2, dtype=torch.float32, device="cuda")
  # the size is checked before anything is launched, so the (small) buffers are never touched
  rc = lib.cdb_rel_l1_static(_p(small), None, _p(small), None, MAX_ELEMS + 1, 1, _p(means), _stream())
  assert rc == 7
  assert b"limit" in lib.cdb_status_string(rc)
  assert b"CDB_REL_L1_STATIC_MAX_ELEMS" in lib.cdb_last_cuda_error()
  assert lib.cdb_rel_l1_static(None, None, None, None, 8, 1, None, None) == 1
  # host memory (or another device's) is refused before anything is launched
  host = torch.zeros(8, dtype=torch.bfloat16).pin_memory()
  assert lib.cdb_rel_l1_static(_p(host), None, _p(small), None, 8, 1, _p(means), _stream()) == 1
  assert b"current device" in lib.cdb_last_cuda_error()
