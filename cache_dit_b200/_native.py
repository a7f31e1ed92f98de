"""ctypes binding of the C ABI declared in include/cache_dit_b200.h.

The shared library is the product: there is no eager or CPU fallback.  `lib()` raises if the
library is missing; every wrapper raises if it is handed a non-CUDA tensor.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int64, c_size_t, c_uint64, c_void_p

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libcache_dit_b200.so")

DTYPE_ID = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
MAX_TAYLOR_TERMS = 5
PRE_NONE, PRE_LAYERNORM_MOD, PRE_GELU_TANH = 0, 1, 2

# name -> (restype, argtypes); mirrors include/cache_dit_b200.h one to one
SIGNATURES = {
  "cdb_abi_version": (c_int, []),
  "cdb_status_string": (c_char_p, [c_int]),
  "cdb_last_cuda_error": (c_char_p, []),
  "cdb_rel_l1_scratch_bytes": (c_size_t, []),
  "cdb_rel_l1": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p,
                         c_size_t, c_void_p]),
  "cdb_rel_l1_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p]),
  "cdb_taylor_apply": (c_int, [c_void_p, POINTER(c_void_p), POINTER(c_float), POINTER(c_float), c_int,
                               c_int, c_void_p, c_int64, c_int, c_void_p]),
  "cdb_taylor_update": (c_int, [c_void_p, c_void_p, POINTER(c_void_p), POINTER(c_void_p), c_int, c_float,
                                c_int64, c_int, c_void_p]),
  "cdb_fp8_quant_rows": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
  "cdb_fp8_quant_rows_fused": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p,
                                       c_int64, c_int64, c_float, c_void_p, c_void_p, c_void_p]),
  "cdb_fp8_quant_rows_fused_pair": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p,
                                            c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64,
                                            c_void_p, c_void_p, c_int64, c_int, c_float, c_void_p]),
  "cdb_fp8_quant_rows_concat_gelu": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
                                             c_void_p, c_void_p, c_void_p]),
  "cdb_fp8_quant_rows_concat": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
                                             c_void_p, c_void_p, c_void_p]),
  "cdb_fp8_gemm_rowscaled": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                     c_int64, c_int64, c_int64, c_void_p, c_void_p]),
  "cdb_fp8_gemm_rowscaled_grouped": (c_int, [c_void_p, c_int, c_void_p, c_void_p]),
  "cdb_fp8_gemm_rowscaled_grouped_act": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
  "cdb_fp8_gemm_plan": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
  "cdb_tuning_set_gemm_tile_cols": (c_int, [c_int]),
  "cdb_tuning_set_gemm_kernel": (c_int, [c_int]),
  "cdb_qk_norm_rope": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                               c_int64, c_int64, c_int, c_int, c_int, c_float, c_void_p]),
  "cdb_gated_residual_pair": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                      c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                      c_int64, c_void_p]),
  "cdb_bf16_gemv": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p]),
  "cdb_peer_enable_access": (c_int, [c_int]),
  "cdb_peer_alloc": (c_int, [c_size_t, POINTER(c_void_p)]),
  "cdb_peer_free": (c_int, [c_void_p]),
  "cdb_peer_export": (c_int, [c_void_p, c_char_p]),
  "cdb_peer_import": (c_int, [c_char_p, POINTER(c_void_p)]),
  "cdb_peer_release": (c_int, [c_void_p]),
  "cdb_scatter_heads": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64,
                                c_int64, c_int64, c_int64, c_int, c_int, c_float, c_void_p]),
  "cdb_scatter_heads_multi": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
  "cdb_peer_barrier": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_uint64, c_void_p]),
  "cdb_gather_tokens": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_void_p, c_int64, c_int, c_int,
                                c_void_p]),
  "cdb_gather_tokens_fp8": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_void_p, c_int64,
                                    c_int, c_int, c_void_p]),
  "cdb_fp8_dequant_heads": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
  "cdb_peer_sync_bytes": (c_size_t, []),
  "cdb_peer_signal": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
  "cdb_peer_wait": (c_int, [c_void_p, c_int, c_void_p, c_uint64, c_void_p]),
  "cdb_gated_residual": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                 c_int64, c_void_p]),
}

_lib = None

# Kernel launches issued through this binding since import (read by the benchmark), and an
# optional per-launch timing hook: when `gemm_timer` is a list, every GEMM launch appends
# (start_event, end_event, flops) recorded on the launching stream.
launch_count = 0
gemm_timer = None


class NativeLibraryError(RuntimeError):
  pass


def lib() -> ctypes.CDLL:
  """Load libcache_dit_b200.so (once). Raises NativeLibraryError when it has not been built."""
  global _lib
  if _lib is None:
    if not os.path.exists(LIB_PATH):
      raise NativeLibraryError(
        f"{LIB_PATH} is missing. Build it with `python -m cache_dit_b200.csrc.build` "
        "(needs nvcc); cache_dit_b200 has no fallback path.")
    handle = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
      fn = getattr(handle, name)
      fn.restype = res
      fn.argtypes = args
    _lib = handle
  return _lib


def check(status: int, what: str, launch: bool = True):
  global launch_count
  if launch:
    launch_count += 1
  if status != 0:
    L = lib()
    msg = L.cdb_status_string(status).decode()
    detail = L.cdb_last_cuda_error().decode() if status == 4 else ""
    raise RuntimeError(f"{what} failed: {msg}" + (f" [{detail}]" if detail else ""))


def _ptr(t):
  return None if t is None else c_void_p(t.data_ptr())


def _stream(t: torch.Tensor):
  return c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _need_cuda(*tensors):
  for t in tensors:
    if t is not None and not t.is_cuda:
      raise RuntimeError("cache_dit_b200 kernels take CUDA tensors only (no CPU fallback)")


def _need_contig(*tensors):
  for t in tensors:
    if t is not None and not t.is_contiguous():
      raise RuntimeError("cache_dit_b200 kernels need contiguous tensors")


# scratch for the relative-L1 reduction: one zero-initialised buffer per (device, stream)
_scratch = {}


def rel_l1_scratch(device, stream_id: int) -> torch.Tensor:
  key = (device.index if device.index is not None else torch.cuda.current_device(), stream_id)
  buf = _scratch.get(key)
  if buf is None:
    buf = torch.zeros(lib().cdb_rel_l1_scratch_bytes(), dtype=torch.uint8, device=device)
    _scratch[key] = buf
  return buf


def rel_l1(cur, base, prev, residual_out, means):
  """See cdb_rel_l1. `means` is a float32[2] CUDA tensor that receives the two local means."""
  _need_cuda(cur, base, prev, residual_out, means)
  _need_contig(cur, base, prev, residual_out)
  n = cur.numel()
  for t in (base, prev, residual_out):
    if t is not None and (t.numel() != n or t.dtype != cur.dtype):
      raise RuntimeError("rel_l1: tensors must share shape and dtype")
  scratch = None
  if prev is not None:
    scratch = rel_l1_scratch(cur.device, torch.cuda.current_stream(cur.device).cuda_stream)
  st = lib().cdb_rel_l1(_ptr(cur), _ptr(base), _ptr(prev), _ptr(residual_out), n, DTYPE_ID[cur.dtype],
                        _ptr(means), _ptr(scratch), 0 if scratch is None else scratch.numel(), _stream(cur))
  check(st, "cdb_rel_l1")


def taylor_apply(hidden, derivs, coef, power, add_hidden: bool, out):
  _need_cuda(hidden, out, *derivs)
  _need_contig(hidden, out, *derivs)
  k = len(derivs)
  n = out.numel()
  for t in list(derivs) + ([hidden] if add_hidden else []):
    if t.numel() != n or t.dtype != out.dtype:
      raise RuntimeError("taylor_apply: tensors must share shape and dtype")
  d = (c_void_p * k)(*[t.data_ptr() for t in derivs])
  c = (c_float * k)(*coef)
  p = (c_float * k)(*power)
  st = lib().cdb_taylor_apply(_ptr(hidden) if add_hidden else None, d, c, p, k, int(add_hidden), _ptr(out),
                              n, DTYPE_ID[out.dtype], _stream(out))
  check(st, "cdb_taylor_apply")


def taylor_update(after, before, prev, cur, n_new: int, window: float):
  _need_cuda(after, before, *prev[:n_new], *cur[:n_new + 1])
  _need_contig(after, before, *prev[:n_new], *cur[:n_new + 1])
  n = after.numel()
  for t in list(prev[:n_new]) + list(cur[:n_new + 1]) + ([before] if before is not None else []):
    if t.numel() != n or t.dtype != after.dtype:
      raise RuntimeError("taylor_update: tensors must share shape and dtype")
  pp = (c_void_p * MAX_TAYLOR_TERMS)(*[t.data_ptr() for t in prev[:n_new]])
  cc = (c_void_p * MAX_TAYLOR_TERMS)(*[t.data_ptr() for t in cur[:n_new + 1]])
  st = lib().cdb_taylor_update(_ptr(after), _ptr(before), pp, cc, n_new, float(window), n,
                               DTYPE_ID[after.dtype], _stream(after))
  check(st, "cdb_taylor_update")


def fp8_quant_rows(x2d, q, scale, preop=PRE_NONE, mod_shift=None, mod_scale=None, rows_per_batch=0,
                   eps=0.0):
  """x2d [rows, cols] bf16 (row stride may exceed cols); q [rows, cols] float8_e4m3fn; scale [rows] f32."""
  _need_cuda(x2d, q, scale, mod_shift, mod_scale)
  if x2d.dtype != torch.bfloat16 or x2d.dim() != 2 or x2d.stride(1) != 1:
    raise RuntimeError("fp8_quant_rows: x must be a bf16 matrix with unit column stride")
  rows, cols = x2d.shape
  _need_contig(q, scale)
  ld_mod = 0
  if preop == PRE_LAYERNORM_MOD:
    if mod_shift.dim() != 2 or mod_scale.dim() != 2 or mod_shift.stride(1) != 1 or mod_scale.stride(1) != 1 \
        or mod_shift.stride(0) != mod_scale.stride(0) or mod_shift.dtype != torch.bfloat16 \
        or mod_scale.dtype != torch.bfloat16:
      raise RuntimeError("fp8_quant_rows: modulation must be two bf16 [batch, cols] matrices")
    ld_mod = mod_shift.stride(0)
  st = lib().cdb_fp8_quant_rows_fused(_ptr(x2d), rows, cols, x2d.stride(0) if rows > 1 else max(cols, x2d.stride(0)),
                                      preop, _ptr(mod_shift), _ptr(mod_scale), rows_per_batch, ld_mod,
                                      float(eps), _ptr(q), _ptr(scale), _stream(x2d))
  check(st, "cdb_fp8_quant_rows")


# One 32-byte "mailbox" per device holds everything the host reads back once per step, so that a single
# small device-to-host copy carries the two means of the relative-L1 check AND the latched status of
# every bounded device-side wait:
#   int32 words  [0:2] the two float32 means   [2] GEMM status word   [4:6] PeerSync {epoch, status}
_mailboxes = {}
MAILBOX_WORDS = 8
MAILBOX_GEMM_STATUS = 2
MAILBOX_PEER_STATUS = 5
_peer_sync_claimed = set()


class DeviceTimeoutError(RuntimeError):
  """A bounded wait inside a kernel ran out (CDB_ERR_DEVICE_TIMEOUT): results after it are not valid."""


def _device_index(device) -> int:
  return device.index if device.index is not None else torch.cuda.current_device()


def device_mailbox(device) -> torch.Tensor:
  idx = _device_index(device)
  box = _mailboxes.get(idx)
  if box is None:
    box = torch.zeros(MAILBOX_WORDS, dtype=torch.int32, device=device)
    _mailboxes[idx] = box
  return box


def mailbox_means(device) -> torch.Tensor:
  """float32[2] view of the mailbox: where `rel_l1` leaves the two local means."""
  return device_mailbox(device)[0:2].view(torch.float32)


def gemm_status_word(device) -> torch.Tensor:
  return device_mailbox(device)[MAILBOX_GEMM_STATUS:MAILBOX_GEMM_STATUS + 1]


def claim_peer_sync(device):
  """The mailbox's PeerSync words for the first exchange object of a device (its latched status then
  travels with the per-step copy); None when they are taken (further exchanges keep their own)."""
  idx = _device_index(device)
  if idx in _peer_sync_claimed:
    return None
  _peer_sync_claimed.add(idx)
  sync = device_mailbox(device)[4:6]
  sync.zero_()
  return sync


def release_peer_sync(device):
  _peer_sync_claimed.discard(_device_index(device))


def raise_on_device_status(gemm_status: int, peer_status: int):
  """Turn the latched status words (host copies) into the C ABI's CDB_ERR_DEVICE_TIMEOUT as an exception."""
  if gemm_status != 0:
    raise DeviceTimeoutError(f"CDB_ERR_DEVICE_TIMEOUT: a bounded wait inside the FP8 GEMM ran out (code {gemm_status}); "
                             "the products launched since are incomplete")
  if peer_status != 0:
    raise DeviceTimeoutError(f"CDB_ERR_DEVICE_TIMEOUT: the signal of peer {peer_status - 1} did not arrive within the "
                             "timeout of the head/token exchange; later blocks ran unsynchronised")


def fp8_gemm_rowscaled(a_q, a_scale, w_q, w_scale, bias, out):
  """out[M,N] bf16 = (a_q[M,K] @ w_q[N,K]^T) * a_scale[M] * w_scale[N] (+ bias[N])."""
  _need_cuda(a_q, a_scale, w_q, w_scale, bias, out)
  _need_contig(a_q, a_scale, w_q, w_scale, bias)
  M, K = a_q.shape
  N = w_q.shape[0]
  if w_q.shape[1] != K or out.shape != (M, N) or out.stride(1) != 1 or out.dtype != torch.bfloat16:
    raise RuntimeError("fp8_gemm_rowscaled: shape mismatch")
  if a_scale.numel() != M or w_scale.numel() != N or a_scale.dtype != torch.float32 \
      or w_scale.dtype != torch.float32:
    raise RuntimeError("fp8_gemm_rowscaled: scales must be float32 [M] and [N]")
  if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != N):
    raise RuntimeError("fp8_gemm_rowscaled: bias must be bf16 [N]")
  timer = gemm_timer
  if timer is not None:
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record()
  st = lib().cdb_fp8_gemm_rowscaled(_ptr(a_q), _ptr(a_scale), _ptr(w_q), _ptr(w_scale), _ptr(bias), _ptr(out),
                                    M, N, K, out.stride(0) if M > 1 else max(N, out.stride(0)),
                                    _ptr(gemm_status_word(out.device)), _stream(out))
  if timer is not None:
    end.record()
    timer.append((start, end, 2.0 * M * N * K, False))
  check(st, "cdb_fp8_gemm_rowscaled")


def gemm_device_status(device) -> int:
  """Non-zero if a bounded wait inside the GEMM kernel expired since the last reset (syncs)."""
  return int(gemm_status_word(device).item())


def check_device_status(device):
  """Read the device's latched status words now (synchronises) and raise DeviceTimeoutError if one is set."""
  host = device_mailbox(device).cpu()
  raise_on_device_status(int(host[MAILBOX_GEMM_STATUS]), int(host[MAILBOX_PEER_STATUS]))


def qk_norm_rope(x, norm_weight, cos, sin, out, pos_offset: int, heads: int, eps: float):
  """Per-head RMSNorm + rotary embedding of x [batch, tokens, heads*head_dim] (rows may be a column
  slice of a wider matrix), written into out[:, pos_offset:pos_offset+tokens] of the joint buffer
  out [batch, total_tokens, heads, head_dim].  cos/sin are bf16 [total_tokens, head_dim]."""
  _need_cuda(x, norm_weight, cos, sin, out)
  _need_contig(norm_weight, cos, sin, out)
  b, t, c = x.shape
  d = c // heads
  if x.dtype != torch.bfloat16 or x.stride(2) != 1 or (b > 1 and x.stride(0) != t * x.stride(1)):
    raise RuntimeError("qk_norm_rope: x must be bf16 with unit column stride and uniformly strided rows")
  if out.shape[0] != b or out.shape[2] != heads or out.shape[3] != d or cos.shape != (out.shape[1], d) \
      or cos.dtype != torch.bfloat16 or sin.dtype != torch.bfloat16 or norm_weight.dtype != torch.bfloat16:
    raise RuntimeError("qk_norm_rope: joint buffer / rotary table shapes do not match the projection")
  st = lib().cdb_qk_norm_rope(_ptr(x), x.stride(1), _ptr(norm_weight), _ptr(cos), _ptr(sin), _ptr(out),
                              heads * d, out.stride(0), b * t, t, int(pos_offset), heads, d, float(eps),
                              _stream(x))
  check(st, "cdb_qk_norm_rope")


def gated_residual(x, gate, y):
  """x + gate[:, None, :] * y for x [batch, tokens, cols] contiguous, gate [batch, cols] (rows may be a
  column slice), y [batch, tokens, cols] (rows may be a column slice).  Returns a new tensor."""
  _need_cuda(x, gate, y)
  _need_contig(x)
  b, t, c = x.shape
  if x.dtype != torch.bfloat16 or y.dtype != x.dtype or gate.dtype != x.dtype or y.stride(2) != 1 \
      or gate.stride(1) != 1 or (b > 1 and y.stride(0) != t * y.stride(1)) or y.shape != x.shape:
    raise RuntimeError("gated_residual: bf16 operands with unit column stride and uniform row strides")
  out = torch.empty_like(x)
  st = lib().cdb_gated_residual(_ptr(x), _ptr(y), y.stride(1), _ptr(gate), gate.stride(0) if b > 1 else c,
                                _ptr(out), b * t, t, c, _stream(x))
  check(st, "cdb_gated_residual")
  return out


def bf16_gemv(x2d, w, bias, out):
  """out[M, N] = bf16(x2d[M, K] @ w[N, K]^T + bias[N]) for M <= 4 (see cdb_bf16_gemv); rows of x2d / out may be strided."""
  _need_cuda(x2d, w, bias, out)
  _need_contig(w, bias)
  m, k = x2d.shape
  n = w.shape[0]
  if x2d.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or w.shape[1] != k \
      or tuple(out.shape) != (m, n) or x2d.stride(1) != 1 or out.stride(1) != 1 \
      or (bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != n)):
    raise RuntimeError("bf16_gemv: bf16 x [M, K], w [N, K], bias [N], out [M, N] with unit column strides")
  st = lib().cdb_bf16_gemv(_ptr(x2d), x2d.stride(0) if m > 1 else max(k, x2d.stride(0)), _ptr(w), _ptr(bias), _ptr(out),
                           out.stride(0) if m > 1 else max(n, out.stride(0)), m, n, k, _stream(x2d))
  check(st, "cdb_bf16_gemv")


def fp8_quant_rows_concat_gelu(head2d, tail2d, q, scale, tail_activated=False):
  """Quantize rows of [head | gelu_tanh(tail)] (bf16 matrices, rows may be strided) into q / scale.  With
  `tail_activated` the tail already holds gelu_tanh(...) (written by a product with an activation in its
  epilogue) and is only concatenated."""
  _need_cuda(head2d, tail2d, q, scale)
  _need_contig(q, scale)
  for t in (head2d, tail2d):
    if t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
      raise RuntimeError("fp8_quant_rows_concat_gelu: bf16 matrices with unit column stride")
  rows, c1 = head2d.shape
  c2 = tail2d.shape[1]
  if tail2d.shape[0] != rows or q.shape != (rows, c1 + c2):
    raise RuntimeError("fp8_quant_rows_concat_gelu: row counts / output width do not match")
  fn = lib().cdb_fp8_quant_rows_concat if tail_activated else lib().cdb_fp8_quant_rows_concat_gelu
  st = fn(_ptr(head2d), c1, head2d.stride(0) if rows > 1 else max(c1, head2d.stride(0)),
          _ptr(tail2d), c2, tail2d.stride(0) if rows > 1 else max(c2, tail2d.stride(0)),
          rows, _ptr(q), _ptr(scale), _stream(head2d))
  check(st, "cdb_fp8_quant_rows_concat" if tail_activated else "cdb_fp8_quant_rows_concat_gelu")


# ---- Ulysses exchange over peer memory ---------------------------------------------------------
def _ptr_array(ptrs):
  return (c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def peer_enable_access(peer_device: int):
  check(lib().cdb_peer_enable_access(int(peer_device)), "cdb_peer_enable_access", launch=False)


def scatter_heads(x, norm_weight, cos, sin, table_row_offset: int, dst_ptrs, dst_batch_stride: int,
                  dst_row_offset: int, heads: int, eps: float = 0.0, across_heads: bool = False):
  """x [batch, tokens, heads*head_dim] bf16 -> head h into rank h // (heads/world)'s joint buffer
  (see cdb_scatter_heads).  norm_weight None copies, else per-head RMSNorm + rotary embedding first."""
  _need_cuda(x, norm_weight, cos, sin)
  b, t, c = x.shape
  d = c // heads
  if x.dtype != torch.bfloat16 or x.stride(2) != 1 or (b > 1 and x.stride(0) != t * x.stride(1)):
    raise RuntimeError("scatter_heads: x must be bf16 with unit column stride and uniformly strided rows")
  if norm_weight is not None:
    _need_contig(norm_weight, cos, sin)
  if norm_weight is not None and norm_weight.numel() != (c if across_heads else d):
    raise RuntimeError("scatter_heads: norm weight is [head_dim] per head or [heads*head_dim] across heads")
  st = lib().cdb_scatter_heads(_ptr(x), x.stride(1), _ptr(norm_weight), int(bool(across_heads)), _ptr(cos), _ptr(sin),
                               int(table_row_offset),
                               _ptr_array(dst_ptrs), len(dst_ptrs), int(dst_batch_stride), b * t, t,
                               int(dst_row_offset), heads, d, float(eps), _stream(x))
  check(st, "cdb_scatter_heads")


def gather_tokens(o, dst_ptrs, my_rank: int, row_starts=None, dst_token_capacity=None):
  """o [batch, tokens_all, heads_per_rank, head_dim] contiguous -> token rows into their owners' buffers
  ([batch, dst_token_capacity, heads, head_dim]); `row_starts` (world + 1 ints) for unequal token ranges."""
  _need_cuda(o)
  _need_contig(o)
  b, s, h, d = o.shape
  world = len(dst_ptrs)
  starts = None if row_starts is None else (c_int64 * (world + 1))(*[int(v) for v in row_starts])
  if dst_token_capacity is None:
    dst_token_capacity = s // world if row_starts is None else max(row_starts[r + 1] - row_starts[r] for r in range(world))
  st = lib().cdb_gather_tokens(_ptr(o), _ptr_array(dst_ptrs), world, int(my_rank), b, s, starts,
                               int(dst_token_capacity), h, d, _stream(o))
  check(st, "cdb_gather_tokens")


def peer_signal(flag_ptrs, my_rank: int, sync, stream_of):
  check(lib().cdb_peer_signal(_ptr_array(flag_ptrs), len(flag_ptrs), int(my_rank), _ptr(sync), _stream(stream_of)),
        "cdb_peer_signal")


def peer_wait(my_flags, world: int, sync, timeout_ns: int):
  check(lib().cdb_peer_wait(_ptr(my_flags), int(world), _ptr(sync), int(timeout_ns), _stream(my_flags)),
        "cdb_peer_wait")


def peer_alloc(nbytes: int) -> int:
  out = c_void_p()
  check(lib().cdb_peer_alloc(int(nbytes), ctypes.byref(out)), "cdb_peer_alloc", launch=False)
  return int(out.value)


def peer_free(ptr: int):
  check(lib().cdb_peer_free(c_void_p(ptr)), "cdb_peer_free", launch=False)


def peer_export(ptr: int) -> bytes:
  buf = ctypes.create_string_buffer(64)
  check(lib().cdb_peer_export(c_void_p(ptr), buf), "cdb_peer_export", launch=False)
  return buf.raw


def peer_import(handle: bytes) -> int:
  out = c_void_p()
  check(lib().cdb_peer_import(ctypes.create_string_buffer(handle, 64), ctypes.byref(out)), "cdb_peer_import", launch=False)
  return int(out.value)


def peer_release(ptr: int):
  check(lib().cdb_peer_release(c_void_p(ptr)), "cdb_peer_release", launch=False)


class ScatterJob(ctypes.Structure):
  """ctypes image of `cdb_scatter_job`."""
  _fields_ = [("x", c_void_p), ("ld_x", c_int64), ("tokens", c_int64), ("tokens_per_batch", c_int64),
              ("norm_weight", c_void_p), ("norm_across_heads", c_int), ("eps", c_float), ("cos_table", c_void_p),
              ("sin_table", c_void_p), ("table_row_offset", c_int), ("dst_ptrs", c_void_p),
              ("dst_batch_stride", c_int64), ("dst_row_offset", c_int64), ("dst_scale_ptrs", c_void_p)]


def scatter_heads_multi(jobs, heads: int):
  """Several `scatter_heads` calls as one launch.  jobs: dicts with x [batch, tokens, heads*head_dim],
  norm_weight / cos / sin (None: copy), table_row_offset, dst_ptrs, dst_batch_stride, dst_row_offset,
  eps, across_heads.  All jobs share heads, head_dim and the number of destinations."""
  if not 1 <= len(jobs) <= 6:
    raise RuntimeError("scatter_heads_multi: 1 to 6 jobs per launch")
  arr = (ScatterJob * len(jobs))()
  keep = []
  world = len(jobs[0]["dst_ptrs"])
  x0 = jobs[0]["x"]
  d = x0.shape[-1] // heads
  for slot, j in zip(arr, jobs):
    x, w = j["x"], j.get("norm_weight")
    _need_cuda(x, w, j.get("cos"), j.get("sin"))
    b, t, c = x.shape
    if x.dtype != torch.bfloat16 or x.stride(2) != 1 or (b > 1 and x.stride(0) != t * x.stride(1)) or c != heads * d \
        or len(j["dst_ptrs"]) != world:
      raise RuntimeError("scatter_heads_multi: bf16 projections of one head layout, uniformly strided rows")
    across = bool(j.get("across_heads", False))
    if w is not None and w.numel() != (c if across else d):
      raise RuntimeError("scatter_heads_multi: norm weight is [head_dim] per head or [heads*head_dim] across heads")
    ptrs = _ptr_array(j["dst_ptrs"])
    keep.append(ptrs)
    slot.x, slot.ld_x, slot.tokens, slot.tokens_per_batch = x.data_ptr(), x.stride(1), b * t, t
    slot.norm_weight = None if w is None else w.data_ptr()
    slot.norm_across_heads, slot.eps = int(across), float(j.get("eps", 0.0))
    slot.cos_table = None if w is None else j["cos"].data_ptr()
    slot.sin_table = None if w is None else j["sin"].data_ptr()
    slot.table_row_offset = int(j.get("table_row_offset", 0))
    slot.dst_ptrs = ctypes.cast(ptrs, c_void_p)
    slot.dst_batch_stride, slot.dst_row_offset = int(j["dst_batch_stride"]), int(j["dst_row_offset"])
    if j.get("dst_scale_ptrs") is not None:  # FP8 on the wire
      sptrs = _ptr_array(j["dst_scale_ptrs"])
      keep.append(sptrs)
      slot.dst_scale_ptrs = ctypes.cast(sptrs, c_void_p)
  st = lib().cdb_scatter_heads_multi(ctypes.cast(arr, c_void_p), len(jobs), world, heads, d, _stream(x0))
  check(st, "cdb_scatter_heads_multi")


def peer_barrier(flag_ptrs, my_flags, my_rank: int, sync, timeout_ns: int):
  check(lib().cdb_peer_barrier(_ptr_array(flag_ptrs), _ptr(my_flags), len(flag_ptrs), int(my_rank), _ptr(sync),
                               int(timeout_ns), _stream(my_flags)), "cdb_peer_barrier")


def gather_tokens_fp8(o, dst_ptrs, dst_scale_ptrs, my_rank: int, row_starts=None, dst_token_capacity=None):
  """`gather_tokens` with e4m3 bytes + one bf16 scale per (token, head) on the wire."""
  _need_cuda(o)
  _need_contig(o)
  b, s, h, d = o.shape
  world = len(dst_ptrs)
  starts = None if row_starts is None else (c_int64 * (world + 1))(*[int(v) for v in row_starts])
  if dst_token_capacity is None:
    dst_token_capacity = s // world if row_starts is None else max(row_starts[r + 1] - row_starts[r] for r in range(world))
  st = lib().cdb_gather_tokens_fp8(_ptr(o), _ptr_array(dst_ptrs), _ptr_array(dst_scale_ptrs), world, int(my_rank), b, s,
                                   starts, int(dst_token_capacity), h, d, _stream(o))
  check(st, "cdb_gather_tokens_fp8")


def fp8_dequant_heads(q_list, scale_list, out_list, head_dim: int):
  """out = bf16(float(q) * scale) per row of head_dim e4m3 bytes; scales float32 or bf16; up to 3 tensors."""
  _need_cuda(*q_list, *scale_list, *out_list)
  _need_contig(*q_list, *scale_list, *out_list)
  n = len(q_list)
  rows = (c_int64 * n)(*[q.numel() * q.element_size() // head_dim for q in q_list])
  bf16_scales = scale_list[0].dtype == torch.bfloat16
  st = lib().cdb_fp8_dequant_heads(_ptr_array([q.data_ptr() for q in q_list]),
                                   _ptr_array([s.data_ptr() for s in scale_list]),
                                   _ptr_array([o.data_ptr() for o in out_list]), rows, n, int(head_dim),
                                   int(bf16_scales), _stream(out_list[0]))
  check(st, "cdb_fp8_dequant_heads")


class GemmProblem(ctypes.Structure):
  """ctypes image of `cdb_gemm_problem`."""
  _fields_ = [("a_q", c_void_p), ("a_scale", c_void_p), ("w_q", c_void_p), ("w_scale", c_void_p), ("bias", c_void_p),
              ("out", c_void_p), ("M", c_int64), ("N", c_int64), ("K", c_int64), ("ld_out", c_int64)]


def fp8_gemm_plan(shapes, sm_count=148):
  """(kind, tile_cols) a launch of these one or two (M, N, K) problems would take on a GPU with `sm_count` SMs:
  kind 1 = single-CTA tile kernel, 2 = CTA-pair kernel, 3 = few-row kernel.  Host arithmetic only (no GPU)."""
  arr = (GemmProblem * len(shapes))()
  for slot, (M, N, K) in zip(arr, shapes):
    slot.M, slot.N, slot.K, slot.ld_out = M, N, K, N
  kind, cols = c_int(0), c_int(0)
  check(lib().cdb_fp8_gemm_plan(ctypes.cast(arr, c_void_p), len(shapes), sm_count, ctypes.byref(kind), ctypes.byref(cols)),
        "cdb_fp8_gemm_plan")
  return kind.value, cols.value


def fp8_gemm_rowscaled_grouped(problems, gelu_from=None):
  """Up to two products (a_q, a_scale, w_q, w_scale, bias, out) in one launch; see fp8_gemm_rowscaled.
  gelu_from: per problem the first output column that passes through tanh-GELU in the epilogue (None: none)."""
  if not 1 <= len(problems) <= 2:
    raise RuntimeError("fp8_gemm_rowscaled_grouped: one or two problems per launch")
  arr = (GemmProblem * len(problems))()
  flops = 0.0
  for slot, (a_q, a_scale, w_q, w_scale, bias, out) in zip(arr, problems):
    _need_cuda(a_q, a_scale, w_q, w_scale, bias, out)
    _need_contig(a_q, a_scale, w_q, w_scale, bias)
    M, K = a_q.shape
    N = w_q.shape[0]
    if w_q.shape[1] != K or tuple(out.shape) != (M, N) or out.stride(1) != 1 or out.dtype != torch.bfloat16:
      raise RuntimeError("fp8_gemm_rowscaled_grouped: shapes do not match / output must be bf16 rows")
    if a_scale.numel() != M or w_scale.numel() != N or a_scale.dtype != torch.float32 or w_scale.dtype != torch.float32 \
        or (bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != N)):
      raise RuntimeError("fp8_gemm_rowscaled_grouped: scales must be float32 [M] / [N], bias bf16 [N]")
    slot.a_q, slot.a_scale, slot.w_q, slot.w_scale = a_q.data_ptr(), a_scale.data_ptr(), w_q.data_ptr(), w_scale.data_ptr()
    slot.bias = None if bias is None else bias.data_ptr()
    slot.out = out.data_ptr()
    slot.M, slot.N, slot.K = M, N, K
    slot.ld_out = out.stride(0) if M > 1 else max(N, out.stride(0))
    flops += 2.0 * M * N * K
  out0 = problems[0][5]
  timer = gemm_timer
  if timer is not None:
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record()
  if gelu_from is not None and any(g is not None for g in gelu_from):
    cols = (c_int64 * len(problems))(*[-1 if g is None else int(g) for g in gelu_from])
    st = lib().cdb_fp8_gemm_rowscaled_grouped_act(ctypes.cast(arr, c_void_p), len(problems), ctypes.cast(cols, c_void_p),
                                                  _ptr(gemm_status_word(out0.device)), _stream(out0))
  else:
    st = lib().cdb_fp8_gemm_rowscaled_grouped(ctypes.cast(arr, c_void_p), len(problems),
                                              _ptr(gemm_status_word(out0.device)), _stream(out0))
  if timer is not None:
    end.record()
    timer.append((start, end, flops, bool(gelu_from is not None and any(g is not None for g in gelu_from))))
  check(st, "cdb_fp8_gemm_rowscaled_grouped")


def fp8_quant_rows_pair(jobs, preop=PRE_NONE, eps=0.0):
  """Two `fp8_quant_rows` jobs of the same width in one launch.  jobs: two dicts with x2d [rows, cols] bf16, q,
  scale and, for the LayerNorm variant, mod_shift / mod_scale [batch, cols] and rows_per_batch."""
  a, b = jobs
  args = []
  cols = a["x2d"].shape[1]
  for j in (a, b):
    x2d, q, scale = j["x2d"], j["q"], j["scale"]
    sh, sc = j.get("mod_shift"), j.get("mod_scale")
    _need_cuda(x2d, q, scale, sh, sc)
    _need_contig(q, scale)
    if x2d.dtype != torch.bfloat16 or x2d.dim() != 2 or x2d.stride(1) != 1 or x2d.shape[1] != cols:
      raise RuntimeError("fp8_quant_rows_pair: bf16 matrices of one width with unit column stride")
    rows = x2d.shape[0]
    ld_mod = 0
    if preop == PRE_LAYERNORM_MOD:
      if sh.dim() != 2 or sc.dim() != 2 or sh.stride(1) != 1 or sc.stride(1) != 1 or sh.stride(0) != sc.stride(0) \
          or sh.dtype != torch.bfloat16 or sc.dtype != torch.bfloat16:
        raise RuntimeError("fp8_quant_rows_pair: modulation must be two bf16 [batch, cols] matrices")
      ld_mod = sh.stride(0)
    args += [_ptr(x2d), rows, x2d.stride(0) if rows > 1 else max(cols, x2d.stride(0)), _ptr(sh), _ptr(sc),
             int(j.get("rows_per_batch", 0)), ld_mod, _ptr(q), _ptr(scale)]
  st = lib().cdb_fp8_quant_rows_fused_pair(*args, cols, int(preop), float(eps), _stream(a["x2d"]))
  check(st, "cdb_fp8_quant_rows_fused_pair")


def gated_residual_pair(xa, gate_a, ya, xb, gate_b, yb):
  """(xa + gate_a * ya, xb + gate_b * yb) with one launch; same rules per set as `gated_residual`."""
  args, outs = [], []
  cols = xa.shape[-1]
  for x, gate, y in ((xa, gate_a, ya), (xb, gate_b, yb)):
    _need_cuda(x, gate, y)
    _need_contig(x)
    b, t, c = x.shape
    if x.dtype != torch.bfloat16 or y.dtype != x.dtype or gate.dtype != x.dtype or y.stride(2) != 1 or c != cols \
        or gate.stride(1) != 1 or (b > 1 and y.stride(0) != t * y.stride(1)) or y.shape != x.shape:
      raise RuntimeError("gated_residual_pair: bf16 operands of one width, unit column stride, uniform row strides")
    out = torch.empty_like(x)
    outs.append(out)
    args += [_ptr(x), _ptr(y), y.stride(1), _ptr(gate), gate.stride(0) if b > 1 else c, _ptr(out), b * t, t]
  st = lib().cdb_gated_residual_pair(*args, cols, _stream(xa))
  check(st, "cdb_gated_residual_pair")
  return outs[0], outs[1]
