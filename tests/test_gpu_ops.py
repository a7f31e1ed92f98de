"""The `torch.library` operators on a B200: same results as the C-ABI calls and as the library product the
reference's operator wraps, leading batch dimensions, and capture in a CUDA graph (the reference's own
tests at this boundary: tests/kernels/test_opaque_scaled_mm.py:46-94 -- finite, bf16, close to eager --
and test_rowwise_cudagraph_partition.py -- graph capture completes)."""
import numpy as np
import pytest
import torch

from oracle import fp8_oracle as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
  import cache_dit_b200  # noqa: F401
  from cache_dit_b200.quantization import ops as module
  return module


def operands(lead, K, N, seed, bias=True):
  g = torch.Generator().manual_seed(seed)
  x = torch.randn(*lead, K, generator=g)
  x = torch.where(torch.rand(*lead, K, generator=g) < 1e-3, x * 20, x).to(torch.bfloat16)
  w = (0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16)
  b = (0.1 * torch.randn(N, generator=g)).to(torch.bfloat16) if bias else None
  return x.cuda(), w.cuda(), None if b is None else b.cuda()


@pytest.mark.parametrize("lead,K,N,bias", [((300, ), 256, 272, False), ((2, 130), 512, 264, True), ((1, 4608), 3072, 3072, True)])
def test_operators_match_abi_calls_and_oracle(ops, lead, K, N, bias):
  from cache_dit_b200 import _native as nat
  x, w, b = operands(lead, K, N, 5 + K + N, bias)
  aq, sa = ops.float8_quantize_rows(x)
  wq, sw = ops.float8_quantize_rows(w)
  assert aq.shape == x.shape and sa.shape == (*lead, 1) and aq.dtype is torch.float8_e4m3fn
  rows = x.reshape(-1, K)
  codes, scale = F.quantize_rows(rows.float().cpu().numpy())
  np.testing.assert_array_equal(aq.reshape(-1, K).view(torch.uint8).cpu().numpy(), codes)
  np.testing.assert_array_equal(sa.reshape(-1).cpu().numpy(), scale)
  y = ops.float8_inference_scaled_mm(aq, sa, wq.t(), sw.t(), b, torch.bfloat16)
  assert y.shape == (*lead, N) and y.dtype is torch.bfloat16 and torch.isfinite(y).all().item()
  direct = torch.empty(rows.shape[0], N, dtype=torch.bfloat16, device="cuda")
  nat.fp8_gemm_rowscaled(aq.reshape(-1, K), sa.reshape(-1), wq, sw.reshape(-1), b, direct)
  assert torch.equal(y.reshape(-1, N), direct)
  take = slice(0, min(rows.shape[0], 512))
  want = F.scaled_mm(codes[take], scale[take], wq.view(torch.uint8).cpu().numpy(), sw.reshape(-1).cpu().numpy(),
                     None if b is None else b.float().cpu().numpy())
  got = y.reshape(-1, N)[take].float().cpu().numpy()
  assert np.linalg.norm(got - want) / np.linalg.norm(want) < 2e-3  # bound of the path: 2e-2


def test_operator_close_to_unquantized_linear(ops):
  """The reference's own criterion at this boundary: finite bf16 output close to the eager linear."""
  x, w, b = operands((64, ), 512, 256, 77)
  aq, sa = ops.float8_quantize_rows(x)
  wq, sw = ops.float8_quantize_rows(w)
  y = ops.float8_inference_scaled_mm(aq, sa, wq.t(), sw.t(), b, torch.bfloat16)
  eager = torch.nn.functional.linear(x, w, b)
  assert (y.float() - eager.float()).abs().max().item() <= 0.5
  assert ((y.float() - eager.float()).norm() / eager.float().norm()).item() < 0.06


def test_only_bf16_output_is_built(ops):
  x, w, _ = operands((16, ), 64, 32, 3, bias=False)
  aq, sa = ops.float8_quantize_rows(x)
  wq, sw = ops.float8_quantize_rows(w)
  with pytest.raises(NotImplementedError):
    ops.float8_inference_scaled_mm(aq, sa, wq.t(), sw.t(), None, torch.float32)


def test_operators_capture_in_a_cuda_graph(ops):
  x, w, b = operands((2, 96), 512, 264, 9)
  wq, sw = ops.float8_quantize_rows(w)

  def linear(inp):
    aq, sa = ops.float8_quantize_rows(inp)
    return ops.float8_inference_scaled_mm(aq, sa, wq.t(), sw.t(), b, torch.bfloat16)

  eager = linear(x)
  static_in = x.clone()
  side = torch.cuda.Stream()
  side.wait_stream(torch.cuda.current_stream())
  with torch.cuda.stream(side):  # warm-up off the capture, as torch's capture rules ask
    linear(static_in)
  torch.cuda.current_stream().wait_stream(side)
  graph = torch.cuda.CUDAGraph()
  with torch.cuda.graph(graph):
    static_out = linear(static_in)
  graph.replay()
  torch.cuda.synchronize()
  assert torch.equal(static_out, eager)
  x2, _, _ = operands((2, 96), 512, 264, 10)
  static_in.copy_(x2)
  graph.replay()
  torch.cuda.synchronize()
  assert torch.equal(static_out, linear(x2))
