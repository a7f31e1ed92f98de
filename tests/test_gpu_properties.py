"""Size-independent properties of the kernels at the full sizes of the benchmark configurations, where
the numpy oracle would take minutes: identities that must hold bit for bit whatever the data."""
import pytest
import torch

pytestmark = pytest.mark.gpu
bf = torch.bfloat16


@pytest.fixture(scope="module")
def nat():
  from cache_dit_b200 import _native
  _native.lib()
  return _native


def _rand(shape, seed, scale=1.0, dtype=bf):
  g = torch.Generator(device="cuda").manual_seed(seed)
  return (torch.randn(shape, device="cuda", generator=g) * scale).to(dtype)


@pytest.mark.parametrize("shape", [(1, 4608, 3072), (1, 9450, 5120), (2, 6889, 3072)])
def test_rel_l1_identities(nat, shape):
  prev = _rand(shape, 1)
  means = torch.zeros(2, dtype=torch.float32, device="cuda")
  # identical tensors: the difference mean is exactly zero, the norm mean is the mean of |prev|
  nat.rel_l1(prev, None, prev, None, means)
  assert means[0].item() == 0.0
  want = prev.float().abs().double().mean().item()
  assert abs(means[1].item() - want) <= 2.0**-8 * want
  # negating both operands changes nothing; scaling both by 2 (exact in bf16) doubles both means
  cur = (prev.float() + 0.05 * _rand(shape, 2).float()).to(bf)
  nat.rel_l1(cur, None, prev, None, means)
  base = means.clone()
  nat.rel_l1(-cur, None, -prev, None, means)
  assert torch.equal(means, base)
  nat.rel_l1(cur * 2, None, prev * 2, None, means)
  assert torch.equal(means, base * 2)
  # the fused form (cur = h - h0 formed inside) equals the two-step form on the materialised residual
  h0 = _rand(shape, 3)
  h = (cur.float() + h0.float()).to(bf)
  res = torch.empty_like(h)
  nat.rel_l1(h, h0, prev, res, means)
  fused = means.clone()
  assert torch.equal(res, h - h0)
  nat.rel_l1(res, None, prev, None, means)
  assert torch.equal(means, fused)


@pytest.mark.parametrize("shape", [(1, 4608, 3072), (1, 9450, 5120)])
def test_taylor_update_then_apply_reproduces_linear_sequences(nat, shape):
  """A residual that grows by a constant tensor every step is extrapolated exactly by order 1 when all
  values are small integers (every bf16 operation involved is then exact)."""
  g = torch.Generator(device="cuda").manual_seed(4)
  a = torch.randint(-8, 9, shape, device="cuda", generator=g).to(bf)
  d = torch.randint(-2, 3, shape, device="cuda", generator=g).to(bf)
  zero = torch.zeros(shape, device="cuda", dtype=bf)
  y0, y1 = a, a + d
  cur = [torch.empty_like(a), torch.empty_like(a)]
  nat.taylor_update(y1, None, [y0], cur, 1, 1.0)  # dY0 = y1, dY1 = (y1 - y0) / 1
  assert torch.equal(cur[0], y1) and torch.equal(cur[1], d)
  out = torch.empty_like(a)
  for elapsed in (1.0, 2.0, 3.0):
    nat.taylor_apply(zero, cur, [1.0, 1.0], [1.0, elapsed], True, out)
    assert torch.equal(out, y1 + d * elapsed)
  # and the add-to-hidden form is the extrapolation plus the hidden states
  hidden = torch.randint(-8, 9, shape, device="cuda", generator=g).to(bf)
  nat.taylor_apply(hidden, cur, [1.0, 1.0], [1.0, 2.0], True, out)
  assert torch.equal(out, hidden + y1 + d * 2)


@pytest.mark.parametrize("rows,cols", [(16384, 5120), (4608, 12288)])
def test_fp8_quant_properties(nat, rows, cols):
  x = _rand((rows, cols), 5)
  q = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device="cuda")
  s = torch.empty(rows, dtype=torch.float32, device="cuda")
  nat.fp8_quant_rows(x, q, s)
  # the row maximum lands on +-448, nothing exceeds it, dequantization is within half an e4m3 step
  codes = q.float()
  assert (codes.abs().amax(dim=1) == 448.0).all().item()
  err = (codes * s[:, None] - x.float()).abs()
  assert (err <= 2.0**-4 * x.float().abs() + s[:, None] * 2.0**-10 + 1e-30).all().item()
  # scaling a row by a power of two scales its scale and leaves the codes unchanged
  q2 = torch.empty_like(q)
  s2 = torch.empty_like(s)
  nat.fp8_quant_rows(x * 4, q2, s2)
  assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and torch.equal(s2, s * 4)


@pytest.mark.parametrize("M,N,K", [(16384, 13824, 5120), (4608, 3072, 12288), (16384, 3072, 3072)])
def test_fp8_gemm_properties(nat, M, N, K):
  g = torch.Generator(device="cuda").manual_seed(6)
  aq = torch.randn(M, K, device="cuda", generator=g).to(torch.float8_e4m3fn)
  wq = torch.randn(N, K, device="cuda", generator=g).to(torch.float8_e4m3fn)
  sa = torch.rand(M, device="cuda", generator=g) + 0.5
  sw = torch.rand(N, device="cuda", generator=g) + 0.5
  out = torch.empty(M, N, dtype=bf, device="cuda")
  nat.fp8_gemm_rowscaled(aq, sa, wq, sw, None, out)
  base = out.clone()
  assert torch.isfinite(base).all().item()
  # run-to-run determinism
  nat.fp8_gemm_rowscaled(aq, sa, wq, sw, None, out)
  assert torch.equal(out, base)
  # scaling the row scales by 2 doubles the output exactly; permuting rows permutes the output
  nat.fp8_gemm_rowscaled(aq, sa * 2, wq, sw, None, out)
  assert torch.equal(out, base * 2)
  perm = torch.randperm(M, device="cuda", generator=g)
  nat.fp8_gemm_rowscaled(aq[perm].contiguous(), sa[perm].contiguous(), wq, sw, None, out)
  assert torch.equal(out, base[perm])
  # a sample of entries against an fp64 dot product of the decoded operands
  rows = torch.randint(0, M, (64, ), device="cuda", generator=g)
  cols = torch.randint(0, N, (64, ), device="cuda", generator=g)
  ref = (aq[rows].double() * wq[cols].double()).sum(dim=1) * sa[rows].double() * sw[cols].double()
  got = base[rows, cols].double()
  assert ((got - ref).abs() <= 2.0**-7 * ref.abs() + 1e-2).all().item()
  assert nat.gemm_device_status(torch.device("cuda:0")) == 0
