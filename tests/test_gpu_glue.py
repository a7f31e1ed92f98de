"""The two block-glue kernels (QK RMSNorm + RoPE into the joint buffer; gated residual add) against
the eager PyTorch ops they replace, and the fused-linear group against its member linears."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nat():
  from cache_dit_b200 import _native
  _native.lib()
  return _native


def _rope_ref(x, cos, sin):
  cos, sin = cos[None, :, None, :], sin[None, :, None, :]
  x1, x2 = x.unflatten(-1, (-1, 2)).unbind(-1)
  rot = torch.stack([-x2, x1], dim=-1).flatten(-2)
  return x * cos + rot * sin


@pytest.mark.parametrize("batch,t_txt,t_img,heads,d", [(1, 7, 33, 4, 64), (2, 16, 48, 3, 128), (1, 512, 4096, 24, 128),
                                                       (1, 5, 9, 2, 256)])
def test_qk_norm_rope_joint_buffer(nat, batch, t_txt, t_img, heads, d):
  g = torch.Generator().manual_seed(batch * 100 + d)
  c = heads * d
  total = t_txt + t_img
  # projections as column slices of a wider matrix, the way a fused q/k/v GEMM produces them
  wide_txt = torch.randn(batch, t_txt, 3 * c, generator=g).to("cuda", torch.bfloat16)
  wide_img = torch.randn(batch, t_img, 3 * c, generator=g).to("cuda", torch.bfloat16)
  x_txt, x_img = wide_txt[..., c:2 * c], wide_img[..., c:2 * c]
  w_txt = (1 + 0.1 * torch.randn(d, generator=g)).to("cuda", torch.bfloat16)
  w_img = (1 + 0.1 * torch.randn(d, generator=g)).to("cuda", torch.bfloat16)
  ang = torch.rand(total, d // 2, generator=g) * 6.28
  cos = torch.cos(ang).repeat_interleave(2, dim=-1).to("cuda", torch.bfloat16).contiguous()
  sin = torch.sin(ang).repeat_interleave(2, dim=-1).to("cuda", torch.bfloat16).contiguous()
  out = torch.full((batch, total, heads, d), float("nan"), device="cuda", dtype=torch.bfloat16)
  nat.qk_norm_rope(x_txt, w_txt, cos, sin, out, 0, heads, 1e-6)
  nat.qk_norm_rope(x_img, w_img, cos, sin, out, t_txt, heads, 1e-6)
  torch.cuda.synchronize()
  # fp32 reference of the same math from the same bf16 inputs
  parts = []
  for x, w in ((x_txt, w_txt), (x_img, w_img)):
    xh = x.float().unflatten(-1, (heads, d))
    parts.append(F.rms_norm(xh, (d, ), w.float(), 1e-6))
  ref = _rope_ref(torch.cat(parts, dim=1), cos.float(), sin.float())
  assert torch.isfinite(out).all().item()
  err = (out.float() - ref).abs()
  # three bf16 roundings on values of magnitude ~|ref|: 2^-8 relative each
  assert (err <= 3 * 2.0**-8 * ref.abs() + 2e-2).all().item(), err.max().item()
  # and the eager bf16 sequence it replaces agrees to bf16 resolution on almost every element
  eager = []
  for x, w in ((x_txt, w_txt), (x_img, w_img)):
    eager.append(F.rms_norm(x.unflatten(-1, (heads, d)), (d, ), w, 1e-6))
  eager = _rope_ref(torch.cat(eager, dim=1), cos, sin)
  close = (out.float() - eager.float()).abs() <= 2.0**-7 * eager.float().abs() + 1e-3
  assert close.float().mean().item() > 0.99


@pytest.mark.parametrize("batch,tokens,cols", [(1, 5, 8), (2, 37, 72), (1, 4608, 3072), (3, 64, 3072)])
def test_gated_residual_is_bitwise_eager(nat, batch, tokens, cols):
  g = torch.Generator().manual_seed(cols + tokens)
  x = torch.randn(batch, tokens, cols, generator=g).to("cuda", torch.bfloat16)
  wide = torch.randn(batch, tokens, 2 * cols, generator=g).to("cuda", torch.bfloat16)
  y = wide[..., cols:]  # a column slice: strided rows
  mod = torch.randn(batch, 6 * cols, generator=g).to("cuda", torch.bfloat16)
  gate = mod.chunk(6, dim=-1)[2]
  out = nat.gated_residual(x, gate, y)
  ref = x + gate[:, None] * y
  assert torch.equal(out, ref)


def test_gated_residual_rejects_odd_width(nat):
  x = torch.zeros(1, 4, 12, device="cuda", dtype=torch.bfloat16)
  with pytest.raises(RuntimeError):
    nat.gated_residual(x, torch.zeros(1, 12, device="cuda", dtype=torch.bfloat16), x.clone())


def test_fused_linear_group_equals_members():
  from cache_dit_b200.quantization.linear import Float8RowwiseLinear, fused_group, quantize_rows_fused
  from cache_dit_b200 import _native
  torch.manual_seed(3)
  dims = [(256, 192), (256, 192), (256, 320)]
  members = []
  for k, n in dims:
    lin = torch.nn.Linear(k, n).to("cuda", torch.bfloat16)
    members.append(Float8RowwiseLinear.from_linear(lin))
  x = torch.randn(2, 50, 256, device="cuda", dtype=torch.bfloat16)
  a_q, a_scale, lead = quantize_rows_fused(x, _native.PRE_NONE)
  separate = [m.forward_quantized(a_q, a_scale, lead) for m in members]
  group = fused_group(members)
  assert fused_group(members) is group  # cached
  fused = group.forward_quantized(a_q, a_scale, lead)
  for s, f in zip(separate, fused):
    assert f.shape == s.shape and torch.equal(f, s)
  # members still work on their own after their storage moved into the group
  for m, s in zip(members, separate):
    assert torch.equal(m.forward_quantized(a_q, a_scale, lead), s)


@pytest.mark.parametrize("rows,c1,c2", [(5, 8, 16), (33, 3072, 12288), (130, 256, 1024), (64, 5120, 13824)])
def test_fp8_quant_concat_gelu_matches_two_step(nat, rows, c1, c2):
  """[head | gelu(tail)] quantized in one pass == GELU kernel output concatenated, then plain quantization."""
  g = torch.Generator().manual_seed(rows + c1)
  wide = torch.randn(rows, c1 + c2 + 8, generator=g).to("cuda", torch.bfloat16)
  head, tail = wide[:, :c1], wide[:, c1 + 8:]  # both strided
  q = torch.empty(rows, c1 + c2, dtype=torch.float8_e4m3fn, device="cuda")
  s = torch.empty(rows, dtype=torch.float32, device="cuda")
  nat.fp8_quant_rows_concat_gelu(head, tail, q, s)
  # two-step construction through the oracle's GELU and the plain kernel
  from oracle import fp8_oracle as FO
  act = torch.from_numpy(FO.gelu_tanh(tail.float().cpu().numpy())).to("cuda", torch.bfloat16)
  cat = torch.cat([head, act], dim=-1).contiguous()
  q2 = torch.empty_like(q)
  s2 = torch.empty_like(s)
  nat.fp8_quant_rows(cat, q2, s2)
  # the fast GELU differs from the oracle's on a few values per million that sit on a bf16 rounding
  # boundary; a row whose maximum is such a value gets a scale one bf16 step away
  same_scale = (s == s2)
  assert same_scale.float().mean().item() >= 0.95
  codes, codes2 = q.view(torch.uint8)[same_scale], q2.view(torch.uint8)[same_scale]
  assert (codes != codes2).float().mean().item() < 1e-3
  torch.testing.assert_close(s, s2, rtol=2.0**-7, atol=0)


def test_gated_residual_pair_equals_separate(nat):
  g = torch.Generator().manual_seed(9)
  cols = 3072
  sets = []
  for batch, tokens in ((1, 4096), (1, 512)):
    x = torch.randn(batch, tokens, cols, generator=g).to("cuda", torch.bfloat16)
    y = torch.randn(batch, tokens, 2 * cols, generator=g).to("cuda", torch.bfloat16)[..., cols:]
    gate = torch.randn(batch, 6 * cols, generator=g).to("cuda", torch.bfloat16).chunk(6, dim=-1)[4]
    sets.append((x, gate, y))
  a, b = nat.gated_residual_pair(*sets[0], *sets[1])
  assert torch.equal(a, sets[0][0] + sets[0][1][:, None] * sets[0][2])
  assert torch.equal(b, sets[1][0] + sets[1][1][:, None] * sets[1][2])


@pytest.mark.parametrize("m,n,k,bias", [(1, 1536, 256, True), (2, 18432, 3072, True), (4, 1000, 512, False), (3, 72, 3072, True)])
def test_bf16_gemv_matches_linear_and_is_slice_independent(m, n, k, bias):
  """`cdb_bf16_gemv` (modulation projections that stay in bf16): fp32-accumulated product within one bf16 step of an
  fp32 reference, rows of x / out strided, and - what the column-sharded modulation bank relies on - a column's
  bits do not depend on which row slice of the weight matrix the call covers."""
  from cache_dit_b200 import _native as nat
  g = torch.Generator().manual_seed(m * n + k)
  x_wide = torch.randn(m, k + 8, generator=g).to("cuda", torch.bfloat16)
  x = x_wide[:, :k]  # strided rows
  w = (0.05 * torch.randn(n, k, generator=g)).to("cuda", torch.bfloat16)
  b = torch.randn(n, generator=g).to("cuda", torch.bfloat16) if bias else None
  out_wide = torch.full((m, n + 16), float("nan"), device="cuda", dtype=torch.bfloat16)
  out = out_wide[:, 8:8 + n]
  nat.bf16_gemv(x, w, b, out)
  torch.cuda.synchronize()
  ref = x.float() @ w.float().t() + (b.float() if bias else 0.0)
  assert torch.isnan(out_wide[:, :8]).all() and torch.isnan(out_wide[:, 8 + n:]).all()
  assert ((out.float() - ref).abs() <= 2.0**-7 * ref.abs() + 1e-3).all().item()
  lo, hi = (n // 3) // 8 * 8, (2 * n // 3) // 8 * 8
  part = torch.empty(m, hi - lo, device="cuda", dtype=torch.bfloat16)
  nat.bf16_gemv(x, w[lo:hi], None if b is None else b[lo:hi], part)
  assert torch.equal(part, out[:, lo:hi])
  from cache_dit_b200.synthetic.layers import modulation_rows
  lin = torch.nn.Linear(k, n, bias=bias).to("cuda", torch.bfloat16)
  with torch.no_grad():
    lin.weight.copy_(w)
    if bias:
      lin.bias.copy_(b)
    got = modulation_rows(x_wide[:, :k].contiguous(), lin)
    want = lin(torch.nn.functional.silu(x_wide[:, :k].contiguous()))
  assert ((got.float() - want.float()).abs() <= 2.0**-6 * want.float().abs() + 2e-3).all().item()
