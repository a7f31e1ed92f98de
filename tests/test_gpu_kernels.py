"""Kernel-level parity on a B200: every C-ABI entry point against the numpy oracle."""
import numpy as np
import pytest
import torch

from oracle import cache_oracle as O
from oracle import fp8_oracle as F

pytestmark = pytest.mark.gpu

TD = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}
ULP = {"fp32": 1e-6, "bf16": 2.0**-8, "fp16": 2.0**-11}


@pytest.fixture(scope="module")
def nat():
  from cache_dit_b200 import _native
  _native.lib()
  return _native


def make(shape, dtype, seed, scale=1.0, device="cuda"):
  g = torch.Generator().manual_seed(seed)
  t = (torch.randn(shape, generator=g) * scale).to(TD[dtype])
  return t.to(device), t.float().numpy()


# ------------------------------------------------------------------------------ rel-L1
@pytest.mark.parametrize("dtype", ["bf16", "fp32", "fp16"])
@pytest.mark.parametrize("shape", [(1, 37, 72), (2, 19, 50), (1, 1, 5), (1, 512, 3072), (1, 4608, 3072)])
@pytest.mark.parametrize("fused_residual", [False, True])
def test_rel_l1_matches_oracle(nat, dtype, shape, fused_residual):
  prev_d, prev = make(shape, dtype, 1)
  means = torch.zeros(2, dtype=torch.float32, device="cuda")
  if fused_residual:
    h0_d, h0 = make(shape, dtype, 2)
    noise_d, noise = make(shape, dtype, 3, 0.05)
    h_d = (prev_d.float() + h0_d.float() + noise_d.float()).to(TD[dtype])
    h = h_d.float().cpu().numpy()
    res_d = torch.empty_like(h_d)
    nat.rel_l1(h_d, h0_d, prev_d, res_d, means)
    cur = O.residual(h, h0, dtype)
    np.testing.assert_array_equal(res_d.float().cpu().numpy(), cur)
  else:
    noise_d, noise = make(shape, dtype, 3, 0.05)
    cur_d = (prev_d.float() + noise_d.float()).to(TD[dtype])
    cur = cur_d.float().cpu().numpy()
    nat.rel_l1(cur_d, None, prev_d, None, means)
  md, mp = O.local_means(prev, cur, dtype)
  got = means.cpu().numpy()
  # sums are accumulated in a different order than numpy's: allow one unit in the last place of
  # the storage dtype on each mean (usually they are identical)
  assert abs(got[0] - md) <= ULP[dtype] * abs(md), (got, md, mp)
  assert abs(got[1] - mp) <= ULP[dtype] * abs(mp), (got, md, mp)
  diff = float(np.asarray(O.rnd(np.float32(got[0]) / np.float32(got[1]), dtype)).reshape(-1)[0])
  assert abs(diff - O.rel_l1(prev, cur, dtype)) <= 1e-3 * diff + 2 * ULP[dtype] * diff


def test_rel_l1_unaligned_views_and_repeat_launches(nat):
  base_d, _ = make((4099, ), "bf16", 5)
  other_d, _ = make((4099, ), "bf16", 6)
  prev_d, cur_d = base_d[1:], other_d[1:]  # 4098 elements each, 2 bytes past a 16-byte boundary
  means = torch.zeros(2, dtype=torch.float32, device="cuda")
  want = O.local_means(prev_d.float().cpu().numpy(), cur_d.float().cpu().numpy(), "bf16")
  for _ in range(3):  # the scratch ticket resets itself between launches
    means.zero_()
    nat.rel_l1(cur_d, None, prev_d, None, means)
    got = means.cpu().numpy()
    assert abs(got[0] - want[0]) <= 2.0**-8 * want[0]
    assert abs(got[1] - want[1]) <= 2.0**-8 * want[1]


def test_rel_l1_residual_only_and_run_to_run_determinism(nat):
  h_d, h = make((1, 333, 129), "bf16", 7)
  h0_d, h0 = make((1, 333, 129), "bf16", 8)
  res_d = torch.empty_like(h_d)
  nat.rel_l1(h_d, h0_d, None, res_d, None)
  np.testing.assert_array_equal(res_d.float().cpu().numpy(), O.residual(h, h0, "bf16"))
  prev_d, _ = make((1, 4608, 3072), "fp32", 9)
  cur_d, _ = make((1, 4608, 3072), "fp32", 10)
  m1 = torch.zeros(2, dtype=torch.float32, device="cuda")
  m2 = torch.zeros(2, dtype=torch.float32, device="cuda")
  nat.rel_l1(cur_d, None, prev_d, None, m1)
  nat.rel_l1(cur_d, None, prev_d, None, m2)
  assert torch.equal(m1, m2)


# ------------------------------------------------------------------------------ Taylor
@pytest.mark.parametrize("dtype", ["bf16", "fp32", "fp16"])
@pytest.mark.parametrize("terms", [1, 2, 3, 5])
@pytest.mark.parametrize("shape,add", [((1, 37, 72), True), ((1, 7, 13), True), ((1, 512, 3072), True),
                                       ((1, 37, 72), False)])
def test_taylor_apply_matches_oracle(nat, dtype, terms, shape, add):
  import math
  hid_d, hid = make(shape, dtype, 20)
  ds = [make(shape, dtype, 21 + i, 0.3**i) for i in range(terms)]
  elapsed = 3
  out_d = torch.empty_like(hid_d)
  nat.taylor_apply(hid_d, [d[0] for d in ds], [1.0 / math.factorial(i) for i in range(terms)],
                   [float(elapsed**i) for i in range(terms)], add, out_d)
  approx = O.taylor_series([d[1] for d in ds], elapsed, dtype)
  want = O.apply_add(approx, hid, dtype) if add else approx
  np.testing.assert_array_equal(out_d.float().cpu().numpy(), want)


def test_taylor_apply_in_place(nat):
  hid_d, hid = make((1, 100, 64), "bf16", 30)
  d0, d0n = make((1, 100, 64), "bf16", 31)
  d1, d1n = make((1, 100, 64), "bf16", 32, 0.1)
  nat.taylor_apply(hid_d, [d0, d1], [1.0, 1.0], [1.0, 2.0], True, hid_d)
  want = O.apply_add(O.taylor_series([d0n, d1n], 2, "bf16"), hid, "bf16")
  np.testing.assert_array_equal(hid_d.float().cpu().numpy(), want)


@pytest.mark.parametrize("dtype", ["bf16", "fp32", "fp16"])
@pytest.mark.parametrize("n_new", [0, 1, 2, 4])
@pytest.mark.parametrize("shape", [(1, 37, 72), (1, 7, 13), (1, 512, 3072)])
@pytest.mark.parametrize("fused_residual", [False, True])
def test_taylor_update_matches_oracle(nat, dtype, n_new, shape, fused_residual):
  after_d, after = make(shape, dtype, 40)
  before_d, before = make(shape, dtype, 41) if fused_residual else (None, None)
  prev = [make(shape, dtype, 42 + i, 0.5) for i in range(n_new)]
  cur_d = [torch.empty_like(after_d) for _ in range(n_new + 1)]
  window = 3
  nat.taylor_update(after_d, before_d, [p[0] for p in prev], cur_d, n_new, float(window))
  y = O.residual(after, before, dtype) if fused_residual else after
  ladder = O.taylor_derivatives(y, [p[1] for p in prev] + [None], window, True, dtype)
  for i in range(n_new + 1):
    np.testing.assert_array_equal(cur_d[i].float().cpu().numpy(), ladder[i], err_msg=f"order {i}")


# ------------------------------------------------------------------------------ FP8 quantization
def activations(rows, cols, seed):
  """N(0,1) with 0.1 % of the elements scaled by 20 (outliers), as bf16."""
  g = torch.Generator().manual_seed(seed)
  x = torch.randn(rows, cols, generator=g)
  mask = torch.rand(rows, cols, generator=g) < 1e-3
  x = torch.where(mask, x * 20.0, x).to(torch.bfloat16)
  return x.cuda(), x.float().numpy()


@pytest.mark.parametrize("rows,cols", [(1, 8), (5, 72), (33, 3072), (257, 5120), (64, 12288), (16, 13824),
                                       (8, 15360), (4, 16384), (4608, 3072)])
def test_fp8_quant_rows_matches_oracle(nat, rows, cols):
  x_d, x = activations(rows, cols, rows + cols)
  if rows > 2:
    x_d[2].zero_()
    x[2] = 0.0
  q = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device="cuda")
  s = torch.empty(rows, dtype=torch.float32, device="cuda")
  nat.fp8_quant_rows(x_d, q, s)
  codes, scale = F.quantize_rows(x)
  np.testing.assert_array_equal(s.cpu().numpy(), scale)
  np.testing.assert_array_equal(q.view(torch.uint8).cpu().numpy(), codes)


def test_fp8_quant_rows_strided_input(nat):
  x_d, x = activations(40, 1024, 3)
  view = x_d[:, 256:768]
  q = torch.empty(40, 512, dtype=torch.float8_e4m3fn, device="cuda")
  s = torch.empty(40, dtype=torch.float32, device="cuda")
  nat.fp8_quant_rows(view, q, s)
  codes, scale = F.quantize_rows(x[:, 256:768])
  np.testing.assert_array_equal(s.cpu().numpy(), scale)
  np.testing.assert_array_equal(q.view(torch.uint8).cpu().numpy(), codes)


def _close_codes(q, s, want_vals, frac=2e-3, rel=2e-3):
  """Fused pre-ops use device transcendental / fp32 statistics: a few elements may land on the
  neighbouring bf16 value before quantization.  Compare dequantized values instead of codes."""
  got = F.e4m3_decode(q.view(torch.uint8).cpu().numpy()) * s.cpu().numpy()[:, None]
  codes, scale = F.quantize_rows(want_vals)
  want = F.e4m3_decode(codes) * scale[:, None]
  mism = np.mean(got != want)
  err = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
  assert mism < frac and err < rel, (mism, err)


@pytest.mark.parametrize("rows,cols,batch", [(6, 72, 2), (512, 3072, 1), (96, 5120, 3)])
def test_fp8_quant_fused_layernorm_modulate(nat, rows, cols, batch):
  x_d, x = activations(rows, cols, 11)
  sh_d, sh = make((batch, cols), "bf16", 12, 0.2)
  sc_d, sc = make((batch, cols), "bf16", 13, 0.2)
  q = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device="cuda")
  s = torch.empty(rows, dtype=torch.float32, device="cuda")
  rpb = rows // batch
  nat.fp8_quant_rows(x_d, q, s, nat.PRE_LAYERNORM_MOD, sh_d, sc_d, rpb, 1e-6)
  want = np.concatenate([F.layernorm_modulate(x[b * rpb:(b + 1) * rpb], sh[b], sc[b], 1e-6)
                         for b in range(batch)])
  _close_codes(q, s, want)


@pytest.mark.parametrize("rows,cols", [(6, 72), (256, 12288)])
def test_fp8_quant_fused_gelu(nat, rows, cols):
  x_d, x = activations(rows, cols, 14)
  q = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device="cuda")
  s = torch.empty(rows, dtype=torch.float32, device="cuda")
  nat.fp8_quant_rows(x_d, q, s, nat.PRE_GELU_TANH)
  _close_codes(q, s, F.gelu_tanh(x))


# ------------------------------------------------------------------------------ FP8 GEMM
def rel_fro(a, b):
  return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) /
               max(np.linalg.norm(b.astype(np.float64)), 1e-30))


@pytest.mark.parametrize("M,N,K,bias", [
  (128, 256, 128, False), (128, 256, 512, True), (1, 8, 16, False), (200, 264, 144, True),
  (130, 520, 3072, False), (512, 3072, 3072, True), (4608, 3072, 3072, False),
  (1024, 12288, 3072, True), (1024, 3072, 12288, False), (640, 13824, 5120, False),
])
def test_fp8_gemm_matches_oracle(nat, M, N, K, bias):
  x_d, x = activations(M, K, M + N + K)
  g = torch.Generator().manual_seed(99)
  w = (0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16)
  b = torch.randn(N, generator=g).to(torch.bfloat16) if bias else None
  w_d = w.cuda()
  aq = torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda")
  sa = torch.empty(M, dtype=torch.float32, device="cuda")
  wq = torch.empty(N, K, dtype=torch.float8_e4m3fn, device="cuda")
  sw = torch.empty(N, dtype=torch.float32, device="cuda")
  nat.fp8_quant_rows(x_d, aq, sa)
  nat.fp8_quant_rows(w_d, wq, sw)
  out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
  nat.gemm_status_word(out.device).zero_()
  nat.fp8_gemm_rowscaled(aq, sa, wq, sw, None if b is None else b.cuda(), out)
  torch.cuda.synchronize()
  assert nat.gemm_device_status(out.device) == 0
  want = F.scaled_mm(aq.view(torch.uint8).cpu().numpy(), sa.cpu().numpy(),
                     wq.view(torch.uint8).cpu().numpy(), sw.cpu().numpy(),
                     None if b is None else b.float().numpy())
  got = out.float().cpu().numpy()
  assert np.isfinite(got).all()
  err = rel_fro(got, want)
  # north-star tolerance is 2e-2 relative Frobenius; identical quantized operands and fp32
  # accumulation leave only bf16 output rounding flips, so hold the kernel to a far tighter bar
  assert err < 2e-3, err
  # and against the un-quantized bf16 linear it must stay inside FP8's own error (~4 %)
  ref = x @ w.float().numpy().T + (0 if b is None else b.float().numpy())
  assert rel_fro(got, ref) < 8e-2


@pytest.mark.parametrize("M,N,K,bias", [(576, 3072, 3072, True), (576, 9216, 1024, False), (70, 1000, 256, True),
                                        (1152, 3080, 512, False)])
def test_fp8_gemm_result_is_independent_of_the_tile_width(nat, M, N, K, bias):
  """The single-CTA kernel picks its tile width (a multiple of 16 columns) so that tiles fill whole waves of
  SMs.  Every width must give the bits the full width gives: widths that end on a 64-column store boundary,
  widths with a ragged last block of 16 / 32 / 48 columns (written with plain stores), N not a multiple of
  the width, a strided output, and what the cost model itself picks."""
  x_d, _ = activations(M, K, M + K)
  w_d, _ = activations(N, K, N + K)
  g = torch.Generator().manual_seed(5)
  b = torch.randn(N, generator=g).to(torch.bfloat16).cuda() if bias else None
  aq = torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda")
  sa = torch.empty(M, dtype=torch.float32, device="cuda")
  wq = torch.empty(N, K, dtype=torch.float8_e4m3fn, device="cuda")
  sw = torch.empty(N, dtype=torch.float32, device="cuda")
  nat.fp8_quant_rows(x_d, aq, sa)
  nat.fp8_quant_rows(w_d, wq, sw)
  lib = nat.lib()
  try:
    assert lib.cdb_tuning_set_gemm_tile_cols(256) == 0
    want = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    nat.fp8_gemm_rowscaled(aq, sa, wq, sw, b, want)
    torch.cuda.synchronize()
    assert torch.isfinite(want).all()
    for cols in (0, 16, 64, 80, 96, 112, 128, 160, 176, 192, 208, 224, 240):
      assert lib.cdb_tuning_set_gemm_tile_cols(cols) == 0
      wide = torch.full((M, N + 24), float("nan"), dtype=torch.bfloat16, device="cuda")
      nat.fp8_gemm_rowscaled(aq, sa, wq, sw, b, wide[:, 8:8 + N])
      torch.cuda.synchronize()
      assert torch.equal(wide[:, 8:8 + N], want), cols
      assert torch.isnan(wide[:, :8]).all() and torch.isnan(wide[:, 8 + N:]).all(), cols  # nothing written outside
    assert lib.cdb_tuning_set_gemm_tile_cols(24) != 0 and lib.cdb_tuning_set_gemm_tile_cols(272) != 0
  finally:
    lib.cdb_tuning_set_gemm_tile_cols(0)
  assert nat.gemm_device_status(want.device) == 0


@pytest.mark.parametrize("shapes", [[(64, 3072, 512)], [(576, 3072, 1024)], [(894, 1000, 256)], [(1152, 3080, 512)],
                                    [(576, 9216, 512), (64, 9216, 512)], [(1024, 3072, 1536), (128, 3072, 1536)]])
def test_fp8_gemm_pair_kernel_gives_the_single_cta_kernels_bits(nat, shapes):
  """Below 4096 rows a wave-count model picks the single-CTA or the CTA-pair kernel per launch (rank shards of a
  context-parallel run).  Both accumulate every output element over the K blocks in the same order, so the
  choice must not change a bit: rows that fill a quarter of a 256-row pair tile, ragged row and column counts,
  a strided output, two products in one launch, and pair tiles narrower than 256 columns (the launch model uses
  128 where the wide tiles would leave most pairs idle)."""
  lib = nat.lib()
  kinds = (1, 2, 0, (2, 128), (2, 192), (2, 64), (2, 32))  # (2, cols): the pair kernel at a forced tile width
  problems = {k: [] for k in kinds}
  wides = {k: [] for k in kinds}
  for i, (M, N, K) in enumerate(shapes):
    x_d, _ = activations(M, K, M + K + i)
    w_d, _ = activations(N, K, N + K + i)
    g = torch.Generator().manual_seed(7 + i)
    b = torch.randn(N, generator=g).to(torch.bfloat16).cuda()
    aq = torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda")
    sa = torch.empty(M, dtype=torch.float32, device="cuda")
    wq = torch.empty(N, K, dtype=torch.float8_e4m3fn, device="cuda")
    sw = torch.empty(N, dtype=torch.float32, device="cuda")
    nat.fp8_quant_rows(x_d, aq, sa)
    nat.fp8_quant_rows(w_d, wq, sw)
    for kind in kinds:
      wide = torch.full((M, N + 24), float("nan"), dtype=torch.bfloat16, device="cuda")
      wides[kind].append(wide)
      problems[kind].append((aq, sa, wq, sw, b, wide[:, 8:8 + N]))
  try:
    for kind in kinds:
      k, cols = kind if isinstance(kind, tuple) else (kind, 0)
      assert lib.cdb_tuning_set_gemm_kernel(k) == 0 and lib.cdb_tuning_set_gemm_tile_cols(cols) == 0
      nat.fp8_gemm_rowscaled_grouped(problems[kind])
      torch.cuda.synchronize()
    assert lib.cdb_tuning_set_gemm_kernel(3) != 0
  finally:
    lib.cdb_tuning_set_gemm_kernel(0)
    lib.cdb_tuning_set_gemm_tile_cols(0)
  for i, (M, N, K) in enumerate(shapes):
    single = wides[1][i]
    assert torch.isfinite(single[:, 8:8 + N]).all()
    for kind in kinds[1:]:
      assert torch.equal(wides[kind][i][:, 8:8 + N], single[:, 8:8 + N]), (kind, i)
      assert torch.isnan(wides[kind][i][:, :8]).all() and torch.isnan(wides[kind][i][:, 8 + N:]).all(), (kind, i)
  assert nat.gemm_device_status(torch.device("cuda")) == 0


@pytest.mark.parametrize("kind,cols", [(1, 0), (1, 80), (2, 0)])
@pytest.mark.parametrize("shapes,gelu_from", [([(320, 1024, 256)], [0]), ([(576, 3072 + 1024, 512)], [3072]),
                                              ([(520, 2048, 256), (72, 2048, 256)], [0, 0]),
                                              ([(300, 1000, 256), (64, 512, 256)], [None, 256])])
def test_fp8_gemm_epilogue_gelu(nat, kind, cols, shapes, gelu_from):
  """An MLP-in product can apply the MLP's tanh-GELU in its epilogue: columns from `gelu_from` on are written as
  bf16(gelu(bf16(y))).  Columns in front of it must keep the plain product's bits; the activated ones must be what
  the GELU variant of the quantization kernel computes from the plain output (same device function, so the
  quantized activations agree: equal scales, and codes that differ only where that variant's uncorrected division
  lands on the other side of a rounding boundary), and within one bf16 step of torch's gelu where that is itself accurate.  Both tile kernels,
  a ragged tile width, two products per launch."""
  lib = nat.lib()
  plain, acted, probs_plain, probs_act = [], [], [], []
  for i, (M, N, K) in enumerate(shapes):
    x_d, _ = activations(M, K, 40 + i)
    w_d, _ = activations(N, K, 50 + i)
    g = torch.Generator().manual_seed(60 + i)
    b = torch.randn(N, generator=g).to(torch.bfloat16).cuda()
    aq = torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda")
    sa = torch.empty(M, dtype=torch.float32, device="cuda")
    wq = torch.empty(N, K, dtype=torch.float8_e4m3fn, device="cuda")
    sw = torch.empty(N, dtype=torch.float32, device="cuda")
    nat.fp8_quant_rows(x_d, aq, sa)
    nat.fp8_quant_rows(w_d, wq, sw)
    plain.append(torch.empty(M, N, dtype=torch.bfloat16, device="cuda"))
    acted.append(torch.empty(M, N, dtype=torch.bfloat16, device="cuda"))
    probs_plain.append((aq, sa, wq, sw, b, plain[-1]))
    probs_act.append((aq, sa, wq, sw, b, acted[-1]))
  try:
    assert lib.cdb_tuning_set_gemm_kernel(kind) == 0 and lib.cdb_tuning_set_gemm_tile_cols(cols) == 0
    nat.fp8_gemm_rowscaled_grouped(probs_plain)
    nat.fp8_gemm_rowscaled_grouped(probs_act, gelu_from)
    torch.cuda.synchronize()
  finally:
    lib.cdb_tuning_set_gemm_kernel(0)
    lib.cdb_tuning_set_gemm_tile_cols(0)
  for (M, N, K), c0, y, z in zip(shapes, gelu_from, plain, acted):
    if c0 is None:
      assert torch.equal(y, z)
      continue
    assert torch.equal(y[:, :c0], z[:, :c0])
    want = torch.nn.functional.gelu(y[:, c0:].float(), approximate="tanh").to(torch.bfloat16)
    got = z[:, c0:]
    # one bf16 step, plus the absolute error of torch's own 0.5 x (1 + tanh u) where 1 + tanh u cancels (x < -4)
    err = (got.float() - want.float()).abs()
    assert bool((err <= 2.0 ** -7 * want.float().abs() + 1e-6).all())
    assert float(((got != want) & (want.float().abs() > 1e-3)).float().mean()) < 2e-3  # away from that tail: rare last-bit ties
    n = N - c0
    qa = torch.empty(M, n, dtype=torch.float8_e4m3fn, device="cuda")
    sa_ = torch.empty(M, dtype=torch.float32, device="cuda")
    qb = torch.empty(M, n, dtype=torch.float8_e4m3fn, device="cuda")
    sb_ = torch.empty(M, dtype=torch.float32, device="cuda")
    nat.fp8_quant_rows(y[:, c0:], qa, sa_, nat.PRE_GELU_TANH)
    nat.fp8_quant_rows(got, qb, sb_)
    assert torch.equal(sa_, sb_)
    assert float((qa.view(torch.uint8) != qb.view(torch.uint8)).float().mean()) < 1e-4
  assert nat.gemm_device_status(torch.device("cuda")) == 0
  assert lib.cdb_fp8_gemm_rowscaled_grouped_act(None, 1, None, None, None) != 0


def test_fp8_quant_concat_with_activated_tail(nat):
  """[head | tail] with a tail that already is activated = the concat + GELU kernel on the plain tail."""
  rows, c1, c2 = 200, 3072, 4096
  head, _ = activations(rows, c1, 71)
  tail, _ = activations(rows, c2, 72)
  want_q = torch.empty(rows, c1 + c2, dtype=torch.float8_e4m3fn, device="cuda")
  want_s = torch.empty(rows, dtype=torch.float32, device="cuda")
  nat.fp8_quant_rows_concat_gelu(head, tail, want_q, want_s)
  # torch's gelu stands in for the product epilogue here; it differs from the device function in the last bf16
  # bit of a few values, hence the tolerances (the epilogue's own bits are held in test_fp8_gemm_epilogue_gelu)
  act = torch.nn.functional.gelu(tail.float(), approximate="tanh").to(torch.bfloat16)
  got_q = torch.empty_like(want_q)
  got_s = torch.empty_like(want_s)
  nat.fp8_quant_rows_concat_gelu(head, act, got_q, got_s, tail_activated=True)
  torch.cuda.synchronize()
  assert float((got_s != want_s).float().mean()) < 1e-2  # torch's gelu may differ from the device function in the last bf16 bit
  close = (got_q.view(torch.uint8).int() - want_q.view(torch.uint8).int()).abs()
  assert float((close != 0).float().mean()) < 2e-3 and int(close.max()) <= 1


def test_fp8_gemm_strided_output_and_back_to_back(nat):
  M, N, K = 256, 512, 256
  x_d, _ = activations(M, K, 1)
  w_d, _ = activations(N, K, 2)
  aq = torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda")
  sa = torch.empty(M, dtype=torch.float32, device="cuda")
  wq = torch.empty(N, K, dtype=torch.float8_e4m3fn, device="cuda")
  sw = torch.empty(N, dtype=torch.float32, device="cuda")
  nat.fp8_quant_rows(x_d, aq, sa)
  nat.fp8_quant_rows(w_d, wq, sw)
  big = torch.zeros(M, 2 * N, dtype=torch.bfloat16, device="cuda")
  dense = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
  for _ in range(3):
    nat.fp8_gemm_rowscaled(aq, sa, wq, sw, None, big[:, N:])
    nat.fp8_gemm_rowscaled(aq, sa, wq, sw, None, dense)
  torch.cuda.synchronize()
  assert torch.equal(big[:, N:], dense)
  assert not big[:, :N].any()
  assert nat.gemm_device_status(dense.device) == 0


# ------------------------------------------------------------------------------ shapes of the sharded configs
# Qwen-Image 1328^2: 6889 image tokens over 8 ranks -> shards of 862 / 861 tokens (uneven), hidden 3072;
# Wan2.1-14B 81x720p: 75600 tokens over 8 ranks -> 9450 tokens, hidden 5120, FFN 13824.
@pytest.mark.parametrize("shape", [(1, 862, 3072), (1, 861, 3072), (1, 256, 3072), (1, 9450, 5120)])
def test_cache_kernels_on_context_parallel_shard_shapes(nat, shape):
  prev_d, prev = make(shape, "bf16", 50)
  h0_d, h0 = make(shape, "bf16", 51)
  noise_d, _ = make(shape, "bf16", 52, 0.05)
  h_d = (prev_d.float() + h0_d.float() + noise_d.float()).to(torch.bfloat16)
  res_d = torch.empty_like(h_d)
  means = torch.zeros(2, dtype=torch.float32, device="cuda")
  nat.rel_l1(h_d, h0_d, prev_d, res_d, means)
  cur = O.residual(h_d.float().cpu().numpy(), h0, "bf16")
  np.testing.assert_array_equal(res_d.float().cpu().numpy(), cur)
  md, mp = O.local_means(prev, cur, "bf16")
  got = means.cpu().numpy()
  assert abs(got[0] - md) <= 2.0**-8 * md and abs(got[1] - mp) <= 2.0**-8 * mp
  d1_d, d1 = make(shape, "bf16", 53, 0.1)
  out_d = torch.empty_like(h_d)
  nat.taylor_apply(h_d, [prev_d, d1_d], [1.0, 1.0], [1.0, 2.0], True, out_d)
  want = O.apply_add(O.taylor_series([prev, d1], 2, "bf16"), h_d.float().cpu().numpy(), "bf16")
  np.testing.assert_array_equal(out_d.float().cpu().numpy(), want)


@pytest.mark.parametrize("M,N,K", [(862, 3072, 3072), (9450, 13824, 5120), (9450, 5120, 13824), (512, 18432, 3072),
                                   (1, 18432, 3072)])
def test_fp8_gemm_on_model_shapes(nat, M, N, K):
  x_d, x = activations(M, K, M + 1)
  g = torch.Generator().manual_seed(98)
  w_d = (0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16).cuda()
  aq = torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda")
  sa = torch.empty(M, dtype=torch.float32, device="cuda")
  wq = torch.empty(N, K, dtype=torch.float8_e4m3fn, device="cuda")
  sw = torch.empty(N, dtype=torch.float32, device="cuda")
  nat.fp8_quant_rows(x_d, aq, sa)
  nat.fp8_quant_rows(w_d, wq, sw)
  out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
  nat.fp8_gemm_rowscaled(aq, sa, wq, sw, None, out)
  torch.cuda.synchronize()
  assert nat.gemm_device_status(out.device) == 0
  rows = slice(0, min(M, 1024))  # the CPU product of the largest shapes is checked on a row block
  want = F.scaled_mm(aq[rows].view(torch.uint8).cpu().numpy(), sa[rows].cpu().numpy(),
                     wq.view(torch.uint8).cpu().numpy(), sw.cpu().numpy())
  got = out[rows].float().cpu().numpy()
  assert torch.isfinite(out).all().item()
  assert rel_fro(got, want) < 2e-3
  if M > 1024:  # and the last row block (ragged M tile)
    rows = slice(M - 300, M)
    want = F.scaled_mm(aq[rows].view(torch.uint8).cpu().numpy(), sa[rows].cpu().numpy(),
                       wq.view(torch.uint8).cpu().numpy(), sw.cpu().numpy())
    assert rel_fro(out[rows].float().cpu().numpy(), want) < 2e-3


# ------------------------------------------------------------------------------ against the library ops the reference calls
@pytest.mark.parametrize("M,N,K,bias", [(300, 272, 256, False), (4608, 3072, 3072, True), (1000, 12288, 3072, False)])
def test_fp8_gemm_matches_library_scaled_mm(nat, M, N, K, bias):
  """`torch._scaled_mm` with row-wise scales is the call the reference makes for this product
  (src/cache_dit/quantization/torchao/_scaled_mm.py:72-91).  Same quantized operands in both."""
  g = torch.Generator().manual_seed(M + N)
  x = torch.randn(M, K, generator=g)
  x = torch.where(torch.rand(M, K, generator=g) < 1e-3, x * 20, x).to("cuda", torch.bfloat16)
  w = (0.02 * torch.randn(N, K, generator=g)).to("cuda", torch.bfloat16)
  b = (0.1 * torch.randn(N, generator=g)).to("cuda", torch.bfloat16) if bias else None
  aq = torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda")
  sa = torch.empty(M, dtype=torch.float32, device="cuda")
  wq = torch.empty(N, K, dtype=torch.float8_e4m3fn, device="cuda")
  sw = torch.empty(N, dtype=torch.float32, device="cuda")
  nat.fp8_quant_rows(x, aq, sa)
  nat.fp8_quant_rows(w, wq, sw)
  out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
  nat.fp8_gemm_rowscaled(aq, sa, wq, sw, b, out)
  try:
    lib = torch._scaled_mm(aq, wq.t(), scale_a=sa.view(M, 1), scale_b=sw.view(1, N), bias=b, out_dtype=torch.bfloat16)
  except Exception as e:  # the library build on this machine has no row-wise FP8 kernel
    pytest.skip(f"torch._scaled_mm row-wise unavailable: {e}")
  err = (out.float() - lib.float()).norm() / lib.float().norm()
  assert err.item() < 2e-3, err.item()  # both round an fp32 accumulation to bf16; bound of the path is 2e-2


@pytest.mark.parametrize("rows,cols", [(64, 3072), (33, 5120)])
def test_fp8_quant_matches_torch_cast_pipeline(nat, rows, cols):
  """Per-row dynamic quantization written with torch's own ops and its e4m3 cast, the primitives the
  reference's torchao configuration lowers to (PerRow, e4m3: src/cache_dit/quantization/torchao/quantize_ao.py:540-558;
  zero scale -> 1 at :43-71)."""
  x_d, _ = activations(rows, cols, 21)
  x_d[3].zero_()
  x_d[min(5, rows - 1), :7] = -0.0  # a negative zero keeps its sign through the division (code 0x80)
  q = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device="cuda")
  s = torch.empty(rows, dtype=torch.float32, device="cuda")
  nat.fp8_quant_rows(x_d, q, s)
  xf = x_d.float()
  scale = xf.abs().amax(dim=1) / 448.0
  scale = torch.where(scale == 0, torch.ones_like(scale), scale)
  want = (xf / scale[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
  assert torch.equal(s, scale)
  assert torch.equal(q.view(torch.uint8), want.view(torch.uint8))


@pytest.mark.parametrize("case", ["small_bias", "odd_rows", "wide"])
def test_fp8_linear_matches_committed_torch_fixture(nat, case):
  """The committed outputs of PyTorch's CUDA ops (tests/golden/make_fp8_torch_fixture.py): codes and scales
  bit for bit, the product within the path's tolerance of the library's."""
  import os
  fx = np.load(os.path.join(os.path.dirname(__file__), "golden", "fp8_torch_cuda.npz"))
  dev = lambda bits: torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).cuda()
  x, w = dev(fx[f"{case}.x"]), dev(fx[f"{case}.w"])
  b = dev(fx[f"{case}.bias"]) if f"{case}.bias" in fx.files else None
  M, K, N = x.shape[0], x.shape[1], w.shape[0]
  aq = torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda")
  sa = torch.empty(M, dtype=torch.float32, device="cuda")
  wq = torch.empty(N, K, dtype=torch.float8_e4m3fn, device="cuda")
  sw = torch.empty(N, dtype=torch.float32, device="cuda")
  nat.fp8_quant_rows(x, aq, sa)
  nat.fp8_quant_rows(w, wq, sw)
  np.testing.assert_array_equal(sa.cpu().numpy(), fx[f"{case}.a_scale"])
  np.testing.assert_array_equal(aq.view(torch.uint8).cpu().numpy(), fx[f"{case}.a_codes"])
  np.testing.assert_array_equal(sw.cpu().numpy(), fx[f"{case}.w_scale"])
  np.testing.assert_array_equal(wq.view(torch.uint8).cpu().numpy(), fx[f"{case}.w_codes"])
  out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
  nat.fp8_gemm_rowscaled(aq, sa, wq, sw, b, out)
  want = dev(fx[f"{case}.out"]).float()
  err = (out.float() - want).norm() / want.norm()
  assert err.item() < 2e-3, err.item()  # bound of the path: 2e-2


@pytest.mark.parametrize("shapes", [((4608, 3072, 3072), (512, 3072, 3072)), ((1000, 520, 256), (130, 264, 256)),
                                    ((300, 272, 512), (700, 1024, 256)), ((4096, 9216, 3072), (512, 9216, 3072))])
def test_fp8_gemm_grouped_equals_separate_launches(nat, shapes):
  """Two products in one launch (the second one's tiles ride in the tail wave of the first) give exactly
  what two launches give, whatever their shapes and order."""
  g = torch.Generator(device="cuda").manual_seed(sum(shapes[0]))
  problems, want = [], []
  for M, N, K in shapes:
    aq = torch.randn(M, K, device="cuda", generator=g).to(torch.float8_e4m3fn)
    wq = torch.randn(N, K, device="cuda", generator=g).to(torch.float8_e4m3fn)
    sa = torch.rand(M, device="cuda", generator=g) + 0.5
    sw = torch.rand(N, device="cuda", generator=g) + 0.5
    bias = torch.randn(N, device="cuda", generator=g).to(torch.bfloat16)
    ref = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    nat.fp8_gemm_rowscaled(aq, sa, wq, sw, bias, ref)
    want.append(ref)
    problems.append((aq, sa, wq, sw, bias, torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")))
  nat.fp8_gemm_rowscaled_grouped(problems)
  torch.cuda.synchronize()
  for (_, _, _, _, _, out), ref in zip(problems, want):
    assert torch.equal(out, ref)
  assert nat.gemm_device_status(torch.device("cuda:0")) == 0


@pytest.mark.parametrize("preop", ["none", "layernorm", "gelu"])
def test_fp8_quant_pair_equals_separate_launches(nat, preop):
  """Two tensors quantized by one launch (different row counts, strides and modulation vectors) give
  exactly what two launches give."""
  code = {"none": nat.PRE_NONE, "layernorm": nat.PRE_LAYERNORM_MOD, "gelu": nat.PRE_GELU_TANH}[preop]
  cols = 3072
  xa_d, _ = activations(2 * 300, cols, 31)
  wide, _ = activations(3 * 37, cols + 64, 32)
  xb_d = wide[:, 64:]  # strided rows
  mods = {}
  for name, batch, seed in (("a", 2, 33), ("b", 3, 34)):
    m, _ = make((batch, 2 * cols), "bf16", seed, 0.2)
    mods[name] = (m[:, :cols], m[:, cols:])
  jobs, want = [], []
  for x, name, batch in ((xa_d, "a", 2), (xb_d, "b", 3)):
    rows = x.shape[0]
    q = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device="cuda")
    s = torch.empty(rows, dtype=torch.float32, device="cuda")
    if preop == "layernorm":
      nat.fp8_quant_rows(x, q, s, code, mods[name][0], mods[name][1], rows // batch, 1e-6)
    else:
      nat.fp8_quant_rows(x, q, s, code)
    want.append((q, s))
    job = dict(x2d=x, q=torch.zeros_like(q), scale=torch.zeros_like(s))
    if preop == "layernorm":
      job.update(mod_shift=mods[name][0], mod_scale=mods[name][1], rows_per_batch=rows // batch)
    jobs.append(job)
  nat.fp8_quant_rows_pair(jobs, code, 1e-6)
  torch.cuda.synchronize()
  for job, (q, s) in zip(jobs, want):
    assert torch.equal(job["scale"], s)
    assert torch.equal(job["q"].view(torch.uint8), q.view(torch.uint8))


def test_fused_linear_group_follows_its_members_when_they_move():
  """q/k/v run as one product over concatenated weights that the member layers view.  Moving the model
  (here: to the CPU and back, which gives the members fresh buffers) must not leave the group computing
  with the weights it cached before the move."""
  from cache_dit_b200.quantization.linear import Float8RowwiseLinear, fused_group
  torch.manual_seed(3)
  dev = torch.device("cuda")
  holder = torch.nn.Module()
  holder.lins = torch.nn.ModuleList(
    [Float8RowwiseLinear.from_linear(torch.nn.Linear(256, 128).to(torch.bfloat16).to(dev)) for _ in range(3)])
  x = torch.randn(64, 256, device=dev).to(torch.bfloat16)
  a_q, a_scale = holder.lins[0].quantize_input(x)
  separate = [l.forward_quantized(a_q, a_scale, (64, )).clone() for l in holder.lins]
  first = fused_group(list(holder.lins))
  outs = first.forward_quantized(a_q, a_scale, (64, ))
  assert all(torch.equal(o, s) for o, s in zip(outs, separate))
  assert fused_group(list(holder.lins)) is first  # cached while the members still view its storage
  holder.to("cpu")
  holder.to(dev)
  with torch.no_grad():  # the moved copies are independent now: change one to prove which weights are used
    holder.lins[1].weight_scale.mul_(2.0)
  second = fused_group(list(holder.lins))
  assert second is not first
  outs = second.forward_quantized(a_q, a_scale, (64, ))
  separate = [l.forward_quantized(a_q, a_scale, (64, )) for l in holder.lins]
  assert all(torch.equal(o, s) for o, s in zip(outs, separate))


@pytest.mark.parametrize("sizes", [(128, 128, 256), (40, 24)])
def test_fused_group_activates_its_last_member(sizes):
  """`gelu_last` returns the last member's output activated by the product's epilogue (FP8 linears have a multiple
  of 8 output features, so a member always starts on a 16-byte chunk): the other members keep the plain product's
  bits and the last one is gelu of them."""
  from cache_dit_b200.quantization.linear import Float8RowwiseLinear, fused_group, grouped_forward_quantized
  torch.manual_seed(4)
  dev = torch.device("cuda")
  lins = [Float8RowwiseLinear.from_linear(torch.nn.Linear(64, n).to(torch.bfloat16).to(dev)) for n in sizes]
  x = torch.randn(40, 64, device=dev).to(torch.bfloat16)
  a_q, a_scale = lins[0].quantize_input(x)
  group = fused_group(lins)
  plain = [o.clone() for o in group.forward_quantized(a_q, a_scale, (40, ))]
  acted = group.forward_quantized(a_q, a_scale, (40, ), gelu_last=True)
  (paired, ) = grouped_forward_quantized([(group, a_q, a_scale, (40, ))], gelu_last=True)
  for got in (acted, paired):
    for a, b in zip(plain[:-1], got[:-1]):
      assert torch.equal(a, b)
    want = torch.nn.functional.gelu(plain[-1].float(), approximate="tanh").to(torch.bfloat16)
    err = (got[-1].float() - want.float()).abs()
    assert bool((err <= 2.0 ** -7 * want.float().abs() + 1e-6).all())
