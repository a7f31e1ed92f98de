"""Host-side (CPU, eager) semantics of the MLP helpers: where the activation is applied must not matter."""
import torch
import torch.nn.functional as F

from cache_dit_b200.synthetic import layers as L


def _mods(b, c, seed):
  g = torch.Generator().manual_seed(seed)
  return 0.1 * torch.randn(b, c, generator=g), 0.1 * torch.randn(b, c, generator=g)


def test_gelu_last_marks_only_the_last_output():
  torch.manual_seed(0)
  x = torch.randn(2, 5, 16)
  shift, scale = _mods(2, 16, 1)
  lins = [torch.nn.Linear(16, 8), torch.nn.Linear(16, 8), torch.nn.Linear(16, 24)]
  plain = L.norm_modulate_linears(x, shift, scale, lins)
  acted = L.norm_modulate_linears(x, shift, scale, lins, gelu_last=True)
  for a, b in zip(plain[:-1], acted[:-1]):
    assert torch.equal(a, b)
  assert torch.equal(acted[-1], F.gelu(plain[-1], approximate="tanh"))
  pa, pb = L.norm_modulate_linears_pair((x, shift, scale, lins[:1]), (x[:, :2], shift, scale, lins[2:]), gelu_last=True)
  assert torch.equal(pa[0], F.gelu(plain[0], approximate="tanh"))
  assert torch.equal(pb[0], F.gelu(lins[2](L.norm_modulate(x[:, :2], shift, scale)), approximate="tanh"))


def test_activated_inputs_skip_the_activation():
  torch.manual_seed(1)
  h, c = torch.randn(2, 5, 24), torch.randn(2, 3, 24)
  la, lb = torch.nn.Linear(24, 16), torch.nn.Linear(24, 16)
  want = L.gelu_linear_pair(h, la, c, lb)
  act = lambda t: F.gelu(t, approximate="tanh")
  got = L.gelu_linear_pair(act(h), la, act(c), lb, activated=True)
  assert torch.equal(want[0], got[0]) and torch.equal(want[1], got[1])
  assert torch.equal(L.gelu_linear(act(h), la, activated=True), L.gelu_linear(h, la))
  o = torch.randn(2, 5, 8)
  lo = torch.nn.Linear(8 + 24, 16)
  assert torch.equal(L.concat_gelu_linear(o, act(h), lo, tail_activated=True), L.concat_gelu_linear(o, h, lo))


def test_switch(monkeypatch):
  monkeypatch.delenv("CACHE_DIT_B200_GELU_IN_PRODUCT", raising=False)
  assert L.gelu_in_product()
  monkeypatch.setenv("CACHE_DIT_B200_GELU_IN_PRODUCT", "0")
  assert not L.gelu_in_product()
