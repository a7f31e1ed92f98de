"""Layer selection of `quantize` on CPU (the FP8 conversion itself is replaced by a marker module).

The reference quantizes repeated block by repeated block (src/cache_dit/quantization/torchao/quantize_ao.py:128-131),
so the names its filter sees are relative to the block: "attn.to_q", never "transformer_blocks.1.attn.to_q".
"""
import pytest
import torch
from torch import nn

import cache_dit_b200 as cd
from cache_dit_b200.quantization import linear as qlinear
from cache_dit_b200.quantization import quantize as qmod


class _Marker(nn.Module):

  def __init__(self, linear):
    super().__init__()
    self.shape = tuple(linear.weight.shape)


class Block(nn.Module):

  def __init__(self):
    super().__init__()
    self.attn = nn.Module()
    self.attn.to_q = nn.Linear(32, 32)
    self.attn.to_k = nn.Linear(32, 32)
    self.norm1 = nn.Module()
    self.norm1.linear = nn.Linear(32, 64)
    self.img_mod = nn.Sequential(nn.SiLU(), nn.Linear(32, 64))


class Model(nn.Module):
  _repeated_blocks = ["Block"]

  def __init__(self):
    super().__init__()
    self.blocks = nn.ModuleList([Block() for _ in range(3)])
    self.proj_out = nn.Linear(32, 16)


@pytest.fixture
def marker_conversion(monkeypatch):
  monkeypatch.setattr(qlinear.Float8RowwiseLinear, "from_linear", classmethod(lambda cls, lin: _Marker(lin)))
  monkeypatch.setattr(qlinear.Float8RowwiseLinear, "supports", staticmethod(lambda lin: True))


def _quantized_names(model):
  return sorted(n for n, m in model.named_modules() if isinstance(m, _Marker))


def test_patterns_match_block_relative_names_only(marker_conversion):
  model = Model().to(torch.bfloat16)
  # "blocks.1" and "s.1" occur only in the path OUTSIDE the repeated block: in the reference they match nothing
  cd.quantize(model, cd.QuantizeConfig(quant_type="float8_per_row", exclude_layers=["blocks.1", "s.1", "mod"]))
  names = _quantized_names(model)
  for i in range(3):
    assert f"blocks.{i}.attn.to_q" in names and f"blocks.{i}.attn.to_k" in names and f"blocks.{i}.norm1.linear" in names
    assert f"blocks.{i}.img_mod.1" not in names  # "mod" is inside the block-relative name
  assert "proj_out" not in names  # outside the repeated blocks: regional quantization leaves it alone
  assert all("blocks." not in line.split("->")[0] for line in model._quantize_stats["skipped"])


def test_custom_filter_sees_block_relative_names(marker_conversion):
  seen = []

  def only_q(m, name):
    seen.append(name)
    return isinstance(m, nn.Linear) and name == "attn.to_q"

  model = Model().to(torch.bfloat16)
  cd.quantize(model, cd.QuantizeConfig(quant_type="float8_per_row", filter_fn=only_q))
  assert _quantized_names(model) == [f"blocks.{i}.attn.to_q" for i in range(3)]
  assert "attn.to_k" in seen and not any(n.startswith("blocks") for n in seen)


def test_whole_module_pass_keeps_full_paths(marker_conversion):
  model = Model().to(torch.bfloat16)
  cd.quantize(model, cd.QuantizeConfig(quant_type="float8_per_row", regional_quantize=False, exclude_layers=["blocks.1"]))
  names = _quantized_names(model)
  assert "proj_out" in names and "blocks.0.attn.to_q" in names
  assert not any(n.startswith("blocks.1.") for n in names)
