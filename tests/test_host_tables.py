"""Pure host logic against tables produced by the reference: step masks and config tags."""
import pytest

import cache_dit_b200 as cd
from tests.golden_io import load_json

TABLES = load_json("host_tables.json")


@pytest.mark.parametrize("key", sorted(k for k in TABLES["steps_mask"] if not k.startswith("bins/")))
def test_predefined_step_masks(key):
  policy, total = key.split("/")
  assert cd.steps_mask(total_steps=int(total), mask_policy=policy) == TABLES["steps_mask"][key]


def test_explicit_bins():
  assert cd.steps_mask(compute_bins=[4, 2, 1], cache_bins=[3, 5, 2]) == TABLES["steps_mask"]["bins/a"]
  assert cd.steps_mask(compute_bins=[6, 1, 1, 1], cache_bins=[1, 2, 5], total_steps=14) == \
      TABLES["steps_mask"]["bins/b"]
  with pytest.raises(AssertionError):
    cd.steps_mask(compute_bins=[1], cache_bins=[1], total_steps=5)
  with pytest.raises(ValueError):
    cd.steps_mask(total_steps=28, mask_policy="warp")


def test_config_tags():
  tags = TABLES["tags"]
  assert cd.DBCacheConfig().strify() == tags["default"]
  assert cd.DBCacheConfig(Fn_compute_blocks=1, max_warmup_steps=4, max_cached_steps=10,
                          max_continuous_cached_steps=3, residual_diff_threshold=0.12,
                          steps_computation_mask=[1, 0, 1, 0], steps_computation_policy="static",
                          num_inference_steps=4, force_refresh_step_hint=2,
                          enable_separate_cfg=True).strify() == tags["scm"]
  assert cd.TaylorSeerCalibratorConfig(taylorseer_order=2).strify() == tags["taylor"]
  assert cd.TaylorSeerCalibratorConfig(taylorseer_order=2).strify(details=True) == tags["taylor_details"]


def test_config_defaults_match_reference_schema():
  c = cd.DBCacheConfig()
  assert (c.Fn_compute_blocks, c.Bn_compute_blocks, c.residual_diff_threshold, c.max_warmup_steps,
          c.warmup_interval, c.max_cached_steps, c.max_continuous_cached_steps) == (8, 0, 0.08, 8, 1, -1, -1)
  assert c.enable_separate_cfg is None and c.cfg_compute_first is False and c.cfg_diff_compute_separate is True
  assert c.steps_computation_policy == "dynamic" and c.force_refresh_step_policy == "once"
  t = cd.TaylorSeerCalibratorConfig()
  assert (t.enable_calibrator, t.enable_encoder_calibrator, t.calibrator_type, t.calibrator_cache_type,
          t.taylorseer_order) == (True, True, "taylorseer", "residual", 1)
  assert t.to_kwargs() == {"n_derivatives": 1}
  q = cd.QuantizeConfig()
  assert q.quant_type == "float8_per_row" and q.exclude_layers == ["embedder", "embed", "modulation", "mod"]
  assert q.regional_quantize is True and q.per_tensor_fallback is True
  with pytest.raises(NotImplementedError):
    cd.QuantizeConfig(quant_type="int8_per_row")
  c.update(Fn_compute_blocks=4, residual_diff_threshold=None)
  assert c.Fn_compute_blocks == 4 and c.residual_diff_threshold == 0.08
  assert cd.DBCacheConfig().empty(num_inference_steps=5).Fn_compute_blocks is None


def test_ulysses_exchange_mode_selection(monkeypatch):
  """Without a process group the attention exchange falls back to collectives; explicit choices win and
  unknown names are refused."""
  import cache_dit_b200 as cd
  monkeypatch.delenv("CACHE_DIT_B200_ULYSSES_EXCHANGE", raising=False)
  assert cd.ParallelismConfig(ulysses_size=2).exchange_mode() == "nccl"
  assert cd.ParallelismConfig(ulysses_size=2, parallel_kwargs={"exchange": "peer"}).exchange_mode() == "peer"
  monkeypatch.setenv("CACHE_DIT_B200_ULYSSES_EXCHANGE", "peer")
  assert cd.ParallelismConfig(ulysses_size=2).exchange_mode() == "peer"
  monkeypatch.setenv("CACHE_DIT_B200_ULYSSES_EXCHANGE", "carrier-pigeon")
  import pytest
  with pytest.raises(ValueError):
    cd.ParallelismConfig(ulysses_size=2).exchange_mode()


def test_token_views_rejoin_without_copy():
  import torch
  from cache_dit_b200.synthetic.layers import join_tokens, split_tokens
  x = torch.arange(2 * 7 * 3, dtype=torch.float32).reshape(2, 7, 3)
  a, b = split_tokens(x, 3)
  assert join_tokens(a, b) is x
  # any other pair is concatenated
  c = b.clone()
  y = join_tokens(a, c)
  assert y is not x and torch.equal(y, x)
  assert torch.equal(join_tokens(b, a), torch.cat([b, a], dim=1))
