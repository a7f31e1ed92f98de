"""Load the committed golden fixtures (written by tests/golden/make_golden.py)."""
import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_json(name):
  with open(os.path.join(GOLDEN, name)) as f:
    return json.load(f)


_npz = {}


def load_arrays(name, prefix):
  if name not in _npz:
    _npz[name] = np.load(os.path.join(GOLDEN, name))
  z = _npz[name]
  return {k[len(prefix) + 1:]: z[k] for k in z.files if k.startswith(prefix + "/")}


def compare_trace(got: dict, want: dict, diff_rtol: float = 1e-3):
  """Masks, step indices and integer counters bit-exact; diffs within `diff_rtol` relative."""
  assert got["hits"] == want["hits"], (got["hits"], want["hits"])
  assert got["step_index"] == want["step_index"]
  gs, ws = got["stats"], want["stats"]
  for k in ("cached_steps", "cfg_cached_steps", "accumulated_cached_steps",
            "cfg_accumulated_cached_steps", "accumulated_executed_steps",
            "accumulated_transformer_executed_steps"):
    assert gs[k] == ws[k], (k, gs[k], ws[k])
  for k in ("residual_diffs", "cfg_residual_diffs"):
    assert sorted(gs[k]) == sorted(ws[k]), (k, sorted(gs[k]), sorted(ws[k]))
    for step, w in ws[k].items():
      g = gs[k][step]
      assert abs(g - w) <= diff_rtol * abs(w) + 1e-12, (k, step, g, w)


def compare_digests(got: dict, want: dict, rtol: float, atol: float):
  assert sorted(got) == sorted(want)
  for k, w in want.items():
    g = got[k]
    np.testing.assert_allclose(g["samples"], w["samples"], rtol=rtol, atol=atol, err_msg=k)
    assert abs(g["abs_sum"] - w["abs_sum"]) <= 1e-5 * abs(w["abs_sum"]), (k, g, w)
    assert abs(g["sum"] - w["sum"]) <= 1e-5 * abs(w["abs_sum"]), (k, g, w)
