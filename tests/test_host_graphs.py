"""Host logic of the CUDA-graph segment runner that needs no GPU: nest flattening, key building and
the eager fall-back for tensors it cannot capture."""
import torch

from cache_dit_b200.caching.block_graphs import BlockGraphRunner, _flatten, _rebuild


def test_flatten_rebuild_round_trip():
  a, b, c = torch.zeros(2), torch.ones(3), torch.full((1, ), 2.0)
  nest = (a, None, (b, [c, 5]), {"k": a, "flag": True})
  flat = []
  spec = _flatten(nest, flat)
  assert [t.data_ptr() for t in flat] == [a.data_ptr(), b.data_ptr(), c.data_ptr(), a.data_ptr()]
  back = _rebuild(spec, flat)
  assert back[0] is a and back[1] is None and back[2][0] is b and back[2][1][0] is c and back[2][1][1] == 5
  assert isinstance(back[2][1], list) and back[3]["k"] is a and back[3]["flag"] is True
  hash(spec)


def test_cpu_tensors_run_eagerly_and_are_never_captured():
  r = BlockGraphRunner(warmup_calls=1)
  calls = []

  def fn(x, k):
    calls.append(1)
    return x + k

  x = torch.arange(4.0)
  for _ in range(5):
    assert torch.equal(r.run(("t", ), fn, (x, 2)), x + 2)
  assert len(calls) == 5 and r.captures == 0 and r.replays == 0 and not r.segments


def test_unhashable_constant_runs_eagerly():
  r = BlockGraphRunner()
  out = r.run(("t", ), lambda x, s: x, (torch.zeros(1), {1, 2}))
  assert out.shape == (1, )
