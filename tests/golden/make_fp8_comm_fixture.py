"""Fixture for the FP8 head/token exchange format, produced by the REFERENCE's own Triton kernels on a B200.

The reference quantizes what crosses the wire under `ulysses_float8` with four Triton kernels
(src/cache_dit/kernels/triton/_float8_comm.py:5-148, launched by the ops registered at
src/cache_dit/kernels/triton/_ops_registery.py:50-180 and called from
src/cache_dit/distributed/core/_distributed_primitives.py:741-813).  They need a GPU, and the reference tree
does not exist on the GPU machine, so this script works in two steps:

  where a checkout of the reference exists (no GPU needed):
      python tests/golden/make_fp8_comm_fixture.py --stage --reference /path/to/cache-dit
    places unmodified copies of the three Triton source files the ops need under baseline/_ref/ (git-ignored: not part
    of this repository's history; a `pip install --target baseline/_ref` of the reference fails here because its build
    needs setuptools-scm, which is not installed);
  on a B200:
      python tests/golden/make_fp8_comm_fixture.py [--out FILE]
    imports the staged ops, runs them on small seeded inputs and stores inputs (bf16 bit patterns) and outputs
    (raw bytes) as tests/golden/fp8_comm_reference.npz, which is committed.

Cases (all bf16 inputs, seeded):
  qkv.<name>  x [B, S, W, N, D] -> fp8_comm_qkv_permute_quant -> [W, S, B, N, D + 4] bytes (D codes + fp32 scale per
              (token, head)); and for every w the receiver side fp8_comm_qkv_permute_dequant([S, B, N, D + 4]) -> [B, S, N, D]
  o.<name>    x [R, D] -> fp8_comm_per_token_quant -> [R, D + 2] bytes (D codes + bf16 scale per row);
              fp8_comm_per_token_dequant -> [R, D]
"""
import argparse
import importlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
STAGED = os.path.join(ROOT, "baseline", "_ref", "cache_dit_triton_kernels")
REFERENCE_SUBDIR = os.path.join("src", "cache_dit", "kernels", "triton")
FILES = ["_float8_comm.py", "_merge_attn_states.py", "_ops_registery.py"]

QKV_CASES = {"w2_d64": (1, 40, 2, 2, 64), "w4_d128": (2, 24, 4, 2, 128), "w8_d128": (1, 33, 8, 3, 128)}
O_CASES = {"d64": (160, 64), "d128": (2 * 24 * 8, 128)}


def stage(reference_root):
  os.makedirs(STAGED, exist_ok=True)
  for name in FILES:
    shutil.copyfile(os.path.join(reference_root, REFERENCE_SUBDIR, name), os.path.join(STAGED, name))
  with open(os.path.join(STAGED, "__init__.py"), "w") as f:
    f.write("")
  print("staged", FILES, "->", STAGED)


def reference_ops():
  """torch.ops.cache_dit_triton_ops of the staged reference files (None if they are not staged)."""
  if not os.path.exists(os.path.join(STAGED, "_ops_registery.py")):
    return None
  import torch
  parent = os.path.dirname(STAGED)
  if parent not in sys.path:
    sys.path.insert(0, parent)
  importlib.import_module("cache_dit_triton_kernels._ops_registery")
  return torch.ops.cache_dit_triton_ops


def seeded_inputs():
  """The inputs of every case (torch bf16 CPU tensors).  Row magnitudes spread over two decades, one all-zero
  head (the scale floors apply) and a few outliers."""
  import torch
  g = torch.Generator().manual_seed(1234)
  inputs = {}
  for name, shape in QKV_CASES.items():
    x = torch.randn(*shape, generator=g) * torch.exp(1.5 * torch.randn(*shape[:-1], 1, generator=g))
    x[0, 3, 0, 0] = 0
    x[0, 5, 1, 1, 7] = 300.0
    inputs[f"qkv.{name}"] = x.to(torch.bfloat16)
  for name, shape in O_CASES.items():
    x = torch.randn(*shape, generator=g) * torch.exp(1.5 * torch.randn(shape[0], 1, generator=g))
    x[2] = 0
    x[4] = 1e-6 * torch.randn(shape[1], generator=g)  # below the 1e-4 floor of the row maximum
    inputs[f"o.{name}"] = x.to(torch.bfloat16)
  return inputs


def generate(out_path):
  import numpy as np
  import torch
  ops = reference_ops()
  if ops is None:
    raise SystemExit("the reference's Triton files are not staged: run with --stage where the reference tree exists")
  bits = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
  raw = lambda t: t.contiguous().view(torch.uint8).cpu().numpy()
  arrays = {}
  for key, x in seeded_inputs().items():
    xd = x.cuda()
    arrays[f"{key}.x"] = bits(xd)
    if key.startswith("qkv."):
      q = ops.fp8_comm_qkv_permute_quant(xd)  # [W, S, B, N, D + 4]
      arrays[f"{key}.wire"] = raw(q)
      deq = [ops.fp8_comm_qkv_permute_dequant(q[w].contiguous()) for w in range(q.shape[0])]  # each [B, S, N, D]
      arrays[f"{key}.dequant"] = bits(torch.stack(deq, dim=0))
    else:
      q = ops.fp8_comm_per_token_quant(xd)  # [R, D + 2]
      arrays[f"{key}.wire"] = raw(q)
      arrays[f"{key}.dequant"] = bits(ops.fp8_comm_per_token_dequant(q))
  torch.cuda.synchronize()
  os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
  np.savez_compressed(out_path, **arrays)
  print("wrote", out_path, {k: v.shape for k, v in arrays.items()})


if __name__ == "__main__":
  ap = argparse.ArgumentParser()
  ap.add_argument("--stage", action="store_true")
  ap.add_argument("--reference", help="root of a checkout of the reference (with --stage)")
  ap.add_argument("--out", default=os.path.join(HERE, "fp8_comm_reference.npz"))
  a = ap.parse_args()
  if a.stage:
    if not a.reference:
      ap.error("--stage needs --reference /path/to/cache-dit")
    stage(a.reference)
  else:
    generate(a.out)
