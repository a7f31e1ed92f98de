"""Writes fp8_torch_cuda.npz: what PyTorch's own CUDA ops give for the FP8 per-row linear on small seeded inputs.

Run on a machine with a CUDA GPU whose `torch._scaled_mm` accepts row-wise scales (sm_89 and later):

    python tests/golden/make_fp8_torch_fixture.py --out tests/golden/fp8_torch_cuda.npz

The reference reaches this arithmetic through torchao (absent here) and `torch._scaled_mm`
(src/cache_dit/quantization/torchao/_scaled_mm.py:72-91).  This script evaluates the published rule with
torch ops on the GPU, the library product included, so the CPU suite can hold the numpy restatement
against values PyTorch itself produced:
  scale = amax(|x|, row) / 448 (1 for an all-zero row), q = e4m3fn(clamp(x / scale, -448, 448)),
  out   = _scaled_mm(q_a, q_w^T, scale_a [M,1], scale_b [1,N], bias, out_dtype=bf16).
Tensors are stored as raw bits (bf16 -> uint16, e4m3 -> uint8) so that nothing is rounded on the way.
"""
import argparse

import numpy as np
import torch

CASES = [  # name, M, K, N, bias
    ("small_bias", 48, 256, 64, True),
    ("odd_rows", 33, 512, 96, False),
    ("wide", 16, 2048, 48, True),
]


def quantize_rows(x: torch.Tensor):
  amax = x.abs().amax(dim=1).float()
  scale = amax / 448.0
  scale = torch.where(scale == 0, torch.ones_like(scale), scale)
  q = (x.float() / scale[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
  return q, scale


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--out", required=True)
  args = ap.parse_args()
  dev = torch.device("cuda:0")
  out = {}
  for i, (name, M, K, N, bias) in enumerate(CASES):
    g = torch.Generator().manual_seed(1234 + i)
    x = torch.randn(M, K, generator=g) * torch.exp(0.5 * torch.randn(M, 1, generator=g))
    x[1] = 0.0  # an all-zero token: scale 1, codes 0
    x[2, 5] = 300.0  # an outlier sets the row's scale
    w = 0.03 * torch.randn(N, K, generator=g)
    b = torch.randn(N, generator=g) if bias else None
    x, w = x.to(torch.bfloat16).to(dev), w.to(torch.bfloat16).to(dev)
    b = b.to(torch.bfloat16).to(dev) if bias else None
    aq, sa = quantize_rows(x)
    wq, sw = quantize_rows(w)
    y = torch._scaled_mm(aq, wq.t(), scale_a=sa.view(M, 1), scale_b=sw.view(1, N), bias=b, out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    out[f"{name}.x"] = x.view(torch.int16).cpu().numpy().view(np.uint16)
    out[f"{name}.w"] = w.view(torch.int16).cpu().numpy().view(np.uint16)
    if bias:
      out[f"{name}.bias"] = b.view(torch.int16).cpu().numpy().view(np.uint16)
    out[f"{name}.a_codes"] = aq.view(torch.uint8).cpu().numpy()
    out[f"{name}.a_scale"] = sa.cpu().numpy()
    out[f"{name}.w_codes"] = wq.view(torch.uint8).cpu().numpy()
    out[f"{name}.w_scale"] = sw.cpu().numpy()
    out[f"{name}.out"] = y.view(torch.int16).cpu().numpy().view(np.uint16)
  out["meta"] = np.array([torch.__version__, torch.cuda.get_device_name(0)])
  np.savez_compressed(args.out, **out)
  print("wrote", args.out, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
  main()
