"""A test-only FP8 linear made of PyTorch library ops: the independent arm for end-to-end FP8 checks.

It does what the reference's float8 per-row inference path does after torchao has quantized the operands:
`scale = amax / 448 -> where(== 0, 1)`, `q = clamp(x / scale, +-448).to(float8_e4m3fn)` with torch ops, then
`torch._scaled_mm(a_q, w_q.t(), scale_a [M, 1], scale_b [1, N], bias, out_dtype=bf16)` - the call at
src/cache_dit/quantization/torchao/_scaled_mm.py:72-91.  None of this package's kernels is involved, and since a
model holding these modules has no `Float8RowwiseLinear`, the block glue around them (adaLN LayerNorm, GELU,
concatenations) runs as eager PyTorch too.
"""
import torch

E4M3_MAX = 448.0


def quantize_rows_torch(x2d: torch.Tensor):
  scale = x2d.abs().amax(dim=1, keepdim=True).float() / E4M3_MAX
  scale = torch.where(scale == 0, torch.ones_like(scale), scale)
  q = (x2d.float() / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
  return q, scale


class LibraryFloat8Linear(torch.nn.Module):

  def __init__(self, linear: torch.nn.Linear):
    super().__init__()
    w = linear.weight.detach().to(torch.bfloat16)
    self.in_features, self.out_features = w.shape[1], w.shape[0]
    w_q, w_scale = quantize_rows_torch(w)
    self.register_buffer("w_q", w_q)                      # [N, K] e4m3
    self.register_buffer("w_scale", w_scale.t().contiguous())  # [1, N] fp32
    self.register_buffer("bias", None if linear.bias is None else linear.bias.detach().to(torch.bfloat16))

  def forward(self, x):
    x2 = x.reshape(-1, self.in_features).to(torch.bfloat16)
    a_q, a_scale = quantize_rows_torch(x2)
    out = torch._scaled_mm(a_q, self.w_q.t(), scale_a=a_scale, scale_b=self.w_scale, bias=self.bias,
                           out_dtype=torch.bfloat16)
    return out.view(*x.shape[:-1], self.out_features)


def swap_repeated_block_linears(model: torch.nn.Module, exclude=("embedder", "embed", "modulation", "mod")) -> int:
  """Replace the nn.Linear layers the product path would make FP8 (inside the repeated block classes, names
  without an excluded pattern; block-relative names as in the reference) by `LibraryFloat8Linear`."""
  repeated = set(getattr(model, "_repeated_blocks", []))
  count = 0

  def walk(root, prefix):
    nonlocal count
    for name, child in list(root.named_children()):
      full = f"{prefix}.{name}" if prefix else name
      if isinstance(child, torch.nn.Linear):
        k, n = child.in_features, child.out_features
        if not any(p in full for p in exclude) and k % 16 == 0 and n % 16 == 0:
          setattr(root, name, LibraryFloat8Linear(child))
          count += 1
      else:
        walk(child, full)

  for _, sub in list(model.named_modules()):
    if sub.__class__.__name__ in repeated:
      walk(sub, "")
  return count
