"""The `torch.library` operators over the FP8 kernels, as far as a machine without a GPU can tell: schema,
shape propagation through the fake implementations, dtype ids, no CPU implementation.

The reference registers its FP8 product the same way (src/cache_dit/quantization/torchao/_scaled_mm.py:38-43,
94-137: schema, dtype ids {fp16: 0, bf16: 1, fp32: 2}, fake impl returning (*a.shape[:-1], b.shape[-1]))."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import cache_dit_b200  # noqa: F401  (registers the operators)
from cache_dit_b200.quantization import ops


def test_schema_is_the_reference_operators():
  schema = str(torch.ops.cache_dit_b200.float8_inference_scaled_mm.default._schema)
  assert schema == ("cache_dit_b200::float8_inference_scaled_mm(Tensor a_data, Tensor a_scale, Tensor b_data, "
                    "Tensor b_scale, Tensor? bias, int out_dtype_id, bool use_fast_accum) -> Tensor")


def test_output_dtype_ids():
  assert [ops.encode_output_dtype(d) for d in (torch.float16, torch.bfloat16, torch.float32)] == [0, 1, 2]
  assert ops.decode_output_dtype(1) is torch.bfloat16
  with pytest.raises(ValueError):
    ops.encode_output_dtype(torch.float64)
  with pytest.raises(ValueError):
    ops.decode_output_dtype(3)


@pytest.mark.parametrize("lead", [(10, ), (2, 5), (1, 3, 4)])
def test_fake_implementations_carry_shapes(lead):
  rows = 1
  for n in lead:
    rows *= n
  with FakeTensorMode():
    a = torch.empty(*lead, 64, dtype=torch.float8_e4m3fn, device="cuda")
    sa = torch.empty(rows, 1, dtype=torch.float32, device="cuda")
    w = torch.empty(48, 64, dtype=torch.float8_e4m3fn, device="cuda")
    sw = torch.empty(1, 48, dtype=torch.float32, device="cuda")
    y = ops.float8_inference_scaled_mm(a, sa, w.t(), sw, None, torch.bfloat16)
    assert tuple(y.shape) == (*lead, 48) and y.dtype is torch.bfloat16 and y.device.type == "cuda"
    y32 = ops.float8_inference_scaled_mm(a, sa, w.t(), sw, None, torch.float32)
    assert y32.dtype is torch.float32  # the fake follows the id; the CUDA kernel itself writes bf16 only
    q, s = ops.float8_quantize_rows(torch.empty(*lead, 64, dtype=torch.bfloat16, device="cuda"))
    assert tuple(q.shape) == (*lead, 64) and q.dtype is torch.float8_e4m3fn
    assert tuple(s.shape) == (*lead, 1) and s.dtype is torch.float32


def test_there_is_no_cpu_implementation():
  with pytest.raises(NotImplementedError):
    ops.float8_quantize_rows(torch.zeros(2, 16, dtype=torch.bfloat16))
  a = torch.zeros(2, 16, dtype=torch.float8_e4m3fn)
  with pytest.raises(NotImplementedError):
    ops.float8_inference_scaled_mm(a, torch.ones(2, 1), a.t(), torch.ones(1, 2))


def test_latched_device_status_becomes_an_exception():
  """The host image of the per-device mailbox: word 2 = FP8 GEMM status, word 5 = peer-exchange status.
  Either non-zero value must stop the step (CDB_ERR_DEVICE_TIMEOUT), zero must not."""
  import pytest
  from cache_dit_b200 import _native as nat
  nat.raise_on_device_status(0, 0)
  with pytest.raises(nat.DeviceTimeoutError, match="FP8 GEMM"):
    nat.raise_on_device_status(13, 0)
  with pytest.raises(nat.DeviceTimeoutError, match="peer 2"):
    nat.raise_on_device_status(0, 3)
  assert issubclass(nat.DeviceTimeoutError, RuntimeError)
  assert nat.MAILBOX_GEMM_STATUS == 2 and nat.MAILBOX_PEER_STATUS == 5 and nat.MAILBOX_WORDS * 4 == 32
