"""Small launches of every kernel for an ncu --set full capture (a few hundred MB on the device)."""
import sys, torch
sys.path.insert(0, __import__('os').path.dirname(__import__('os').path.dirname(__import__('os').path.abspath(__file__))))
from cache_dit_b200 import _native as nat
nat.lib()
dev = 'cuda'
S, C = 8192, 3072            # bf16 [1, 8192, 3072] = 50 MB per tensor: 2-5 tensors per kernel > L2
mk = lambda: torch.randn(1, S, C, device=dev).to(torch.bfloat16)
h, h0, p, d = mk(), mk(), mk(), mk()
o, o2 = torch.empty_like(h), torch.empty_like(h)
means = torch.zeros(2, device=dev)
flush = torch.empty(1 << 28, dtype=torch.uint8, device=dev)
M, K, N = 4608, 3072, 12288
x = torch.randn(M, K, device=dev).to(torch.bfloat16)
w = (0.02 * torch.randn(N, K, device=dev)).to(torch.bfloat16)
aq = torch.empty(M, K, device=dev, dtype=torch.float8_e4m3fn); sa = torch.empty(M, device=dev)
wq = torch.empty(N, K, device=dev, dtype=torch.float8_e4m3fn); sw = torch.empty(N, device=dev)
out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
nat.fp8_quant_rows(w, wq, sw)
for rep in range(2):
    flush.zero_()
    nat.rel_l1(h, None, p, None, means)
    flush.zero_()
    nat.rel_l1(h, h0, p, o, means)
    flush.zero_()
    nat.taylor_apply(h, [p, d], [1.0, 1.0], [1.0, 2.0], True, o)
    flush.zero_()
    nat.taylor_update(h, h0, [p], [o, o2], 1, 3.0)
    flush.zero_()
    nat.fp8_quant_rows(x, aq, sa)
    flush.zero_()
    nat.fp8_gemm_rowscaled(aq, sa, wq, sw, None, out)
torch.cuda.synchronize()
print('ok', means.tolist(), nat.gemm_device_status(torch.device('cuda:0')))
