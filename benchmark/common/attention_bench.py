"""Times the fused attention forward and backward on the GPT-2 XL head layout (B x 64 heads x 1024 x 25 by default; env B, DH).
"""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import torch
from cubework_b200 import ops
B, H, T, dh = int(os.environ.get("B", 8)), 64, 1024, int(os.environ.get("DH", 25))
torch.manual_seed(0)
qkv = (torch.randn(B, T, H, 3 * dh, device="cuda") * 0.5).bfloat16().requires_grad_(True)
kb = torch.zeros(B, T, device="cuda")
for it in range(3):
    out = ops.attention_packed(qkv, True, kb)
    out.backward(torch.ones_like(out))
torch.cuda.synchronize()
e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
e[0].record(); out = ops.attention_packed(qkv, True, kb); e[1].record(); out.backward(torch.ones_like(out)); e[2].record()
torch.cuda.synchronize()
print("fwd ms", e[0].elapsed_time(e[1]), "bwd ms", e[1].elapsed_time(e[2]))
