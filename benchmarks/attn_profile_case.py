"""Small attention case for profiler captures: causal forward + backward, T = 16384, 8 heads, head_dim 128, twice.

    python benchmarks/attn_profile_case.py        (small enough for a profiler capture: 3 kernels per pass, a few GB)
"""
import math, torch, sys
import os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from odysseus_transformer_b200.ops import native
native.set_backend("fused"); lib=native.lib()
T,H=16384,8
q,k,v,do=[(torch.randn(T,H,128,device='cuda')*0.5).bfloat16() for _ in range(4)]
sc=1/math.sqrt(128)
for _ in range(2):
    o,lse=lib.attn_fwd(q,k,v,True,sc)
    lib.attn_bwd(do,q,k,v,o,lse,True,sc)
torch.cuda.synchronize()
print("ok")
