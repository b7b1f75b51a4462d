import math, torch, sys
sys.path.insert(0,'.')
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
