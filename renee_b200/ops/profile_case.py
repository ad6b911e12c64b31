"""Small-case launcher for profiling: ``python renee_b200/ops/profile_case.py [repeats]`` launches each
hand-written kernel once per repeat at the headline benchmark's shapes (encoder: T=8192 tokens, H=768,
F=3072, 256 sequences of 32 tokens and 64 sequences of 128 tokens, 12 heads; classifier: B=256, D=768, a 16384-label shard = the per-GPU
shard at 8 GPUs; AdamW over 66.4M parameters).  About 1.5 GB on the device, a few milliseconds of work:
sized so that ``ncu --set full`` on it ends by itself within a minute or two."""
import os, sys, torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from renee_b200 import ops
from renee_b200.ops import cuda as cu
from renee_b200.optim.hparams import HP, HyperParams
dev = torch.device("cuda", 0)
T, H, F = 8192, 768, 3072
dt = torch.bfloat16
rng = ops.StepRNG(1, torch.tensor([1], dtype=torch.int32, device=dev))
x = torch.randn(T, H, device=dev).to(dt); pre = torch.randn(T, H, device=dev).to(dt)
gam = torch.ones(H, device=dev, dtype=dt); mean = torch.zeros(T, device=dev); rstd = torch.ones(T, device=dev)
o1, o2 = torch.empty_like(x), torch.empty_like(x)
dg, db, dbias = [torch.empty(H, device=dev, dtype=dt) for _ in range(3)]
xf = torch.randn(T, F, device=dev).to(dt); da = torch.randn(T, F, device=dev).to(dt); bf = torch.zeros(F, device=dev, dtype=dt)
dxf = torch.empty_like(xf); dbf = torch.empty(F, device=dev, dtype=dt)
q = torch.randn(T, 3 * H, device=dev).to(dt); dq = torch.empty(3 * H, device=dev, dtype=dt)
B, D, L = 256, 768, 16384
X = (torch.randn(B, D, device=dev) * 0.5).half(); W = (torch.randn(L, D, device=dev) * 0.05).half(); M = torch.zeros_like(W)
Gt = torch.zeros(L, B, dtype=torch.float16, device=dev); dX = torch.zeros(B, D, device=dev)
hp = HyperParams(dev); hp.buf[HP.LR_XFC] = 0.05
n0 = torch.zeros(1, dtype=torch.int32, device=dev); e = torch.zeros(1, dtype=torch.int32, device=dev)
b_, S_, nh_ = 256, 32, 12
mask = torch.ones(b_, S_, dtype=torch.int32, device=dev)
aws = ops.attention_workspace(b_, S_, nh_, dev, dt)
mask_long = torch.ones(64, 128, dtype=torch.int32, device=dev)
aws_long = ops.attention_workspace(64, 128, nh_, dev, dt)
bq = torch.zeros(3 * H, device=dev, dtype=dt); ctx = torch.empty(T, H, device=dev, dtype=dt); dqkv = torch.empty_like(q)
Zt = torch.empty(B, L, device=dev); ov = torch.empty(B, 100, device=dev); oi = torch.empty(B, 100, dtype=torch.int32, device=dev)
n_ad = 66_400_000 // 1024 * 1024
p32 = torch.zeros(n_ad, device=dev); am = torch.zeros_like(p32); av = torch.zeros_like(p32)
ag = torch.zeros(n_ad, device=dev, dtype=dt); p16 = torch.zeros(n_ad, device=dev, dtype=dt); hp.buf[HP.LR_ENC] = 1e-5
for it in range(int(sys.argv[1]) if len(sys.argv) > 1 else 1):
    ops.bias_dropout_add_ln_bwd(x, pre, gam, mean, rstd, 0.1, rng, 3, dg, db, dbias, o1, o2)
    ops.bias_gelu_bwd(da, xf, bf, dbf, dxf)
    ops.bias_gelu_fwd(xf, bf, dxf)
    cu.colsum(q, dq)
    cu.xfc_logits_grad(W, X, Gt, B, e, e, n0, 0)
    cu.xfc_dx(Gt, B, W, B, dX, hp.buf, cu.dx_splits(B, D, L))
    cu.xfc_dw_sgd(Gt, B, X, W, M, hp.buf, 0.9, 1e-4)
    ops.attention_fwd(q, bq, mask, nh_, 0.1, rng, 4, ctx, aws)
    ops.attention_bwd(ctx, q, bq, mask, nh_, 0.1, rng, 4, aws, dqkv, dq)
    ops.attention_fwd(q, bq, mask_long, nh_, 0.1, rng, 4, ctx, aws_long)
    ops.attention_bwd(ctx, q, bq, mask_long, nh_, 0.1, rng, 4, aws_long, dqkv, dq)
    cu.xfc_logits_grad(W, X, None, L, None, None, None, 0, raw_out=Zt)
    cu.topk_rows(Zt, L, 100, 0, ov, oi)
    ops.adamw_step(p32, am, av, ag, p16, hp, 0.9, 0.999, 1e-6, 0.01, n_ad // 2)
torch.cuda.synchronize()
cu.check_status()
print("ok")
