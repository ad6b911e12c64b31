"""``python -m renee_b200.utils.memory_plan --labels 100000000 --gpus 8 --batch 1024 --seq 32``: per-GPU device
memory of a training configuration, without a GPU.

The plan is not a formula kept beside the code: it builds the real ``XCTrainer`` (flat encoder buffers,
activation arena, classifier shard, momentum, scratch, staging buffers) on PyTorch's ``meta`` device in guard
mode and adds up what the framework's allocation sites asked for, so it follows the code when the code changes
(``tests/test_memory_plan.py`` checks it against a real CPU instantiation).  Added on top: the symmetric
peer-memory buffers of the fused collectives (computed from the same shapes ``parallel/fused.py`` uses) and a
fixed allowance for what the framework does not allocate itself (CUDA context, library workspaces, allocator
slack).  For comparison the line ``reference_layout_gb`` gives the classifier state of the reference's layout on the
same shard: fp32 master + fp32 gradient + fp32 momentum + the per-step fp16 copy (dl_base.py:185, 562, 625-633).
"""
from __future__ import annotations

import argparse
import collections
import json

import torch

HBM_BYTES = 180e9                 # B200
OTHER_ALLOWANCE_BYTES = 3e9       # CUDA context + cuBLAS/NCCL workspaces + caching-allocator slack (not ours)


def plan(labels: int, gpus: int, global_batch: int, seq: int, enc_cfg=None, fp16xfc: bool = True,
         fp32encoder: bool = False, bottleneck_dims: int = 0, accum: int = 1, pooling: str = "cls") -> dict:
    from ..models.encoder import EncoderConfig
    from ..parallel.dist import DistContext
    from ..train import TrainConfig, XCTrainer
    from . import guard
    from .sharding import shard_labels

    enc_cfg = enc_cfg or EncoderConfig()
    if global_batch % gpus:
        raise ValueError("the global batch must be a multiple of the number of GPUs")
    b = global_batch // gpus
    sh = shard_labels(labels, gpus)
    cfg = TrainConfig(batch_size=b, epochs=1, seed=0, dropout=0.5, lr1=0.05, lr2=1e-5, warmup=10, wd1=1e-4,
                      noloss=True, fp16xfc=fp16xfc, fp32encoder=fp32encoder, maxlen=seq, pooling=pooling,
                      bottleneck_dims=bottleneck_dims, accum=accum)
    ctx = DistContext(rank=0, world_size=gpus, local_rank=0, device=torch.device("meta"), backend=None)
    by_kind: collections.Counter = collections.Counter()
    with guard.enabled_for_test():
        tr = XCTrainer(cfg, enc_cfg, sh, ctx, steps_per_epoch=100)
        tr.encoder._alloc(b + 1, seq)            # the trainer's staging buffers hold b + 1 rows (ragged final batch)
        tr.xfc.scratch(global_batch)
        for e in guard._registry:
            kind = e.name.rsplit(".", 1)[0] if not e.name.startswith("encoder.act") else "encoder.activations"
            if e.name.startswith("xfc."):
                kind = e.name
            by_kind[kind] += e.hi - e.lo
        D = tr.encoder.out_dims
        n_enc = tr.encoder.numel
        act_bytes = 4 if fp32encoder else 2
    if gpus > 1:
        rows = global_batch + gpus
        # parity double-buffered X (fp16) and dX partials (fp32), flags; the gradient and bf16 parameter copies move
        # from private to symmetric memory (already counted under "encoder"), plus the fp32 slice sum of the optimizer
        by_kind["peer.X_dX"] = 2 * rows * D * (2 + 4) + 128 * 4
        by_kind["peer.optimizer_slice_sum"] = (n_enc // gpus + 16) * 4
    ours = sum(by_kind.values())
    ls = sh.labels_per_rank
    ref_xfc = ls * D * (4 + 4 + 4 + (2 if fp16xfc else 0)) + (global_batch // max(accum, 1)) * ls * (2 if fp16xfc else 4)
    return {
        "config": {"labels": labels, "gpus": gpus, "global_batch": global_batch, "seq": seq, "labels_per_gpu": ls,
                   "fp16xfc": fp16xfc, "activation_bytes": act_bytes},
        "per_gpu_gb": {k: round(v / 1e9, 3) for k, v in sorted(by_kind.items(), key=lambda kv: -kv[1])},
        "framework_total_gb": round(ours / 1e9, 2),
        "with_allowance_gb": round((ours + OTHER_ALLOWANCE_BYTES) / 1e9, 2),
        "fits_180gb": bool(ours + OTHER_ALLOWANCE_BYTES < HBM_BYTES),
        "reference_layout_gb": {"classifier_state_and_logits": round(ref_xfc / 1e9, 2)},
    }


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--labels", type=int, required=True)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--batch", type=int, default=256, help="global batch")
    ap.add_argument("--seq", type=int, default=32)
    ap.add_argument("--fp32xfc", action="store_true")
    ap.add_argument("--fp32encoder", action="store_true")
    ap.add_argument("--bottleneck-dims", type=int, default=0)
    ap.add_argument("--accum", type=int, default=1)
    a = ap.parse_args(argv)
    print(json.dumps(plan(a.labels, a.gpus, a.batch, a.seq, fp16xfc=not a.fp32xfc, fp32encoder=a.fp32encoder,
                          bottleneck_dims=a.bottleneck_dims, accum=a.accum), indent=1))


if __name__ == "__main__":
    main()
