"""``python -m renee_b200.utils.phase_report [--config 131k-s32]``: device-timed phases of the training
step on one GPU (eager launches, CUDA events; see ``XCTrainer.profile_step``)."""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch


def main(argv=None) -> None:
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    from bench import CONFIGS
    from renee_b200.data import xcrepo
    from renee_b200.data.collate import XCCollator
    from renee_b200.data.synthetic import SyntheticSpec, SyntheticXC
    from renee_b200.models.encoder import EncoderConfig
    from renee_b200.parallel.dist import DistContext
    from renee_b200.train import TrainConfig, XCTrainer
    from renee_b200.utils.sharding import shard_labels

    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="131k-s32", choices=sorted(CONFIGS))
    ap.add_argument("--repeats", type=int, default=5)
    a = ap.parse_args(argv)
    c = CONFIGS[a.config]
    dev = torch.device("cuda", 0)
    B = c["batch"]
    spec = SyntheticSpec(num_labels=c["labels"], seq_len=c["seq"], len_lo=c["len_lo"], len_hi=c["seq"],
                         poisson_lam=c["lam"], zipf_s=c["zipf"], seed=0)
    ids, mask, lab = SyntheticXC(spec).rows(np.arange(2 * B))
    ds = xcrepo.InMemoryDataset(ids, mask, lab)
    sh = shard_labels(c["labels"], 1)
    cfg = TrainConfig(batch_size=B, epochs=1, seed=0, dropout=c["dropout"], lr1=0.05, lr2=1e-5, warmup=5000, wd1=1e-4,
                      noloss=True, fp16xfc=True, maxlen=c["seq"], pooling="cls", cuda_graph=False)
    tr = XCTrainer(cfg, EncoderConfig(), sh, DistContext(device=dev), steps_per_epoch=1000)
    coll = XCCollator(sh, ds, 0, 1, B, True)
    batches = [coll(np.arange(i * B, (i + 1) * B)).pin() for i in range(2)]
    for i in range(3):
        tr.train_step(batches[i % 2])
    acc: dict = {}
    for i in range(a.repeats):
        for k, v in tr.profile_step(batches[i % 2]).items():
            acc[k] = acc.get(k, 0.0) + v / a.repeats
    acc["total"] = sum(acc.values())
    print(json.dumps({"config": a.config, "phases_ms": {k: round(v, 4) for k, v in acc.items()}}))


if __name__ == "__main__":
    main()
