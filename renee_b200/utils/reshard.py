"""Consolidate or re-shard per-rank state dicts.

The reference writes one ``{name}_{rank}_state_dict.pt`` per rank, each holding a copy of the encoder and
that rank's ``xfc_weight [Ls, D]`` rows (dl_base.py:448-451), so a model trained on G GPUs can only be
loaded on G GPUs.  These helpers stitch the classifier shards back together (dropping the padded rows)
and cut them again for a different world size, following the padding rule of
:func:`renee_b200.utils.sharding.shard_labels`.

    python -m renee_b200.utils.reshard --dir OUT --name renee-exp --from-world 8 --to-world 2 --labels 131072
"""
from __future__ import annotations

import argparse
import os

import torch

from .sharding import shard_labels


def consolidate(shards: list[dict], num_labels: int) -> dict:
    """Per-rank state dicts (rank order) → one state dict with the full ``xfc_weight [L, D]``."""
    W = torch.cat([sd["xfc_weight"] for sd in shards], dim=0)[:num_labels]
    out = {k: v for k, v in shards[0].items() if k != "xfc_weight"}
    out["xfc_weight"] = W.contiguous()
    return out


def reshard(full: dict, num_labels: int, world_size: int) -> list[dict]:
    """Consolidated state dict → ``world_size`` per-rank dicts (padded rows are zero)."""
    sh = shard_labels(num_labels, world_size)
    W = full["xfc_weight"]
    pad = torch.zeros(sh.padded_labels - W.shape[0], W.shape[1], dtype=W.dtype)
    Wp = torch.cat([W, pad], dim=0)
    outs = []
    for r in range(world_size):
        lo, hi = sh.shard_range(r)
        sd = {k: v for k, v in full.items() if k != "xfc_weight"}
        sd["xfc_weight"] = Wp[lo:hi].clone()
        outs.append(sd)
    return outs


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--dir", required=True)
    ap.add_argument("--name", default="renee-exp")
    ap.add_argument("--from-world", type=int, required=True)
    ap.add_argument("--to-world", type=int, required=True)
    ap.add_argument("--labels", type=int, required=True)
    ap.add_argument("--out-dir", default="")
    a = ap.parse_args(argv)
    shards = [torch.load(os.path.join(a.dir, f"{a.name}_{r}_state_dict.pt"), map_location="cpu") for r in range(a.from_world)]
    full = consolidate(shards, a.labels)
    out_dir = a.out_dir or a.dir
    os.makedirs(out_dir, exist_ok=True)
    if a.to_world == 0:
        torch.save(full, os.path.join(out_dir, f"{a.name}_consolidated_state_dict.pt"))
        return
    for r, sd in enumerate(reshard(full, a.labels, a.to_world)):
        torch.save(sd, os.path.join(out_dir, f"{a.name}_{r}_state_dict.pt"))


if __name__ == "__main__":
    main()
