"""Per-rank training checkpoints with RNG state, written atomically.

Parity: ``GenericModel.checkpoint/resume`` (reference dl_base.py:412-446).  File
``{dir}/{name}_{rank}_checkpoint.pt``; the previous file is rotated to ``..._checkpoint_prev.pt``.
Keys kept from the reference: ``epoch, model_dict, loss, scaler, py_rng, torch_rng,
torch_cuda_rng, torch_random_rng, np_rng, xfc_optimizer_state_dict, tf_optimizer_state_dict,
xfc_scheduler_state_dict, tf_scheduler_state_dict``.  Added: ``dropout_rng`` (the counter-based
kernel RNG), ``count`` (steps taken) and ``world_size``/``labels_per_rank`` so that a resume under a
different sharding is refused instead of silently mis-loading.  Unlike the reference the new file is
written to a temporary name and renamed, so a crash never leaves a truncated checkpoint.

Interchangeable with files written by the reference: ``model_dict`` (same keys and shapes) and ``scaler``.
NOT interchangeable: the optimizer and scheduler sub-dicts.  The reference stores apex/torch optimizer
state dicts (``state`` / ``param_groups`` keyed by parameter index); here ``xfc_optimizer_state_dict`` is
``{"momentum_buffer": [Ls, D]}``, ``tf_optimizer_state_dict`` holds the flat ``exp_avg`` / ``exp_avg_sq``
buffers of the encoder engine and the schedulers store ``base_lr`` and their step.  A reference checkpoint
can therefore initialise the weights of a run here, not resume its optimizer trajectory.
"""
from __future__ import annotations

import os
import random

import numpy as np
import torch


def checkpoint_path(out_dir: str, name: str, rank: int, prev: bool = False) -> str:
    return os.path.join(out_dir, f"{name}_{rank}_checkpoint{'_prev' if prev else ''}.pt")


def _optimizer_states(tr) -> tuple[dict, dict]:
    if tr.cfg.default_impl:
        return tr.xfc_optimizer.state_dict(), tr.tf_optimizer.state_dict()
    enc = tr.encoder
    return tr.xfc.optimizer_state_dict(), {"exp_avg": enc.m.detach().clone(), "exp_avg_sq": enc.v.detach().clone(),
                                           "layout": _flat_layout(enc)}


def _flat_layout(enc) -> list:
    """(name, offset, numel) of every parameter in the flat buffers: the moments are stored flat, so a checkpoint
    carries the layout it was written with."""
    return [(n, int(s.offset), int(s.numel)) for n, s in enc.slots.items()]


def _load_flat_moments(enc, tf_opt: dict, device) -> None:
    """Copy the flat moments back; a checkpoint written under another ordering of the flat buffer is re-mapped by
    parameter name (one without a recorded layout is taken to have this build's ordering only if the sizes agree)."""
    here = _flat_layout(enc)
    there = tf_opt.get("layout")
    for key, dst in (("exp_avg", enc.m), ("exp_avg_sq", enc.v)):
        src = tf_opt[key]
        if there is None or [tuple(x) for x in there] == here:
            if src.numel() != dst.numel():
                raise RuntimeError(f"optimizer state {key}: {src.numel()} elements in the checkpoint, {dst.numel()} here")
            dst.copy_(src.to(device))
            continue
        old = {n: (o, k) for n, o, k in there}
        for n, o, k in here:
            if n not in old or old[n][1] != k:
                raise RuntimeError(f"optimizer state {key}: parameter {n!r} missing or of another size in the checkpoint")
            dst[o:o + k].copy_(src[old[n][0]:old[n][0] + k].to(device))


def save_checkpoint(tr, out_dir: str, loss: float) -> str:
    os.makedirs(out_dir, exist_ok=True)
    xfc_opt, tf_opt = _optimizer_states(tr)
    sd = {"epoch": tr.epoch, "model_dict": tr.state_dict(), "loss": loss,
          "scaler": tr.hp.state_dict(),
          "py_rng": random.getstate(),
          "torch_rng": torch.get_rng_state(),
          "torch_cuda_rng": torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
          "torch_random_rng": torch.random.get_rng_state(),
          "np_rng": np.random.get_state(),
          "xfc_optimizer_state_dict": xfc_opt, "tf_optimizer_state_dict": tf_opt,
          "xfc_scheduler_state_dict": tr.xfc_sched.state_dict(),
          "tf_scheduler_state_dict": tr.tf_sched.state_dict(),
          "dropout_rng": tr.rng.state_dict(), "count": tr.count, "best_score": tr.best_score,
          "world_size": tr.G, "labels_per_rank": tr.Ls}
    path = checkpoint_path(out_dir, tr.name, tr.rank)
    tmp = path + ".tmp"
    torch.save(sd, tmp)
    if os.path.exists(path):
        os.replace(path, checkpoint_path(out_dir, tr.name, tr.rank, prev=True))
    os.replace(tmp, path)
    return path


def load_checkpoint(tr, out_dir: str) -> float:
    path = checkpoint_path(out_dir, tr.name, tr.rank)
    sd = torch.load(path, map_location="cpu", weights_only=False)
    if sd.get("world_size", tr.G) != tr.G or sd.get("labels_per_rank", tr.Ls) != tr.Ls:
        raise RuntimeError(f"checkpoint {path} was written for world_size={sd.get('world_size')} / "
                           f"labels_per_rank={sd.get('labels_per_rank')}, not {tr.G} / {tr.Ls}")
    tr.epoch = int(sd["epoch"]) + 1
    tr.load_state_dict(sd["model_dict"])
    tr.hp.load_state_dict(sd["scaler"])
    random.setstate(sd["py_rng"])
    torch.set_rng_state(sd["torch_rng"])
    if sd.get("torch_cuda_rng") is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state(sd["torch_cuda_rng"])
    torch.random.set_rng_state(sd["torch_random_rng"])
    np.random.set_state(sd["np_rng"])
    if tr.cfg.default_impl:
        tr.xfc_optimizer.load_state_dict(sd["xfc_optimizer_state_dict"])
        tr.tf_optimizer.load_state_dict(sd["tf_optimizer_state_dict"])
    else:
        tr.xfc.load_optimizer_state_dict(sd["xfc_optimizer_state_dict"])
        _load_flat_moments(tr.encoder, sd["tf_optimizer_state_dict"], tr.device)
    tr.xfc_sched.load_state_dict(sd["xfc_scheduler_state_dict"])
    tr.tf_sched.load_state_dict(sd["tf_scheduler_state_dict"])
    tr.rng.load_state_dict(sd.get("dropout_rng", tr.rng.state_dict()))
    tr.count = int(sd.get("count", 0))
    tr.best_score = float(sd.get("best_score", tr.best_score))
    return sd["loss"]


def maybe_resume(tr, out_dir: str):
    if os.path.isfile(checkpoint_path(out_dir, tr.name, tr.rank)):
        return load_checkpoint(tr, out_dir)
    return None
