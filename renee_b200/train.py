"""Training runtime: the optimized loss-skipping step, the autograd baseline step, the epoch loop.

Parity with the reference's ``GenericModel`` (dl_base.py:146-455):

* ``XCTrainer.train_step``  ↔ the optimized branch of ``fit`` (dl_base.py:297-378): encoder forward,
  embedding all-gather, manual classifier forward/backward with loss skipping, SGD-momentum on the
  classifier (unscaled), hand-off of the encoder-input gradient ``dX`` (scaled by the loss scale),
  encoder backward, Adam on the encoder, both cosine schedules stepped every iteration;
* ``XCTrainer.default_step`` ↔ ``--default-impl`` (dl_base.py:274-295): dense targets,
  ``BCEWithLogitsLoss(sum)`` and autograd — the numerical oracle of the optimized path;
* ``fit`` ↔ the epoch loop with evaluation every ``evaluation_epochs`` epochs and on the last one,
  and a checkpoint per epoch (dl_base.py:382-393).

On a GPU the optimized step is a fixed sequence of kernel launches on static buffers (no autograd
graph, no allocation), which is what allows it to be captured in a CUDA graph; step-varying values
(learning rates, dropout seed, loss scale) are read from device memory.
"""
from __future__ import annotations

import os
import random
import sys
import time
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn as nn

from . import ops
from .data.collate import XCBatch
from .models.encoder import (DistilEncoder, EncoderConfig, FP32Linear, TransformerInputLayer)
from .models.flat_encoder import FlatEncoder
from .models.xfc import XFCClassifier
from .optim.hparams import HP, HyperParams
from .optim.schedule import CosineWarmupSchedule
from .ops.rng import DropoutRNG
from .parallel.collectives import TorchCollectives
from .parallel.dist import DistContext
from .utils import guard
from .utils.timing import nvtx_range
from .utils.sharding import LabelSharding

LOSS_SAMPLE_FREQ = 100   # dl_base.py:144
_S_CLS_DROPOUT = 5


@dataclass
class TrainConfig:
    batch_size: int = 8            # per GPU
    epochs: int = 50
    expname: str = "renee-exp"
    seed: int = 42
    bottleneck_dims: int = 0
    dropout: float = 0.5
    lr1: float = 0.0025
    lr2: float = 1e-5
    mo: float = 0.9
    wd1: float = 0.01
    wd2: float = 0.01
    fp32encoder: bool = False
    fp16xfc: bool = False
    noloss: bool = False
    checkpoint_resume: str = ""
    warmup: int = 140000
    accum: int = 1
    maxlen: int = 32
    default_impl: bool = False
    custom_cuda: bool = False
    pooling: str = "mean"
    encoder_dtype: str = "bf16"      # compute dtype of the encoder on a GPU unless fp32encoder
    adam_eps: float = 1e-6           # main.py:181
    evaluation_epochs: int = 5       # main.py:184
    cuda_graph: bool = True
    fused_comm: bool = True
    stochastic_round: bool = True     # fp16 W storage: round the updated weights stochastically (see models/xfc.py)
    overlap_dw: bool = False         # issue the last dW+SGD kernel on a side stream, under the encoder backward
    out_dir: str = ""

    @classmethod
    def from_args(cls, args) -> "TrainConfig":
        names = cls.__dataclass_fields__.keys()
        return cls(**{k: getattr(args, k) for k in names if hasattr(args, k)})


class DefaultModel(nn.Module):
    """Module layout of the reference's ``GenericModel``: ``embed = Sequential(encoder wrapper,
    [bottleneck], dropout)`` and ``xfc_weight [Ls, D]`` (dl_base.py:147-187)."""

    def __init__(self, enc_cfg: EncoderConfig, labels_per_rank: int, cfg: TrainConfig):
        super().__init__()
        mods = [TransformerInputLayer(DistilEncoder(enc_cfg), cfg.pooling)]
        D = enc_cfg.dim
        if cfg.bottleneck_dims > 0:
            mods.append(FP32Linear(enc_cfg.dim, cfg.bottleneck_dims, bias=False))
            D = cfg.bottleneck_dims
        mods.append(nn.Dropout(cfg.dropout))
        self.embed = nn.Sequential(*mods)
        self.xfc_weight = nn.Parameter(torch.empty(labels_per_rank, D))
        nn.init.normal_(self.xfc_weight, mean=0.0, std=0.02)


def split_param_groups(named_params, wd2: float):
    """The reference's grouping (dl_base.py:219-236): names containing ``xfc`` → SGD; everything else
    → Adam with a no-decay group for names containing ``bias`` / ``LayerNorm.bias`` /
    ``LayerNorm.weight``."""
    xfc, tf = [], []
    for n, p in named_params:
        if p.requires_grad:
            (xfc if "xfc" in n else tf).append((n, p))
    nd = ("bias", "LayerNorm.bias", "LayerNorm.weight")
    groups = [{"params": [p for n, p in tf if not any(k in n for k in nd)], "weight_decay": wd2},
              {"params": [p for n, p in tf if any(k in n for k in nd)], "weight_decay": 0.0}]
    return [p for _, p in xfc], groups


class XCTrainer:
    def __init__(self, cfg: TrainConfig, enc_cfg: EncoderConfig, sharding: LabelSharding, ctx: DistContext,
                 steps_per_epoch: int, comm=None):
        self.cfg = cfg
        self.enc_cfg = enc_cfg
        self.sharding = sharding
        self.ctx = ctx
        self.rank, self.G = ctx.rank, ctx.world_size
        self.device = ctx.device
        self.comm = comm if comm is not None else TorchCollectives(ctx)
        self.steps_per_epoch = int(steps_per_epoch)
        self.total_steps = int(steps_per_epoch * cfg.epochs)
        self.epoch = 0
        self.count = 0                      # optimizer steps taken (dl_base.py:363)
        self.best_score = -9999999.0
        self.name = cfg.expname
        self.out_dir = cfg.out_dir
        if self.out_dir:
            os.makedirs(self.out_dir, exist_ok=True)
        self.B = cfg.batch_size * self.G
        self.Ls = sharding.labels_per_rank
        on_gpu = self.device.type in ("cuda", "meta")     # meta: size-accounting dry runs plan for a GPU
        self.act_dtype = torch.float32 if (cfg.fp32encoder or not on_gpu) else \
            (torch.bfloat16 if cfg.encoder_dtype == "bf16" else torch.float16)
        self.xfc_sched = CosineWarmupSchedule(cfg.lr1, cfg.warmup, self.total_steps)
        self.tf_sched = CosineWarmupSchedule(cfg.lr2, cfg.warmup, self.total_steps)
        self.rng = DropoutRNG(cfg.seed)
        self.hp = HyperParams(self.device, init_scale=2.0 ** 12 if cfg.fp16xfc else 2.0 ** 16,
                              enabled=not cfg.fp32encoder)
        self.step_rng = ops.StepRNG(0, self.hp.seed_tensor())
        self.loss_sum = 0.0
        self.loss_steps = 0
        self._graphs: dict = {}
        self._graph_warm: dict = {}
        self._graph_generation = -1
        self._pending_loss = None
        self._side_stream = None
        self._aborted = False
        self.n_captures = 0         # CUDA-graph captures so far (a benchmark checks that none lands in its timed region)
        self.watchdog = None        # optional parallel.watchdog.Heartbeat, consulted before each step's launches
        if cfg.default_impl:
            self._init_default()
        else:
            self._init_optimized()

    # ------------------------------------------------------------------ construction
    def _init_default(self) -> None:
        cfg = self.cfg
        torch.manual_seed(cfg.seed)
        self.model = DefaultModel(self.enc_cfg, self.Ls, cfg).to(self.device)
        xfc_params, tf_groups = split_param_groups(self.model.named_parameters(), cfg.wd2)
        self.xfc_optimizer = torch.optim.SGD(xfc_params, lr=cfg.lr1, momentum=cfg.mo, weight_decay=cfg.wd1)
        self.tf_optimizer = torch.optim.AdamW(tf_groups, lr=cfg.lr2, eps=cfg.adam_eps)
        self.loss_fn = nn.BCEWithLogitsLoss(reduction="sum")

    def _init_optimized(self) -> None:
        cfg = self.cfg
        D = cfg.bottleneck_dims if cfg.bottleneck_dims > 0 else self.enc_cfg.dim
        self.D = D
        self.comm.setup(self.B, D)
        self.encoder = FlatEncoder(self.enc_cfg, self.device, self.act_dtype, cfg.pooling, cfg.bottleneck_dims,
                                   seed=cfg.seed, grad_alloc=getattr(self.comm, "alloc_grad", None),
                                   p16_alloc=getattr(self.comm, "alloc_p16", None))
        self.xfc = XFCClassifier(self.Ls, D, self.device, cfg.fp16xfc,
                                 rank=self.rank, seed=cfg.seed, max_batch=self.B, accum=cfg.accum,
                                 stochastic_round=cfg.stochastic_round)
        dev = self.device
        b, S = cfg.batch_size + 1, cfg.maxlen
        self.max_nnz = 0
        self.buf = dict(
            ids=guard.zeros(b, S, dtype=torch.int32, device=dev, name="step.ids"),
            mask=guard.zeros(b, S, dtype=torch.int32, device=dev, name="step.mask"),
            x_local=guard.zeros(b, D, dtype=self.xfc.dtype, device=dev, name="step.x_local"),
            X=guard.zeros(self.B + self.G, D, dtype=self.xfc.dtype, device=dev, name="step.X"),
            dX=guard.zeros(self.B + self.G, D, dtype=torch.float32, device=dev, name="step.dX"),
            dx_local=guard.zeros(b, D, dtype=torch.float32, device=dev, name="step.dx_local"),
            de=guard.zeros(b, D, dtype=torch.float32, device=dev, name="step.de"),
            nnz=guard.zeros(1, dtype=torch.int32, device=dev, name="step.nnz"),
            loss=guard.zeros(1, dtype=torch.float32, device=dev, name="step.loss"),
        )
        self._ensure_pos_capacity(max(1024, self.B * 8))
        if self.device.type == "cuda" and cfg.fp16xfc and cfg.overlap_dw:
            # measured on B200 (131k-s32): 4.27 ms/step with the overlap vs 4.23 ms without at one GPU,
            # 2.86 vs 2.67 ms at two — the kernel competes with the backward GEMMs for HBM — so it is off by default
            self._side_stream = torch.cuda.Stream(device=self.device)

    def _ensure_pos_capacity(self, n: int) -> None:
        if n <= self.max_nnz:
            return
        cap = 1
        while cap < n:
            cap *= 2
        self.max_nnz = cap
        self.buf["pos_rows"] = guard.zeros(cap, dtype=torch.int32, device=self.device, name="step.pos_rows")
        self.buf["pos_labels"] = guard.zeros(cap, dtype=torch.int32, device=self.device, name="step.pos_labels")
        self._graphs, self._graph_warm = {}, {}   # static addresses changed: captured graphs are stale

    # ------------------------------------------------------------------ one step (optimized)
    def _set_hparams(self) -> None:
        seed = self.rng.seed_for_step()
        self.step_rng.set(seed)
        self.hp.set_step(self.xfc_sched.lr(), self.tf_sched.lr(), seed)
        self.hp.upload()

    def _upload(self, batch: XCBatch) -> tuple[int, int]:
        b = batch.input_ids.shape[0]
        nnz = int(batch.pos_rows.numel())
        self._ensure_pos_capacity(nnz)
        bf = self.buf
        bf["ids"][:b].copy_(batch.input_ids, non_blocking=True)
        bf["mask"][:b].copy_(batch.attention_mask, non_blocking=True)
        bf["pos_rows"][:nnz].copy_(batch.pos_rows, non_blocking=True)
        bf["pos_labels"][:nnz].copy_(batch.pos_labels, non_blocking=True)
        bf["nnz"].fill_(nnz)
        if batch.uploaded is not None:
            batch.uploaded()            # the loader may refill the batch's staging buffers once these copies are done
        return b, nnz

    def h2d_bytes(self, batch: XCBatch) -> int:
        return int(batch.input_ids.numel() * 4 + batch.attention_mask.numel() * 4 + batch.pos_rows.numel() * 8
                   + HP.HOST_SLOTS * 4)

    def stage_batch(self, batch: XCBatch) -> None:
        """Host→device part of a step: this step's hyper-parameters (32 bytes) and inputs."""
        self._set_hparams()
        b, nnz = self._upload(batch)
        want_loss = (not self.cfg.noloss) and (self.count % LOSS_SAMPLE_FREQ == 0)
        self._staged = (b, batch.batch_size, nnz, want_loss)

    def device_step(self):
        """Device part of a step on the staged batch: a CUDA-graph replay when one has been captured
        for this shape, the same launch sequence issued eagerly otherwise."""
        b, B, nnz, want_loss = self._staged
        self.comm.host_begin()
        key = (b, B, self.comm.parity)
        use_graph = (self.cfg.cuda_graph and self.device.type == "cuda" and not want_loss
                     and getattr(self.comm, "graph_safe", self.G == 1))
        if use_graph and self._graph_generation != self.encoder.generation:
            self._graphs, self._graph_warm = {}, {}          # the encoder re-allocated its activations
            self._graph_generation = self.encoder.generation
        if use_graph:
            g = self._graphs.get(key)
            if g is not None:
                g.replay()
                return None
            seen = self._graph_warm.get(key, 0)
            self._graph_warm[key] = seen + 1
            if seen >= 2:
                self._capture(key, b, B, nnz)
                self._graphs[key].replay()
                return None
        return self._device_step(b, B, nnz, want_loss)

    def _capture(self, key, b: int, B: int, nnz: int) -> None:
        from .ops import cuda as cu
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        n0 = cu.launch_count()
        with torch.cuda.graph(graph):
            self._device_step(b, B, nnz, False)
        self._graph_launches = cu.launch_count() - n0
        self._graphs[key] = graph
        self.n_captures += 1

    def graph_active(self) -> bool:
        return bool(self._graphs)

    def graphs_ready(self, b: int, B: int) -> bool:
        """True once every graph that steps of this shape will replay exists: one per buffer parity with the
        peer-memory backend, one otherwise.  Until then a step may still capture (synchronise + instantiate)."""
        if not (self.cfg.cuda_graph and self.device.type == "cuda"
                and getattr(self.comm, "graph_safe", self.G == 1)):
            return True                                     # nothing will ever be captured
        if self._graph_generation != self.encoder.generation:
            return False
        parities = (0, 1) if hasattr(self.comm, "host_step") else (self.comm.parity,)
        return all((b, B, q) in self._graphs for q in parities)

    def launches_per_step(self) -> int:
        return int(getattr(self, "_graph_launches", 0))

    def train_step(self, batch: XCBatch) -> torch.Tensor | None:
        """Runs one optimized step; returns the sampled loss tensor (device, un-normalised) on
        sampling steps, else ``None``.  No host synchronisation happens here."""
        if self._aborted:
            raise RuntimeError("this trainer was aborted after a peer or kernel failure; restart from a checkpoint")
        if self.watchdog is not None:
            try:
                self.watchdog.check()   # a dead or failed peer is noticed on the host, before any kernel waits for it
            except Exception:
                self.abort()
                raise
        if self.cfg.default_impl:
            return self.default_step(batch)
        self.stage_batch(batch)
        want_loss = self._staged[3]
        loss = self.device_step()
        self.count += 1
        self.rng.advance()
        self.xfc_sched.step()
        self.tf_sched.step()
        if want_loss:
            self._pending_loss = (loss, batch.batch_size)
        return loss

    def _device_step(self, b: int, B: int, nnz: int, want_loss: bool):
        cfg, bf, enc, comm = self.cfg, self.buf, self.encoder, self.comm
        ids, mask = bf["ids"][:b], bf["mask"][:b]
        comm.device_begin()
        with nvtx_range("encoder_forward"):
            emb = enc.forward(ids, mask, self.step_rng, train=True)
        with nvtx_range("allgather_classifier"):
            # classifier-input dropout + cast + all-gather (fused into one kernel on the peer-memory backend)
            X, wait = comm.embeddings_to_X(emb, B, cfg.dropout, self.step_rng, _S_CLS_DROPOUT, bf)
            dX, signal = comm.dx_buffer(B, bf)
            loss = self.xfc.step(X, bf["pos_rows"], bf["pos_labels"], bf["nnz"] if X.is_cuda else nnz, dX,
                                 self.hp, cfg.mo, cfg.wd1, want_loss, wait=wait, signal=signal,
                                 side_stream=self._side_stream)
            if want_loss:
                loss = comm.allreduce_scalar(loss.reshape(1))
        with nvtx_range("reduce_scatter"):
            de = comm.dx_to_local(dX, B, cfg.dropout, self.step_rng, _S_CLS_DROPOUT, bf)
        with nvtx_range("encoder_backward"):
            # with the peer-memory backend the gradient reduce-scatter runs bucket by bucket under the backward pass
            hook = getattr(comm, "on_layer_done", None)
            if hook is not None:
                comm.backward_begin(enc)
            enc.backward(de, on_layer_done=(lambda l: hook(enc, l)) if hook is not None else None)
        with nvtx_range("optimizer"):
            comm.optimizer_step(enc, self.hp, 0.9, 0.999, cfg.adam_eps, cfg.wd2)
            self.hp.update_scale()
        if self._side_stream is not None:
            torch.cuda.current_stream().wait_stream(self._side_stream)   # the overlapped dW+SGD kernel joins here
        return loss

    def profile_step(self, batch: XCBatch) -> dict:
        """Runs one optimized step eagerly with device-side timers around its phases and returns
        ``{phase: milliseconds}`` (it is a real training step: weights are updated)."""
        from .utils.timing import PhaseTimer
        cfg, bf, enc, comm = self.cfg, self.buf, self.encoder, self.comm
        tm = PhaseTimer(self.device)
        with tm.phase("h2d"):
            self.stage_batch(batch)
        b, B, nnz, _ = self._staged
        comm.host_begin()
        with tm.phase("encoder_forward"):
            comm.device_begin()
            emb = enc.forward(bf["ids"][:b], bf["mask"][:b], self.step_rng, train=True)
        with tm.phase("allgather_classifier"):
            X, wait = comm.embeddings_to_X(emb, B, cfg.dropout, self.step_rng, _S_CLS_DROPOUT, bf)
            dX, signal = comm.dx_buffer(B, bf)
            self.xfc.step(X, bf["pos_rows"], bf["pos_labels"], bf["nnz"] if X.is_cuda else nnz, dX, self.hp, cfg.mo,
                          cfg.wd1, False, wait=wait, signal=signal)
        with tm.phase("reduce_scatter"):
            de = comm.dx_to_local(dX, B, cfg.dropout, self.step_rng, _S_CLS_DROPOUT, bf)
        with tm.phase("encoder_backward"):
            enc.backward(de)
        with tm.phase("optimizer"):
            comm.optimizer_step(enc, self.hp, 0.9, 0.999, cfg.adam_eps, cfg.wd2)
            self.hp.update_scale()
        self.count += 1
        self.rng.advance()
        self.xfc_sched.step()
        self.tf_sched.step()
        return tm.result_ms()

    def pop_loss(self) -> float | None:
        """Normalised sampled loss of the most recent sampling step (synchronises)."""
        pend = getattr(self, "_pending_loss", None)
        if pend is None:
            return None
        loss, B = pend
        self._pending_loss = None
        return float(loss.item()) / (B * self.sharding.padded_labels)

    # ------------------------------------------------------------------ one step (autograd baseline)
    def default_step(self, batch: XCBatch):
        cfg, m = self.cfg, self.model
        dev = self.device
        B = batch.batch_size
        data = {"input_ids": batch.input_ids.to(dev), "attention_mask": batch.attention_mask.to(dev)}
        embed = m.embed(data)
        X = _AllGatherRows.apply(embed, self.comm, B) if self.G > 1 else embed
        out = X @ m.xfc_weight.t()
        y = batch.dense_targets.to(dev)
        loss = self.loss_fn(out, y)
        loss.backward()
        if self.G > 1:  # DDP semantics: encoder gradients are averaged over ranks
            for n, p in m.named_parameters():
                if "xfc" not in n and p.grad is not None:
                    torch.distributed.all_reduce(p.grad)
                    p.grad.mul_(1.0 / self.G)
        for opt, sched in ((self.xfc_optimizer, self.xfc_sched), (self.tf_optimizer, self.tf_sched)):
            for g in opt.param_groups:
                g["lr"] = sched.lr()
            opt.step()
            opt.zero_grad(set_to_none=True)
            sched.step()
        self.count += 1
        self._pending_loss = (loss.detach().reshape(1).clone(), B)
        if self.G > 1:
            self.comm.allreduce_scalar(self._pending_loss[0])
        return self._pending_loss[0]

    # ------------------------------------------------------------------ state dict (reference layout)
    def state_dict(self) -> dict:
        if self.cfg.default_impl:
            return {k: v.detach().clone() for k, v in self.model.state_dict().items()}
        self.comm.sync_master(self.encoder)     # collective when the optimizer is sharded over ranks
        sd = {"xfc_weight": self.xfc.state_dict_weight()}
        for k, v in self.encoder.encoder_state_dict().items():
            sd[f"embed.0.transformer.{k}"] = v
        if self.cfg.bottleneck_dims > 0:
            sd["embed.1.transformer_weight"] = self.encoder.bottleneck_weight().detach().clone()
        return sd

    def load_state_dict(self, sd: dict) -> None:
        sd = normalise_state_dict_keys(sd)
        if self.cfg.default_impl:
            self.model.load_state_dict(sd)
            return
        self.xfc.load_weight(sd["xfc_weight"])
        pre = "embed.0.transformer."
        self.encoder.load_encoder_state_dict({k[len(pre):]: v for k, v in sd.items() if k.startswith(pre)})
        if self.cfg.bottleneck_dims > 0:
            self.encoder.bottleneck_weight().copy_(sd["embed.1.transformer_weight"].to(self.device, torch.float32))
            self.encoder.sync_compute_copy()

    # ------------------------------------------------------------------ epoch loop
    def fit(self, loader, evaluator=None, log=print) -> None:
        from .checkpoint import maybe_resume, save_checkpoint
        from .utils.logging import JsonlLogger
        cfg = self.cfg
        jl = JsonlLogger(os.path.join(self.out_dir, f"{self.name}_log.jsonl") if self.out_dir else None,
                         enabled=self.ctx.is_main, echo=None)
        if cfg.checkpoint_resume:
            prev = maybe_resume(self, cfg.checkpoint_resume)
            if prev is not None:
                log(f"Resuming training from epoch:  {self.epoch} with loss:  {prev}")
            else:
                log("No checkpoint file to resume. Starting training from scratch")
        for epoch in range(self.epoch, cfg.epochs):
            self.epoch = epoch
            self.loss_sum, self.loss_steps = 0.0, 0
            t0 = time.time()
            n_rows = 0
            for batch in loader.epoch(epoch):
                self.train_step(batch)
                n_rows += batch.batch_size
                l = self.pop_loss()
                if l is not None:
                    self.loss_sum += l
                    self.loss_steps += 1
            if self.device.type == "cuda":
                torch.cuda.synchronize()
                self.check_device_status()
            mean_loss = self.loss_sum / self.loss_steps if self.loss_steps else 0.0
            if self.ctx.is_main:
                log(f"mean loss after epoch {epoch} : {'%.4E' % mean_loss}")
                log(f"Scale:  {self.hp.get_scale()}")
                log(f"epoch {epoch}: {n_rows / max(time.time() - t0, 1e-9):.1f} samples/s (wall)")
                sys.stdout.flush()
                jl.log("epoch", epoch=epoch, mean_loss=mean_loss, loss_scale=self.hp.get_scale(), steps=self.count,
                       optimizer_steps=int(self.hp.buf[HP.ADAM_STEP]), rows=n_rows,
                       samples_per_s=n_rows / max(time.time() - t0, 1e-9), world_size=self.G)
            last = epoch == cfg.epochs - 1
            if evaluator is not None and (((epoch + 1) % cfg.evaluation_epochs == 0) or last):
                evaluator(self, epoch, mean_loss, self.out_dir, self.name)
            if cfg.checkpoint_resume:
                save_checkpoint(self, cfg.checkpoint_resume, mean_loss)
        self.epoch = cfg.epochs

    def abort(self) -> None:
        """After a peer or kernel failure: launch nothing more and wait for what is in flight (every device-side
        wait is bounded, so this returns) before the process tears its memory mappings down."""
        self._aborted = True
        if self.device.type == "cuda":
            try:
                torch.cuda.synchronize()
            except RuntimeError:
                pass

    def check_device_status(self) -> None:
        """Raise (and tell the other ranks) if a bounded device-side wait has expired since the last check, or
        (guard mode) if something wrote outside a framework buffer."""
        if guard.enabled():
            try:
                guard.assert_clean()
            except guard.GuardError as exc:
                if self.watchdog is not None:
                    self.watchdog.post_failure(str(exc))
                raise
        if self.device.type != "cuda":
            return
        from .ops import cuda as cu
        try:
            cu.check_status(self.device)
        except cu.KernelError as exc:
            if self.watchdog is not None:
                self.watchdog.post_failure(str(exc))
            self.abort()
            raise

    def save(self, out_dir: str | None = None) -> str:
        out_dir = out_dir or self.out_dir
        os.makedirs(out_dir, exist_ok=True)
        path = os.path.join(out_dir, f"{self.name}_{self.rank}_state_dict.pt")
        torch.save(self.state_dict(), path)
        return path

    def load(self, out_dir: str | None = None) -> None:
        out_dir = out_dir or self.out_dir
        path = os.path.join(out_dir, f"{self.name}_{self.rank}_state_dict.pt")
        self.load_state_dict(torch.load(path, map_location="cpu"))

    # ------------------------------------------------------------------ inference helpers
    @torch.no_grad()
    def embed_eval(self, batch: XCBatch) -> torch.Tensor:
        """Embeddings of this rank's rows in eval mode (no dropout), classifier dtype."""
        dev = self.device
        if self.cfg.default_impl:
            self.model.eval()
            e = self.model.embed({"input_ids": batch.input_ids.to(dev), "attention_mask": batch.attention_mask.to(dev)})
            self.model.train()
            return e
        b = batch.input_ids.shape[0]
        ids = batch.input_ids.to(dev, non_blocking=True)
        mask = batch.attention_mask.to(dev, non_blocking=True)
        emb = self.encoder.forward(ids, mask, self.step_rng, train=False)
        return emb.to(self.xfc.dtype)

    def local_topk(self, X: torch.Tensor, k: int):
        if self.cfg.default_impl:
            Z = X.float() @ self.model.xfc_weight.float().t()
            return torch.topk(Z, min(k, Z.shape[1]), dim=1)
        return self.xfc.topk(X, k)


class _AllGatherRows(torch.autograd.Function):
    """All-gather with gradient: the backward sums every rank's gradient and returns this rank's
    rows — the reference's ``AllGather`` autograd function (dl_base.py:457-481)."""

    @staticmethod
    def forward(ctx, x_local, comm, B):
        ctx.comm, ctx.B, ctx.b = comm, B, x_local.shape[0]
        out = torch.empty(B, x_local.shape[1], dtype=x_local.dtype, device=x_local.device)
        return comm.gather_embeddings(x_local.detach(), B, out).clone()

    @staticmethod
    def backward(ctx, grad):
        out = torch.empty(ctx.b, grad.shape[1], dtype=grad.dtype, device=grad.device)
        return ctx.comm.reduce_scatter_dx(grad.contiguous(), ctx.B, out).clone(), None, None


def normalise_state_dict_keys(sd: dict) -> dict:
    """Accept the key variants the reference's wrappers produce: DDP inserts ``module.`` after
    ``embed.`` (main.py:161) and ``torch.compile`` inserts ``_orig_mod.`` (main.py:156)."""
    out = {}
    for k, v in sd.items():
        k2 = k.replace("embed.module.", "embed.").replace("._orig_mod.", ".")
        out[k2] = v
    return out


def seed_everything(seed: int) -> None:
    torch.manual_seed(seed)
    random.seed(seed)
    np.random.seed(seed)
