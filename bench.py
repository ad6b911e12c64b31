"""Headline benchmark: training throughput (samples/s) of the label-sharded XC trainer.

    python bench.py --gpus N --steps K --warmup W [--config 131k-s32] [--impl ours|reference]

For N > 1 launch with ``python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr
127.0.0.1 --master-port P bench.py --gpus N ...`` (one rank per GPU, NCCL).  Rank 0 prints ONE JSON
line.  ``value`` is the whole-job samples/s of K device-timed steps (CUDA events, max over ranks)
with inputs already resident (``ms_per_step_min/median/max`` come from one event per step); ``e2e``
times K steps the way ``XCTrainer.fit`` runs them: batches drawn from the prefetching loader (sampling,
collation and pinning inside the timed region), the public ``XCTrainer.train_step`` call with its
pinned host→device copy of every step's inputs, and a device→host read of the step's result;
``e2e_precollated`` is the same without the loader.  Warm-up continues past ``--warmup`` until every
CUDA graph the run replays exists, and the run asserts that no capture happened while timing.  The
global batch is fixed, so scaling is strong.
Synthetic seeded data of the configuration's shape, random-init weights.

``--impl reference`` runs the unmodified reference (``baseline/_ref``) through its own ``start()``
on the same workload written in its on-disk formats; see ``baseline/run_reference.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # the benchmark workloads: 131 K labels at sequence lengths 32 and 128, 1.3 M and 100 M labels (the small CPU
    # plumbing workload is tests/test_cpu_plumbing.py)
    "131k-s32": dict(labels=131072, seq=32, len_lo=6, batch=256, lam=1.3, zipf=1.1, dropout=0.85),
    "131k-s128": dict(labels=131072, seq=128, len_lo=32, batch=128, lam=4.5, zipf=1.1, dropout=0.85),
    "1.3m": dict(labels=1310720, seq=32, len_lo=6, batch=512, lam=21.0, zipf=1.05, dropout=0.85),
    "100m": dict(labels=100_000_000, seq=32, len_lo=6, batch=1024, lam=3.0, zipf=1.1, dropout=0.85),
    # the per-GPU share of 131k-s32 at 8 GPUs, runnable on one GPU (profiling of the small-shape regime)
    "131k-s32-shard8": dict(labels=16384, seq=32, len_lo=6, batch=32, lam=1.3, zipf=1.1, dropout=0.85),
    "131k-s32-shard4": dict(labels=32768, seq=32, len_lo=6, batch=64, lam=1.3, zipf=1.1, dropout=0.85),
    "131k-s32-shard2": dict(labels=65536, seq=32, len_lo=6, batch=128, lam=1.3, zipf=1.1, dropout=0.85),
    "tiny": dict(labels=8192, seq=32, len_lo=6, batch=64, lam=1.3, zipf=1.1, dropout=0.85),
}


class ClockSampler:
    """Samples ``nvidia-smi`` clocks and throttle reasons every 200 ms while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_ours(args) -> dict:
    import numpy as np
    import torch
    import torch.distributed as dist

    from renee_b200.data import xcrepo
    from renee_b200.data.collate import GlobalBatchSampler, PrefetchLoader, XCCollator
    from renee_b200.data.synthetic import SyntheticSpec, SyntheticXC
    from renee_b200.models.encoder import EncoderConfig
    from renee_b200.ops import cuda as cu
    from renee_b200.parallel.dist import init_distributed
    from renee_b200.train import TrainConfig, XCTrainer
    from renee_b200.utils.sharding import shard_labels

    c = CONFIGS[args.config]
    ctx = init_distributed()
    G, rank = ctx.world_size, ctx.rank
    assert G == args.gpus, f"launched with {G} ranks but --gpus {args.gpus}"
    B = c["batch"]
    assert B % G == 0
    K, W = args.steps, args.warmup
    spec = SyntheticSpec(num_labels=c["labels"], seq_len=c["seq"], len_lo=c["len_lo"], len_hi=c["seq"],
                         poisson_lam=c["lam"], zipf_s=c["zipf"], seed=0)
    n_batches = min(max(W + K, 8), 48)
    ids, mask, lab = SyntheticXC(spec).rows(np.arange(n_batches * B))
    ds = xcrepo.InMemoryDataset(ids, mask, lab)
    sh = shard_labels(c["labels"], G)
    enc_cfg = EncoderConfig()
    cfg = TrainConfig(batch_size=B // G, epochs=1, seed=0, dropout=c["dropout"], lr1=0.05, lr2=1e-5, warmup=5000,
                      wd1=1e-4, noloss=True, fp16xfc=True, maxlen=c["seq"], pooling="cls", accum=args.accum,
                      cuda_graph=not args.no_graph, fused_comm=not args.no_fused_comm)
    if args.persistent_logits:
        cu.set_xfc_persistent(True)
    comm = None
    if G > 1 and cfg.fused_comm:
        from renee_b200.parallel.fused import PeerCollectives
        comm = PeerCollectives(ctx, use_nvls=True if args.nvls else None)
    tr = XCTrainer(cfg, enc_cfg, sh, ctx, steps_per_epoch=100000, comm=comm)
    if G > 1 and not args.no_watchdog:
        # the CLI's training path runs with the heartbeat watchdog; so does the benchmark
        from renee_b200.parallel.watchdog import Heartbeat
        store = dist.distributed_c10d._get_default_store()
        tr.watchdog = Heartbeat(store, rank, G, interval=1.0, timeout=60.0).start()
    coll = XCCollator(sh, ds, rank, args.accum, max(1, B // args.accum), True)
    batches = [coll(np.arange(i * B, (i + 1) * B)).pin() for i in range(n_batches)]
    b_local = batches[0].input_ids.shape[0]

    def barrier():
        if G > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up: at least W steps, and until every CUDA graph the run will replay has been captured
    warm = 0
    while warm < W or (not tr.graphs_ready(b_local, B) and warm < W + 12):
        tr.train_step(batches[warm % n_batches])
        warm += 1
    barrier()
    cu.check_status()
    if cfg.cuda_graph:
        assert tr.graphs_ready(b_local, B) and tr.graph_active(), "CUDA graphs not captured during warm-up"
    captures0 = tr.n_captures

    # ---- device-timed region: inputs resident, K full steps, one event per step
    sampler = ClockSampler(ctx.device.index or 0)
    if rank == 0:
        sampler.start()
    tr.stage_batch(batches[warm % n_batches])
    barrier()
    l0 = cu.launch_count()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(K + 1)]
    evs[0].record()
    for i in range(K):
        tr.device_step()
        evs[i + 1].record()
    barrier()
    launches = tr.launches_per_step() * K if tr.graph_active() else cu.launch_count() - l0
    ms = evs[0].elapsed_time(evs[K])
    per_step = sorted(evs[i].elapsed_time(evs[i + 1]) for i in range(K))

    # ---- end to end, pre-collated: public train_step (pinned H2D of each step's inputs) + D2H of its result
    result_host = torch.zeros(K, 16, dtype=torch.float32).pin_memory()
    h2d = 0
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        b = batches[(warm + i) % n_batches]
        tr.train_step(b)
        result_host[i].copy_(tr.hp.buf, non_blocking=True)
        h2d += tr.h2d_bytes(b)
    e1.record()
    barrier()
    pre_ms = e0.elapsed_time(e1)

    # ---- end to end through the loader, as `fit` runs: sampling, collation and pinning of every batch happen
    # (on the loader's thread) inside the timed region, then the same train_step + D2H
    loader = PrefetchLoader(GlobalBatchSampler(n_batches * B, B, True, 0), coll, pin=True)
    h2d_l = 0
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    done, epoch = 0, 0
    while done < K:
        for b in loader.epoch(epoch):
            if b.batch_size != B:
                continue
            tr.train_step(b)
            result_host[done].copy_(tr.hp.buf, non_blocking=True)
            h2d_l += tr.h2d_bytes(b)
            done += 1
            if done == K:
                break
        epoch += 1
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None
    cu.check_status()
    tr.check_device_status()          # bounded waits all met; with RENEE_B200_GUARD=1 also every guard band intact
    assert tr.n_captures == captures0, "a CUDA-graph capture landed inside a timed region"
    t = torch.tensor([ms, pre_ms, e2e_ms, per_step[0], per_step[K // 2], per_step[-1]], dtype=torch.float64,
                     device=ctx.device)
    if G > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, pre_ms, e2e_ms, s_min, s_med, s_max = (float(x) for x in t)
    assert torch.isfinite(result_host).all()
    if tr.watchdog is not None:
        tr.watchdog.stop()
    value = B * K / (ms / 1e3)
    out = {"metric": "train samples/sec (device-timed, max over ranks)", "value": round(value, 2), "unit": "samples/s",
           "n_gpus": G, "steps": K, "warmup": W, "warmup_run": warm, "ms_per_step": round(ms / K, 4),
           "ms_per_step_min": round(s_min, 4), "ms_per_step_median": round(s_med, 4), "ms_per_step_max": round(s_max, 4),
           "higher_is_better": True, "scaling": "strong",
           "vs_baseline": None,      # the reference publishes epoch times on V100s, no samples/s for this config
           "dtype": "bf16 encoder, fp16 classifier W+momentum",
           "data": "synthetic seeded (Zipf labels, Poisson positives), random-init weights", "impl": "ours",
           "config": {"model": f"DistilBERT-style 6x768 encoder + label-sharded XFC, L={c['labels']}",
                      "name": args.config, "global_batch": B, "seq_len": c["seq"], "labels": c["labels"],
                      "parallelism": f"dp{G} encoder + label-sharded classifier x{G}",
                      "flags": "--fp16xfc --noloss --dropout 0.85 --lr1 0.05 --lr2 1e-5 --wd1 1e-4"
                               + (f" --accum {args.accum}" if args.accum > 1 else ""),
                      "arm": "own flat encoder engine, CLS pooling, bf16",
                      "l2": "per-step working set (W, momentum, encoder params/moments/activations) exceeds the 126 MB L2",
                      "cuda_graph": tr.graph_active(), "fused_comm": comm is not None,
                      "nvls": bool(comm is not None and comm.use_nvls), "watchdog": tr.watchdog is not None,
                      "own_gemm": bool(getattr(tr.encoder, "own_gemm", False)),
                      "guard_bands": "intact" if os.environ.get("RENEE_B200_GUARD") == "1" else "off",
                      "persistent_logits": bool(args.persistent_logits)},
           "clocks": clocks,
           "e2e": {"value": round(B * K / (e2e_ms / 1e3), 2), "unit": "samples/s", "ms_per_step": round(e2e_ms / K, 4),
                   "h2d_bytes_per_step": h2d_l // K, "d2h_bytes_per_step": 64,
                   "path": "GlobalBatchSampler -> XCCollator -> pin (loader thread) -> XCTrainer.train_step -> D2H"},
           "e2e_precollated": {"value": round(B * K / (pre_ms / 1e3), 2), "unit": "samples/s",
                               "ms_per_step": round(pre_ms / K, 4), "h2d_bytes_per_step": h2d // K,
                               "d2h_bytes_per_step": 64},
           "memory_gb": round(torch.cuda.max_memory_allocated() / 1e9, 2),
           "gpu_launches": int(launches)}
    if G > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out if rank == 0 else None


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="131k-s32", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-fused-comm", action="store_true")
    ap.add_argument("--persistent-logits", action="store_true",
                    help="classifier logits GEMM: persistent CTAs with double-buffered TMEM accumulators")
    ap.add_argument("--custom-cuda", action="store_true", help="reference arm: route its GEMMs to its CUTLASS extension")
    ap.add_argument("--accum", type=int, default=1, help="split accumulation factor (both arms)")
    ap.add_argument("--nvls", action="store_true", help="gradient reduction and parameter push through NVLS multimem")
    ap.add_argument("--no-watchdog", action="store_true", help="run multi-GPU steps without the heartbeat watchdog")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        from baseline.run_reference import run_reference
        out = run_reference(args, CONFIGS[args.config])
    else:
        out = run_ours(args)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
