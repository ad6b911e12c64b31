"""Reference arm of ``bench.py``: runs the UNMODIFIED reference (``baseline/_ref/main.py`` +
``dl_base.py`` + its compiled ``xfc_gemm_cuda`` extension) through its own ``start()`` entry point on
the benchmark's synthetic workload.

What is supplied around it (nothing of ``renee_b200`` is imported here):

* the workload written in the reference's on-disk formats (``trn_X_Y.txt``, ``tst_X_Y.txt``,
  ``tst_filter_labels.txt``, int64 ``*_doc_{input_ids,attention_mask}.dat``) — generated with plain
  numpy from the same distributions as the benchmark configuration;
* a randomly initialised DistilBERT saved with ``save_pretrained`` (no hub access);
* ``baseline/shims``: minimal stand-ins for ``apex.optimizers`` (→ torch fused SGD/AdamW) and for the
  three pyxclib functions the reference imports — neither package can be installed offline;
* timing: ``dl_base.trange`` is wrapped so that CUDA events bracket exactly K iterations of the
  reference's own training loop (data loading, H2D, forward, XFC step, backward, both optimizers),
  with a barrier + synchronize on both sides, max over ranks.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SHIMS = os.path.join(HERE, "shims")


_ZIPF_CUM: dict = {}


def _zipf_sample(rng, L, s, n):
    head = min(L, 1 << 20)
    cum = _ZIPF_CUM.get((head, s))
    if cum is None:
        cum = _ZIPF_CUM[(head, s)] = np.cumsum(np.power(np.arange(1, head + 1, dtype=np.float64), -s))
    tail = 0.0
    if L > head:
        tail = ((L + 0.5) ** (1 - s) - (head + 0.5) ** (1 - s)) / (1 - s)
    u = rng.random(n) * (cum[-1] + tail)
    out = np.searchsorted(cum, np.minimum(u, cum[-1] * (1 - 1e-12)), side="right")
    far = u >= cum[-1]
    if far.any():
        r = u[far] - cum[-1]
        x = np.power((head + 0.5) ** (1 - s) + r * (1 - s), 1.0 / (1 - s))
        out[far] = np.clip(np.floor(x + 0.5).astype(np.int64) - 1, head, L - 1)
    return np.minimum(out, L - 1)


def _write_dataset(root, c, n_trn, n_tst, seed=0):
    """Synthetic dataset in the XC-repository layout under ``root`` (written once, atomically)."""
    if os.path.exists(os.path.join(root, ".done")):
        return
    tmp = root + f".tmp{os.getpid()}"
    tok = os.path.join(tmp, f"bert-base-uncased-{c['seq']}")
    os.makedirs(tok, exist_ok=True)
    rng = np.random.default_rng(seed)
    L, S = c["labels"], c["seq"]
    for name, n in (("trn", n_trn), ("tst", n_tst)):
        lens = rng.integers(c["len_lo"], S + 1, size=n)
        mask = (np.arange(S)[None] < lens[:, None]).astype(np.int64)
        ids = rng.integers(1000, 30522, size=(n, S), dtype=np.int64) * mask
        ids.tofile(os.path.join(tok, f"{name}_doc_input_ids.dat"))
        mask.tofile(os.path.join(tok, f"{name}_doc_attention_mask.dat"))
        npos = 1 + rng.poisson(c["lam"], size=n)
        with open(os.path.join(tmp, f"{name}_X_Y.txt"), "w") as f:
            f.write(f"{n} {L}\n")
            for r in range(n):
                cols = np.unique(_zipf_sample(rng, L, c["zipf"], int(npos[r])))
                f.write(" ".join(f"{int(x)}:1.00000" for x in cols) + "\n")
    with open(os.path.join(tmp, "tst_filter_labels.txt"), "w") as f:
        f.write("0 0\n")
    open(os.path.join(tmp, ".done"), "w").close()
    try:
        os.rename(tmp, root)
    except OSError:
        pass  # another rank won the race


def _preflight(c, G, B, accum, custom_cuda, local):
    """Sizes the reference's classifier state from its source before anything is allocated, so that a
    configuration it cannot hold is reported instead of driving the box out of memory.  Per rank, with
    ``n = Ls * 768`` elements: fp32 parameter built on the HOST first (dl_base.py:185-187, then ``model.cuda()``,
    main.py:157); on the device fp32 W + fp32 .grad + fp32 momentum + the per-step fp16 copy (dl_base.py:562) =
    14 n bytes, the fp16 ``[B/accum, Ls]`` logits buffer (dl_base.py:176), and on the cuBLAS path an fp16
    ``[Ls, 768]`` product before its fp32 cast (dl_base.py:625-631); about 3 GB for the encoder, its
    optimizer state, activations and the CUDA context."""
    import torch
    per_rank = (c["labels"] + G - 1) // G
    Ls = (per_rank + 15) // 16 * 16                      # main.py:76-87
    n = Ls * 768
    dev = 14 * n + 2 * (B // accum) * Ls + (0 if custom_cuda else 2 * n) + 3e9
    total = torch.cuda.get_device_properties(local).total_memory
    if dev > total:
        return (f"reference classifier state needs about {dev / 1e9:.0f} GB per GPU at {Ls} labels per rank "
                f"(fp32 W+grad+momentum, fp16 copy, [B/accum, Ls] logits, cuBLAS temporaries; accum={accum}) "
                f"but the device has {total / 1e9:.0f} GB")
    host = 4 * n * G * 1.25
    try:
        import psutil
        avail = psutil.virtual_memory().available
    except Exception:
        avail = None
    if avail is not None and host > avail:
        return (f"reference builds its fp32 classifier on the host first: {host / 1e9:.0f} GB for {G} ranks, "
                f"{avail / 1e9:.0f} GB of host memory available")
    return None


def _wait_for(path, timeout=600.0):
    t0 = time.time()
    while not os.path.exists(path):
        if time.time() - t0 > timeout:
            raise RuntimeError(f"timed out waiting for {path}")
        time.sleep(0.2)


def run_reference(args, c) -> dict | None:
    if not (os.path.exists(os.path.join(REF, "main.py")) and os.path.exists(os.path.join(REF, "dl_base.py"))):
        return {"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref"}
    import torch
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}
    rank = int(os.environ.get("RANK", 0))
    G = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    K, W, B = args.steps, args.warmup, c["batch"]
    accum = max(1, int(getattr(args, "accum", 1)))
    why = _preflight(c, G, B, accum, bool(getattr(args, "custom_cuda", False)), local)
    if why is not None:
        return {"impl": "reference", "unavailable": why} if rank == 0 else None
    work = os.environ.get("RENEE_REF_WORKDIR", "/tmp/renee_ref")
    data = os.path.join(work, f"LF-Synthetic-{c['labels']}-s{c['seq']}-n{(W + K) * B}")
    model_dir = os.path.join(work, "distilbert-random-init")
    os.makedirs(work, exist_ok=True)
    if rank == 0:
        _write_dataset(data, c, (W + K) * B, B)
        if not os.path.exists(os.path.join(model_dir, "config.json")):
            from transformers import DistilBertConfig, DistilBertModel
            torch.manual_seed(0)
            DistilBertModel(DistilBertConfig()).save_pretrained(model_dir)
    _wait_for(os.path.join(data, ".done"))
    _wait_for(os.path.join(model_dir, "config.json"))
    time.sleep(0.5 if rank else 0.0)

    sys.path.insert(0, SHIMS)
    sys.path.insert(0, REF)
    os.chdir(work)
    if not hasattr(np, "bool"):
        np.bool = bool
    import dl_base
    import main as refmain
    import torch.distributed as dist

    state = {"ev0": None, "ev1": None, "sampler": None, "clocks": None}
    orig_trange = dl_base.trange

    def timed_trange(*a, **kw):
        if kw.get("desc") != "Iteration":
            for x in orig_trange(*a, **kw):
                yield x
            return
        n = a[0]
        for i in range(n):
            if i == W:
                if G > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                if rank == 0:
                    from bench import ClockSampler
                    state["sampler"] = ClockSampler(local)
                    state["sampler"].start()
                state["ev0"] = torch.cuda.Event(enable_timing=True)
                state["ev0"].record()
            yield i
        state["ev1"] = torch.cuda.Event(enable_timing=True)
        state["ev1"].record()
        torch.cuda.synchronize()
        if G > 1:
            dist.barrier()
        if state["sampler"] is not None:
            state["clocks"] = state["sampler"].stop()

    dl_base.trange = timed_trange
    # The reference opens its own tcp:// rendezvous with rank 0 as the store's host.  Under torchrun the
    # variable below makes every rank connect as a client to a store the launcher is assumed to host on
    # that port, and the rendezvous never completes — so it is cleared for this process.
    os.environ.pop("TORCHELASTIC_USE_AGENT_STORE", None)
    port = int(os.environ.get("MASTER_PORT", "29500")) + 17
    ns = argparse.Namespace(
        data_dir=data, custom_cuda=bool(getattr(args, "custom_cuda", False)), default_impl=False, batch_size=B // G,
        epochs=1, expname="bench", device=None, dist_url=f"tcp://127.0.0.1:{port}", rank=0, world_size=G, seed=42,
        bottleneck_dims=0, dropout=c["dropout"], lr1=0.05, lr2=1e-5, mo=0.9, wd1=1e-4, wd2=0.01, fp32encoder=False,
        fp16xfc=True, noloss=True, checkpoint_resume="", infer=False, warmup=5000, accum=accum, pre_tok=True,
        maxlen=c["seq"], tf=model_dir, use_ngame_encoder="", compile=False)
    try:
        refmain.start(local, max(G, 1), ns)
    except torch.cuda.OutOfMemoryError as exc:
        msg = str(exc).splitlines()[0][:300]
        print(f"reference arm, rank {rank}: {msg}", file=sys.stderr, flush=True)
        out = {"impl": "reference", "unavailable": f"reference ran out of device memory: {msg}"}
        if G > 1:
            # ranks that did not fail sit in a collective: print the verdict and leave without joining it
            if rank == 0:
                import json
                print(json.dumps(out), flush=True)
            sys.stdout.flush()
            os._exit(0)
        return out
    if state["ev0"] is None or state["ev1"] is None:
        return {"impl": "reference", "unavailable": "reference loop ended before the timed region"} if rank == 0 else None
    ms = state["ev0"].elapsed_time(state["ev1"])
    t = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local}")
    if G > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    if G > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return None
    value = B * K / (ms / 1e3)
    b = B // G
    h2d = b * c["seq"] * 8 * 2 + int(B * (1 + c["lam"]) / G) * 16
    return {"metric": "train samples/sec (device-timed, max over ranks)", "value": round(value, 2), "unit": "samples/s",
            "n_gpus": G, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp16 autocast encoder, fp16 classifier compute (fp32 master)",
            "data": "synthetic seeded, random-init weights", "impl": "reference",
            "config": {"model": f"DistilBERT-style 6x768 encoder + label-sharded XFC, L={c['labels']}",
                       "name": getattr(args, "config", ""), "global_batch": B,
                       "seq_len": c["seq"], "labels": c["labels"],
                       "parallelism": f"dp{G} encoder + label-sharded classifier x{G}",
                       "flags": "--fp16xfc --noloss --dropout 0.85 --lr1 0.05 --lr2 1e-5 --wd1 1e-4"
                                + (f" --accum {accum}" if accum > 1 else ""),
                       "arm": "HF DistilBertModel under DDP, mean pooling, fp16 autocast"
                              + (", --custom-cuda" if ns.custom_cuda else ""),
                       "note": "the reference's loop is end to end by construction: DataLoader, pageable H2D, step"},
            "clocks": state["clocks"],
            "e2e": {"value": round(value, 2), "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 0},
            "gpu_launches": None}
