"""Command line of the trainer — flag-compatible with the reference's ``main.py``.

All 30 reference flags are accepted with the same names, types and defaults (main.py:190-255);
``--pre-tok`` and ``--compile`` are parsed for compatibility and have no effect (data is always
pre-tokenised, as in the reference; the encoder here is hand-fused, so there is nothing to hand to a
tracing compiler).  ``--world-size`` counts nodes and ``--rank`` is the node rank, exactly as in the
reference (main.py:263-264); under ``torchrun`` the environment's rank/world take precedence.

Additional flags select the pooling, the synthetic workload generator and engine options.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="BERT XFC (Blackwell-native)")
    p.add_argument("--data-dir", type=str, default="", help="Path to dataset directory")
    p.add_argument("--custom-cuda", action="store_true", default=False,
                   help="Accepted for compatibility: the fused sm_100a kernels are always used with --fp16xfc on a GPU")
    p.add_argument("--default-impl", action="store_true", default=False,
                   help="Autograd baseline: dense targets + BCEWithLogitsLoss")
    p.add_argument("--batch-size", type=int, default=8, metavar="N", help="per GPU batch size (default: 8)")
    p.add_argument("--epochs", type=int, default=50, metavar="N")
    p.add_argument("--expname", type=str, default="renee-exp", metavar="N")
    p.add_argument("--device", type=int, default=None, metavar="N", help="Single device training")
    p.add_argument("--dist-url", default="tcp://localhost:23456", type=str)
    p.add_argument("--rank", type=int, default=0, metavar="N", help="Rank of node")
    p.add_argument("--world-size", type=int, default=1, metavar="N", help="Number of nodes")
    p.add_argument("--seed", type=int, default=42, metavar="N")
    p.add_argument("--bottleneck-dims", type=int, default=0, metavar="N")
    p.add_argument("--dropout", type=float, default=0.5, metavar="N")
    p.add_argument("--lr1", type=float, default=0.0025, metavar="LR", help="learning rate for xfc layer")
    p.add_argument("--lr2", type=float, default=1e-5, metavar="LR", help="learning rate for encoder")
    p.add_argument("--mo", type=float, default=0.9, metavar="MO")
    p.add_argument("--wd1", type=float, default=0.01, metavar="WD")
    p.add_argument("--wd2", type=float, default=0.01, metavar="WD")
    p.add_argument("--fp32encoder", action="store_true", default=False)
    p.add_argument("--fp16xfc", action="store_true", default=False)
    p.add_argument("--noloss", action="store_true", default=False)
    p.add_argument("--checkpoint-resume", type=str, default="")
    p.add_argument("--infer", action="store_true", default=False)
    p.add_argument("--warmup", type=int, default=140000, metavar="N")
    p.add_argument("--accum", type=int, default=1, metavar="N")
    p.add_argument("--pre-tok", action="store_true", default=False)
    p.add_argument("--maxlen", type=int, default=32, metavar="N")
    p.add_argument("--tf", type=str, default="distilbert-base-uncased", metavar="N")
    p.add_argument("--use-ngame-encoder", type=str, default="")
    p.add_argument("--compile", action="store_true", default=False)
    # ---- extensions
    p.add_argument("--pooling", choices=["mean", "cls"], default="mean")
    p.add_argument("--encoder-dtype", choices=["bf16", "fp16"], default="bf16")
    p.add_argument("--encoder-weights", type=str, default="", help="state_dict (.pt) with HF DistilBERT keys")
    p.add_argument("--synthetic-labels", type=int, default=0, help="generate a synthetic workload with this many labels")
    p.add_argument("--synthetic-train", type=int, default=4096)
    p.add_argument("--synthetic-test", type=int, default=512)
    p.add_argument("--synthetic-lam", type=float, default=1.3)
    p.add_argument("--synthetic-zipf", type=float, default=1.1)
    p.add_argument("--synthetic-len-lo", type=int, default=6)
    p.add_argument("--no-cuda-graph", dest="cuda_graph", action="store_false", default=True)
    p.add_argument("--no-fused-comm", dest="fused_comm", action="store_false", default=True)
    p.add_argument("--no-stochastic-round", dest="stochastic_round", action="store_false", default=True,
                   help="with --fp16xfc: round the updated fp16 classifier weights to nearest instead of stochastically")
    p.add_argument("--cpu", action="store_true", default=False, help="force CPU (gloo) execution")
    p.add_argument("--heartbeat-timeout", type=float, default=60.0,
                   help="seconds without a peer heartbeat before a step is refused (0 disables the watchdog)")
    p.add_argument("--results-dir", type=str, default="./Results/Bert-XC/")
    return p


def _load_data(args, rank: int):
    """Returns ``(trn_dataset, tst_dataset, num_labels, tst_labels, filter_mat, inv_prop)``."""
    from .data import xcrepo
    from .data.synthetic import SyntheticSpec, SyntheticXC
    from .utils.metrics import compute_inv_propensity, propensity_constants

    if args.synthetic_labels > 0:
        spec = SyntheticSpec(num_labels=args.synthetic_labels, seq_len=args.maxlen, len_lo=min(args.synthetic_len_lo, args.maxlen),
                             len_hi=args.maxlen, poisson_lam=args.synthetic_lam, zipf_s=args.synthetic_zipf, seed=args.seed)
        gen = SyntheticXC(spec)
        ids, mask, labels = gen.rows(np.arange(args.synthetic_train))
        tids, tmask, tlabels = gen.rows(np.arange(args.synthetic_train, args.synthetic_train + args.synthetic_test))
        trn = xcrepo.InMemoryDataset(ids, mask, labels)
        tst = xcrepo.InMemoryDataset(tids, tmask, tlabels)
        filt = None
        dataset_name = "synthetic"
    else:
        d = args.data_dir
        labels = xcrepo.read_sparse_file(os.path.join(d, "trn_X_Y.txt"))
        tlabels = xcrepo.read_sparse_file(os.path.join(d, "tst_X_Y.txt"))
        folder = os.path.join(d, f"{xcrepo.tokenizer_folder(args.tf)}-{args.maxlen}")
        trn = xcrepo.PreTokDataset(folder, labels, labels.shape[0], args.maxlen, "trn")
        tst = xcrepo.PreTokDataset(folder, tlabels, tlabels.shape[0], args.maxlen, "tst")
        filt = xcrepo.read_filter_file(os.path.join(d, "tst_filter_labels.txt"), tlabels.shape)
        dataset_name = d.rstrip("/").split("/")[-1]
    A, B = propensity_constants(dataset_name)
    inv_prop = compute_inv_propensity(labels, A, B)
    return trn, tst, labels.shape[1], tlabels, filt, inv_prop, dataset_name


def start(local_device: int, ngpus_per_node: int, args) -> None:
    """Per-process entry (the reference's ``start``, main.py:20-186)."""
    from .data.collate import GlobalBatchSampler, PrefetchLoader, XCCollator
    from .evaluate import FullPredictor, PrecEvaluator
    from .models.encoder import config_from_name, strip_ngame_prefix
    from .parallel.dist import env_world, init_distributed, shutdown
    from .train import TrainConfig, XCTrainer, seed_everything
    from .utils.sharding import shard_labels

    seed_everything(args.seed)
    env = env_world()
    if env is not None:
        ctx = init_distributed(device="cpu" if args.cpu else None)
    elif args.world_size > 1:
        rank = args.rank * ngpus_per_node + local_device if args.world_size > ngpus_per_node else local_device
        ctx = init_distributed(rank, args.world_size, local_device, init_method=args.dist_url,
                               device="cpu" if args.cpu else None)
    else:
        ctx = init_distributed(0, 1, local_device or 0, device="cpu" if args.cpu else None)
    rank, G = ctx.rank, ctx.world_size

    trn, tst, L, tst_labels, filt, inv_prop, dataset_name = _load_data(args, rank)
    sharding = shard_labels(L, G)
    if ctx.is_main:
        if sharding.padded_labels != L:
            print("Rounding numy to", sharding.padded_labels)
        print("Final numy_per_gpu: ", sharding.labels_per_rank)

    gbsz = args.batch_size * G
    xfcz = max(1, gbsz // args.accum)
    trn_loader = PrefetchLoader(GlobalBatchSampler(len(trn), gbsz, True, args.seed),
                                XCCollator(sharding, trn, rank, args.accum, xfcz, True, args.default_impl),
                                pin=ctx.device.type == "cuda")
    tst_loader = PrefetchLoader(GlobalBatchSampler(len(tst), gbsz, False, args.seed),
                                XCCollator(sharding, tst, rank, args.accum, xfcz, False, False),
                                pin=ctx.device.type == "cuda")

    enc_cfg = config_from_name(args.tf)
    cfg = TrainConfig.from_args(args)
    cfg.out_dir = os.path.join(args.results_dir, dataset_name, args.expname)
    comm = None
    if G > 1 and ctx.device.type == "cuda" and args.fused_comm and not args.default_impl:
        import socket
        import torch.distributed as dist
        hosts = [None] * G
        dist.all_gather_object(hosts, socket.gethostname())
        if len(set(hosts)) == 1:
            from .parallel.fused import PeerCollectives
            comm = PeerCollectives(ctx)          # NVLink peer memory: all ranks on one node
        elif ctx.is_main:
            print("ranks span several nodes: using the NCCL collectives (peer-memory kernels are intra-node)")
    trainer = XCTrainer(cfg, enc_cfg, sharding, ctx, steps_per_epoch=len(trn_loader), comm=comm)
    if G > 1 and args.heartbeat_timeout > 0:
        import torch.distributed as dist
        from .parallel.watchdog import Heartbeat
        store = dist.distributed_c10d._get_default_store()
        trainer.watchdog = Heartbeat(store, rank, G, interval=1.0, timeout=args.heartbeat_timeout).start()

    init_sd = None
    if args.use_ngame_encoder:
        print(f"Using NGAME pretrained encoder. Loading from {args.use_ngame_encoder}")
        init_sd = strip_ngame_prefix(torch.load(args.use_ngame_encoder, map_location="cpu"))
    elif args.encoder_weights:
        init_sd = torch.load(args.encoder_weights, map_location="cpu")
    if init_sd is not None and any("attention.self.query.weight" in k for k in init_sd):
        from .models.encoder import convert_bert_state_dict
        init_sd = convert_bert_state_dict(init_sd, roberta="roberta" in args.tf.lower())   # BERT / RoBERTa / MiniLM keys
    if init_sd is not None:
        if args.default_impl:
            trainer.model.embed[0].transformer.load_state_dict(init_sd, strict=True)
        else:
            trainer.encoder.load_encoder_state_dict(init_sd, strict=True)

    evaluator = PrecEvaluator(tst_loader, FullPredictor(), tst_labels if ctx.is_main else None,
                              filter_mat=filt, inv_prop=inv_prop)
    if args.infer:
        trainer.load()
        evaluator(trainer, -1, -1.0, None, trainer.name)
    else:
        trainer.fit(trn_loader, evaluator)
    shutdown()


def main(argv=None) -> None:
    args = build_parser().parse_args(argv)
    print(args)
    from .parallel.dist import env_world
    if args.device is not None:
        print("Specific device chosen. Starting single device training")
        start(args.device, 1, args)
        return
    if env_world() is not None:
        start(int(os.environ.get("LOCAL_RANK", 0)), max(1, torch.cuda.device_count()), args)
        return
    ngpus = torch.cuda.device_count() if (torch.cuda.is_available() and not args.cpu) else 1
    args.world_size *= ngpus
    if args.batch_size * args.world_size % args.accum != 0:
        print("Code currently expects  args.accum cleanly divides args.batch_size*args.world_size")
        sys.exit(-1)
    if args.world_size == 1:
        start(0, 1, args)
        return
    print("Starting multi device training on ", args.world_size, " devices")
    import torch.multiprocessing as mp
    mp.spawn(start, nprocs=ngpus, args=(ngpus, args), join=True)


if __name__ == "__main__":
    main()
