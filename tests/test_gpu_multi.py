"""Real multi-GPU check (needs >= 2 devices): the peer-memory collectives fused into the kernels give
the same training trajectory as the NCCL library collectives, eagerly and from CUDA graphs."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import numpy as np
    from renee_b200.data import xcrepo
    from renee_b200.data.collate import XCCollator
    from renee_b200.data.synthetic import SyntheticSpec, SyntheticXC
    from renee_b200.models.encoder import EncoderConfig
    from renee_b200.ops import cuda as cu
    from renee_b200.parallel.dist import init_distributed, shutdown
    from renee_b200.parallel.fused import PeerCollectives
    from renee_b200.train import TrainConfig, XCTrainer
    from renee_b200.utils.sharding import shard_labels

    ctx = init_distributed(rank, world, rank, timeout_s=120)
    enc = EncoderConfig(dim=256, n_layers=2, n_heads=4, hidden_dim=1024)
    L, B, S = 4096, 64, 16
    spec = SyntheticSpec(num_labels=L, seq_len=S, len_lo=4, len_hi=S, poisson_lam=2.0, seed=0)
    ids, mask, lab = SyntheticXC(spec).rows(np.arange(B * 4))
    ds = xcrepo.InMemoryDataset(ids, mask, lab)
    sh = shard_labels(L, world)
    coll = XCCollator(sh, ds, rank, 1, B, True)
    batches = [coll(np.arange(i * B, (i + 1) * B)) for i in range(4)]
    results = {}
    for name, fused, graph in (("nccl", False, False), ("peer", True, False), ("peer_graph", True, True)):
        cfg = TrainConfig(batch_size=B // world, epochs=1, seed=0, dropout=0.5, lr1=1e-3, lr2=1e-5, warmup=2, wd1=1e-4,
                          noloss=True, fp16xfc=True, maxlen=S, pooling="cls", cuda_graph=graph)
        # eager run on plain peer loads/stores, graph run with NVLS multimem where the allocation offers it
        comm = PeerCollectives(ctx, use_nvls=graph) if fused else None
        tr = XCTrainer(cfg, enc, sh, ctx, steps_per_epoch=100, comm=comm)
        for i in range(6):
            tr.train_step(batches[i % 4])
        torch.cuda.synchronize()
        cu.check_status()
        if graph:
            assert tr.graph_active()
            print(f"rank {rank}: multicast grad={comm._mc_grad != 0} p16={comm._mc_p16 != 0}", flush=True)
        results[name] = {k: v.cpu() for k, v in tr.state_dict().items()}
        if name == "peer":
            # cross-rank top-k merge over peer memory equals the NCCL all-gather + topk merge (several calls:
            # the buffers alternate by call parity; two sizes: the buffers grow on demand)
            from renee_b200.parallel.collectives import TorchCollectives
            lib_comm = TorchCollectives(ctx)
            g = torch.Generator(device=ctx.device).manual_seed(100 + rank)
            for n_rows, kk in ((37, 5), (64, 5), (64, 100), (37, 5)):
                vals = torch.randn(n_rows, kk, generator=g, device=ctx.device)
                idxs = torch.randint(0, 1 << 20, (n_rows, kk), generator=g, device=ctx.device) + rank * (1 << 20)
                v1, i1 = comm.merge_topk(vals, idxs, kk)
                v2, i2 = lib_comm.merge_topk(vals, idxs, kk)
                torch.testing.assert_close(v1, v2, rtol=0, atol=0)
                assert torch.equal(i1, i2)
            torch.cuda.synchronize()
            cu.check_status()
        torch.distributed.barrier()
    torch.save(results, os.path.join(out_dir, f"r{rank}.pt"))
    shutdown()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_peer_collectives_match_nccl(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), f"r{r}.pt"), weights_only=False)
        for name in ("peer", "peer_graph"):
            for k, v in res["nccl"].items():
                # same math, different summation order (atomics, bf16 all-reduce): agreement to bf16 precision
                torch.testing.assert_close(res[name][k], v, rtol=3e-2, atol=3e-3, msg=lambda m: f"{name}/{k}: {m}")


def _shard_worker(rank, world, port, out_dir):
    """Four steps at dropout 0 (dropout masks are indexed by the LOCAL row, so they differ between world sizes)
    with the default peer-memory backend (plain peer mappings, CUDA graphs); saves this rank's state."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import numpy as np
    from renee_b200.data import xcrepo
    from renee_b200.data.collate import XCCollator
    from renee_b200.data.synthetic import SyntheticSpec, SyntheticXC
    from renee_b200.models.encoder import EncoderConfig
    from renee_b200.ops import cuda as cu
    from renee_b200.parallel.dist import DistContext, init_distributed, shutdown
    from renee_b200.parallel.fused import PeerCollectives
    from renee_b200.train import TrainConfig, XCTrainer
    from renee_b200.utils.sharding import shard_labels

    if world > 1:
        ctx = init_distributed(rank, world, rank, timeout_s=120)
    else:
        torch.cuda.set_device(0)
        ctx = DistContext(device=torch.device("cuda", 0))
    enc = EncoderConfig(dim=256, n_layers=2, n_heads=4, hidden_dim=1024, dropout=0.0, attention_dropout=0.0)
    L, B, S = 4000, 64, 16
    spec = SyntheticSpec(num_labels=L, seq_len=S, len_lo=4, len_hi=S, poisson_lam=2.0, seed=0)
    ids, mask, lab = SyntheticXC(spec).rows(np.arange(B * 4))
    ds = xcrepo.InMemoryDataset(ids, mask, lab)
    sh = shard_labels(L, world)
    coll = XCCollator(sh, ds, rank, 1, B, True)
    cfg = TrainConfig(batch_size=B // world, epochs=1, seed=0, dropout=0.0, lr1=1e-2, lr2=1e-5, warmup=2, wd1=1e-4,
                      noloss=True, fp16xfc=True, maxlen=S, pooling="cls", stochastic_round=False)
    comm = PeerCollectives(ctx) if world > 1 else None
    if comm is not None:
        assert not comm.use_nvls            # the default binds no multicast object
    tr = XCTrainer(cfg, enc, sh, ctx, steps_per_epoch=100, comm=comm)
    for i in range(4):
        tr.train_step(coll(np.arange(i * B, (i + 1) * B)))
    torch.cuda.synchronize()
    cu.check_status()
    sd = {k: v.cpu() for k, v in tr.state_dict().items()}
    torch.save(sd, os.path.join(out_dir, f"g{world}_r{rank}.pt"))
    if world > 1:
        torch.distributed.barrier()
        shutdown()


@pytest.mark.parametrize("world,overlap", [(2, "0"), (2, "1"), (4, "0"), (8, "0")])
def test_sharding_invariance_against_one_gpu(tmp_path, world, overlap, monkeypatch):
    """Label-sharded training on G GPUs gives the single-GPU weights: the classifier shards, concatenated, equal
    the G = 1 matrix and every rank's encoder equals the G = 1 encoder (up to summation order in 16 bits).  With
    two GPUs also with the gradient reduce-scatter issued bucket by bucket under the backward pass (opt-in)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    monkeypatch.setenv("RENEE_B200_RS_OVERLAP", overlap)      # inherited by the spawned ranks
    out = str(tmp_path)
    mp.spawn(_shard_worker, args=(1, _free_port(), out), nprocs=1, join=True)
    mp.spawn(_shard_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    one = torch.load(os.path.join(out, "g1_r0.pt"), weights_only=False)
    parts = [torch.load(os.path.join(out, f"g{world}_r{r}.pt"), weights_only=False) for r in range(world)]
    W = torch.cat([p["xfc_weight"] for p in parts])[:4000]
    torch.testing.assert_close(W, one["xfc_weight"][:4000], rtol=3e-2, atol=2e-3)
    for r, p in enumerate(parts):
        for k, v in one.items():
            if k != "xfc_weight":
                torch.testing.assert_close(p[k], v, rtol=3e-2, atol=3e-3, msg=lambda m: f"rank {r} {k}: {m}")


def _leave_worker(rank, world, port, out_dir):
    """Rank 1 leaves between steps (no kernel or collective of its own in flight); rank 0 must notice on the host,
    before launching anything that would wait for it.  NVLS is off in NCCL and the trainer's own buffers are plain
    peer mappings (the default), so no multicast object exists in this run."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", RENEE_B200_NVLS="0")
    import time
    import numpy as np
    import torch.distributed as dist
    from renee_b200.data import xcrepo
    from renee_b200.data.collate import XCCollator
    from renee_b200.data.synthetic import SyntheticSpec, SyntheticXC
    from renee_b200.models.encoder import EncoderConfig
    from renee_b200.ops import cuda as cu
    from renee_b200.parallel.dist import init_distributed
    from renee_b200.parallel.fused import PeerCollectives
    from renee_b200.parallel.watchdog import Heartbeat, PeerFailure
    from renee_b200.train import TrainConfig, XCTrainer
    from renee_b200.utils.sharding import shard_labels

    ctx = init_distributed(rank, world, rank, timeout_s=60)
    enc = EncoderConfig(dim=256, n_layers=2, n_heads=4, hidden_dim=1024)
    L, B, S = 4096, 32, 16
    spec = SyntheticSpec(num_labels=L, seq_len=S, len_lo=4, len_hi=S, poisson_lam=2.0, seed=0)
    ids, mask, lab = SyntheticXC(spec).rows(np.arange(B * 2))
    ds = xcrepo.InMemoryDataset(ids, mask, lab)
    sh = shard_labels(L, world)
    coll = XCCollator(sh, ds, rank, 1, B, True)
    cfg = TrainConfig(batch_size=B // world, epochs=1, seed=0, dropout=0.5, lr1=1e-3, lr2=1e-5, warmup=2, wd1=1e-4,
                      noloss=True, fp16xfc=True, maxlen=S, pooling="cls")
    comm = PeerCollectives(ctx)
    assert not comm.use_nvls and comm._mc_grad == 0 and comm._mc_p16 == 0
    tr = XCTrainer(cfg, enc, sh, ctx, steps_per_epoch=100, comm=comm)
    store = dist.distributed_c10d._get_default_store()
    tr.watchdog = Heartbeat(store, rank, world, interval=0.2, timeout=1.5).start()
    batch = coll(np.arange(B))
    for _ in range(4):
        tr.train_step(batch)
    torch.cuda.synchronize()                 # nothing of this rank is in flight any more
    cu.check_status()
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 1:
        tr.watchdog.stop()
        os._exit(0)                          # leaves between steps, without any tear-down collective
    t0 = time.time()
    caught = None
    while time.time() - t0 < 20.0:
        try:
            tr.watchdog.check()
        except PeerFailure as exc:
            caught = exc
            break
        time.sleep(0.1)
    ok = caught is not None and caught.ranks == [1]
    raised_before_launch = False
    n0 = cu.launch_count()
    try:
        tr.train_step(batch)
    except PeerFailure:
        raised_before_launch = cu.launch_count() == n0
    # the context is intact: an ordinary kernel still runs and no bounded wait has expired
    x = torch.randn(64, 256, device=ctx.device).bfloat16()
    s = torch.empty(256, device=ctx.device, dtype=torch.bfloat16)
    cu.colsum(x, s)
    torch.cuda.synchronize()
    cu.check_status()
    with open(os.path.join(out_dir, "leave.txt"), "w") as f:
        f.write(f"{int(ok)} {int(raised_before_launch)} {int(tr._aborted)} {time.time() - t0:.2f}")
    tr.watchdog.stop()
    os._exit(0)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_rank_leaving_between_steps_is_noticed_before_any_launch(tmp_path):
    mp.spawn(_leave_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    ok, before, aborted, secs = open(os.path.join(str(tmp_path), "leave.txt")).read().split()
    assert ok == "1" and before == "1" and aborted == "1" and float(secs) < 10.0
