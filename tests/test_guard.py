"""Guard-band allocation (``renee_b200/utils/guard.py``): detection logic on CPU, the trainer's buffers
under guard mode on CPU and (GPU) the same after real kernel launches."""
import numpy as np
import pytest
import torch

from renee_b200.utils import guard


def test_disabled_returns_plain_tensors():
    guard.enable(False)
    t = guard.zeros(3, 5, dtype=torch.float16)
    assert t.shape == (3, 5) and t.dtype == torch.float16 and guard.registered() == 0
    assert guard.from_allocator(lambda n, dt: torch.empty(n, dtype=dt), 7, torch.float32).numel() == 7
    assert guard.check() == []


def test_detects_writes_on_either_side_and_names_the_buffer():
    with guard.enabled_for_test():
        a = guard.zeros(10, 3, dtype=torch.float32, name="a")
        b = guard.empty(5, dtype=torch.int32, name="b")
        c = guard.from_allocator(lambda n, dt: torch.empty(n, dtype=dt), 100, torch.float16, name="c")
        assert a.shape == (10, 3) and float(a.abs().sum()) == 0.0 and c.numel() == 100
        for t in (a, b, c):
            assert t.data_ptr() % 64 == 0      # the band keeps the allocator's alignment (64 B on CPU, 512 B on CUDA)
        a.fill_(1.0); b.fill_(7); c.fill_(2.0)          # in-bounds writes leave the bands alone
        guard.assert_clean()
        # one element past the end of `a`, one element before the start of `c`
        torch.as_strided(a, (1,), (1,), storage_offset=a.storage_offset() + a.numel()).fill_(3.0)
        torch.as_strided(c, (1,), (1,), storage_offset=c.storage_offset() - 1).fill_(3.0)
        bad = guard.check()
        assert len(bad) == 2
        assert bad[0].startswith("a: 4 byte(s) after the buffer, nearest at offset 120")
        assert bad[1].startswith("c: 2 byte(s) before the buffer, nearest at offset -1")
        with pytest.raises(guard.GuardError):
            guard.assert_clean()
    assert not guard.enabled() and guard.registered() == 0


def _tiny_trainer(device, fp16xfc, B=24, S=20):
    from renee_b200.data import xcrepo
    from renee_b200.data.collate import XCCollator
    from renee_b200.data.synthetic import SyntheticSpec, SyntheticXC
    from renee_b200.models.encoder import EncoderConfig
    from renee_b200.parallel.dist import DistContext
    from renee_b200.train import TrainConfig, XCTrainer
    from renee_b200.utils.sharding import shard_labels
    L = 1000                        # ragged on purpose: B not a multiple of 8, L not of 16, S not of 16
    spec = SyntheticSpec(num_labels=L, seq_len=S, len_lo=3, len_hi=S, poisson_lam=2.0, zipf_s=1.1, seed=1)
    ids, mask, lab = SyntheticXC(spec).rows(np.arange(4 * B))
    ds = xcrepo.InMemoryDataset(ids, mask, lab)
    sh = shard_labels(L, 1)
    ctx = DistContext(rank=0, world_size=1, local_rank=0, device=torch.device(device), backend=None)
    enc = EncoderConfig(vocab_size=30522, dim=128, n_layers=2, n_heads=2, hidden_dim=256,
                        max_position_embeddings=max(64, S))
    cfg = TrainConfig(batch_size=B, epochs=1, seed=0, dropout=0.5, lr1=0.05, lr2=1e-4, warmup=10, wd1=1e-4,
                      noloss=False, fp16xfc=fp16xfc, maxlen=S, pooling="mean")
    tr = XCTrainer(cfg, enc, sh, ctx, steps_per_epoch=100)
    coll = XCCollator(sh, ds, 0, 1, B, True)
    return tr, [coll(np.arange(i * B, (i + 1) * B)) for i in range(4)]


def test_trainer_buffers_are_guarded_and_clean_on_cpu():
    with guard.enabled_for_test():
        tr, batches = _tiny_trainer("cpu", fp16xfc=False)
        for b in batches:
            tr.train_step(b)
        assert guard.registered() > 20
        tr.check_device_status()
        w_guarded = tr.xfc.W.clone()
    tr2, batches2 = _tiny_trainer("cpu", fp16xfc=False)
    for b in batches2:
        tr2.train_step(b)
    torch.testing.assert_close(tr2.xfc.W, w_guarded, rtol=0, atol=0)     # guard mode changes no result


@pytest.mark.gpu
def test_kernels_leave_guard_bands_intact():
    """Every kernel of the training step, eagerly and from the CUDA graph, on ragged shapes: nothing may land in
    the bands around the framework's buffers."""
    from renee_b200.ops import cuda as cu
    with guard.enabled_for_test():
        tr, batches = _tiny_trainer("cuda:0", fp16xfc=True)
        for i in range(8):
            tr.train_step(batches[i % len(batches)])
        torch.cuda.synchronize()
        assert guard.registered() > 20
        tr.check_device_status()
        cu.check_status()
        assert torch.isfinite(tr.xfc.W.float()).all()


@pytest.mark.gpu
def test_long_sequence_step_from_graph_leaves_guard_bands_intact():
    """Sequences of 129..512 tokens take the blocked attention kernels (two-pass forward, dQ and dK/dV backward
    kernels with a softmax-gradient scratch): a few steps, eager and replayed from the CUDA graph."""
    from renee_b200.ops import cuda as cu
    with guard.enabled_for_test():
        tr, batches = _tiny_trainer("cuda:0", fp16xfc=True, B=6, S=164)
        w0 = tr.encoder.p32.clone()
        for i in range(6):
            tr.train_step(batches[i % len(batches)])
        torch.cuda.synchronize()
        tr.check_device_status()
        cu.check_status()
        assert tr.graph_active()
        assert "ds" in tr.encoder._acts["layers"][0]["att"]
        assert torch.isfinite(tr.encoder.p32).all() and not torch.equal(w0, tr.encoder.p32)


def test_symmetric_allocation_addresses_follow_the_payload(monkeypatch):
    """``PeerCollectives._symm`` with a stand-in for the symmetric-memory module: without guard mode the peer and
    multicast addresses are the allocation's own; in guard mode they are shifted by one band, like the payload."""
    import sys
    import types
    from renee_b200.parallel import fused

    class Handle:
        def __init__(self, t):
            self.buffer_ptrs = [t.data_ptr(), t.data_ptr() + (1 << 30)]
            self.multicast_ptr = 1 << 40

    fake = types.ModuleType("torch.distributed._symmetric_memory")
    fake.empty = lambda n, dtype, device: torch.empty(n, dtype=dtype, device=device)
    fake.rendezvous = lambda t, group: Handle(t)
    monkeypatch.setitem(sys.modules, "torch.distributed._symmetric_memory", fake)
    import torch.distributed as dist
    monkeypatch.setattr(dist, "_symmetric_memory", fake, raising=False)

    class Ctx:
        device = torch.device("cpu")

    def make():
        pc = fused.PeerCollectives.__new__(fused.PeerCollectives)
        pc.ctx, pc.group, pc._handles, pc.use_nvls = Ctx(), None, [], True
        return pc

    guard.enable(False)
    pc = make()
    t, ptrs = pc._symm(1000, torch.float16)
    assert t.numel() == 1000 and ptrs[0] == t.data_ptr() and ptrs[1] == t.data_ptr() + (1 << 30)
    assert pc._last_multicast == 1 << 40
    with guard.enabled_for_test():
        pc = make()
        t, ptrs = pc._symm(1000, torch.float16)
        assert t.numel() == 1000 and ptrs[0] == t.data_ptr() and ptrs[1] == t.data_ptr() + (1 << 30)
        assert pc._last_multicast == (1 << 40) + guard.BAND_BYTES
        t.fill_(1.0)
        guard.assert_clean()
        # without NVLS the buffers come from plain CUDA IPC mappings instead (no multicast object at all)
        pc.use_nvls = False
        called = []
        monkeypatch.setattr(fused.PeerCollectives, "_ipc", lambda self, n, dt, name: called.append((n, dt)) or ("t", [0]))
        assert pc._symm(10, torch.int32) == ("t", [0]) and called == [(10, torch.int32)]
