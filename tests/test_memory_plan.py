"""``utils/memory_plan.py``: the meta-device dry run must add up to what a real instantiation allocates."""
import torch

from renee_b200.utils import guard
from renee_b200.utils.memory_plan import plan


def _real_bytes(labels, batch, seq, enc):
    from renee_b200.parallel.dist import DistContext
    from renee_b200.train import TrainConfig, XCTrainer
    from renee_b200.utils.sharding import shard_labels
    cfg = TrainConfig(batch_size=batch, epochs=1, seed=0, dropout=0.5, lr1=0.05, lr2=1e-5, warmup=10, wd1=1e-4,
                      noloss=True, fp16xfc=False, fp32encoder=True, maxlen=seq, pooling="cls")
    ctx = DistContext(rank=0, world_size=1, local_rank=0, device=torch.device("cpu"), backend=None)
    with guard.enabled_for_test():
        tr = XCTrainer(cfg, enc, shard_labels(labels, 1), ctx, steps_per_epoch=10)
        tr.encoder._alloc(batch + 1, seq)
        tr.xfc.scratch(batch)
        return sum(e.hi - e.lo for e in guard._registry)


def test_plan_matches_a_real_cpu_instantiation():
    from renee_b200.models.encoder import EncoderConfig
    enc = EncoderConfig(vocab_size=1000, dim=128, n_layers=2, n_heads=2, hidden_dim=256, max_position_embeddings=32)
    p = plan(labels=3000, gpus=1, global_batch=16, seq=24, enc_cfg=enc, fp16xfc=False, fp32encoder=True)
    real = _real_bytes(3000, 16, 24, enc)
    assert abs(p["framework_total_gb"] * 1e9 - real) <= 0.005e9 + 1      # the plan rounds to 10 MB
    exact = sum(v for v in p["per_gpu_gb"].values())
    assert exact > 0 and p["fits_180gb"]


def test_plan_of_the_100m_label_config_fits_and_the_reference_layout_does_not():
    p = plan(labels=100_000_000, gpus=8, global_batch=1024, seq=32)
    assert p["config"]["labels_per_gpu"] == 12_500_000
    assert abs(p["per_gpu_gb"]["xfc.W"] - 19.2) < 0.01 and abs(p["per_gpu_gb"]["xfc.M"] - 19.2) < 0.01
    assert p["with_allowance_gb"] < 60 and p["fits_180gb"]
    # fp32 master + gradient + momentum + fp16 copy + the [B, Ls] fp16 logits buffer of the reference's layout
    assert p["reference_layout_gb"]["classifier_state_and_logits"] > 150
