"""Label padding/sharding rule (reference main.py:76-97) and batch row split (dl_base.py:348-358)."""
import pytest

from renee_b200.utils.sharding import batch_row_range, shard_labels


def test_padding_rule_matches_reference_arithmetic():
    for L in (131072, 131073, 4096, 1310720, 100_000_000, 17, 670091):
        for G in (1, 2, 3, 4, 8, 16):
            padded = L
            if padded % G != 0:
                padded = G * ((L + G - 1) // G)
            per = padded // G
            if per % 16 != 0:
                padded = G * 16 * ((per + 15) // 16)
                per = padded // G
            s = shard_labels(L, G)
            assert (s.padded_labels, s.labels_per_rank) == (padded, per)
            assert s.labels_per_rank % 16 == 0 and s.padded_labels >= L
            assert s.shard_range(G - 1)[1] == s.padded_labels


def test_batch_rows_cover_and_spread_remainder():
    for B in (256, 250, 7, 9):
        for G in (1, 2, 4, 8):
            rows = [batch_row_range(B, G, r) for r in range(G)]
            assert rows[0][0] == 0 and rows[-1][1] == B
            for a, b in zip(rows, rows[1:]):
                assert a[1] == b[0]
            sizes = [e - s for s, e in rows]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


@pytest.mark.parametrize("G", [2, 3, 8])
def test_gradient_buckets_partition_the_flat_buffer(G):
    """Every rank owns 1/G of every bucket of the flat gradient buffer: over all ranks the owned ranges cover the
    buffer exactly once, on 16-byte boundaries, and the reduce plan of a rank is its owned ranges in backward order
    with consecutive offsets into its fp32 sum buffer."""
    from types import SimpleNamespace

    import torch

    from renee_b200.models.encoder import EncoderConfig
    from renee_b200.models.flat_encoder import FlatEncoder
    from renee_b200.parallel.fused import PeerCollectives

    enc = FlatEncoder(EncoderConfig(dim=128, n_layers=3, n_heads=2, hidden_dim=256, vocab_size=200, max_position_embeddings=16),
                      "cpu", torch.float32, "cls", 0, seed=1)
    covered = torch.zeros(enc.numel, dtype=torch.int32)
    for rank in range(G):
        pc = SimpleNamespace(G=G, rank=rank, gsum=None, ctx=SimpleNamespace(device=torch.device("cpu")))
        plan = PeerCollectives._buckets(pc, enc)
        pc._buckets = lambda e, _pc=pc: _pc._bucket_plan
        owned = PeerCollectives.owned_ranges(pc, enc, rank)
        assert sorted((a * 8, b * 8) for _, a, b, _ in plan) == sorted(owned)
        stages = [s for s, _, _, _ in plan]
        assert stages == sorted(stages) and stages[0] == 1 and stages[-1] == enc.cfg.n_layers + 1
        g = 0
        for _, a, b, g0 in plan:
            assert g0 == g and b > a
            g += b - a
        assert pc.gsum.numel() >= g * 8
        for a, b in owned:
            assert a % 8 == 0 and b % 8 == 0
            covered[a:b] += 1
    n = enc.numel // 8 * 8
    assert int(covered[:n].min()) == 1 and int(covered[:n].max()) == 1
