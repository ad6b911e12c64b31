"""Label padding/sharding rule (reference main.py:76-97) and batch row split (dl_base.py:348-358)."""
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
