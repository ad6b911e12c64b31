"""On-disk formats, synthetic generator determinism and the collator's sharded positives."""
import numpy as np
import scipy.sparse as sp
import torch

from renee_b200.data import xcrepo
from renee_b200.data.collate import GlobalBatchSampler, XCCollator
from renee_b200.data.synthetic import SyntheticSpec, SyntheticXC, ZipfSampler
from renee_b200.utils.sharding import batch_row_range, shard_labels


def test_sparse_file_roundtrip(tmp_path):
    m = sp.random(20, 50, density=0.1, format="csr", random_state=0, dtype=np.float32)
    m.data[:] = 1.0
    p = tmp_path / "trn_X_Y.txt"
    xcrepo.write_sparse_file(m, str(p))
    assert open(p).readline().split() == ["20", "50"]
    back = xcrepo.read_sparse_file(str(p))
    assert (back != m).nnz == 0


def test_reads_reference_sample_format(tmp_path):
    p = tmp_path / "tst_X_Y.txt"
    p.write_text("2 131073\n42537:1.00000 43834:1.00000\n\n")
    m = xcrepo.read_sparse_file(str(p))
    assert m.shape == (2, 131073) and m[0].indices.tolist() == [42537, 43834] and m[1].nnz == 0


def test_filter_and_token_files(tmp_path):
    xcrepo.write_filter_file(np.array([[0, 3], [1, 2]]), str(tmp_path / "f.txt"))
    f = xcrepo.read_filter_file(str(tmp_path / "f.txt"), (2, 5))
    assert f[0, 3] == 1 and f[1, 2] == 1 and f.nnz == 2
    ids = np.arange(12).reshape(3, 4)
    xcrepo.write_token_files(str(tmp_path / "bert-base-uncased-4"), "trn_doc", ids, (ids > 0).astype(np.int64))
    ds = xcrepo.PreTokDataset(str(tmp_path / "bert-base-uncased-4"), None, 3, 4, "trn")
    a, b = ds.get_fts([2, 0])
    assert a.tolist() == [[8, 9, 10, 11], [0, 1, 2, 3]] and b[1].tolist() == [0, 1, 1, 1]
    assert xcrepo.tokenizer_folder("sentence-transformers/msmarco-distilbert-base-v4") == "bert-base-uncased"
    assert xcrepo.tokenizer_folder("paraphrase-distilroberta-base-v2") == "roberta-base"


def test_synthetic_is_deterministic_and_well_formed():
    spec = SyntheticSpec(num_labels=4096, seq_len=32, len_lo=8, len_hi=32, poisson_lam=2.0, seed=0)
    a = SyntheticXC(spec).rows(np.arange(100, 140))
    b = SyntheticXC(spec).rows(np.arange(100, 140))
    assert (a[0] == b[0]).all() and (a[2] != b[2]).nnz == 0
    ids, mask, lab = a
    lens = mask.sum(1)
    assert lens.min() >= 8 and lens.max() <= 32
    assert ((ids == 0) == (mask == 0)).all() and ids[mask == 1].min() >= 1000 and ids.max() < 30522
    nnz = np.diff(lab.indptr)
    assert nnz.min() >= 1 and lab.indices.max() < 4096
    for r in range(lab.shape[0]):
        assert len(set(lab[r].indices.tolist())) == nnz[r]


def test_zipf_head_heavier_than_tail():
    z = ZipfSampler(10_000_000, 1.1)
    x = z.sample(np.random.default_rng(0), 20000)
    assert x.min() >= 0 and x.max() < 10_000_000
    assert (x < 10).mean() > (x > 1_000_000).mean() > 0


def test_collator_shards_positives_sorted_by_label():
    spec = SyntheticSpec(num_labels=1000, seq_len=16, len_lo=4, len_hi=16, poisson_lam=3.0, seed=1)
    ids, mask, lab = SyntheticXC(spec).rows(np.arange(64))
    ds = xcrepo.InMemoryDataset(ids, mask, lab)
    G = 4
    sh = shard_labels(1000, G)
    rows = np.arange(10, 31)     # 21 rows: remainder spread over first rank
    seen = sp.lil_matrix((len(rows), sh.padded_labels))
    for r in range(G):
        b = XCCollator(sh, ds, r, accum=1, xfc_batch=len(rows))(rows)
        s, e = batch_row_range(len(rows), G, r)
        assert b.input_ids.shape[0] == e - s and (b.input_ids.numpy() == ids[rows[s:e]]).all()
        lbl = b.pos_labels.numpy()
        assert (np.diff(lbl) >= 0).all() and (lbl < sh.labels_per_rank).all()
        for rr, ll in zip(b.pos_rows.numpy(), lbl):
            seen[rr, ll + r * sh.labels_per_rank] = 1
        assert b.z.shape[0] == 2 and b.z.dtype == torch.int64
    assert (seen.tocsr()[:, :1000] != lab[rows]).nnz == 0


def test_collator_layout_does_not_depend_on_accum():
    """Global rows sorted by label for every ``accum``: the classifier splits the label axis, not the rows."""
    spec = SyntheticSpec(num_labels=500, seq_len=8, len_lo=2, len_hi=8, poisson_lam=2.0, seed=2)
    ids, mask, lab = SyntheticXC(spec).rows(np.arange(32))
    ds = xcrepo.InMemoryDataset(ids, mask, lab)
    sh = shard_labels(500, 1)
    a = XCCollator(sh, ds, 0, accum=1, xfc_batch=30)(np.arange(30))
    b = XCCollator(sh, ds, 0, accum=4, xfc_batch=8)(np.arange(30))
    assert (a.pos_rows == b.pos_rows).all() and (a.pos_labels == b.pos_labels).all()
    assert (np.diff(b.pos_labels.numpy()) >= 0).all() and b.pos_rows.max() >= 8
    assert b.pos_rows.numel() == lab[:30].nnz


def test_sampler_same_on_every_rank_and_keeps_partial_batch():
    s = GlobalBatchSampler(103, 16, True, seed=7)
    a = [x.tolist() for x in s.epoch(3)]
    b = [x.tolist() for x in GlobalBatchSampler(103, 16, True, seed=7).epoch(3)]
    assert a == b and len(a) == len(s) == 7 and len(a[-1]) == 7
    assert sorted(sum(a, [])) == list(range(103))
    assert a != [x.tolist() for x in s.epoch(4)]


def test_prefetch_loader_staging_ring_delivers_the_collated_batches():
    """``pin=True``: batches are copied into a fixed ring of staging buffers (page-locked on a GPU box).  Every batch
    must arrive intact although the ring is shorter than the epoch, a slot is refilled only after its batch was
    handed over and acknowledged, and the ring does not grow."""
    from renee_b200.data.collate import PrefetchLoader
    spec = SyntheticSpec(num_labels=512, seq_len=12, len_lo=3, len_hi=12, poisson_lam=2.0, seed=5)
    ids, mask, lab = SyntheticXC(spec).rows(np.arange(90))
    ds = xcrepo.InMemoryDataset(ids, mask, lab)
    sh = shard_labels(512, 2)
    coll = XCCollator(sh, ds, 1, 1, 8, True)
    loader = PrefetchLoader(GlobalBatchSampler(90, 8, True, 3), coll, depth=2, pin=True)
    assert len(loader._slots) == 4
    for epoch in range(2):
        want = [coll(rows) for rows in GlobalBatchSampler(90, 8, True, 3).epoch(epoch)]
        n, acked = 0, []
        for got, ref_b in zip(loader.epoch(epoch), want):
            for name in ("input_ids", "attention_mask", "pos_rows", "pos_labels"):
                assert torch.equal(getattr(got, name), getattr(ref_b, name)), (epoch, n, name)
            assert got.batch_size == ref_b.batch_size and callable(got.uploaded)
            acked.append(got.input_ids.data_ptr())
            got.uploaded()
            n += 1
        assert n == len(want) == 12
        assert len(set(acked)) <= 4                       # the same four slots, over and over
