"""Every reference flag parses with the reference's name, type and default (main.py:190-255)."""
from renee_b200.cli import build_parser

REFERENCE_DEFAULTS = {
    "data_dir": "", "custom_cuda": False, "default_impl": False, "batch_size": 8, "epochs": 50,
    "expname": "renee-exp", "device": None, "dist_url": "tcp://localhost:23456", "rank": 0, "world_size": 1,
    "seed": 42, "bottleneck_dims": 0, "dropout": 0.5, "lr1": 0.0025, "lr2": 1e-5, "mo": 0.9, "wd1": 0.01,
    "wd2": 0.01, "fp32encoder": False, "fp16xfc": False, "noloss": False, "checkpoint_resume": "",
    "infer": False, "warmup": 140000, "accum": 1, "pre_tok": False, "maxlen": 32,
    "tf": "distilbert-base-uncased", "use_ngame_encoder": "", "compile": False,
}


def test_defaults():
    a = vars(build_parser().parse_args([]))
    assert len(REFERENCE_DEFAULTS) == 30
    for k, v in REFERENCE_DEFAULTS.items():
        assert a[k] == v, k


def test_headline_recipe_parses():
    argv = ("--data-dir Datasets/LF-AmazonTitles-131K --maxlen 32 --epochs 100 --batch-size 32 --lr1 0.05 "
            "--lr2 1e-5 --warmup 5000 --dropout 0.85 --wd1 1e-4 --noloss --fp16xfc --expname x "
            "--tf sentence-transformers/msmarco-distilbert-base-v4 --custom-cuda --accum 2 "
            "--checkpoint-resume ck --compile --pre-tok --device 0").split()
    a = build_parser().parse_args(argv)
    assert a.fp16xfc and a.noloss and a.dropout == 0.85 and a.lr1 == 0.05 and a.wd1 == 1e-4 and a.accum == 2
