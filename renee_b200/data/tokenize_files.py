"""Offline tokenisation tool: raw text files → int64 token memmaps.

    python -m renee_b200.data.tokenize_files --data-dir DIR [--max-length 32]
        [--tokenizer-type bert-base-uncased] [--num-threads 32] [--output-folder DIR]
        [--tokenize-label-texts] [--tokenizer-path LOCAL_DIR]

Reads ``trn_X.txt`` / ``tst_X.txt`` (and ``Y.txt`` with ``--tokenize-label-texts``), one text per line,
and writes ``{trn_doc,tst_doc,lbl}_{input_ids,attention_mask}.dat`` (int64 ``[N, max_length]``,
padded/truncated to ``max_length`` with special tokens) into ``{output}/{tokenizer-type}-{max-length}``
— the layout the trainer's ``PreTokDataset`` reads.  Same flags and outputs as the reference's
``utils/CreateTokenizedFiles.py`` (lines 34-111).  The work is streamed in bounded chunks written
straight into the memmap, so peak memory does not grow with the corpus.  ``--tokenizer-path`` points at
a local tokenizer directory for machines without hub access.
"""
from __future__ import annotations

import argparse
import os
import time
from concurrent.futures import ProcessPoolExecutor

import numpy as np

_TOK = None


def _init(tokenizer_path: str) -> None:
    global _TOK
    from transformers import AutoTokenizer
    _TOK = AutoTokenizer.from_pretrained(tokenizer_path, do_lower_case=True)


def _encode(job):
    texts, max_len = job
    enc = _TOK(texts, add_special_tokens=True, max_length=max_len, padding="max_length", truncation=True,
               return_attention_mask=True, return_tensors="np")
    return enc["input_ids"].astype(np.int64), enc["attention_mask"].astype(np.int64)


def read_lines(path: str) -> list[str]:
    with open(path, "r", encoding="utf-8") as f:
        return [line.strip() for line in f]


def tokenize_to_memmap(texts: list[str], folder: str, prefix: str, max_len: int, tokenizer_path: str,
                       num_threads: int = 8, chunk: int = 20000, encode_fn=None) -> tuple[int, int]:
    """Writes ``{prefix}_input_ids.dat`` and ``{prefix}_attention_mask.dat``.  ``encode_fn(texts, max_len)
    -> (ids, mask)`` replaces the HF tokenizer (used by tests and for custom tokenisers)."""
    os.makedirs(folder, exist_ok=True)
    n = len(texts)
    ii = np.memmap(os.path.join(folder, f"{prefix}_input_ids.dat"), dtype=np.int64, mode="w+", shape=(n, max_len))
    am = np.memmap(os.path.join(folder, f"{prefix}_attention_mask.dat"), dtype=np.int64, mode="w+", shape=(n, max_len))
    jobs = [(texts[s: s + chunk], max_len) for s in range(0, n, chunk)]
    if encode_fn is not None:
        results = (encode_fn(*j) for j in jobs)
        pool = None
    else:
        pool = ProcessPoolExecutor(max_workers=max(1, num_threads), initializer=_init, initargs=(tokenizer_path,))
        results = pool.map(_encode, jobs)
    row = 0
    for ids, mask in results:
        ii[row: row + len(ids)] = ids
        am[row: row + len(ids)] = mask
        row += len(ids)
    if pool is not None:
        pool.shutdown()
    ii.flush(); am.flush()
    return n, max_len


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--data-dir", type=str, required=True)
    ap.add_argument("--max-length", type=int, default=32)
    ap.add_argument("--tokenizer-type", type=str, default="bert-base-uncased")
    ap.add_argument("--num-threads", type=int, default=32)
    ap.add_argument("--output-folder", type=str, default="")
    ap.add_argument("--tokenize-label-texts", action="store_true", default=False)
    ap.add_argument("--tokenizer-path", type=str, default="", help="local tokenizer directory (defaults to --tokenizer-type)")
    a = ap.parse_args(argv)
    out = a.output_folder or a.data_dir
    folder = os.path.join(out, f"{a.tokenizer_type}-{a.max_length}")
    tok = a.tokenizer_path or a.tokenizer_type
    todo = [("trn_doc", "trn_X.txt"), ("tst_doc", "tst_X.txt")]
    if a.tokenize_label_texts:
        todo.append(("lbl", "Y.txt"))
    for prefix, fname in todo:
        t0 = time.perf_counter()
        texts = read_lines(os.path.join(a.data_dir, fname))
        n, _ = tokenize_to_memmap(texts, folder, prefix, a.max_length, tok, a.num_threads)
        print(f"{prefix}: {n} texts -> {folder} in {time.perf_counter() - t0:.2f} s")


if __name__ == "__main__":
    main()
