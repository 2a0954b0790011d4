"""Prepare a token-shard dataset for the ``shards:`` data source from LOCAL text: ``.txt`` files (one document per file or
per blank-line-separated paragraph with --split-paragraphs) or ``.jsonl`` files with a text field.  Documents are
tokenized, terminated with the tokenizer's end-of-text id and written as ``<out>/<name>_{train,val}_NNNNNN.bin`` shards.

    python tools/train/fetch_dataset.py --inputs corpus/*.txt --out data/mine --tokenizer bytes --shard-tokens 1000000

This box has no network, so nothing is downloaded: the reference's tool of the same name fetches public corpora
(``tools/train/fetch_dataset.py``); this one covers the "tokenize and shard" half for data that is already on disk.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import _cli  # noqa: E402,F401


def documents(paths, text_field: str, split_paragraphs: bool):
    for p in paths:
        if p.endswith(".jsonl"):
            with open(p) as f:
                for line in f:
                    if line.strip():
                        t = json.loads(line).get(text_field)
                        if t:
                            yield t
        else:
            text = open(p, encoding="utf-8", errors="replace").read()
            if split_paragraphs:
                yield from (x for x in text.split("\n\n") if x.strip())
            elif text.strip():
                yield text


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--inputs", nargs="+", required=True, help="files or globs (.txt, .jsonl)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--name", default="corpus")
    ap.add_argument("--tokenizer", default="bytes", help="bytes | gpt2 | tiktoken:NAME | hf:NAME")
    ap.add_argument("--text-field", default="text")
    ap.add_argument("--split-paragraphs", action="store_true")
    ap.add_argument("--shard-tokens", type=int, default=10_000_000)
    ap.add_argument("--val-fraction", type=float, default=0.01, help="every 1/fraction-th document goes to the val split")
    a = ap.parse_args(argv)
    import numpy as np
    from dataflow_b200.data.sources.shards import write_shard
    from dataflow_b200.data.tokenizers import resolve_tokenizer
    tok = resolve_tokenizer(a.tokenizer)
    if tok.vocab_size > 65536:
        raise SystemExit(f"tokenizer {a.tokenizer!r} has {tok.vocab_size} ids; shards hold uint16")
    paths = sorted(p for pat in a.inputs for p in glob.glob(pat))
    if not paths:
        raise SystemExit("no input files")
    os.makedirs(a.out, exist_ok=True)
    every = int(round(1 / a.val_fraction)) if a.val_fraction > 0 else 0
    bufs = {"train": [], "val": []}
    counts = {"train": 0, "val": 0}
    shards = {"train": 0, "val": 0}
    totals = {"train": 0, "val": 0, "documents": 0}

    def flush(split):
        if bufs[split]:
            path = os.path.join(a.out, f"{a.name}_{split}_{shards[split]:06d}.bin")
            write_shard(path, np.concatenate(bufs[split]))
            shards[split] += 1
            bufs[split], counts[split] = [], 0

    for n, doc in enumerate(documents(paths, a.text_field, a.split_paragraphs)):
        ids = tok.encode(doc) + ([tok.eot_id] if tok.eot_id is not None else [])
        split = "val" if every and n % every == every - 1 else "train"
        bufs[split].append(np.asarray(ids, dtype=np.uint16))
        counts[split] += len(ids)
        totals[split] += len(ids)
        totals["documents"] += 1
        if counts[split] >= a.shard_tokens:
            flush(split)
    flush("train")
    flush("val")
    meta = {"tokenizer": tok.describe(), "tokens": totals, "shards": shards, "delimiter": tok.eot_id}
    json.dump(meta, open(os.path.join(a.out, f"{a.name}.meta.json"), "w"), indent=1)
    print(json.dumps(meta))
    print(f"use it with:  --data 'shards:{a.out},delimiter={tok.eot_id}'")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
