"""Data plane: source determinism and cursor resume, feed order (threaded == synchronous), packing policies,
exact resume of the packed-step sequence, capture -> replay."""
import json

import numpy as np
import pytest

from dataflow_b200.data import DataFeed, DataPipeline, Packer, Sequence, resolve_data
from dataflow_b200.data.sources.shards import write_shard


def take(source, n, cursor=None):
    out = []
    for seq, cur in source.sequences(cursor):
        out.append((seq, cur))
        if len(out) == n:
            break
    return out


@pytest.fixture
def shard_root(tmp_path):
    g = np.random.default_rng(0)
    for k in range(2):
        ids = g.integers(0, 1000, size=5000)
        ids[g.integers(0, 5000, size=40)] = 50256          # document delimiters
        write_shard(str(tmp_path / f"tiny_train_{k:03d}.bin"), ids)
    return str(tmp_path)


@pytest.fixture
def jsonl_file(tmp_path):
    p = tmp_path / "docs.jsonl"
    with open(p, "w") as f:
        for i in range(30):
            f.write(json.dumps({"text": f"document number {i} " + "word " * (i % 7 + 1)}) + "\n")
        f.write(json.dumps({"instruction": "Q: two plus two?", "output": " four"}) + "\n")
    return str(p)


@pytest.mark.parametrize("spec", ["synthetic:vocab=300,mean_len=40,seed=3", "SHARDS", "SHARDS,window=64", "JSONL"])
def test_sources_are_pure_functions_of_their_cursor(spec, shard_root, jsonl_file):
    spec = spec.replace("SHARDS", f"shards:{shard_root}").replace("JSONL", f"jsonl:{jsonl_file},tokenizer=bytes")
    src = resolve_data(spec, vocab_size=65536, max_seqlen=128)
    a = take(src, 25)
    b = take(resolve_data(spec, vocab_size=65536, max_seqlen=128), 25)
    for (s1, c1), (s2, c2) in zip(a, b):
        assert np.array_equal(s1.tokens, s2.tokens) and np.array_equal(s1.targets, s2.targets) and c1 == c2
    # resuming from the cursor after item 9 yields item 10 onwards
    c = take(src, 15, a[9][1])
    for (s1, _), (s2, _) in zip(a[10:], c):
        assert np.array_equal(s1.tokens, s2.tokens)
    assert all(len(s) <= 128 for s, _ in a)
    json.dumps(a[-1][1])          # cursors are JSON-clean


def test_document_targets_shift_inside_the_document_and_end_with_eot(shard_root):
    src = resolve_data(f"shards:{shard_root}", max_seqlen=100000)
    seq, _ = next(iter(src.sequences()))
    assert np.array_equal(seq.targets[:-1], seq.tokens[1:]) and seq.targets[-1] == 50256
    assert 50256 not in seq.tokens


def test_long_policies(tmp_path):
    write_shard(str(tmp_path / "one_train.bin"), list(range(1, 301)) + [50256] + list(range(1, 21)) + [50256])
    root = str(tmp_path)
    lens = lambda lp: [len(s) for s, _ in take(resolve_data(f"shards:{root},long_policy={lp}", max_seqlen=128), 4)]
    assert lens("exclude")[:2] == [20, 20]            # the 300-token document is dropped; epochs wrap
    assert lens("trim")[:2] == [128, 20]
    assert lens("chunk")[:4] == [128, 128, 44, 20]
    assert lens("whole")[:2] == [300, 20]
    # a cursor that points into the middle of a chunked document resumes at the next piece
    src = resolve_data(f"shards:{root},long_policy=chunk", max_seqlen=128)
    items = take(src, 4)
    again = take(src, 2, items[0][1])
    assert [len(s) for s, _ in again] == [128, 44] and np.array_equal(again[0][0].tokens, items[1][0].tokens)


def test_instruction_records_mask_the_prompt(jsonl_file):
    src = resolve_data(f"jsonl:{jsonl_file},tokenizer=bytes")
    seqs = [s for s, _ in take(src, 31)]
    last = seqs[30]
    n_prompt = len("Q: two plus two?".encode())
    assert (last.targets[:n_prompt - 1] == -1).all() and (last.targets[n_prompt - 1:] >= 0).all()


def test_threaded_feed_hands_out_source_order():
    src = resolve_data("synthetic:vocab=100,mean_len=20,seed=1")
    a, b = DataFeed(src, prefetch_sequences=0), DataFeed(src, prefetch_sequences=8)
    try:
        for _ in range(50):
            (s1, c1), (s2, c2) = a.next_sequence(), b.next_sequence()
            assert np.array_equal(s1.tokens, s2.tokens) and c1 == c2
    finally:
        a.close()
        b.close()


@pytest.mark.parametrize("policy,split", [("ffd", False), ("greedy", False), ("greedy", True)])
def test_packing_invariants_and_exact_resume(policy, split):
    def pipe():
        return DataPipeline("synthetic:vocab=500,mean_len=60,seed=5", 256, 3, max_seqlen=128, vocab_size=500,
                            policy=policy, allow_round_split=split, prefetch_sequences=0)
    st = pipe()(None)
    steps = [st.next_step() for _ in range(6)]
    st.close()
    for s in steps:
        assert len(s.rounds) == 3
        for r in s.rounds:
            assert r.bounds[0] == 0 and r.bounds[-1] == r.content <= 256
            assert (r.targets[r.content:] == -1).all()
            assert all(b - a <= 128 for a, b in zip(r.bounds, r.bounds[1:]))
            if split:
                assert r.content == 256
        assert s.valid_rows == sum(int((r.targets >= 0).sum()) for r in s.rounds)
        json.dumps(s.cursor_after)
    if policy == "ffd":
        assert np.mean([s.fill for s in steps]) > 0.9
    # resume after step 2: steps 3.. are byte-identical
    st2 = pipe()(steps[2].cursor_after)
    again = [st2.next_step() for _ in range(3)]
    st2.close()
    assert [s.digest() for s in again] == [s.digest() for s in steps[3:]]
    assert again[0].index == 3


def test_capture_replays_exactly(tmp_path):
    cap = str(tmp_path / "run.capture")
    p = DataPipeline("synthetic:vocab=500,mean_len=60,seed=9", 256, 2, max_seqlen=128, vocab_size=500, capture=cap,
                     prefetch_sequences=4)
    st = p(None)
    steps = [st.next_step() for _ in range(4)]
    st.close()
    q = DataPipeline(f"capture:{cap}", 256, 2, max_seqlen=128, policy="greedy", prefetch_sequences=0)
    st = q(None)
    toks = np.concatenate([np.concatenate([r.tokens[:r.content] for r in s.rounds]) for s in steps])
    got = []
    while (s := st.next_step()) is not None:
        got.append(np.concatenate([r.tokens[:r.content] for r in s.rounds]))
    st.close()
    assert sorted(np.concatenate(got).tolist()) == sorted(toks.tolist())
    assert sum(len(g) for g in got) == len(toks)


def test_text_sources_name_the_bad_line_and_do_not_read_an_empty_corpus_for_ever(tmp_path):
    good = json.dumps({"text": "a perfectly fine document"})
    cases = {"broken.jsonl": (good + "\n{\"text\": \"cut sho\n", r"broken\.jsonl:2: not a JSON document"),
             "list.jsonl": (good + "\n[1, 2, 3]\n", r"list\.jsonl:2: a record must be a JSON object, this line is a list")}
    for name, (body, needle) in cases.items():
        p = tmp_path / name
        p.write_text(body)
        src = resolve_data(f"jsonl:{p},tokenizer=bytes", vocab_size=65536, max_seqlen=64)
        with pytest.raises(ValueError, match=needle):
            take(src, 5)
    # nothing usable: no text field anywhere, or only documents shorter than two tokens.  Epochs wrap, so without a check
    # the source would spin through the files for ever
    empty = tmp_path / "empty.jsonl"
    empty.write_text(json.dumps({"title": "no text field"}) + "\n" + json.dumps({"text": ""}) + "\n\n")
    with pytest.raises(ValueError, match="no usable document"):
        take(resolve_data(f"jsonl:{empty},tokenizer=bytes", vocab_size=65536, max_seqlen=64), 1)
    # a corpus with one usable document wraps as before
    one = tmp_path / "one.jsonl"
    one.write_text(json.dumps({"title": "skip me"}) + "\n" + good + "\n")
    got = take(resolve_data(f"jsonl:{one},tokenizer=bytes", vocab_size=65536, max_seqlen=64), 3)
    assert len(got) == 3 and [c["epoch"] for _, c in got] == [0, 1, 2]


def test_shards_with_nothing_usable_end_with_an_error(tmp_path):
    write_shard(str(tmp_path / "tiny_train_000.bin"), np.arange(40) % 7)            # 40 tokens, no delimiter id among them
    with pytest.raises(ValueError, match="no window of 64 \\+ 1 tokens fits any shard"):
        take(resolve_data(f"shards:{tmp_path},window=64", vocab_size=65536, max_seqlen=128), 1)
    with pytest.raises(ValueError, match="no document ends with the delimiter"):
        take(resolve_data(f"shards:{tmp_path}", vocab_size=65536, max_seqlen=128), 1)
    assert len(take(resolve_data(f"shards:{tmp_path},window=16", vocab_size=65536, max_seqlen=128), 5)) == 5     # wraps as before


def test_parquet_source_reads_resumes_and_refuses_an_empty_column(tmp_path):
    pa = pytest.importorskip("pyarrow")
    import pyarrow.parquet as pq
    docs = [f"parquet document {i} " + "word " * (i % 5 + 1) for i in range(12)]
    pq.write_table(pa.table({"text": docs[:6] + [""]}), tmp_path / "a.parquet", row_group_size=3)
    pq.write_table(pa.table({"text": docs[6:]}), tmp_path / "b.parquet", row_group_size=4)
    spec = f"parquet:{tmp_path}/*.parquet,tokenizer=bytes"
    got = take(resolve_data(spec, vocab_size=65536, max_seqlen=256), 14)
    assert [c["epoch"] for _, c in got] == [0] * 12 + [1, 1] and len({bytes(s.tokens) for s, _ in got[:12]}) == 12
    again = take(resolve_data(spec, vocab_size=65536, max_seqlen=256), 4, got[7][1])          # resume after the eighth document
    assert all(np.array_equal(a.tokens, b.tokens) for (a, _), (b, _) in zip(again, got[8:12]))
    pq.write_table(pa.table({"text": ["", "", "x"]}), tmp_path / "none.pq")
    with pytest.raises(ValueError, match="no usable document"):
        take(resolve_data(f"parquet:{tmp_path}/none.pq,tokenizer=bytes", vocab_size=65536, max_seqlen=64), 1)
