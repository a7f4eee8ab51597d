# SPDX-License-Identifier: Apache-2.0
"""Offline data preparation of the embedding project: parquet collections, sharded pre-tokenisation jobs that write
what the training loader reads, dense retrieval."""

import json
from pathlib import Path

import numpy as np
import pyarrow as pa
import pyarrow.parquet as pq
import pytest
import torch

from arctictraining_b200.embed.data import PretokenizedBatchLoader
from arctictraining_b200.embed.data_processing import MinedDataJob
from arctictraining_b200.embed.data_processing import PairsJob
from arctictraining_b200.embed.data_processing import ParquetCollection
from arctictraining_b200.embed.data_processing import dense_retrieval
from arctictraining_b200.embed.data_processing import pretokenize_mined_data
from arctictraining_b200.embed.data_processing import pretokenize_pairs
from arctictraining_b200.embed.data_processing import shard_row_range
from arctictraining_b200.embed.data_processing.embedders import read_embeddings
from arctictraining_b200.embed.data_processing.embedders import write_embeddings


def toy_tokenize(texts):
    return [[1] + [2 + ord(c) % 40 for c in t] for t in texts]


def write_pairs(root, n_files=3, rows_per_file=7):
    root.mkdir(parents=True, exist_ok=True)
    k = 0
    for f in range(n_files):
        rows = []
        for _ in range(rows_per_file):
            rows.append({"QUERY_ID": f"q{k}", "DOCUMENT_ID": f"d{k % 5}" if k % 4 else None, "QUERY_TEXT": f"query {k}",
                         "DOCUMENT_TEXT": f"document {k % 5}"})
            k += 1
        pq.write_table(pa.Table.from_pylist(rows), root / f"part_{f}.parquet")
    return k


def test_parquet_collection_streams_row_ranges_across_files(tmp_path):
    n = write_pairs(tmp_path / "pairs")
    ds = ParquetCollection.from_location(str(tmp_path / "pairs"))
    assert ds.num_files == 3 and ds.num_rows == n == 21 and ds.batches_per_epoch(4) == 5
    got = pa.concat_tables(list(ds.stream_tables(["QUERY_ID"], (5, 16))))["QUERY_ID"].to_pylist()
    assert got == [f"q{i}" for i in range(5, 16)]
    sizes = [t.num_rows for t in ds.stream_chunks(8)]
    assert sizes == [8, 8, 5]
    one = ParquetCollection.from_location(str(tmp_path / "pairs" / "part_1.parquet"))
    assert one.num_rows == 7


def test_shard_row_range_hands_out_whole_chunks():
    spans = [shard_row_range(103, 10, s, 4) for s in range(4)]
    assert spans[0][0] == 0 and spans[-1][1] == 103
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert all(a % 10 == 0 for a, _ in spans)
    assert sorted((b - a + 9) // 10 for a, b in spans) == [2, 3, 3, 3]
    with pytest.raises(ValueError):
        shard_row_range(10, 2, 4, 4)


def test_pairs_job_sharded_output_is_what_the_loader_reads(tmp_path):
    write_pairs(tmp_path / "pairs")
    job = PairsJob(tokenizer_id="toy", query_doc_pair_dir=str(tmp_path / "pairs"), output_dir=str(tmp_path / "out"),
                   batch_size=8, query_prefix="Q:", document_prefix="D:", max_seq_length=6)
    shards = job.split_to_shards(2)
    with pytest.raises(ValueError):
        shards[0].split_to_shards(2)
    assert sum(pretokenize_pairs(s, toy_tokenize) for s in shards) == 3
    meta = json.loads((tmp_path / "out" / "metadata.json").read_text())
    assert meta["batch_size"] == 8 and meta["query_prefix"] == "Q:"
    batches = list(PretokenizedBatchLoader(tmp_path / "out", 0, 1))
    assert len(batches) == 3
    b = batches[0]
    # 8 pairs; documents de-duplicated by id (d1..d4 + two rows without id that share text with d0 / d4)
    assert b.query_tokens.shape == (8, 6)           # truncated to max_seq_length
    assert b.relevance_labels.to_dense().sum() == 8  # every pair a positive
    assert b.document_tokens.shape[0] < 8
    assert b.query_tokens[0, :3].tolist() == toy_tokenize(["Q:"])[0]
    ids = pq.read_table(tmp_path / "out" / "batch_00000000" / "did_map.parquet")["DOCUMENT_ID"].to_pylist()
    assert any(i.startswith("__MISSING_ID__") for i in ids)


def test_mined_job_reuses_queries_with_disjoint_negatives(tmp_path):
    nq, nd = 8, 40
    pq.write_table(pa.table({"QUERY_ID": np.arange(nq), "QUERY_TEXT": [f"q{i}" for i in range(nq)]}), tmp_path / "q.parquet")
    pq.write_table(pa.table({"DOCUMENT_ID": np.arange(nd), "DOCUMENT_TEXT": [f"doc{i}" for i in range(nd)]}), tmp_path / "d.parquet")
    rows = []
    for q in range(nq):
        rows.append((q, q, 1.0))
        rows += [(q, (q + 1 + j) % nd + 0, -float(j)) for j in range(1, 7) if (q + 1 + j) % nd != q]
    lq, ld, lr = zip(*rows)
    pq.write_table(pa.table({"QUERY_ID": lq, "DOCUMENT_ID": ld, "RELEVANCE": lr}), tmp_path / "labels.parquet")
    job = MinedDataJob(tokenizer_id="toy", query_loc=str(tmp_path / "q.parquet"), document_loc=str(tmp_path / "d.parquet"),
                       labels_loc=str(tmp_path / "labels.parquet"), output_loc=str(tmp_path / "mined"), queries_per_batch=4,
                       num_query_uses=2, num_negatives_per_query_per_batch=3)
    assert pretokenize_mined_data(job, toy_tokenize) == 4
    batches = list(PretokenizedBatchLoader(tmp_path / "mined" / "data", 0, 1))
    assert len(batches) == 4
    for b in batches:
        dense = b.relevance_labels.to_dense()
        assert dense.shape[0] == 4
        assert ((dense == 1).sum(1) == 1).all() and ((dense == -1).sum(1) == 3).all()
    # a query's negatives in its two uses do not overlap
    seen = {}
    for i in range(4):
        d = tmp_path / "mined" / "data" / f"batch_{i:08d}"
        q_tok = {r["BATCH_QUERY_ID"]: tuple(r["QUERY_TOKEN_ID_LIST"]) for r in pq.read_table(d / "queries.parquet").to_pylist()}
        d_tok = {r["BATCH_DOCUMENT_ID"]: tuple(r["DOCUMENT_TOKEN_ID_LIST"]) for r in pq.read_table(d / "documents.parquet").to_pylist()}
        for r in pq.read_table(d / "relations.parquet").to_pylist():
            if r["RELEVANCE"] < 0:
                seen.setdefault(q_tok[r["BATCH_QUERY_ID"]], []).append(d_tok[r["BATCH_DOCUMENT_ID"]])
    assert len(seen) == 8 and all(len(v) == 6 and len(set(v)) == 6 for v in seen.values())
    assert json.loads((tmp_path / "mined" / "metadata.json").read_text())["num_query_uses"] == 2


def test_dense_retrieval_matches_brute_force_across_slices():
    g = torch.Generator().manual_seed(0)
    q = torch.nn.functional.normalize(torch.randn(37, 16, generator=g), dim=-1)
    d = torch.nn.functional.normalize(torch.randn(211, 16, generator=g), dim=-1)
    idx, val = dense_retrieval(q.numpy(), d.numpy(), retrieval_depth=10, item_slice_size=50, query_slice_size=16, device="cpu")
    ref_val, ref_idx = torch.topk(q @ d.t(), 10, dim=1)
    assert np.array_equal(idx, ref_idx.numpy().astype(np.int32))
    assert np.allclose(val, ref_val.numpy(), atol=1e-6)
    idx2, _ = dense_retrieval(q.numpy(), d.numpy(), retrieval_depth=500, device="cpu")
    assert idx2.shape == (37, 211)


def test_embedding_parquet_round_trip(tmp_path):
    m = np.random.default_rng(0).standard_normal((5, 8)).astype(np.float32)
    write_embeddings(str(tmp_path / "e.parquet"), [f"id{i}" for i in range(5)], m)
    ids, back = read_embeddings(str(tmp_path / "e.parquet"))
    assert list(ids) == [f"id{i}" for i in range(5)] and np.array_equal(back, m)


def test_embed_all_keeps_input_order_and_config_cli_runs_a_shard(tmp_path):
    from arctictraining_b200.embed.data_processing import Embedder
    from arctictraining_b200.embed.data_processing import run_config_file_cli

    class LengthEmbedder(Embedder):
        def to_device(self, device):
            pass

        def embed_batch(self, texts, is_query, **kw):
            return np.array([[len(t), float(is_query)] for t in texts], dtype=np.float32)

    texts = ["aaa", "b", "cccccc", "dd", "eeee"]
    out = LengthEmbedder().embed_all(texts, is_query=True, batch_size=2)
    assert out[:, 0].tolist() == [3, 1, 6, 2, 4] and out[:, 1].tolist() == [1] * 5

    write_pairs(tmp_path / "pairs")
    cfg = tmp_path / "job.yaml"
    cfg.write_text(f"tokenizer_id: toy\nquery_doc_pair_dir: {tmp_path / 'pairs'}\noutput_dir: {tmp_path / 'o'}\nbatch_size: 8\n")
    ran = []
    run_config_file_cli(PairsJob, lambda c: ran.append(pretokenize_pairs(c, toy_tokenize)), [str(cfg), "--num-shards", "3", "--shard", "2"])
    assert ran == [1] and (tmp_path / "o" / "batch_00000002").is_dir() and not (tmp_path / "o" / "batch_00000000").exists()


def test_hard_negative_mining_respects_the_false_negative_threshold():
    from arctictraining_b200.embed.data_processing import mine_hard_negatives

    # query 1: positive doc 10 scores 0.9; docs 11 (0.89: too close, unlabelled positive?), 12 (0.8), 13 (0.5), 14 (0.1)
    # query 2: its positive (doc 20) was not retrieved -> dropped;  query 3: only one eligible negative -> dropped
    sq = np.array([1, 1, 1, 1, 1, 2, 2, 3, 3, 3])
    sd = np.array([10, 11, 12, 13, 14, 21, 22, 30, 31, 32])
    sc = np.array([0.9, 0.89, 0.8, 0.5, 0.1, 0.7, 0.6, 0.9, 0.88, 0.3])
    lq, ld = np.array([1, 2, 3]), np.array([10, 20, 30])
    q, d, r, stats = mine_hard_negatives(sq, sd, sc, lq, ld, threshold=0.95, negatives_per_query=2, max_positives_per_query=1)
    assert q.tolist() == [1, 1, 1] and d.tolist() == [10, 12, 13] and r.tolist() == [1, -1, -1]
    assert stats["kept_queries"] == 1 and stats["dropped_no_positive_retrieved"] == 1 and stats["dropped_too_few_negatives"] == 1
    # against a plain per-query loop on random data
    rng = np.random.default_rng(0)
    nq, depth = 40, 30
    sq = np.repeat(np.arange(nq), depth)
    sd = np.concatenate([rng.permutation(200)[:depth] for _ in range(nq)])
    sc = rng.random(nq * depth).astype(np.float32)
    lq = np.repeat(np.arange(nq), 3)
    ld = rng.integers(0, 200, nq * 3)
    q, d, r, _ = mine_hard_negatives(sq, sd, sc, lq, ld, threshold=0.9, negatives_per_query=5, max_positives_per_query=2)
    want = []
    for qi in range(nq):
        m = sq == qi
        docs, scores = sd[m], sc[m]
        pos = np.isin(docs, ld[lq == qi])
        if not pos.any():
            continue
        o = np.argsort(-scores[pos], kind="stable")
        use_pos, pos_scores = docs[pos][o][:2], scores[pos][o][:2]
        ok = (~pos) & (scores < 0.9 * pos_scores.min())
        o2 = np.argsort(-scores[ok], kind="stable")
        negs = docs[ok][o2][:5]
        if len(negs) < 5:
            continue
        want += [(qi, int(x), 1) for x in use_pos] + [(qi, int(x), -1) for x in negs]
    assert list(zip(q.tolist(), d.tolist(), r.tolist())) == want


def test_combining_sources_keeps_ids_apart():
    from arctictraining_b200.embed.data_processing import combine_datasets
    from arctictraining_b200.embed.data_processing import scramble_ids

    a = scramble_ids(np.arange(1000), 0)
    b = scramble_ids(np.arange(1000), 1)
    assert len(np.unique(a)) == 1000 and len(np.intersect1d(a, b)) == 0 and np.array_equal(a, scramble_ids(np.arange(1000), 0))

    def source(n):
        return {"queries": pa.table({"QUERY_ID": np.arange(n, dtype=np.uint64), "QUERY_TEXT": [f"q{i}" for i in range(n)]}),
                "documents": pa.table({"DOCUMENT_ID": np.arange(n, dtype=np.uint64), "DOCUMENT_TEXT": [f"d{i}" for i in range(n)]}),
                "labels": pa.table({"QUERY_ID": np.arange(n, dtype=np.uint64), "DOCUMENT_ID": np.arange(n, dtype=np.uint64),
                                    "RELEVANCE": np.ones(n, dtype=np.int8)})}

    out = combine_datasets([source(5), source(7)])
    assert out["queries"].num_rows == 12 and out["labels"].num_rows == 12
    # labels still point at rows of their own source: the scrambled (query, document) ids of a label exist in the tables
    qid = set(out["queries"]["QUERY_ID"].to_pylist())
    did = set(out["documents"]["DOCUMENT_ID"].to_pylist())
    assert all(r["QUERY_ID"] in qid and r["DOCUMENT_ID"] in did for r in out["labels"].to_pylist())


def test_staged_preparation_script_runs_end_to_end_on_a_toy_dataset(tmp_path):
    """embed -> retrieve -> mine -> combine -> batch -> dev-split of the fine-tuning example, with a stand-in embedder
    and tokenizer; the result is what the training loader reads."""
    import argparse
    import sys

    from arctictraining_b200.embed.data_processing import Embedder

    root = Path(__file__).resolve().parent.parent
    sys.path.insert(0, str(root / "projects" / "arctic_embed" / "examples" / "finetune_models"))
    import prepare_data as prep

    class BagOfLetters(Embedder):  # texts that share letters are close
        def to_device(self, device):
            pass

        def embed_batch(self, texts, is_query, **kw):
            out = np.zeros((len(texts), 26), dtype=np.float32)
            for i, t in enumerate(texts):
                for ch in t.lower():
                    if "a" <= ch <= "z":
                        out[i, ord(ch) - 97] += 1
            return out / np.maximum(np.linalg.norm(out, axis=1, keepdims=True), 1e-6)

    words = ["alpha", "bravo", "charlie", "delta", "echo", "foxtrot", "golf", "hotel", "india", "juliet", "kilo", "lima"]
    for name in ("a", "b"):
        d = tmp_path / name
        d.mkdir()
        pq.write_table(pa.table({"QUERY_ID": np.arange(12, dtype=np.uint64), "QUERY_TEXT": [f"{w} {w}" for w in words]}), d / "queries.parquet")
        pq.write_table(pa.table({"DOCUMENT_ID": np.arange(12, dtype=np.uint64), "DOCUMENT_TEXT": [f"about {w}" for w in words]}), d / "documents.parquet")
        pq.write_table(pa.table({"QUERY_ID": np.arange(12, dtype=np.uint64), "DOCUMENT_ID": np.arange(12, dtype=np.uint64)}), d / "labels.parquet")
        ns = argparse.Namespace(dataset=str(d), batch_size=5, device="", pooling="", query_prefix="", document_prefix="", max_seq_len=32, model="")
        prep.stage_embed(ns, embedder=BagOfLetters())
        prep.stage_retrieve(argparse.Namespace(dataset=str(d), depth=12, device="cpu"))
        prep.stage_mine(argparse.Namespace(dataset=str(d), threshold=0.99, negatives=3, max_positives=1))
        mined = pq.read_table(d / "mined_labels.parquet").to_pandas()
        assert (mined.groupby("QUERY_ID")["RELEVANCE"].apply(lambda r: (r == 1).sum()) == 1).all()
        assert (mined.groupby("QUERY_ID")["RELEVANCE"].apply(lambda r: (r == -1).sum()) == 3).all()
    prep.stage_combine(argparse.Namespace(datasets=[str(tmp_path / "a"), str(tmp_path / "b")], out=str(tmp_path / "combined")))
    for d in ("a", "b", "combined"):
        prep.stage_batch(argparse.Namespace(dataset=str(tmp_path / d), tokenizer="toy", name="v1", query_prefix="q: ", document_prefix="d: ",
                                            queries_per_batch=4, negatives=3, max_seq_len=16), tokenize=toy_tokenize)
    prep.stage_dev_split(argparse.Namespace(datasets=[str(tmp_path / "a"), str(tmp_path / "b")], name="v1", out=str(tmp_path / "eval"), batches=1))
    train = list(PretokenizedBatchLoader(tmp_path / "combined" / "pretokenized" / "v1" / "data", 0, 1))
    assert len(train) >= 4 and train[0].query_tokens.shape[0] == 4
    dense = train[0].relevance_labels.to_dense()
    assert ((dense == 1).sum(1) == 1).all() and ((dense == -1).sum(1) == 3).all()
    assert len(list(PretokenizedBatchLoader(tmp_path / "eval" / "a", 0, 1))) == 1
    assert json.loads((tmp_path / "eval" / "metadata.json").read_text())["query_prefix"] == "q: "


def test_download_tables_are_deduplicated_and_stable(tmp_path):
    import importlib.util

    import pyarrow.parquet as pq

    path = Path(__file__).resolve().parent.parent / "projects" / "arctic_embed" / "examples" / "finetune_models" / "download_data.py"
    spec = importlib.util.spec_from_file_location("_embed_download", path)
    dl = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(dl)

    q = ["who", "what", "who", "who"]
    d = ["doc a", "doc b", "doc a", "doc c"]
    tables = dl.pairs_to_tables(q, d, extra_documents=["doc z", "doc b"])
    assert len(tables["queries"]) == 2 and len(tables["documents"]) == 4 and len(tables["labels"]) == 3
    ids = dict(zip(tables["queries"]["QUERY_TEXT"].to_pylist(), tables["queries"]["QUERY_ID"].to_pylist()))
    assert ids["who"] == int(dl.text_ids(["who"])[0])  # the id depends on the text alone
    doc_ids = set(tables["documents"]["DOCUMENT_ID"].to_pylist())
    assert set(tables["labels"]["DOCUMENT_ID"].to_pylist()) <= doc_ids
    assert set(tables["labels"]["QUERY_ID"].to_pylist()) == set(ids.values())
    dl.write_tables(tables, tmp_path / "toy")
    assert pq.read_table(tmp_path / "toy" / "labels.parquet").num_rows == 3
    with pytest.raises(ValueError):
        dl.pairs_to_tables(["a"], [])

    assert dl.title_and_text(" T ", "x") == "T\nx" and dl.title_and_text("", "x") == "x"
    index = dl.BodyIndex(["the body text that is long enough to fill the whole tail key", "short", "a short"])
    assert index.split("My title the body text that is long enough to fill the whole tail key") == (
        "My title", "the body text that is long enough to fill the whole tail key")
    assert index.split("Title: a short") == ("Title:", "a short")  # the longest matching body wins
    assert index.split("nothing known") is None
