# SPDX-License-Identifier: Apache-2.0
"""Fine-tuning data with mined hard negatives, stage by stage.

Every source dataset is a directory with ``queries.parquet`` (QUERY_ID, QUERY_TEXT), ``documents.parquet``
(DOCUMENT_ID, DOCUMENT_TEXT) and ``labels.parquet`` (QUERY_ID, DOCUMENT_ID; the annotated positives).

    python prepare_data.py embed    --dataset data/nq --model Snowflake/snowflake-arctic-embed-l-v2.0
    python prepare_data.py retrieve --dataset data/nq --depth 300
    python prepare_data.py mine     --dataset data/nq --threshold 0.95 --negatives 10
    python prepare_data.py combine  --datasets data/nq data/msmarco --out data/combined
    python prepare_data.py batch    --dataset data/combined --tokenizer intfloat/e5-base-unsupervised --name example_dot95
    python prepare_data.py dev-split --datasets data/nq data/msmarco --name example_dot95 --out data/eval --batches 5

Stages of the reference: projects/arctic_embed/examples/finetune_models/data_processing_scripts/stage_1..6_*.py.
"""

import argparse
import json
import shutil
import sys
from pathlib import Path

import numpy as np
import pyarrow as pa
import pyarrow.parquet as pq

sys.path.insert(0, str(Path(__file__).resolve().parents[4]))

from arctictraining_b200.embed.data_processing import MinedDataJob  # noqa: E402
from arctictraining_b200.embed.data_processing import HFEmbedder  # noqa: E402
from arctictraining_b200.embed.data_processing import combine_datasets  # noqa: E402
from arctictraining_b200.embed.data_processing import dense_retrieval  # noqa: E402
from arctictraining_b200.embed.data_processing import mine_hard_negatives  # noqa: E402
from arctictraining_b200.embed.data_processing import pretokenize_mined_data  # noqa: E402
from arctictraining_b200.embed.data_processing.embedders import normalize_embeddings  # noqa: E402
from arctictraining_b200.embed.data_processing.embedders import read_embeddings  # noqa: E402
from arctictraining_b200.embed.data_processing.embedders import write_embeddings  # noqa: E402


def stage_embed(args, embedder=None) -> None:
    """Teacher embeddings of all queries and documents -> ``embeddings/{queries,documents}.parquet``."""
    root = Path(args.dataset)
    embedder = embedder or HFEmbedder(args.model, args.pooling, args.query_prefix, args.document_prefix, args.max_seq_len)
    if embedder is not None and args.device:
        embedder.to_device(args.device)
    for name, id_col, text_col, is_query in (("queries", "QUERY_ID", "QUERY_TEXT", True), ("documents", "DOCUMENT_ID", "DOCUMENT_TEXT", False)):
        t = pq.read_table(root / f"{name}.parquet")
        vecs = embedder.embed_all(t[text_col].to_pylist(), is_query, batch_size=args.batch_size)
        write_embeddings(str(root / "embeddings" / f"{name}.parquet"), t[id_col].to_pylist(), vecs.astype(np.float32))
        print(f"{name}: {vecs.shape[0]} x {vecs.shape[1]}")


def stage_retrieve(args) -> None:
    """Top-``depth`` documents per query by inner product -> ``retrieval_scores.parquet`` (QUERY_ID, DOCUMENT_ID, SCORE)."""
    root = Path(args.dataset)
    qid, q = read_embeddings(str(root / "embeddings" / "queries.parquet"))
    did, d = read_embeddings(str(root / "embeddings" / "documents.parquet"))
    idx, val = dense_retrieval(normalize_embeddings(q.astype(np.float32)), normalize_embeddings(d.astype(np.float32)),
                               retrieval_depth=args.depth, device=args.device or None)
    k = idx.shape[1]
    pq.write_table(pa.table({"QUERY_ID": np.repeat(np.asarray(qid), k), "DOCUMENT_ID": np.asarray(did)[idx.ravel()],
                             "SCORE": val.ravel().astype(np.float32)}), root / "retrieval_scores.parquet")
    print(f"{len(qid)} queries x {k} documents")


def stage_mine(args) -> None:
    """Positives + hard negatives per query -> ``mined_labels.parquet`` (QUERY_ID, DOCUMENT_ID, RELEVANCE)."""
    root = Path(args.dataset)
    s = pq.read_table(root / "retrieval_scores.parquet")
    lab = pq.read_table(root / "labels.parquet")
    q, d, r, stats = mine_hard_negatives(s["QUERY_ID"].to_numpy(), s["DOCUMENT_ID"].to_numpy(), s["SCORE"].to_numpy(),
                                         lab["QUERY_ID"].to_numpy(), lab["DOCUMENT_ID"].to_numpy(), args.threshold,
                                         args.negatives, args.max_positives)
    pq.write_table(pa.table({"QUERY_ID": q, "DOCUMENT_ID": d, "RELEVANCE": r}), root / "mined_labels.parquet")
    print(json.dumps(stats))


def stage_combine(args) -> None:
    """Several mined datasets -> one (ids re-hashed per source so that they cannot collide)."""
    sources = []
    for ds in args.datasets:
        root = Path(ds)
        sources.append({"queries": pq.read_table(root / "queries.parquet"), "documents": pq.read_table(root / "documents.parquet"),
                        "labels": pq.read_table(root / "mined_labels.parquet")})
    out = combine_datasets(sources)
    Path(args.out).mkdir(parents=True, exist_ok=True)
    for name, fname in (("queries", "queries.parquet"), ("documents", "documents.parquet"), ("labels", "mined_labels.parquet")):
        pq.write_table(out[name], Path(args.out) / fname)
    print({k: v.num_rows for k, v in out.items()})


def stage_batch(args, tokenize=None) -> None:
    """Pre-tokenised training batches under ``<dataset>/pretokenized/<name>/``."""
    root = Path(args.dataset)
    job = MinedDataJob(tokenizer_id=args.tokenizer, query_loc=str(root / "queries.parquet"), document_loc=str(root / "documents.parquet"),
                       labels_loc=str(root / "mined_labels.parquet"), output_loc=str(root / "pretokenized" / args.name),
                       query_prefix=args.query_prefix, document_prefix=args.document_prefix, queries_per_batch=args.queries_per_batch,
                       num_negatives_per_query_per_batch=args.negatives, max_seq_length=args.max_seq_len)
    print(f"{pretokenize_mined_data(job, tokenize)} batches")


def stage_dev_split(args) -> None:
    """The first ``--batches`` batches of every source become its evaluation set (their tokenisation metadata must agree)."""
    meta = None
    for ds in args.datasets:
        src = Path(ds) / "pretokenized" / args.name
        m = json.loads((src / "metadata.json").read_text())
        if meta is not None and m != meta:
            raise ValueError(f"{src}: tokenisation metadata differs from the other datasets")
        meta = m
        for b in sorted((src / "data").iterdir())[: args.batches]:
            shutil.copytree(b, Path(args.out) / Path(ds).name / b.name, dirs_exist_ok=True)
    (Path(args.out) / "metadata.json").write_text(json.dumps(meta, indent=2))


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="stage", required=True)
    e = sub.add_parser("embed"); e.add_argument("--dataset", required=True); e.add_argument("--model", default="Snowflake/snowflake-arctic-embed-l-v2.0")
    e.add_argument("--pooling", default="first_token"); e.add_argument("--query-prefix", default="query: "); e.add_argument("--document-prefix", default="")
    e.add_argument("--max-seq-len", type=int, default=512); e.add_argument("--batch-size", type=int, default=256); e.add_argument("--device", default="cuda")
    r = sub.add_parser("retrieve"); r.add_argument("--dataset", required=True); r.add_argument("--depth", type=int, default=300); r.add_argument("--device", default="")
    m = sub.add_parser("mine"); m.add_argument("--dataset", required=True); m.add_argument("--threshold", type=float, default=0.95)
    m.add_argument("--negatives", type=int, default=10); m.add_argument("--max-positives", type=int, default=1)
    c = sub.add_parser("combine"); c.add_argument("--datasets", nargs="+", required=True); c.add_argument("--out", required=True)
    b = sub.add_parser("batch"); b.add_argument("--dataset", required=True); b.add_argument("--tokenizer", required=True); b.add_argument("--name", default="example_dot95")
    b.add_argument("--query-prefix", default="query: "); b.add_argument("--document-prefix", default="passage: "); b.add_argument("--queries-per-batch", type=int, default=256)
    b.add_argument("--negatives", type=int, default=10); b.add_argument("--max-seq-len", type=int, default=512)
    d = sub.add_parser("dev-split"); d.add_argument("--datasets", nargs="+", required=True); d.add_argument("--name", default="example_dot95")
    d.add_argument("--out", required=True); d.add_argument("--batches", type=int, default=5)
    return ap


STAGES = {"embed": stage_embed, "retrieve": stage_retrieve, "mine": stage_mine, "combine": stage_combine, "batch": stage_batch,
          "dev-split": stage_dev_split}

if __name__ == "__main__":
    a = parser().parse_args()
    STAGES[a.stage](a)
