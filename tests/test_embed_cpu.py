# SPDX-License-Identifier: Apache-2.0
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F
import yaml

from arctictraining_b200.embed.data import slice_sparse_coo_tensor
from arctictraining_b200.embed.losses import info_nce_loss
from arctictraining_b200.embed.losses import one_size_truncated_mrl_info_nce_loss
from arctictraining_b200.embed.model import pool

ROOT = Path(__file__).resolve().parent.parent


def test_infonce_matches_cross_entropy_for_one_positive_per_query():
    torch.manual_seed(0)
    scores = torch.randn(6, 9, requires_grad=True)
    rel = -torch.ones(6, 9, dtype=torch.long)
    target = torch.tensor([3, 0, 8, 2, 5, 1])
    rel[torch.arange(6), target] = 1
    loss = info_nce_loss(scores, rel, 0.05)
    ref_scores = scores.detach().clone().requires_grad_(True)
    ref = F.cross_entropy(ref_scores / 0.05, target)
    loss.backward()
    ref.backward()
    assert torch.allclose(loss, ref, atol=1e-6) and torch.allclose(scores.grad, ref_scores.grad, atol=1e-6)


def test_infonce_multi_positive_and_unlabelled_pairs():
    torch.manual_seed(0)
    scores = torch.randn(3, 5, requires_grad=True)
    rel = torch.tensor([[1, 1, -1, 0, -1], [-1, 0, 1, -1, 0], [0, -1, -1, 1, -1]])
    loss = info_nce_loss(scores, rel, 0.1)
    # naive: one softmax row per positive, other positives of that query and unlabelled columns masked
    s = scores.detach().clone().requires_grad_(True)
    rows = []
    for q, d in [(0, 0), (0, 1), (1, 2), (2, 3)]:
        mask = (rel[q] == -1).clone()
        mask[d] = True
        logits = (s[q] / 0.1).masked_fill(~mask, -1e12)
        rows.append(F.cross_entropy(logits.unsqueeze(0), torch.tensor([d])))
    ref = torch.stack(rows).mean()
    loss.backward()
    ref.backward()
    assert torch.allclose(loss, ref, atol=1e-6) and torch.allclose(scores.grad, s.grad, atol=1e-6)


def test_mrl_loss_combines_full_and_truncated():
    torch.manual_seed(0)
    q, d = torch.randn(4, 16), torch.randn(4, 16)
    rel = -torch.ones(4, 4, dtype=torch.long)
    rel.fill_diagonal_(1)
    loss, full, trunc = one_size_truncated_mrl_info_nce_loss(q, d, rel, truncated_dimension=8, mrl_weight=0.25)
    assert torch.allclose(loss, 0.75 * full + 0.25 * trunc)
    only, full2, none = one_size_truncated_mrl_info_nce_loss(q, d, rel)
    assert none is None and torch.allclose(only, full2)


def test_pooling_modes():
    h = torch.arange(2 * 4 * 3, dtype=torch.float32).view(2, 4, 3)
    mask = torch.tensor([[1, 1, 0, 0], [1, 1, 1, 1]])
    assert torch.equal(pool(h, mask, "first"), h[:, 0])
    assert torch.equal(pool(h, mask, "last"), torch.stack([h[0, 1], h[1, 3]]))
    assert torch.allclose(pool(h, mask, "mean"), torch.stack([h[0, :2].mean(0), h[1].mean(0)]))


def test_slice_sparse_coo_tensor():
    dense = torch.tensor([[0, 1, 0, -1], [1, 0, 0, 0], [0, 0, -1, 1]])
    sp = dense.to_sparse()
    assert torch.equal(slice_sparse_coo_tensor(sp, slice(1, 3), slice(0, 3)).to_dense(), dense[1:3, 0:3])


def test_biencoder_trainer_learns_on_synthetic_batches(tiny_recipe, tmp_path):
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    r = tiny_recipe(
        type="biencoder", code=str(ROOT / "projects" / "arctic_embed" / "train.py"),
        model={"name_or_path": "tiny-llama", "dtype": "fp32", "pooling": "mean", "disable_activation_checkpoint": True},
        tokenizer={"type": "fake"}, micro_batch_size=1, exit_iteration=12, optimizer={"lr": 2e-3, "weight_decay": 0.0},
        use_in_batch_negatives=True, loss_temperature=0.05, mrl_dim=32,
        checkpoint=[{"type": "biencoder", "output_dir": str(tmp_path / "ck"), "save_end_of_training": True}],
    )
    r["data"] = {"synthetic_batches": 12, "synthetic_global_queries": 8, "synthetic_docs_per_query": 2,
                 "synthetic_seq_len": 12, "synthetic_vocab": 1024, "cache_dir": str(tmp_path / "cache")}
    r["deepspeed"] = {"zero_optimization": {"stage": 1}}
    p = tmp_path / "embed.yaml"
    p.write_text(yaml.safe_dump(r))
    cfg = get_config(p)
    tr = get_registered_trainer(cfg.type)(cfg)
    first = tr.eval(next(iter(tr.train_dataloader)))["infoNCE"]
    tr.train()
    last = tr.eval(next(iter(tr.train_dataloader)))["infoNCE"]
    assert tr.global_step == 12 and last < first
    out = next((tmp_path / "ck").glob("global_step_*"))
    assert (out / "biencoder_config.json").exists() and (out / "model.safetensors").exists()


def _write_memory_dataset(fs, root, n_batches=3, nq=8, dpq=2):
    import io

    import pyarrow as pa
    import pyarrow.parquet as pq

    rng = np.random.default_rng(0)
    fs.pipe(f"{root}/metadata.json", b'{"tokenizer": "toy"}')
    for b in range(n_batches):
        base = f"{root}/data/batch_{b:08d}"
        # ids deliberately out of order: the loader must sort by id and map relations through the ids
        qid = rng.permutation(nq) + 100
        did = rng.permutation(nq * dpq) + 500
        tables = {
            "queries.parquet": pa.table({"BATCH_QUERY_ID": qid,
                                         "QUERY_TOKEN_ID_LIST": [list(range(1, 2 + int(i) % 5)) for i in qid]}),
            "documents.parquet": pa.table({"BATCH_DOCUMENT_ID": did,
                                           "DOCUMENT_TOKEN_ID_LIST": [[int(i)] * (1 + int(i) % 7) for i in did]}),
            "relations.parquet": pa.table({"BATCH_QUERY_ID": np.repeat(np.sort(qid), dpq),
                                           "BATCH_DOCUMENT_ID": np.sort(did),
                                           "RELEVANCE": np.tile([1, -1], nq)}),
        }
        for name, t in tables.items():
            buf = io.BytesIO()
            pq.write_table(t, buf)
            fs.pipe(f"{base}/{name}", buf.getvalue())
    return f"{root}/data"


def test_loader_streams_from_an_fsspec_object_store_and_shards_consistently():
    from arctictraining_b200.embed.data import PretokenizedBatchLoader
    from arctictraining_b200.embed.data import open_filesystem
    from arctictraining_b200.embed.data import read_dataset_metadata

    fs = open_filesystem("memory")
    root = _write_memory_dataset(fs, "/embed_ds")
    assert read_dataset_metadata(root, fs) == {"tokenizer": "toy"}
    whole = list(PretokenizedBatchLoader(root, 0, 1, filesystem=fs))
    assert len(whole) == 3
    b = whole[0]
    # rows come out sorted by id: query i has id 100 + i and 1 + (100 + i) % 5 tokens
    lens = b.query_attention_mask.sum(1).tolist()
    assert lens == [1 + (100 + i) % 5 for i in range(8)]
    assert b.document_tokens[:, 0].tolist() == list(range(500, 516))
    dense = b.relevance_labels.to_dense()
    assert dense.shape == (8, 16) and all(dense[i, 2 * i] == 1 and dense[i, 2 * i + 1] == -1 for i in range(8))
    # two ranks see disjoint contiguous slices of the same batch and the same (global) labels
    r0 = list(PretokenizedBatchLoader(root, 0, 2, filesystem=fs, read_ahead=1))
    r1 = list(PretokenizedBatchLoader(root, 1, 2, filesystem=fs, read_ahead=3))
    assert torch.equal(torch.cat([r0[1].query_tokens[:, :1], r1[1].query_tokens[:, :1]]), whole[1].query_tokens[:, :1])
    assert torch.equal(r0[1].relevance_labels.to_dense(), whole[1].relevance_labels.to_dense())
    # split_factor=2 yields two sub-batches per directory with re-based labels
    halves = list(PretokenizedBatchLoader(root, 0, 1, filesystem=fs, split_factor=2))
    assert len(halves) == 6 and halves[0].relevance_labels.shape == (4, 8)
    assert torch.equal(halves[1].relevance_labels.to_dense(), dense[4:, 8:])


def test_collate_truncates_and_left_pads():
    import pyarrow as pa

    from arctictraining_b200.embed.data import collate_token_column

    col = pa.chunked_array([pa.array([[1, 2, 3, 4, 5], [6], [7, 8]], type=pa.list_(pa.int64()))])
    ids, mask = collate_token_column(col, pad_id=0, max_len=3)
    assert ids.tolist() == [[1, 2, 3], [6, 0, 0], [7, 8, 0]] and mask.tolist() == [[1, 1, 1], [1, 0, 0], [1, 1, 0]]
    ids, mask = collate_token_column(col, pad_id=9, max_len=None, left_pad=True)
    assert ids.tolist() == [[1, 2, 3, 4, 5], [9, 9, 9, 9, 6], [9, 9, 9, 7, 8]]
    assert mask.sum(1).tolist() == [5, 1, 2]
