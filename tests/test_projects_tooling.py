# SPDX-License-Identifier: Apache-2.0
"""Pure-Python project tooling: SQL extraction / execution-based verification and the SFT / DPO sampling of ExCoT."""

import sqlite3
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "projects" / "excot_dpo"))

from excot.pipeline import sample_dpo  # noqa: E402
from excot.pipeline import sample_sft  # noqa: E402
from excot.sql_exec import execute  # noqa: E402
from excot.sql_exec import extract_sql  # noqa: E402
from excot.sql_exec import is_correct  # noqa: E402
from excot.sql_exec import same_result  # noqa: E402


def _make_db(root: Path) -> None:
    d = root / "shop"
    d.mkdir(parents=True)
    con = sqlite3.connect(d / "shop.sqlite")
    con.execute("CREATE TABLE items (name TEXT, price REAL)")
    con.executemany("INSERT INTO items VALUES (?, ?)", [("a", 1.0), ("b", 2.5), ("c", 4.0)])
    con.commit()
    con.close()


def test_sql_extraction_and_execution(tmp_path):
    _make_db(tmp_path)
    answer = "First find prices.\n```sql\nSELECT name FROM items WHERE price > 2\n```\nDone."
    sql = extract_sql(answer)
    assert sql == "SELECT name FROM items WHERE price > 2;"
    assert extract_sql("no query here") is None
    status, rows = execute(str(tmp_path / "shop" / "shop.sqlite"), sql)
    assert status == "ok" and same_result(rows, [("c",), ("b",)])
    assert execute(str(tmp_path / "shop" / "shop.sqlite"), "SELECT nope FROM items")[0] == "error"
    assert is_correct(str(tmp_path), "shop", sql, "SELECT name FROM items WHERE price >= 2.5")
    assert not is_correct(str(tmp_path), "shop", "SELECT name FROM items;", "SELECT name FROM items WHERE price >= 2.5")


def test_sft_and_dpo_sampling():
    def cand(qid, correct, text):
        return {"qid": qid, "schema": "s", "question": f"q{qid}", "evidence": "", "answer": text, "correct": correct,
                "pred_sql": "SELECT 1;"}

    rows = [cand(0, True, "good0"), cand(0, False, "bad0"), cand(1, True, "good1"), cand(2, False, "bad2")]
    sft = sample_sft(rows, per_question=1, seed=0)
    assert [m["messages"][-1]["content"] for m in sft] == ["good0", "good1"]
    dpo = sample_dpo(rows, per_question=1, seed=0)
    assert len(dpo) == 1 and dpo[0]["chosen"] == "good0" and dpo[0]["rejected"] == "bad0"


def test_embed_pretokenize_writes_the_layout_the_loader_reads(tmp_path):
    import torch

    sys.path.insert(0, str(ROOT / "projects" / "arctic_embed" / "data_processing"))
    from mine_hard_negatives import mine
    from pretokenize import build_batches

    from arctictraining_b200.embed.data import PretokenizedBatchLoader

    rows = [{"query": f"q{i}", "document": f"d{i % 3}"} for i in range(8)]  # documents shared between queries
    # mining on hand-made embeddings: every query's positive is its own document; one confusable neighbour each
    uniq = {}
    doc_of_row = [uniq.setdefault(r["document"], len(uniq)) for r in rows]
    d = torch.nn.functional.normalize(torch.eye(3) + 0.1, dim=-1)
    q = d[doc_of_row]
    mined = mine(rows, q, d, doc_of_row, num_negatives=1, k=3, max_ratio=0.95)
    assert all(len(m["negatives"]) == 1 and m["negatives"][0] != m["document"] for m in mined)

    def tokenize(texts, is_query):
        return [[1] + [ord(c) % 50 + 2 for c in t] for t in texts]

    n = build_batches(mined, tokenize, batch_size=4, negatives_per_query=1, seed=0, out_dir=tmp_path)
    assert n == 2
    loader = PretokenizedBatchLoader(tmp_path, rank=0, world=1)
    batches = list(loader)
    assert len(batches) == 2
    b = batches[0]
    assert b.query_tokens.shape[0] == 4 and b.relevance_labels.shape[0] == 4
    dense = b.relevance_labels.to_dense()
    assert (dense > 0).sum(1).min() >= 1  # every query has its positive
    assert (dense < 0).any()              # mined negatives are marked


def test_ci_helpers_resolve_extras_upgrade_user_code_and_check_licences(tmp_path):
    sys.path.insert(0, str(ROOT / "ci"))
    import check_license
    import install_extras
    import prefetch_assets
    import upgrade_user_code

    groups = {"__name__": ["arctictraining-b200"], "dev": ["pytest", "arctictraining_b200[embed, dev]"], "embed": ["pyarrow"]}
    assert install_extras.resolve(["dev"], groups) == ["pyarrow", "pytest"]
    assert "dev" in install_extras.load_groups()
    assert install_extras.main(["dev", "--dry-run"]) == 0

    old = '"""doc."""\nfrom x import A, B\n\nclass T(Trainer):\n    config_type = MyConfig  # keep\n    data_factory_type = [A, B]\n    model_factory_type = [A]\n'
    new, n = upgrade_user_code.upgrade_source(old)
    assert n == 3 and "    config: MyConfig  # keep" in new and "    data_factory: Union[A, B]" in new and "    model_factory: A\n" in new
    assert new.startswith('"""doc."""\nfrom typing import Union')
    assert upgrade_user_code.upgrade_source(new)[1] == 0  # idempotent

    f = tmp_path / "m.py"
    f.write_text("#!/usr/bin/env python\nimport os\n")
    assert not check_license.has_identifier(f)
    check_license.insert_identifier(f)
    assert f.read_text().split("\n")[1] == "# " + check_license.SPDX and check_license.has_identifier(f)
    assert check_license.main([]) == 0  # the repository itself is clean

    cfg = {"data": {"sources": ["org/ds", {"name_or_path": "org/other", "split": "train[:10]", "kwargs": {"name": "x"}}]},
           "model": {"name_or_path": "org/model"}, "tokenizer": {"name_or_path": "org/model"}}
    assert list(prefetch_assets.iter_sources(cfg)) == [("org/ds", None, {}), ("org/other", "train[:10]", {"name": "x"})]
    assert prefetch_assets.model_ids(cfg) == ["org/model"]


def test_recipe_reference_is_up_to_date():
    """``docs/config.md`` is generated from the configuration classes; a field added without regenerating fails here."""
    import subprocess

    res = subprocess.run([sys.executable, str(ROOT / "docs" / "gen_config_reference.py"), "--check"], cwd=ROOT)
    assert res.returncode == 0, "run `python docs/gen_config_reference.py`"
