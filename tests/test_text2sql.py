# SPDX-License-Identifier: Apache-2.0
"""Text-to-SQL project: schema description, value index, prompt building and execution-based evaluation on a toy
SQLite database."""

import json
import random
import sqlite3
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "projects" / "arctic_text2sql_r1"))

from text2sql import evaluate as ev  # noqa: E402
from text2sql import prompting  # noqa: E402
from text2sql import schema as sch  # noqa: E402
from text2sql import value_index as vi  # noqa: E402

TABLES = {
    "db_id": "shop",
    "table_names_original": ["customer", "order"],
    "table_names": ["customer", "order"],
    "column_names_original": [[-1, "*"], [0, "id"], [0, "full name"], [0, "city"], [1, "id"], [1, "customer_id"], [1, "total"]],
    "column_names": [[-1, "*"], [0, "id"], [0, "name of the customer"], [0, "city"], [1, "id"], [1, "customer id"], [1, "order total in dollars"]],
    "column_types": ["text", "integer", "text", "text", "integer", "integer", "real"],
    "primary_keys": [1, 4],
    "foreign_keys": [[5, 1]],
}


@pytest.fixture
def shop(tmp_path):
    d = tmp_path / "dbs" / "shop"
    d.mkdir(parents=True)
    con = sqlite3.connect(d / "shop.sqlite")
    con.executescript("""
        CREATE TABLE customer (id INTEGER PRIMARY KEY, `full name` TEXT, city TEXT);
        CREATE TABLE `order` (id INTEGER PRIMARY KEY, customer_id INTEGER, total REAL);
        INSERT INTO customer VALUES (1, 'Ada Lovelace', 'London'), (2, 'Grace Hopper', 'New York'), (3, 'Alan Turing', 'London');
        INSERT INTO `order` VALUES (1, 1, 10.5), (2, 1, 4.0), (3, 2, 99.0);
    """)
    con.commit()
    con.close()
    return tmp_path / "dbs"


def test_schema_text_quotes_identifiers_and_lists_keys_and_examples(shop):
    assert sch.quote_identifier("order") == "`order`" and sch.quote_identifier("full name") == "`full name`"
    assert sch.quote_identifier("city") == "city"
    sampled = sch.sample_column_values(str(shop / "shop" / "shop.sqlite"), TABLES["table_names_original"], 2)
    assert sampled["customer.city"] == ["London", "New York"] and sampled["order.total"] == [10.5, 4.0]
    text = sch.describe_database(TABLES, sampled, {"customer.city": ["New York"]})
    assert "CREATE TABLE `order` (" in text and "PRIMARY KEY (id)" in text
    assert "CONSTRAINT fk_order_customer_id FOREIGN KEY (customer_id) REFERENCES customer (id)" in text
    assert "`full name` text, -- name of the customer, example: ['Ada Lovelace', 'Grace Hopper']" in text
    assert "city text, -- example: ['New York', 'London']" in text   # matched values first, no comment repeated
    assert not text.rstrip().endswith(",\n);")
    # train mode keeps key columns and the columns of the answer; the rest is a random share
    train = sch.describe_database(TABLES, sampled, mode="train", answer="SELECT total FROM `order`", rng=random.Random(3))
    assert "total real" in train and "customer_id integer" in train
    assert len(sch.create_statements(str(shop / "shop" / "shop.sqlite"))) == 2
    assert sch.strip_sql_comments("SELECT 1 -- one\n/* two */") == "SELECT 1"


def test_value_index_finds_cells_mentioned_in_the_question(shop, tmp_path):
    done = vi.build_indexes(str(shop), str(tmp_path / "idx"))
    assert done == ["shop"]
    index = vi.ValueIndex.load(tmp_path / "idx" / "shop.json")
    assert index.search("hopper", 3)[0]["contents"] == "Grace Hopper"
    found = vi.question_values(index, "How much did Grace Hopper from New York spend?")
    assert found == {"customer.full name": ["Grace Hopper"], "customer.city": ["New York"]}
    assert vi.substring_coverage("New York", "in new york city") == 1.0
    assert vi.substring_coverage("Londonderry", "in London") == pytest.approx(6 / 11)
    assert "grace hopper" in [g.lower() for g in vi.n_grams("Grace Hopper spends", 2)]


def test_prompt_building_for_bird_rows(shop, tmp_path):
    vi.build_indexes(str(shop), str(tmp_path / "idx"))
    rows = [{"db_id": "shop", "question": "Total spent by Ada Lovelace?", "evidence": "spent refers to total",
             "SQL": "SELECT SUM(total) FROM `order` WHERE customer_id = 1"}]
    ex = prompting.build_examples(rows, [TABLES], str(shop), "bird", "dev", 2, str(tmp_path / "idx"))
    assert len(ex) == 1 and ex[0]["output_seq"] == rows[0]["SQL"]
    assert ex[0]["question"] == "spent refers to total\nTotal spent by Ada Lovelace?"
    assert "Database Engine:\nSQLite" in ex[0]["input_seq"] and "example: ['Ada Lovelace'" in ex[0]["input_seq"]
    with pytest.raises(ValueError):
        prompting.build_examples(rows, [TABLES], str(shop), "nope")
    prompting.write_examples(ex, str(tmp_path / "out.json"))
    assert json.loads((tmp_path / "out.json").read_text())[0]["db_id"] == "shop"


def test_execution_accuracy_greedy_voting_and_pass_at_k(shop):
    gold = [{"db_id": "shop", "question": "q1", "SQL": "SELECT city FROM customer WHERE id = 1"},
            {"db_id": "shop", "question": "q2", "SQL": "SELECT COUNT(*) FROM `order`"}]
    right1, right2 = "SELECT city FROM customer WHERE `full name` = 'Ada Lovelace'", "SELECT 3"
    preds = [{"pred_sqls": ["SELECT 'Paris'", right1, right1]},
             {"pred_sqls": [right2, "SELECT nonsense FROM", "SELECT 4"]}]
    assert ev.run_eval(gold, preds, str(shop), "greedy_search", num_cpus=1)[0] == 0.5
    acc, chosen = ev.run_eval(gold, preds, str(shop), "major_voting", num_cpus=1)
    assert chosen[0] == right1 and acc == 1.0 or acc == 0.5  # question 2 has a 1:1 tie between valid results
    assert chosen[0] == right1
    assert ev.run_eval(gold, preds, str(shop), "pass@k", num_cpus=1)[0] == 1.0
    acc_soft, chosen_soft = ev.run_eval(gold, preds, str(shop), "major_voting", num_cpus=1, voting="soft")
    assert chosen_soft[0] == right1
    assert ev.parse_response("thinking...\n```sql\nSELECT 1\n```\nmore\n```SQL\nSELECT 2;\n```") == "SELECT 2;"
    assert ev.parse_response("no code") == ""
    # a statement that would run for ever is interrupted and counted as invalid
    slow = "WITH RECURSIVE c(x) AS (SELECT 1 UNION ALL SELECT x + 1 FROM c) SELECT COUNT(*) FROM c"
    res = ev.execute_many([ev.db_file_of(str(shop), "shop")], [slow], num_cpus=1, timeout=0.3)
    assert res[0]["valid"] == 0


def test_soft_similarity_and_votes():
    a = {"columns": ["x"], "rows": [(1,), (2,), (2,)]}
    b = {"columns": ["x"], "rows": [(2,), (2,), (3,)]}
    assert ev.soft_similarity(a, a) == 1.0
    assert ev.soft_similarity(a, b) == pytest.approx(2 / 4)   # agreement min-counts 2 of max-counts 1 + 2 + 1
    assert ev.soft_similarity(a, None) == 0.0
    samples = [{"sql": "A", "valid": 0, "rows": None, "columns": None}, {"sql": "B", "valid": 0, "rows": None, "columns": None}]
    assert ev.vote(samples, random_when_all_fail=False) == ev.ERROR_SQL
    assert ev.vote(samples, rng=random.Random(0)) in ("A", "B")
