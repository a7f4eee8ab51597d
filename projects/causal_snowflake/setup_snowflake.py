# SPDX-License-Identifier: Apache-2.0
"""Creates the Snowflake objects the `run-causal-snowflake-*.yml` recipes read: a database / schema, a table with one
TEXT column filled from a Hugging Face text dataset, and (optionally) a Snowflake Dataset version of that table.

    python projects/causal_snowflake/setup_snowflake.py --dataset stas/gutenberg-100 --split train --limit 100

Needs `snowflake-snowpark-python` (and `snowflake-ml-python` for `--make-dataset`) plus credentials in the environment
or in ~/.snowflake/connections.toml.  The reference ships the same helper as projects/causal_snowflake/setup_snowflake.py.
"""

import argparse


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--database", default="ARCTIC_TRAINING")
    ap.add_argument("--schema", default="CAUSAL_DEMO")
    ap.add_argument("--table", default="GUTENBERG_100")
    ap.add_argument("--dataset", default="stas/gutenberg-100")
    ap.add_argument("--split", default="train")
    ap.add_argument("--column", default="text")
    ap.add_argument("--limit", type=int, default=100)
    ap.add_argument("--connection", default=None, help="name of a connection in connections.toml")
    ap.add_argument("--make-dataset", action="store_true", help="also create <table>_DS version v1 as a Snowflake Dataset")
    args = ap.parse_args()

    try:
        from snowflake.snowpark import Session
    except ImportError as e:  # pragma: no cover - optional dependency
        raise SystemExit("snowflake-snowpark-python is not installed") from e
    import pandas as pd
    from datasets import load_dataset

    builder = Session.builder
    if args.connection:
        builder = builder.config("connection_name", args.connection)
    session = builder.create()
    fq_schema = f"{args.database}.{args.schema}"
    session.sql(f"CREATE DATABASE IF NOT EXISTS {args.database}").collect()
    session.sql(f"CREATE SCHEMA IF NOT EXISTS {fq_schema}").collect()

    rows = load_dataset(args.dataset, split=args.split)
    if args.limit:
        rows = rows.select(range(min(args.limit, len(rows))))
    frame = pd.DataFrame({"TEXT": [r[args.column] for r in rows]})
    session.write_pandas(frame, args.table, database=args.database, schema=args.schema, auto_create_table=True, overwrite=True)
    print(f"wrote {len(frame)} rows to {fq_schema}.{args.table}")

    if args.make_dataset:
        from snowflake.ml import dataset as sf_dataset

        ds = sf_dataset.create_from_dataframe(
            session, f"{fq_schema}.{args.table}_DS", "v1", input_dataframe=session.table(f"{fq_schema}.{args.table}")
        )
        print(f"created dataset {ds.fully_qualified_name} version v1")
    session.close()


if __name__ == "__main__":
    main()
