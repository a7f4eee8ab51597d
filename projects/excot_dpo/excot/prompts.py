# SPDX-License-Identifier: Apache-2.0
"""Prompt of the divide-and-conquer chain-of-thought text-to-SQL generation."""

SYSTEM = "You are an expert data analyst who writes correct SQLite queries."

DIVIDE_AND_CONQUER = """Database schema:
{schema}

Question: {question}
{evidence}
Work in three steps.
1. Divide: split the question into sub-questions that can each be answered by one simple query.
2. Conquer: write the SQL of every sub-question and explain how the pieces combine.
3. Assemble: give the final query in a single ```sql fenced block.
"""


def build_messages(schema: str, question: str, evidence: str = "") -> list:
    ev = f"Hint: {evidence}\n" if evidence else ""
    return [
        {"role": "system", "content": SYSTEM},
        {"role": "user", "content": DIVIDE_AND_CONQUER.format(schema=schema, question=question, evidence=ev)},
    ]
