# SPDX-License-Identifier: Apache-2.0
"""Text-to-SQL data preparation and BIRD / Spider evaluation (the reference's projects/arctic_text2sql_r1: value index,
prompt construction, sampling with vLLM, execution-based scoring with self-consistency)."""
