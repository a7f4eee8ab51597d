# SPDX-License-Identifier: Apache-2.0
"""A directory (or explicit list) of parquet files treated as one table, streamed file by file.

Parity: projects/arctic_embed/src/arctic_embed/data_processing/many_parquet_dataset.py:36-196.  Row counts come from
the parquet footers (fetched concurrently — on an object store each is one small ranged read), streaming keeps one file
in memory while the next is being fetched.
"""

from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from typing import Iterator
from typing import List
from typing import Optional
from typing import Sequence
from typing import Tuple


def filesystem_for(path: str):
    """``(filesystem, path without protocol)`` for a local path or a URL such as ``s3://bucket/prefix``."""
    import fsspec

    fs, stripped = fsspec.core.url_to_fs(path)
    return fs, stripped


@dataclass
class ParquetCollection:
    paths: List[str]
    rows_per_file: List[int]
    fs: object

    @property
    def num_rows(self) -> int:
        return sum(self.rows_per_file)

    @property
    def num_files(self) -> int:
        return len(self.paths)

    def batches_per_epoch(self, batch_size: int) -> int:
        return self.num_rows // batch_size

    @classmethod
    def from_location(cls, location: str, threads: int = 16) -> "ParquetCollection":
        """``location`` is one parquet file or a directory searched recursively."""
        fs, root = filesystem_for(location)
        if fs.isfile(root):
            paths = [root]
        else:
            paths = sorted(p for p in fs.find(root) if p.endswith(".parquet"))
        if not paths:
            raise FileNotFoundError(f"no parquet files under {location}")
        return cls.from_paths(paths, fs, threads)

    @classmethod
    def from_paths(cls, paths: Sequence[str], fs, threads: int = 16) -> "ParquetCollection":
        import pyarrow.parquet as pq

        def rows(p: str) -> int:
            with fs.open(p, "rb") as f:
                return pq.ParquetFile(f).metadata.num_rows

        with ThreadPoolExecutor(max_workers=max(1, min(threads, len(paths)))) as pool:
            counts = list(pool.map(rows, paths))
        return cls(list(paths), counts, fs)

    def stream_tables(self, columns: Optional[Sequence[str]] = None, row_range: Optional[Tuple[int, int]] = None) -> Iterator:
        """Tables in file order, restricted to the global row range ``[start, stop)``; files entirely outside it are
        never opened.  The next file is fetched while the caller works on the current one."""
        import pyarrow.parquet as pq

        start, stop = row_range if row_range is not None else (0, self.num_rows)
        todo = []
        first = 0
        for path, n in zip(self.paths, self.rows_per_file):
            lo, hi = max(start, first), min(stop, first + n)
            if lo < hi:
                todo.append((path, lo - first, hi - lo))
            first += n

        def read(item):
            path, off, length = item
            t = pq.read_table(path, columns=list(columns) if columns else None, filesystem=self.fs)
            return t.slice(off, length)

        with ThreadPoolExecutor(max_workers=1) as pool:
            nxt = pool.submit(read, todo[0]) if todo else None
            for i in range(len(todo)):
                table = nxt.result()
                nxt = pool.submit(read, todo[i + 1]) if i + 1 < len(todo) else None
                yield table

    def stream_chunks(self, chunk_rows: int, columns: Optional[Sequence[str]] = None,
                      row_range: Optional[Tuple[int, int]] = None) -> Iterator:
        """Tables of exactly ``chunk_rows`` rows (the last may be shorter), re-cut across file boundaries."""
        import pyarrow as pa

        held, held_rows = [], 0
        for t in self.stream_tables(columns, row_range):
            held.append(t)
            held_rows += t.num_rows
            while held_rows >= chunk_rows:
                whole = pa.concat_tables(held)
                yield whole.slice(0, chunk_rows)
                rest = whole.slice(chunk_rows)
                held, held_rows = ([rest] if rest.num_rows else []), rest.num_rows
        if held_rows:
            yield pa.concat_tables(held)

    def read_all(self, columns: Optional[Sequence[str]] = None):
        import pyarrow as pa

        return pa.concat_tables(list(self.stream_tables(columns)))
