# SPDX-License-Identifier: Apache-2.0
"""Small helpers of the data layer.  Parity: arctic_training/data/utils.py:32-97."""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any
from typing import Iterator

from torch.utils.data import DataLoader

_NETWORK_FS = {"nfs", "nfs4", "lustre", "gpfs", "ceph", "cifs", "smb", "fuse.s3fs", "fuse.gcsfuse", "beegfs", "afs", "glusterfs"}


def is_local_fs(path: Path) -> bool:
    """Best-effort test whether ``path`` sits on a node-local file system (vs. a shared network one)."""
    try:
        import psutil

        path = Path(path).resolve()
        best, fstype = "", ""
        for part in psutil.disk_partitions(all=True):
            mp = part.mountpoint
            if str(path).startswith(mp) and len(mp) > len(best):
                best, fstype = mp, part.fstype.lower()
        return not any(fstype.startswith(n) for n in _NETWORK_FS)
    except Exception:
        return True


def calculate_hash_from_args(*args: Any) -> str:
    """Stable md5 of JSON-serialisable arguments (cache directory names)."""
    h = hashlib.md5()
    for a in args:
        h.update(json.dumps(a, sort_keys=True, default=str).encode("utf-8"))
    return h.hexdigest()


class OverfitOneBatchDataLoader:
    """Yields the first batch of a dataloader again and again (``overfit_first_batch``)."""

    def __init__(self, dataloader: DataLoader, num_batches: int = 0) -> None:
        self.dataloader = dataloader
        self.num_batches = num_batches or len(dataloader)
        self.batch = next(iter(dataloader))

    def __len__(self) -> int:
        return self.num_batches

    def __iter__(self) -> Iterator[Any]:
        for _ in range(self.num_batches):
            yield self.batch

    def __getattr__(self, name: str) -> Any:
        return getattr(self.dataloader, name)
