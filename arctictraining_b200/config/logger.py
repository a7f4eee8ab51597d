# SPDX-License-Identifier: Apache-2.0
"""``logger:`` section.  Parity: arctic_training/config/logger.py:29-66."""

from __future__ import annotations

import os
from pathlib import Path
from typing import List
from typing import Literal
from typing import Union

from pydantic import model_validator
from typing_extensions import Self

from .base import BaseConfig

_NULL = Path("/dev/null")


class LoggerConfig(BaseConfig):
    output_dir: Path = _NULL
    """ Output directory for log files (``/dev/null`` disables file logging). """

    level: str = "INFO"
    """ Log level. """

    print_output_ranks: Union[Literal["*"], List[int]] = [0]
    """ Local ranks that print to the console; ``"*"`` for all. """

    file_output_ranks: Union[Literal["*"], List[int]] = "*"
    """ Local ranks that write a log file; ``"*"`` for all. """

    @model_validator(mode="after")
    def _expand_star(self) -> Self:
        for field in ("print_output_ranks", "file_output_ranks"):
            if getattr(self, field) == "*":
                object.__setattr__(self, field, list(range(max(self.world_size, 1))))
        os.environ.setdefault("WANDB_DATA_DIR", str(self.output_dir))
        return self

    @property
    def log_file(self) -> Path:
        return self.output_dir / "logs" / f"rank_{self.local_rank}.log"

    @property
    def file_enabled(self) -> bool:
        return self.output_dir != _NULL and self.local_rank in self.file_output_ranks

    @property
    def print_enabled(self) -> bool:
        return self.local_rank in self.print_output_ranks
