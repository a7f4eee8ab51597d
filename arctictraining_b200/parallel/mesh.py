# SPDX-License-Identifier: Apache-2.0
"""Process groups for data / sequence / expert parallelism.

Ranks are laid out as consecutive blocks: the ``sp`` ranks ``[k*sp, (k+1)*sp)`` form one sequence-parallel
group (one model replica), the ``ep`` ranks ``[k*ep, (k+1)*ep)`` one expert-parallel group, and ranks with
the same position inside their expert-parallel group form an expert-data-parallel group.  ZeRO always
shards dense parameters over the whole world (sequence-parallel ranks count as data-parallel ranks for
that purpose), expert parameters over their expert-data-parallel group.  Parity: the reference gets
these groups from its engine dependency (arctic_training/trainer/trainer.py:271-275,329-336) and has an
unused mesh helper (arctic_training/trainer/parallel_groups.py:19-129).
"""

from __future__ import annotations

from typing import List
from typing import Optional

import torch.distributed as dist


class ParallelGroups:
    def __init__(self, sequence_parallel_size: int = 1, expert_parallel_size: int = 1) -> None:
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.sp_size, self.ep_size = sequence_parallel_size, expert_parallel_size
        for name, n in (("sequence_parallel_size", self.sp_size), ("expert_parallel_size", self.ep_size)):
            if self.world % n != 0:
                raise ValueError(f"world size {self.world} is not divisible by {name}={n}")
        self.dp_size = self.world // self.sp_size
        self.sp_group: Optional[dist.ProcessGroup] = None
        self.ep_group: Optional[dist.ProcessGroup] = None
        self.expert_dp_group: Optional[dist.ProcessGroup] = None
        self.sp_rank = self.rank % self.sp_size
        self.ep_rank = self.rank % self.ep_size
        self.sp_ranks: List[int] = [self.rank]
        self.ep_ranks: List[int] = [self.rank]
        if self.world > 1:
            self._build()

    def _build(self) -> None:
        if self.sp_size > 1:
            for start in range(0, self.world, self.sp_size):
                ranks = list(range(start, start + self.sp_size))
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    self.sp_group, self.sp_ranks = g, ranks
        if self.ep_size > 1:
            for start in range(0, self.world, self.ep_size):
                ranks = list(range(start, start + self.ep_size))
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    self.ep_group, self.ep_ranks = g, ranks
            for pos in range(self.ep_size):
                ranks = list(range(pos, self.world, self.ep_size))
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    self.expert_dp_group = g

    @property
    def dp_rank(self) -> int:
        return self.rank // self.sp_size
