# SPDX-License-Identifier: Apache-2.0
from .mesh import ParallelGroups
from .ulysses import UlyssesContext
from .ulysses import UlyssesDataLoaderAdapter

__all__ = ["ParallelGroups", "UlyssesContext", "UlyssesDataLoaderAdapter"]
