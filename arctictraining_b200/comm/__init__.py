# SPDX-License-Identifier: Apache-2.0
from .dist import all_gather_object
from .dist import barrier
from .dist import get_rank
from .dist import get_world_size
from .dist import init_distributed

__all__ = ["all_gather_object", "barrier", "get_rank", "get_world_size", "init_distributed"]
