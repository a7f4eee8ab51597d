# SPDX-License-Identifier: Apache-2.0
"""Arctic-Embed project: importing this file registers the ``biencoder`` trainer, model factory, checkpoint engine and
the ``contrastive_pretokenized`` data factory (implementation: ``arctictraining_b200/embed``)."""

from arctictraining_b200.embed.trainer import BiencoderCheckpointEngine  # noqa: F401
from arctictraining_b200.embed.trainer import BiencoderModelFactory  # noqa: F401
from arctictraining_b200.embed.trainer import BiencoderTrainer  # noqa: F401
