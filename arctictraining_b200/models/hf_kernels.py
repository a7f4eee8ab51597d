# SPDX-License-Identifier: Apache-2.0
"""This package's kernels inside models of the ``transformers`` library (``model.type: liger``).

The own architectures use the kernels everywhere.  A library model (an architecture without an own implementation) can
still take two of them, the way the reference patches such models with an external kernel package
(arctic_training/model/liger_factory.py:24-69): RMSNorm modules run :func:`arctictraining_b200.ops.rms_norm`, and the
trainer computes the loss from the model body's hidden states with the tiled fused output-projection + cross-entropy
(:func:`arctictraining_b200.ops.fused_linear_cross_entropy`), so ``[tokens, vocabulary]`` logits never exist.  Both ops
fall back to their PyTorch reference implementations off the GPU or for shapes the kernels do not cover.
"""

from __future__ import annotations

import types
from typing import Dict

import torch

from .. import ops


def _rms_norm_forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
    return ops.rms_norm(hidden_states, self.weight, self._atb_eps)


def apply_kernels_to_hf_model(model: torch.nn.Module) -> Dict[str, int]:
    """Patch ``model`` in place; returns how many modules of each kind were switched."""
    counts = {"rms_norm": 0}
    for mod in model.modules():
        name = type(mod).__name__
        weight = getattr(mod, "weight", None)
        # variants that scale by (1 + weight) or carry no weight keep their own forward
        if not name.endswith("RMSNorm") or "Gemma" in name or not isinstance(weight, torch.nn.Parameter) or weight.dim() != 1:
            continue
        eps = getattr(mod, "variance_epsilon", None)
        if eps is None:
            eps = getattr(mod, "eps", None)
        if eps is None or getattr(mod, "_atb_eps", None) is not None:
            continue
        mod._atb_eps = float(eps)
        mod.forward = types.MethodType(_rms_norm_forward, mod)
        counts["rms_norm"] += 1
    head = model.get_output_embeddings() if hasattr(model, "get_output_embeddings") else None
    # the fused loss multiplies by the output projection's weight itself: it needs a plain bias-free linear layer
    model._atb_fused_loss = bool(isinstance(head, torch.nn.Linear) and head.bias is None)
    return counts
