# SPDX-License-Identifier: Apache-2.0
"""Token generation with a key/value cache for the native decoder models.

Used where training needs samples from the model itself (the MLP speculator's generation modes).  The reference
generates through Hugging Face's ``DynamicCache`` and also returns the final hidden state of every processed position
(projects/mlp_speculator/train.py:224-291); this does the same on the native model: the prompt is processed once, every
further token costs one forward of a single position, and the layers run through their usual (engine-wrapped) forward
so that ZeRO-3 parameter gathering keeps working.
"""

from __future__ import annotations

from typing import Optional
from typing import Tuple

import torch
import torch.nn.functional as F


@torch.no_grad()
def generate(
    model: torch.nn.Module,
    input_ids: torch.Tensor,
    max_new_tokens: int,
    do_sample: bool = True,
    temperature: float = 1.0,
    top_k: int = 10,
    generator: Optional[torch.Generator] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(tokens [B, S0 + new], hidden [B, S0 + new - 1, H])``: the prompt followed by the generated tokens, and
    the final (normed) hidden state of every position that was fed to the model (the state at position ``t`` predicts
    token ``t + 1``)."""
    assert input_ids.dim() == 2, "generate: input_ids must be [batch, length]"
    B, S0 = input_ids.shape
    dev = input_ids.device
    n_layers = len(model.model.layers)
    cache = [None] * n_layers
    tokens = input_ids
    step_ids, pos0 = input_ids, 0
    hidden_parts = []
    lm_w = model.lm_head.weight
    for _ in range(max_new_tokens):
        S = step_ids.shape[1]
        position_ids = torch.arange(pos0, pos0 + S, device=dev).unsqueeze(0).expand(B, S)
        ctx = model.model.make_context(position_ids, "sdpa")
        ctx.kv_cache = cache
        h = model.model(step_ids, position_ids, ctx)
        hidden_parts.append(h)
        logits = F.linear(h[:, -1], lm_w).float()
        if do_sample:
            logits = logits / max(temperature, 1e-6)
            if top_k:
                kth = torch.topk(logits, min(top_k, logits.shape[-1])).values[:, -1:]
                logits = logits.masked_fill(logits < kth, float("-inf"))
            nxt = torch.multinomial(torch.softmax(logits, dim=-1), 1, generator=generator)
        else:
            nxt = logits.argmax(-1, keepdim=True)
        tokens = torch.cat([tokens, nxt], dim=1)
        pos0 += S
        step_ids = nxt
    return tokens, torch.cat(hidden_parts, dim=1)
