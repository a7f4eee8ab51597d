# SPDX-License-Identifier: Apache-2.0
"""Floating-point operation estimates for decoder transformers (used for the tflops metrics).

Convention as in the reference (arctic_training/trainer/flops_counter.py:58-377): a matmul with N
weights costs 2N flop per token forward; with backward the multiplier is 6 (8 with activation
checkpointing, which replays the forward); attention scores/values cost ``seqlen^2 * head_dim * heads``
per layer with multiplier 12 (16 with checkpointing) and are computed per packed sample, because tokens
only attend inside their own sample.  Mixture-of-experts layers count the ``top_k`` active experts plus
the router.
"""

from __future__ import annotations

from typing import Any
from typing import Iterable
from typing import Sequence
from typing import Tuple


def _get(cfg: Any, key: str, default: Any = None) -> Any:
    if isinstance(cfg, dict):
        v = cfg.get(key, default)
    else:
        v = getattr(cfg, key, default)
    return default if v is None else v


class FlopsCounter:
    def __init__(self, config: Any, model_size: int, enable_gradient_checkpointing: bool = False) -> None:
        self.config = _get(config, "text_config", config)
        self.model_size = model_size
        self.dense_mult = 8 if enable_gradient_checkpointing else 6
        self.attn_mult = 16 if enable_gradient_checkpointing else 12

    def _mults(self, forward_only: bool) -> Tuple[int, int]:
        return (2, 2) if forward_only else (self.dense_mult, self.attn_mult)

    def _decoder(self, seqlens: Sequence[int], forward_only: bool) -> float:
        c = self.config
        hidden, vocab, layers = _get(c, "hidden_size"), _get(c, "vocab_size"), _get(c, "num_hidden_layers")
        heads = _get(c, "num_attention_heads")
        kv_heads = _get(c, "num_key_value_heads", heads)
        head_dim = _get(c, "head_dim", hidden // heads)
        n_exp = _get(c, "num_experts", 0) or _get(c, "num_local_experts", 0)
        dense_m, attn_m = self._mults(forward_only)
        tokens = sum(seqlens)
        if n_exp:
            mlp = hidden * _get(c, "num_experts_per_tok", 1) * _get(c, "moe_intermediate_size", _get(c, "intermediate_size")) * 3
            mlp += hidden * n_exp
            shared = _get(c, "shared_expert_intermediate_size", 0)
            if shared:
                mlp += hidden * shared * 3
        else:
            mlp = hidden * _get(c, "intermediate_size") * 3
        attn_linear = hidden * (heads * head_dim + 2 * kv_heads * head_dim + heads * head_dim)
        full_every = _get(c, "full_attention_interval", 1)
        full_layers = layers // full_every
        linear_layers = layers - full_layers
        dense_n = mlp * layers + attn_linear * full_layers + self._gated_delta_net_weights() * linear_layers + vocab * hidden
        dense_flops = dense_m * dense_n * tokens
        attn_flops = attn_m * sum(s * s for s in seqlens) * head_dim * heads * full_layers
        return (dense_flops + attn_flops) / 1e12

    def _gated_delta_net_weights(self) -> int:
        """Per-token multiply-accumulates of one linear-attention (gated delta rule) layer, the hybrid layers of
        Qwen3-Next: input projections, short convolution, the four ``d_v x d_v`` state products per value head, output
        projection.  Zero for models without such layers."""
        c = self.config
        kd, vd = _get(c, "linear_key_head_dim", 0), _get(c, "linear_value_head_dim", 0)
        if not kd:
            return 0
        kh, vh = _get(c, "linear_num_key_heads"), _get(c, "linear_num_value_heads")
        hidden, conv = _get(c, "hidden_size"), _get(c, "linear_conv_kernel_dim", 4)
        qk, v = kd * kh, vd * vh
        return hidden * (2 * qk + 2 * v + 2 * vh) + conv * (2 * qk + v) + vh * vd * vd * 4 + hidden * v

    def _mla_moe(self, seqlens: Sequence[int], forward_only: bool) -> float:
        """DeepSeek-V2 / V3: multi-head latent attention (low-rank query and joint key/value projections, a shared
        rotary key) and routed + shared experts after ``first_k_dense_replace`` dense layers."""
        c = self.config
        hidden, vocab, layers = _get(c, "hidden_size"), _get(c, "vocab_size"), _get(c, "num_hidden_layers")
        heads = _get(c, "num_attention_heads")
        nope, rope, v_dim = _get(c, "qk_nope_head_dim"), _get(c, "qk_rope_head_dim"), _get(c, "v_head_dim")
        q_rank, kv_rank = _get(c, "q_lora_rank", 0), _get(c, "kv_lora_rank")
        q_dim = nope + rope
        attn = hidden * heads * q_dim if not q_rank else hidden * q_rank + q_rank * heads * q_dim
        attn += hidden * (kv_rank + rope)             # down-projection to the latent + the shared rotary key
        attn += heads * (nope + v_dim) * kv_rank      # up-projection of keys (non-rotary part) and values
        attn += heads * v_dim * hidden                # output projection
        routed = _get(c, "n_routed_experts", 0)
        dense_first = _get(c, "first_k_dense_replace", 0) if routed else layers
        moe_layer = hidden * routed + hidden * _get(c, "moe_intermediate_size", 0) * 3 * (
            _get(c, "num_experts_per_tok", 0) + _get(c, "n_shared_experts", 0))
        dense_layer = hidden * _get(c, "intermediate_size") * 3
        n = (moe_layer + attn) * (layers - dense_first) + (dense_layer + attn) * dense_first + vocab * hidden
        dense_m, attn_m = self._mults(forward_only)
        flops = dense_m * n * sum(seqlens) + attn_m * sum(s * s for s in seqlens) * layers * q_dim * heads
        return flops / 1e12

    def _generic(self, seqlens: Sequence[int], forward_only: bool) -> float:
        c = self.config
        dense_m, attn_m = self._mults(forward_only)
        hidden, layers = _get(c, "hidden_size", 0), _get(c, "num_hidden_layers", 0)
        total = 0.0
        for s in seqlens:
            total += dense_m * self.model_size * s + attn_m * layers * hidden * s * s
        return total / 1e12

    def estimate_tflos(self, batch_seqlens: Sequence[int], delta_time: float = 1, forward_only: bool = False) -> float:
        c = self.config
        if _get(c, "kv_lora_rank") and _get(c, "qk_rope_head_dim"):
            return self._mla_moe(batch_seqlens, forward_only)
        if _get(c, "num_attention_heads") and _get(c, "intermediate_size", _get(c, "moe_intermediate_size")):
            return self._decoder(batch_seqlens, forward_only)
        return self._generic(batch_seqlens, forward_only)


def estimate_decoder_transformer_tflos(
    hf_model_config: Any, model_size: int, batch_of_seqlens: Iterable[Sequence[int]],
    enable_gradient_checkpointing: bool, forward_only: bool = False,
) -> Tuple[float, int]:
    """``batch_of_seqlens`` has one list per batch row with the lengths of the samples packed in it."""
    counter = FlopsCounter(hf_model_config, model_size, enable_gradient_checkpointing)
    tflos, tokens = 0.0, 0
    for seqlens in batch_of_seqlens:
        seqlens = list(seqlens)
        tflos += counter.estimate_tflos(seqlens, forward_only=forward_only)
        tokens += sum(seqlens)
    return tflos, tokens
