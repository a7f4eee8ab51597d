# SPDX-License-Identifier: Apache-2.0
"""Architecture descriptions: built-in presets and ``config.json`` loading, without ``transformers``.

A model is described by a plain dict with Hugging Face key names (``hidden_size``,
``num_attention_heads`` ...), so ``config.json`` files written by this framework load in
``transformers`` / vLLM and vice versa.  ``model.name_or_path`` may be a directory that holds a
``config.json`` or the name of a preset below (random initialisation, no files needed) — the reference
needs a model directory even for random-init runs (arctic_training/config/trainer.py:187-199,406-418).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any
from typing import Dict
from typing import Optional
from typing import Union


class ArchConfig(dict):
    """Dict with attribute access; unknown attributes read as ``None`` through ``get``."""

    def __getattr__(self, key: str) -> Any:
        try:
            return self[key]
        except KeyError as exc:
            raise AttributeError(key) from exc

    def __setattr__(self, key: str, value: Any) -> None:
        self[key] = value

    @property
    def head_dim_(self) -> int:
        return int(self.get("head_dim") or self["hidden_size"] // self["num_attention_heads"])

    @property
    def is_moe(self) -> bool:
        return bool(self.get("num_experts") or self.get("num_local_experts") or self.get("n_routed_experts"))

    def to_json_dict(self) -> Dict[str, Any]:
        return {k: v for k, v in self.items() if not k.startswith("_")}

    def to_hf(self) -> Any:
        """The same architecture as a config object of the transformers library, e.g. for a custom model factory that
        builds its model with ``AutoModelForCausalLM.from_config(model_config.to_hf())``."""
        from transformers import AutoConfig

        fields = {k: v for k, v in self.to_json_dict().items() if k not in ("model_type", "transformers_version")}
        return AutoConfig.for_model(self["model_type"], **fields)


def _llama(hidden, layers, heads, kv_heads, inter, vocab, theta, max_pos, **extra) -> Dict[str, Any]:
    cfg = dict(
        architectures=["LlamaForCausalLM"],
        model_type="llama",
        hidden_size=hidden,
        num_hidden_layers=layers,
        num_attention_heads=heads,
        num_key_value_heads=kv_heads,
        intermediate_size=inter,
        vocab_size=vocab,
        rope_theta=theta,
        max_position_embeddings=max_pos,
        rms_norm_eps=1e-5,
        hidden_act="silu",
        tie_word_embeddings=False,
        attention_bias=False,
        mlp_bias=False,
        bos_token_id=1,
        eos_token_id=2,
        torch_dtype="bfloat16",
    )
    cfg.update(extra)
    return cfg


PRESETS: Dict[str, Dict[str, Any]] = {
    # 2 layers, hidden 64, 4 q heads / 2 kv heads, SwiGLU 128, vocab 1024 (CPU plumbing tests)
    "tiny-llama": _llama(64, 2, 4, 2, 128, 1024, 10000.0, 2048),
    "llama-3.1-8b": _llama(4096, 32, 32, 8, 14336, 128256, 500000.0, 131072, bos_token_id=128000, eos_token_id=128001),
    "llama-3.1-70b": _llama(8192, 80, 64, 8, 28672, 128256, 500000.0, 131072),
    "llama-3.1-405b": _llama(16384, 126, 128, 8, 53248, 128256, 500000.0, 131072),
    "llama-3.3-70b": _llama(8192, 80, 64, 8, 28672, 128256, 500000.0, 131072),
    "llama-3.2-3b": _llama(3072, 28, 24, 8, 8192, 128256, 500000.0, 131072, tie_word_embeddings=True, head_dim=128),
    "mistral-7b": _llama(
        4096, 32, 32, 8, 14336, 32768, 1000000.0, 32768, architectures=["MistralForCausalLM"], model_type="mistral",
    ),
    "qwen2.5-32b": _llama(
        5120, 64, 40, 8, 27648, 152064, 1000000.0, 32768,
        architectures=["Qwen2ForCausalLM"], model_type="qwen2", attention_bias=True, rms_norm_eps=1e-6,
    ),
    "qwen3-8b": _llama(
        4096, 36, 32, 8, 12288, 151936, 1000000.0, 40960,
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", head_dim=128, rms_norm_eps=1e-6, qk_norm=True,
    ),
    "llama-3.2-1b": _llama(2048, 16, 32, 8, 8192, 128256, 500000.0, 131072, tie_word_embeddings=True, head_dim=64),
    "qwen2.5-7b": _llama(
        3584, 28, 28, 4, 18944, 152064, 1000000.0, 32768,
        architectures=["Qwen2ForCausalLM"], model_type="qwen2", attention_bias=True, rms_norm_eps=1e-6,
    ),
    "qwen3-32b": _llama(
        5120, 64, 64, 8, 25600, 151936, 1000000.0, 40960,
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", head_dim=128, rms_norm_eps=1e-6, qk_norm=True,
    ),
    "tiny-qwen3": _llama(
        64, 2, 4, 2, 128, 1024, 10000.0, 2048,
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", head_dim=16, rms_norm_eps=1e-6, qk_norm=True,
    ),
    "qwen3-30b-a3b": _llama(
        2048, 48, 32, 4, 6144, 151936, 1000000.0, 40960,
        architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", head_dim=128, rms_norm_eps=1e-6, qk_norm=True,
        num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True,
        router_aux_loss_coef=0.001, decoder_sparse_step=1, mlp_only_layers=[],
    ),
    "tiny-qwen3-moe": _llama(
        64, 2, 4, 2, 128, 1024, 10000.0, 2048,
        architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", head_dim=16, rms_norm_eps=1e-6, qk_norm=True,
        num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, norm_topk_prob=True,
        router_aux_loss_coef=0.001, decoder_sparse_step=1, mlp_only_layers=[],
    ),
}


def load_arch_config(
    name_or_path: Union[str, Path], overrides: Optional[Dict[str, Any]] = None
) -> ArchConfig:
    """Resolve a preset name or a model directory into an :class:`ArchConfig` and apply overrides."""
    key = str(name_or_path)
    if key.lower().startswith(("deepseek", "tiny-deepseek")):
        from . import deepseek  # noqa: F401  (registers the DeepSeek presets and converters)
    if key.lower() in PRESETS:
        cfg = ArchConfig(json.loads(json.dumps(PRESETS[key.lower()])))
        cfg["_source"] = "preset"
    else:
        path = Path(key)
        cfg_file = path / "config.json" if path.is_dir() else path
        if not cfg_file.exists():
            raise FileNotFoundError(
                f"{name_or_path!r} is neither a built-in architecture preset ({sorted(PRESETS)}) "
                "nor a directory containing config.json"
            )
        with open(cfg_file) as fh:
            cfg = ArchConfig(json.load(fh))
        cfg["_source"] = str(cfg_file.parent)
        if cfg.get("text_config"):
            inner = dict(cfg["text_config"])
            inner.setdefault("architectures", cfg.get("architectures"))
            cfg = ArchConfig(inner)
    for k, v in (overrides or {}).items():
        cfg[k] = v
    if cfg.get("rope_theta") is None and isinstance(cfg.get("rope_parameters"), dict):
        cfg["rope_theta"] = cfg["rope_parameters"].get("rope_theta", 10000.0)
        if cfg.get("rope_scaling") is None and cfg["rope_parameters"].get("rope_type", "default") != "default":
            cfg["rope_scaling"] = {k: v for k, v in cfg["rope_parameters"].items() if k != "rope_theta"}
    if cfg.get("model_type") == "deepseek_v2":
        from . import deepseek  # noqa: F401,F811
    return cfg
